"""The decoder stack on the SharQ linears against the same stack with unquantised bf16 weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("qkv_bias", [False, True])
def test_small_decoder_tracks_bf16_reference(qkv_bias):
    from sharq_b200 import ops
    from sharq_b200.decoder import DecoderConfig, SharqDecoder

    cfg = DecoderConfig(hidden=512, layers=2, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, qkv_bias=qkv_bias)
    model = SharqDecoder(cfg, torch.device("cuda"), keep_reference=True, seed=3)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (2, 160), generator=g).cuda()
    got = model.prefill(ids)
    ops.check_device_errors()
    want = model.prefill(ids, reference=True)
    assert got.shape == (2, cfg.vocab) and torch.isfinite(got).all()
    rel = (got - want).norm() / want.norm()
    assert rel < 0.35, float(rel)  # W4A4 error accumulated over two layers, far from uncorrelated (~1.4)
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)
    assert cos > 0.93, float(cos)
