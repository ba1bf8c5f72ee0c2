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


def test_small_moe_decoder_tracks_bf16_reference():
    """Mixtral-shaped layer: bf16 router, top-2 of 4 experts, per-expert SharQ FFNs."""
    from sharq_b200 import ops
    from sharq_b200.decoder import DecoderConfig, SharqDecoder

    cfg = DecoderConfig(hidden=512, layers=2, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, experts=4, top_k=2)
    model = SharqDecoder(cfg, torch.device("cuda"), keep_reference=True, seed=5)
    ids = torch.randint(0, cfg.vocab, (2, 192), generator=torch.Generator().manual_seed(1)).cuda()
    got = model.prefill(ids)
    ops.check_device_errors()
    assert torch.isfinite(got).all()
    # One MoE block on the same normalised input, so that both sides route identically (with a
    # random router the logits are nearly tied and whole-stack outputs diverge through routing).
    import torch.nn.functional as F
    from sharq_b200.decoder import _route

    layer = model.layers[0]
    hn = torch.randn(384, cfg.hidden, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).cuda()
    mine = layer._moe(hn)
    routing, selected = _route(hn, layer.router, cfg.top_k)
    want = torch.zeros_like(hn)
    mask = F.one_hot(selected, num_classes=cfg.experts).permute(2, 1, 0)
    for e, (wg, wu, wd) in enumerate(layer.ref["experts"]):
        idx, top_x = torch.where(mask[e])
        cur = hn[top_x]
        want.index_add_(0, top_x, F.linear(F.silu(F.linear(cur, wg)) * F.linear(cur, wu), wd) * routing[top_x, idx, None])
    rel = (mine.float() - want.float()).norm() / want.float().norm()
    assert rel < 0.25, float(rel)
    cos = F.cosine_similarity(mine.float().flatten(), want.float().flatten(), dim=0)
    assert cos > 0.97, float(cos)
    plain = SharqDecoder(cfg, torch.device("cuda"), seed=5, fused_glue=False).prefill(ids)
    assert torch.equal(got, plain)  # SwiGLU fused into the w2 prepare changes no bit
