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


@pytest.mark.parametrize("tokens", [384, 1000])
def test_grouped_experts_equal_the_per_expert_loop(tokens):
    """One grouped launch per step over all experts (sorted token slots, per-expert tensor scales, grouped
    GEMMs, ordered combine) gives the bits of the reference-style per-expert loop, and the layer can be
    captured in a CUDA graph (no host synchronisation)."""
    from sharq_b200 import ops
    from sharq_b200.decoder import DecoderConfig, SharqDecoder

    cfg = DecoderConfig(hidden=512, layers=1, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000, experts=4, top_k=2)
    model = SharqDecoder(cfg, torch.device("cuda"), seed=9)
    layer = model.layers[0]
    hn = torch.randn(tokens, cfg.hidden, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    hn[:, 7] *= 20
    layer.grouped_experts = False
    loop = layer._moe(hn).clone()
    layer.grouped_experts = True
    grouped = layer._moe(hn).clone()
    ops.check_device_errors()
    assert torch.isfinite(grouped).all()
    assert torch.equal(grouped, loop), float((grouped.float() - loop.float()).abs().max())
    # a skewed routing: every token to experts 1 and 3 (experts 0 and 2 get no rows)
    saved = layer.router.clone()
    layer.router.zero_()
    layer.router[1] = 1.0
    layer.router[3] = 0.5
    hn_pos = hn.abs()
    layer.grouped_experts = False
    loop = layer._moe(hn_pos).clone()
    layer.grouped_experts = True
    grouped = layer._moe(hn_pos).clone()
    assert torch.equal(grouped, loop)
    layer.router.copy_(saved)
    # graph capture
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer._moe(hn)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = layer._moe(hn)
    g.replay()
    torch.cuda.synchronize()
    ops.check_device_errors()
    layer.grouped_experts = False
    assert torch.equal(out, layer._moe(hn))


@pytest.mark.parametrize("world", [4, 8])
def test_padded_tensor_parallel_layout_matches_single_rank(world):
    """A Qwen-like shape that does not divide (7 query heads on 1 KV head, FFN 1920): the KV
    head is replicated, query heads are dealt with zero padding heads, the FFN is padded with
    zero rows.  The ranks run as threads of this process on one GPU and exchange their partial
    sums on the host (no collective, no kernel waits on another); the result must track the
    single-rank model."""
    import threading

    from sharq_b200 import ops
    from sharq_b200.decoder import DecoderConfig, SharqDecoder

    cfg = DecoderConfig(hidden=896, layers=2, heads=7, kv_heads=1, head_dim=128, ffn=1920, vocab=1500, qkv_bias=True)
    dev = torch.device("cuda")
    ids = torch.randint(0, cfg.vocab, (2, 96), generator=torch.Generator().manual_seed(3)).cuda()
    want = SharqDecoder(cfg, dev, seed=11).prefill(ids)

    barrier = threading.Barrier(world)
    parts, results, errors = [None] * world, [None] * world, []

    def hook_for(rank):
        def hook(t):
            torch.cuda.synchronize()
            parts[rank] = t
            barrier.wait()
            total = torch.stack([p.float() for p in parts]).sum(0).to(torch.bfloat16)
            torch.cuda.synchronize()
            barrier.wait()
            return total
        return hook

    def run(rank):
        try:
            torch.cuda.set_device(0)
            model = SharqDecoder(cfg, dev, world=world, rank=rank, seed=11, reduce_hook=hook_for(rank))
            results[rank] = model.prefill(ids)
            torch.cuda.synchronize()
        except Exception as exc:  # release the others instead of leaving them at the barrier
            errors.append(exc)
            barrier.abort()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not errors, errors
    ops.check_device_errors()
    for r in range(1, world):
        assert torch.equal(results[r], results[0])  # every rank ends with the same logits
    got = results[0]
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)
    rel = (got - want).norm() / want.norm()
    assert cos > 0.99 and rel < 0.15, (float(cos), float(rel))
