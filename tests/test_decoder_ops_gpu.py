"""The decoder-layer element-wise kernels against the ATen compositions they replace
(HuggingFace's rotary embedding and act_fn(gate) * up as the reference's layer wrappers
run them): every intermediate is rounded to bf16 in the same places, so the outputs must be
bit-identical."""
import pytest
import torch
import torch.nn.functional as F

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _rope_tables(seq, d, theta=5e5):
    from sharq_b200.decoder import rope_tables

    return rope_tables(seq, d, theta, torch.device("cuda"))


@pytest.mark.parametrize("b,s,heads,kv,d", [(1, 2048, 32, 8, 128), (2, 160, 4, 2, 128), (3, 77, 5, 1, 64), (1, 33, 2, 2, 32)])
def test_rope_inplace_equals_aten(b, s, heads, kv, d):
    from sharq_b200 import ops
    from sharq_b200.decoder import apply_rope

    g = torch.Generator().manual_seed(b * s + d)
    width = (heads + 2 * kv) * d
    qkv = torch.randn(b * s, width, generator=g).to(torch.bfloat16).cuda()
    cos, sin = _rope_tables(s, d)
    nq, nk = heads * d, kv * d
    q = qkv[:, :nq].view(b, s, heads, d).transpose(1, 2)
    k = qkv[:, nq:nq + nk].view(b, s, kv, d).transpose(1, 2)
    want_q, want_k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    v_before = qkv[:, nq + nk:].clone()
    got = ops.rope_inplace_(qkv.clone(), heads + kv, d, cos, sin, s)
    assert torch.equal(got[:, :nq].view(b, s, heads, d).transpose(1, 2), want_q)
    assert torch.equal(got[:, nq:nq + nk].view(b, s, kv, d).transpose(1, 2), want_k)
    assert torch.equal(got[:, nq + nk:], v_before)  # value heads untouched


@pytest.mark.parametrize("m,f", [(2048, 14336), (300, 1024), (17, 128)])
def test_swiglu_equals_aten(m, f):
    from sharq_b200 import ops

    g = torch.Generator().manual_seed(m + f)
    gu = (3.0 * torch.randn(m, 2 * f, generator=g)).to(torch.bfloat16).cuda()
    gu[0, :8] = torch.tensor([0.0, -0.0, 30.0, -30.0, 88.0, -88.0, 1e-3, -1e-3], dtype=torch.bfloat16)
    want = F.silu(gu[:, :f]) * gu[:, f:]
    got = ops.swiglu(gu)
    assert torch.equal(got, want)


@pytest.mark.parametrize("m,f", [(2048, 14336), (130, 1024)])
def test_swiglu_prepare_equals_two_step(m, f):
    """SwiGLU fused with the scaled prepare against SwiGLU by ATen followed by the plain scaled prepare."""
    from sharq_b200 import ops

    gu = torch.cat((H.config0_x(m, f, 1), H.config0_x(m, f, 2)), dim=1).cuda()
    h = F.silu(gu[:, :f]) * gu[:, f:]
    want = ops.scaled_sparse_residual_quantize_x(h.contiguous(), 4096)
    got = ops.swiglu_sparse_residual_quantize_x(gu, 4096)
    for name, a, b in zip(("a_comp", "e", "sfa", "q_res", "sf_res", "scale"), got, want):
        assert torch.equal(a.reshape(-1), b.reshape(-1)), name


def test_decoder_fused_glue_equals_aten_glue():
    from sharq_b200 import ops
    from sharq_b200.decoder import DecoderConfig, SharqDecoder

    cfg = DecoderConfig(hidden=512, layers=2, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2000)
    dev = torch.device("cuda")
    ids = torch.randint(0, cfg.vocab, (2, 160), generator=torch.Generator().manual_seed(0)).cuda()
    fused = SharqDecoder(cfg, dev, seed=3, fused_glue=True).prefill(ids)
    plain = SharqDecoder(cfg, dev, seed=3, fused_glue=False).prefill(ids)
    ops.check_device_errors()
    assert torch.equal(fused, plain)


@pytest.mark.parametrize("m,k", [(2048, 4096), (130, 512), (64, 14336)])
def test_add_rmsnorm_prepare_equals_two_step(m, k):
    """Residual add folded into the row statistics pass against the ATen add followed by the
    RMSNorm-fused prepare: the sum and every prepared byte must be identical."""
    from sharq_b200 import ops

    x = H.config0_x(m, k, 11).cuda()
    r = H.config0_x(m, k, 12).cuda()
    gamma = H.config0_gamma(k, 3).cuda()
    total = x + r
    want = ops.fused_rmsnorm_sparse_residual_quantize_x(total, gamma, 1e-6, 4096)
    got = ops.fused_add_rmsnorm_sparse_residual_quantize_x(x, r, gamma, 1e-6, 4096)
    assert torch.equal(got[6], total)
    for name, a, b in zip(("a_comp", "e", "sfa", "q_res", "sf_res", "scale"), got[:6], want):
        assert torch.equal(a.reshape(-1), b.reshape(-1)), name


def test_scatter_add_scaled_equals_aten():
    from sharq_b200 import ops

    g = torch.Generator().manual_seed(4)
    out0 = torch.randn(1000, 512, generator=g).to(torch.bfloat16).cuda()
    rows = torch.randperm(1000, generator=g)[:300].cuda()
    y = torch.randn(300, 512, generator=g).to(torch.bfloat16).cuda()
    w = torch.rand(300, generator=g).to(torch.bfloat16).cuda()
    want = out0.clone().index_add_(0, rows, y * w[:, None])
    got = ops.scatter_add_scaled_(out0.clone(), y, rows, w)
    assert torch.equal(got, want)
    # indices outside the output are skipped, the other rows are still added
    bad = rows.clone()
    bad[0], bad[1] = -1, 1000
    want = out0.clone().index_add_(0, rows[2:], (y * w[:, None])[2:])
    assert torch.equal(ops.scatter_add_scaled_(out0.clone(), y, bad, w), want)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,k,with_residual", [(300, 4096, True), (64, 3584, True), (17, 8192, False), (1, 128, False)])
def test_add_rmsnorm_equals_the_float_composition(rows, k, with_residual):
    """bf16(S * rsqrt(mean(S^2) + eps) * gamma), S = bf16(x + residual): the sum S is bit-equal to the
    ATen add; the normalised values equal the float composition except where the order of the
    float sum of squares moves a value across a bf16 rounding boundary (at most one bf16 ulp, rare)."""
    from sharq_b200 import ops

    g = torch.Generator().manual_seed(rows + k)
    x = torch.randn(rows, k, generator=g).to(torch.bfloat16).cuda()
    x[:, :: 97] *= 20.0
    r = torch.randn(rows, k, generator=g).to(torch.bfloat16).cuda() if with_residual else None
    gamma = (1 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16).cuda()
    eps = 1e-5
    if with_residual:
        y, s = ops.add_rmsnorm(x, gamma, eps, residual=r)
        assert torch.equal(s, x + r)
    else:
        y = ops.add_rmsnorm(x, gamma, eps)
        s = x
    sd = s.double()
    want64 = sd * torch.rsqrt(sd.pow(2).mean(-1, keepdim=True) + eps) * gamma.double()
    sf = s.float()
    want = (sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()).to(torch.bfloat16)
    differing = (y != want).float().mean().item()
    assert differing <= 2e-3, differing
    # never further than one bf16 spacing (2^-8 relative) plus float noise from the exact value
    err = (y.double() - want64).abs()
    assert bool((err <= want64.abs() * 2.0 ** -8 + 1e-30).all())
