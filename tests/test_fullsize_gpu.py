"""Full-size checks at the benchmark's shapes (M = 2048 tokens, Llama-3-8B projections),
where the CPU oracle would take too long.  The reference here is plain PyTorch on the GPU:
the packed operands are dequantised with index arithmetic (no kernels of this project) and
multiplied in float32 (TF32 off); plus size-independent properties of the prepare output."""
import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu

E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def _ue4m3_table(device):
    v = []
    for c in range(256):
        e, m = (c >> 3) & 0xF, c & 7
        v.append(m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7))
    return torch.tensor(v, dtype=torch.float32, device=device)


def _scales(sf: torch.Tensor, rows: int, k: int, group: int, oracle) -> torch.Tensor:
    off = torch.from_numpy(oracle.sf_offsets(rows, k // group)).to(sf.device)
    return _ue4m3_table(sf.device)[sf[off].long()]  # [rows, k/group]


def _dequant_dense(q: torch.Tensor, sf: torch.Tensor, group: int, oracle) -> torch.Tensor:
    rows, kh = q.shape
    lut = torch.tensor(E2M1, dtype=torch.float32, device=q.device)
    vals = torch.stack([lut[(q & 0xF).long()], lut[(q >> 4).long()]], dim=-1).reshape(rows, kh * 2)
    s = _scales(sf, rows, kh * 2, group, oracle)
    return vals * s.repeat_interleave(group, dim=1)


def _dequant_sparse(a_comp, e, sfa, m: int, k: int, oracle) -> torch.Tensor:
    dev = a_comp.device
    lut = torch.tensor(E2M1, dtype=torch.float32, device=dev)
    am = (m + 127) // 128 * 128
    et = e.reshape(k // 256, am, 16)[:, :m, :].permute(1, 0, 2).reshape(m, k // 16)  # byte per 16 K
    nib = torch.stack([et & 0xF, et >> 4], dim=-1).reshape(m, k // 8).long()       # nibble per 8 K
    idx0, idx1 = nib & 3, nib >> 2
    pairs = a_comp.reshape(m, k // 8, 2)                                            # two kept pair-bytes
    out = torch.zeros(m, k // 8, 4, 2, dtype=torch.float32, device=dev)
    for j, idx in enumerate((idx0, idx1)):
        b = pairs[:, :, j]
        v = torch.stack([lut[(b & 0xF).long()], lut[(b >> 4).long()]], dim=-1)     # [m, k/8, 2]
        out.scatter_(2, idx[..., None, None].expand(-1, -1, 1, 2), v.unsqueeze(2))
    s = _scales(sfa, m, k, 32, oracle)
    return out.reshape(m, k) * s.repeat_interleave(32, dim=1)


@pytest.mark.parametrize("n,k,fused_norm", [(6144, 4096, True), (4096, 14336, False)])
def test_full_size_linear_against_torch(oracle, n, k, fused_norm):
    from sharq_b200 import ops

    torch.backends.cuda.matmul.allow_tf32 = False
    m = 2048
    x = H.config0_x(m, k, 11).cuda()
    w = H.config0_w(n, k, 11).cuda()
    w_scale = torch.clamp(w.abs().max().float() / 2688.0, min=1e-9)
    qw, sfs, sfd = ops.quantize_w32_shared((w / w_scale).to(torch.bfloat16))
    if fused_norm:
        gamma = H.config0_gamma(k, 11).cuda()
        a_comp, e, sfa, q_res, sf_res, scale = ops.fused_rmsnorm_sparse_residual_quantize_x(x, gamma, 1e-6, n)
        xf = x.float()
        x_in = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float()).to(torch.bfloat16).float()
    else:
        a_comp, e, sfa, q_res, sf_res, scale = ops.scaled_sparse_residual_quantize_x(x, n)
        x_in = x.float()
    y = ops.sharq_linear_gemm(a_comp, e, sfa, q_res, sf_res, qw, sfs, sfd, scale.reshape(1),
                              alpha_host=float(w_scale.item()))
    ops.check_device_errors()

    xs = _dequant_sparse(a_comp, e, sfa, m, k, oracle)
    xr = _dequant_dense(q_res, sf_res, 16, oracle)
    wd = _dequant_dense(qw, sfs, 32, oracle)
    assert torch.equal(wd, _dequant_dense(qw, sfd, 16, oracle))  # shared payload, two scale views

    # (1) GEMM: float32 product of the dequantised operands, tolerance 1e-2 relative Frobenius
    ref = ((xs + xr) @ wd.T) * (scale * w_scale)
    err = (y.float() - ref).norm() / ref.norm()
    assert err <= 1e-2, float(err)

    # (2) prepare properties: pair-wise 4:8 structure, reconstruction of the scaled activation
    kept = (xs.reshape(m, k // 8, 4, 2) != 0).any(-1).sum(-1)
    assert int(kept.max()) <= 2
    x_scaled = x_in / scale
    rec = (xs + xr - x_scaled).norm() / x_scaled.norm()
    assert rec < 0.06, float(rec)           # two-stage 4-bit quantisation error level
    only_main = (xs - x_scaled).norm() / x_scaled.norm()
    assert rec < only_main                   # the residual pass must improve on the main path alone

    # (3) whole layer against the unquantised bf16 linear: W4A4 error level, not garbage
    full = x_in @ w.float().T
    assert (y.float() - full).norm() / full.norm() < 0.2


def test_full_size_scaling_and_bias_properties():
    """alpha is linear, bias lands on the bf16 result, fused == two-launch composition up to one rounding."""
    from sharq_b200 import ops

    m, n, k = 2048, 4096, 4096
    x = H.config0_x(m, k, 5).cuda()
    w = H.config0_w(n, k, 5).cuda()
    qw, sfs, sfd = ops.quantize_w32_shared((w.float() / (w.float().abs().max() / 2688)).to(torch.bfloat16))
    a_comp, e, sfa, q_res, sf_res, scale = ops.scaled_sparse_residual_quantize_x(x, n)
    y1 = ops.sharq_linear_gemm(a_comp, e, sfa, q_res, sf_res, qw, sfs, sfd, 1.0)
    y2 = ops.sharq_linear_gemm(a_comp, e, sfa, q_res, sf_res, qw, sfs, sfd, 2.0)
    assert torch.equal(y2.float(), 2 * y1.float())  # power-of-two alpha commutes with bf16 rounding
    bias = torch.randn(n, device="cuda").to(torch.bfloat16)
    yb = ops.sharq_linear_gemm(a_comp, e, sfa, q_res, sf_res, qw, sfs, sfd, 1.0, bias=bias)
    assert torch.equal(yb, y1 + bias)
    ys = ops.sparse_matmul(a_comp, qw, e, sfa, sfs, m, n, k, alpha=1.0)
    y_two = ops.matmul_accum(q_res, qw, sf_res, sfd, 1.0, ys, 1.0)
    rel = (y_two.float() - y1.float()).norm() / y1.float().norm()
    assert rel < 4e-3  # differs only by the intermediate bf16 rounding of the sparse result
    ops.check_device_errors()
