"""Bit-exact parity of the activation prepare kernels with the CPU oracle (through the C ABI)."""
import ctypes

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu

SHAPES = [(1, 128), (31, 128), (33, 256), (129, 384), (130, 512), (128, 1024), (512, 4096), (96, 3584)]
NAMES = ("a_comp", "e", "sfa_sparse", "q_res", "sf_res")


def _run_prepare(x: torch.Tensor, n: int = 256):
    from tests.gpu_util import Buf, call, dptr, sizes5, stream_ptr

    m, k = x.shape
    xd = x.cuda()
    bufs = [Buf(s) for s in sizes5(m, n, k)]
    call("sharq_fused_sparse_residual_quantize_x", dptr(xd), m, n, k, *[b.ptr for b in bufs], stream_ptr())
    return [b.get() for b in bufs]


def _compare(got, want, what):
    for name, g, w in zip(NAMES, got, want):
        w = np.asarray(w).reshape(-1)
        assert g.shape == w.shape, (what, name, g.shape, w.shape)
        bad = np.nonzero(g != w)[0]
        assert bad.size == 0, f"{what}: {name} differs at {bad.size} bytes, first {bad[:8]} got {g[bad[:8]]} want {w[bad[:8]]}"


@pytest.mark.parametrize("m,k", SHAPES)
def test_prepare_matches_oracle_config0(oracle, m, k):
    x = H.config0_x(m, k, seed=m + k)
    x = (x.float() / (x.float().abs().max() / 2688.0)).to(torch.bfloat16)  # pre-scaled, as the op expects
    got = _run_prepare(x)
    want = oracle.prepare(H.bits(x))
    _compare(got, want, f"config0 {m}x{k}")


@pytest.mark.parametrize("case", sorted(H.MATRIX_SUITE))
def test_prepare_matrix_suite(oracle, case):
    m, k = 8, 1024
    x = H.MATRIX_SUITE[case](m, k)
    got = _run_prepare(x)
    want = oracle.prepare(H.bits(x))
    _compare(got, want, case)


def test_prepare_extreme_values(oracle):
    m, k = 16, 256
    g = torch.Generator().manual_seed(5)
    x = torch.randn(m, k, generator=g)
    x[0] *= 1e-6        # scales clamp at 2^-9
    x[1] *= 1e5         # scales saturate at 448, values clamp at +-6
    x[2] = 0.0
    x[3, ::2] = -0.0
    x[4] = 2688.0
    x[5] = torch.tensor([3.0e-3, -2.9e-3] * (k // 2))  # UE4M3 subnormal range after /6
    xb = x.to(torch.bfloat16)
    got = _run_prepare(xb)
    want = oracle.prepare(H.bits(xb))
    _compare(got, want, "extremes")


def test_prepare_debug_payload(oracle):
    from tests.gpu_util import Buf, call, dptr, stream_ptr

    m, k, n = 40, 512, 128
    x = H.outlier_rich_x(m, k, 3)
    xd = x.cuda()
    sf = (m // 128 + 1) * 128 * k // 16
    bufs = [Buf(m * k // 2), Buf(sf), Buf(m * k // 2), Buf(sf)]
    call("sharq_fused_sparse_residual_quantize_x_debug", dptr(xd), m, n, k, *[b.ptr for b in bufs], stream_ptr())
    got = [b.get() for b in bufs]
    want = oracle.prepare(H.bits(x), debug=True)
    for name, g, w in zip(("q_sparse", "sfa", "q_res", "sf_res"), got, want):
        assert np.array_equal(g, np.asarray(w).reshape(-1)), name
    # the reference's invariant: never more than two non-zero bytes per 4-byte chunk
    assert H.raw_violation_rate(got[0].reshape(m, k // 2)) == 0.0


@pytest.mark.parametrize("m,k", [(1, 128), (37, 256), (130, 512), (512, 4096), (64, 14336), (3, 32768)])  # 32768: K/32 = 1024, the limit
def test_rmsnorm_prepare_matches_oracle(oracle, m, k):
    from tests.gpu_util import Buf, call, dptr, sizes5, stream_ptr

    n = 128
    x = H.config0_x(m, k, seed=7 * m + k)
    gamma = H.config0_gamma(k, seed=m)
    eps = 1e-6
    xd, gd = x.cuda(), gamma.cuda()
    bufs = [Buf(s) for s in sizes5(m, n, k)]
    ws_bytes = 256 + 4 * m
    ws = Buf(ws_bytes)
    scale = Buf(4)
    call("sharq_fused_rmsnorm_sparse_residual_quantize_x", dptr(xd), dptr(gd), ctypes.c_float(eps), m, n, k, ws.ptr,
         ws_bytes, *[b.ptr for b in bufs], scale.ptr, stream_ptr())
    got = [b.get() for b in bufs]
    wsh = ws.get()
    inv_gpu = wsh[256:256 + 4 * m].view(np.float32)
    amax_gpu = wsh[:4].view(np.float32)[0]
    scale_gpu = scale.get().view(np.float32)[0]

    # row statistics: the sum of squares is order-exact, rsqrtf is a <= 2 ulp approximation
    inv_cpu, _, _ = oracle.rmsnorm_row_stats(H.bits(x), H.bits(gamma), eps)
    ulp = np.abs(inv_gpu.view(np.int32).astype(np.int64) - inv_cpu.view(np.int32).astype(np.int64))
    assert ulp.max() <= 2, f"inv_rms differs by {ulp.max()} ulp"
    # everything downstream is bit-exact given the device's inv_rms
    _, amax_rows, _ = oracle.rmsnorm_row_stats(H.bits(x), H.bits(gamma), eps, inv_rms_in=inv_gpu)
    assert np.float32(amax_rows.max()) == amax_gpu
    want_scale = oracle.tensor_scale(amax_gpu, cuda_mode=True)
    assert want_scale == scale_gpu
    want = oracle.rmsnorm_prepare(H.bits(x), H.bits(gamma), inv_gpu, scale_gpu)
    _compare(got, want, f"rmsnorm {m}x{k}")


def test_tensor_scale_matches_torch_cuda():
    """clamp(amax / 2688, 1e-9) as ATen evaluates it on the device."""
    from tests.gpu_util import Buf, call, dptr, sizes5, stream_ptr

    m, k, n = 4, 128, 128
    for seed in range(6):
        x = (H.config0_x(m, k, seed).float() * (3.0 ** seed)).to(torch.bfloat16)
        xd = x.cuda()
        bufs = [Buf(s) for s in sizes5(m, n, k)]
        ws, scale = Buf(256 + 4 * m), Buf(4)
        call("sharq_scaled_sparse_residual_quantize_x", dptr(xd), m, n, k, ws.ptr, 256 + 4 * m, *[b.ptr for b in bufs],
             scale.ptr, stream_ptr())
        got = scale.get().view(np.float32)[0]
        want = torch.clamp(xd.abs().max().float() / (448.0 * 6.0), min=1e-9).item()
        assert got == np.float32(want)


@pytest.mark.parametrize("m,k", [(5, 128), (130, 384), (256, 4096)])
def test_scaled_prepare_matches_oracle(oracle, m, k):
    from tests.gpu_util import Buf, call, dptr, sizes5, stream_ptr

    n = 64
    x = H.config0_x(m, k, seed=m)
    xd = x.cuda()
    bufs = [Buf(s) for s in sizes5(m, n, k)]
    ws, scale = Buf(256 + 4 * m), Buf(4)
    call("sharq_scaled_sparse_residual_quantize_x", dptr(xd), m, n, k, ws.ptr, 256 + 4 * m, *[b.ptr for b in bufs],
         scale.ptr, stream_ptr())
    got = [b.get() for b in bufs]
    s = oracle.tensor_scale(oracle.absmax_bf16(H.bits(x)), cuda_mode=True)
    assert scale.get().view(np.float32)[0] == s
    want = oracle.prepare(oracle.scale_bf16(H.bits(x), s, cuda_mode=True))
    _compare(got, want, f"scaled {m}x{k}")


@pytest.mark.parametrize("cap", [64.0, 38.0, 84.0, 1.0, 255.0, 0.0030975341796875, 3.3895313892515355e38, 1.0e-30,
                                 7.52316384526264e-37, 1.7e9, 2.0 ** 100])
def test_scaled_prepare_division_is_ieee_for_every_bf16_value(cap):
    """The tensor-scale division bf16(x / scale) inside the scaled prepare equals the IEEE
    division ATen performs, for every finite bf16 value up to a given absmax (absmax values
    with short mantissas make exact rounding ties frequent; tiny and huge ones reach the
    subnormal guards).  Checked through the outputs: the scaled prepare must produce the bytes
    of the plain prepare applied to torch's own quotient."""
    from sharq_b200 import ops

    allv = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    keep = allv[torch.isfinite(allv.float()) & (allv.float().abs() <= cap)]
    assert keep.numel() > 0 and float(keep.float().abs().max()) > 0
    m, k = 1024, 512  # more than 256 K elements: the one-launch kernel, not the small-input path
    reps = (m * k + keep.numel() - 1) // keep.numel()
    g = torch.Generator().manual_seed(3)
    x = keep.repeat(reps)[torch.randperm(reps * keep.numel(), generator=g)][: m * k].reshape(m, k).contiguous().cuda()
    got = ops.scaled_sparse_residual_quantize_x(x, 128)
    scale = torch.clamp(x.abs().max().float() / (448.0 * 6.0), min=1e-9)
    assert torch.equal(got[5].reshape(()), scale.reshape(()))
    want = ops.fused_sparse_residual_quantize_x((x / scale).to(torch.bfloat16), 128)
    for name, a, b in zip(("a_comp", "e", "sfa_sparse", "q_res", "sf_res"), got[:5], want):
        assert torch.equal(a, b), (name, cap)


def test_prepare_rejects_bad_k():
    from sharq_b200 import ops

    x = torch.zeros(4, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 128"):
        ops.fused_sparse_residual_quantize_x(x, 64)
    with pytest.raises(RuntimeError, match="torch.bfloat16"):
        ops.fused_sparse_residual_quantize_x(torch.zeros(4, 128, device="cuda"), 64)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.fused_sparse_residual_quantize_x(torch.zeros(4, 128, dtype=torch.bfloat16), 64)


_DIGEST_SNIPPET = """
import hashlib, sys, torch
sys.path.insert(0, {root!r})
from sharq_b200 import ops
from tests import helpers as H
h = hashlib.sha1()
for m, k in ((1024, 4096), (300, 14336)):
    x = H.config0_x(m, k, 21).cuda(); r = H.config0_x(m, k, 22).cuda(); g = H.config0_gamma(k, 21).cuda()
    outs = list(ops.fused_rmsnorm_sparse_residual_quantize_x(x, g, 1e-6, 4096))
    outs += list(ops.fused_add_rmsnorm_sparse_residual_quantize_x(x, r, g, 1e-6, 4096))
    outs += list(ops.scaled_sparse_residual_quantize_x(x, 4096))
    for t in outs:
        t = t.reshape(-1) if t.dim() else t.reshape(1)
        h.update(t.view(torch.uint8).cpu().numpy().tobytes())
ops.check_device_errors()
print("DIGEST", h.hexdigest())
"""


def test_one_launch_and_separate_kernels_give_the_same_bytes():
    """The scaled prepares run as one cooperative launch for small tensors and as statistics +
    prepare kernels for large ones (or when SHARQ_PREPARE_FUSED=0): both must produce the same
    bytes.  The switch is read once per process, so each variant runs in its own interpreter."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = str(Path(__file__).resolve().parents[1])
    digests = []
    for fused in ("1", "0"):
        env = dict(os.environ, SHARQ_PREPARE_FUSED=fused)
        out = subprocess.run([sys.executable, "-c", _DIGEST_SNIPPET.format(root=root)], env=env, capture_output=True,
                             text=True, timeout=300)
        assert out.returncode == 0, out.stderr[-2000:]
        digests.append([l for l in out.stdout.splitlines() if l.startswith("DIGEST")][-1])
    assert digests[0] == digests[1]
