"""GEMM outputs against the REFERENCE's own CUTLASS GEMMs, and their times side by side.

oracle/_ref/libsharq_ref_gemm.so holds the reference's dense (kernels/src/nvfp4.cu) and
sparse (kernels/src/sparse_nvfp4.cu) block-scaled GEMMs compiled in place from its sources
(recipe: `python oracle/build_ref.py <reference checkout> --gemm`).  Both libraries are
called through their C entry points on the same device buffers.  The sparse GEMM and the
two-launch composition (sparse, then dense with beta = 1, model/qLinearLayer.py:130-154)
must be bit-identical to the reference; the single-launch fused GEMM rounds to bf16 once
instead of twice and must stay within the GEMM tolerance of the reference result.  The
tests skip when the library has not been built.

The timing test asserts with few iterations and prints one line per shape (run with -s)."""
import ctypes
from pathlib import Path

import pytest
import torch

from tests import helpers as H
from tests.gpu_util import call, dptr, stream_ptr

pytestmark = pytest.mark.gpu

REF_SO = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libsharq_ref_gemm.so"
TOL = 1e-2  # relative Frobenius norm


@pytest.fixture(scope="module")
def ref():
    if not REF_SO.exists():
        pytest.skip("oracle/_ref/libsharq_ref_gemm.so not built")
    lib = ctypes.CDLL(str(REF_SO))
    if not hasattr(lib, "ref_matmul_sparse"):
        pytest.skip("reference library was built without its GEMMs")
    return lib


class Case:
    """One linear's quantised operands on the device plus output buffers for both sides."""

    def __init__(self, m, n, k, seed=1):
        from sharq_b200 import ops

        self.m, self.n, self.k = m, n, k
        x = H.config0_x(m, k, seed).cuda()
        w = H.config0_w(n, k, seed).cuda()
        w = (w.float() / (w.float().abs().max() / 2688)).to(torch.bfloat16)
        self.qw, self.sfs, self.sfd = ops.quantize_w32_shared(w)
        self.a_comp, self.e, self.sfa, self.q_res, self.sf_res, scale = ops.scaled_sparse_residual_quantize_x(x, n)
        self.alpha = float(scale.item()) / 2688.0
        self.err = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.out = [torch.empty(m, n, dtype=torch.bfloat16, device="cuda") for _ in range(4)]

    # reference side (default stream)
    def ref_sparse(self, lib, d):
        return lib.ref_matmul_sparse(dptr(self.a_comp), dptr(self.qw), dptr(self.e), self.m, self.n, self.k, dptr(d),
                                     dptr(self.sfa), dptr(self.sfs), ctypes.c_float(self.alpha))

    def ref_dense(self, lib, c, d, beta):
        return lib.ref_matmul_dense(dptr(self.q_res), dptr(self.qw), self.m, self.n, self.k, dptr(c), dptr(d),
                                    dptr(self.sf_res), dptr(self.sfd), ctypes.c_float(self.alpha), ctypes.c_float(beta))

    # this project's side, straight through the C ABI
    def my_sparse(self, d):
        call("sharq_sparse_matmul", dptr(self.a_comp), dptr(self.qw), dptr(self.e), dptr(self.sfa), dptr(self.sfs), self.m,
             self.n, self.k, self.alpha, None, 0.0, dptr(d), dptr(self.err), stream_ptr())

    def my_dense(self, c, d, beta):
        call("sharq_matmul", dptr(self.q_res), dptr(self.qw), dptr(self.sf_res), dptr(self.sfd), self.m, self.n, self.k,
             self.alpha, None, dptr(c) if c is not None else None, beta, dptr(d), dptr(self.err), stream_ptr())

    def my_fused(self, d):
        call("sharq_linear_gemm", dptr(self.a_comp), dptr(self.e), dptr(self.sfa), dptr(self.q_res), dptr(self.sf_res),
             dptr(self.qw), dptr(self.sfs), dptr(self.sfd), self.m, self.n, self.k, self.alpha, None, None, dptr(d),
             dptr(self.err), stream_ptr())


@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (300, 384, 1024), (2048, 4096, 4096), (1024, 6144, 4096),
                                   (2048, 28672, 4096), (8192, 4096, 14336), (2100, 4096, 4096)])
def test_gemms_equal_reference_cutlass(ref, m, n, k):
    c = Case(m, n, k)
    ys, yd, ms, md = c.out
    with torch.cuda.stream(torch.cuda.default_stream()):
        assert c.ref_sparse(ref, ys) == 0
        assert c.ref_dense(ref, ys, yd, 1.0) == 0
        torch.cuda.synchronize()
        c.my_sparse(ms)
        c.my_dense(ms, md, 1.0)
        fused = torch.empty_like(md)
        c.my_fused(fused)
        dense_only_ref, dense_only = torch.empty_like(md), torch.empty_like(md)
        assert c.ref_dense(ref, dense_only_ref, dense_only_ref, 0.0) == 0
        c.my_dense(None, dense_only, 0.0)
        torch.cuda.synchronize()
    assert int(c.err.item()) == 0
    assert torch.equal(ms, ys), "sparse GEMM differs from the reference's CUTLASS sparse GEMM"
    assert torch.equal(dense_only, dense_only_ref), "dense GEMM differs from the reference's CUTLASS dense GEMM"
    assert torch.equal(md, yd), "two-launch composition differs from the reference's"
    rel = float((fused.float() - yd.float()).norm() / yd.float().norm())
    assert rel <= TOL, rel


def _time_us(fn, iters=30):
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


STANDALONE_SLACK = 1.6  # stand-alone dense / sparse GEMM time allowed relative to the reference's CUTLASS kernels
SHAPES_M2048 = {"o_proj": (4096, 4096), "qkv_proj": (6144, 4096), "down_proj": (4096, 14336), "gate_up_proj": (28672, 4096)}


@pytest.mark.parametrize("name", list(SHAPES_M2048))
def test_fused_launch_beats_reference_pair(ref, name):
    """The single fused launch must be faster than the reference's sparse + dense(beta = 1) pair
    on the same device and buffers at the Llama-3-8B projection shapes, M = 2048; the
    stand-alone dense and sparse variants must stay within STANDALONE_SLACK of the reference kernels.
    Few iterations: this is an assertion, not a benchmark.  One line per shape with -s."""
    n, k = SHAPES_M2048[name]
    m = 2048
    with torch.cuda.stream(torch.cuda.default_stream()):
        c = Case(m, n, k)
        ys, yd, ms, md = c.out
        t = {
            "ref_sparse": _time_us(lambda: c.ref_sparse(ref, ys), 10),
            "ref_dense_beta1": _time_us(lambda: c.ref_dense(ref, ys, yd, 1.0), 10),
            "my_sparse": _time_us(lambda: c.my_sparse(ms), 10),
            "my_dense_beta1": _time_us(lambda: c.my_dense(ms, md, 1.0), 10),
            "my_fused": _time_us(lambda: c.my_fused(md), 10),
        }
    pair = t["ref_sparse"] + t["ref_dense_beta1"]
    print(f"\n{name} M={m} N={n} K={k} us: " + " ".join(f"{k_}={v:.1f}" for k_, v in t.items())
          + f" | reference pair {pair:.1f} -> fused is {pair / t['my_fused']:.2f}x", flush=True)
    assert int(c.err.item()) == 0
    assert t["my_fused"] < pair, t
    assert t["my_sparse"] <= STANDALONE_SLACK * t["ref_sparse"], t
    assert t["my_dense_beta1"] <= STANDALONE_SLACK * t["ref_dense_beta1"], t
