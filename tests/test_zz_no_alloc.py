"""The entry point for callers that cannot allocate device memory.

sharq_fused_rmsnorm_sparse_residual_quantize_x_noalloc keeps its scratch in a fixed array
inside the library, for hosts that own no spare workspace (all HBM already given to a pool,
or cudaMalloc forbidden on the calling thread).  It must produce exactly the bytes of the
workspace-taking entry point, also when the shared scratch still holds the previous call's
contents, so two calls with different shapes and data are made back to back and each is
compared with the existing entry point.  This file is named to be collected last.
"""
import ctypes

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _both(m, k, seed, scale_up):
    from sharq_b200 import _lib
    from tests.gpu_util import Buf, call, dptr, sizes5, stream_ptr

    n = 128
    x = (H.config0_x(m, k, seed).float() * scale_up).to(torch.bfloat16)
    gamma = H.config0_gamma(k, seed)
    xd, gd = x.cuda(), gamma.cuda()
    eps = ctypes.c_float(1e-6)

    ref = [Buf(s) for s in sizes5(m, n, k)]
    ws, ref_scale = Buf(256 + 4 * m), Buf(4)
    call("sharq_fused_rmsnorm_sparse_residual_quantize_x", dptr(xd), dptr(gd), eps, m, n, k, ws.ptr, 256 + 4 * m,
         *[b.ptr for b in ref], ref_scale.ptr, stream_ptr())

    new = [Buf(s) for s in sizes5(m, n, k)]
    new_scale = Buf(4)
    rc = _lib.lib().sharq_fused_rmsnorm_sparse_residual_quantize_x_noalloc(
        dptr(xd), dptr(gd), eps, m, n, k, *[b.ptr for b in new], new_scale.ptr, stream_ptr())
    assert rc == 0, _lib.lib().sharq_noalloc_last_error()
    for name, a, b in zip(("a_comp", "e", "sfa_sparse", "q_res", "sf_res"), new, ref):
        assert np.array_equal(a.get(), b.get()), name
    assert np.array_equal(new_scale.get(), ref_scale.get())


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    _both(700, 512, seed=1, scale_up=50.0)   # leaves a large absmax and 700 inv_rms values behind
    _both(130, 1024, seed=2, scale_up=0.01)  # smaller values, fewer rows: stale scratch must not matter


def test_noalloc_rejects_more_rows_than_its_scratch_holds():
    from sharq_b200 import _lib

    L = _lib.lib()
    cap = L.sharq_noalloc_max_rows()
    assert cap == 65536
    one = ctypes.c_void_p(16)  # never dereferenced: the size check comes first
    rc = L.sharq_fused_rmsnorm_sparse_residual_quantize_x_noalloc(one, one, ctypes.c_float(1e-6), cap + 1, 128, 128,
                                                                  one, one, one, one, one, None, None)
    assert rc != 0
    assert b"exceeds the built-in scratch capacity" in L.sharq_noalloc_last_error()
