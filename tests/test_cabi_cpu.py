"""The C-ABI library builds for sm_100a without a GPU, loads, and exports every symbol that
include/sharq_b200.h declares; the ctypes table matches the header; argument checks that
need no device work."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def header_symbols():
    text = (ROOT / "include" / "sharq_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sharq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from sharq_b200 import _build, _lib

    _build.build()
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    names = header_symbols()
    assert len(names) >= 17
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/sharq_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table out of sync with the header"


def test_size_queries_and_argument_errors_without_gpu():
    from sharq_b200 import _lib, ops

    assert _lib.lib().sharq_version() >= 100
    assert ops.get_fused_sparse_residual_buffer_sizes(512, 4096, 4096) == (524288, 131072, 163840, 1048576, 163840)
    assert ops.get_sparse_nvfp4_buffer_sizes(130, 256, 512) == (16640, 8192, 8192, 12288)
    assert _lib.lib().sharq_prepare_workspace_bytes(100) == 256 + 400
    L = _lib.lib()
    # K not a multiple of 128 is rejected before any launch
    rc = L.sharq_fused_sparse_residual_quantize_x(None, 4, 4, 96, None, None, None, None, None, None)
    assert rc != 0 and b"multiple of 128" in L.sharq_last_error()
    rc = L.sharq_sparse_matmul(None, None, None, None, None, 128, 128, 256, 1.0, None, 1.0, None, None, None)
    assert rc != 0 and b"beta == 0" in L.sharq_last_error()
    with pytest.raises(_lib.SharqError):
        _lib.check(L.sharq_set_gemm_tile_n(64))
    # tensor-parallel and grouped entry points reject shapes they cannot split, before any launch
    rc = L.sharq_tp_reduce_rmsnorm_prepare_allgather(None, None, None, None, 1e-6, 2048 + 128, 0, 4096, None, 0, None, None,
                                                     None, None, None, 0, None, None, 0, 8, None, None)
    assert rc != 0 and b"128 * world" in L.sharq_last_error()
    rc = L.sharq_linear_gemm_scatter(None, None, None, None, None, None, None, None, 2048, 4096, 512, 1.0, None, None, 0, 1,
                                     None, None)
    assert rc != 0 and b"world must be in [2" in L.sharq_last_error()
    rc = L.sharq_linear_gemm_grouped(None, None, None, None, None, 17, None, None, None, None, None, 1.0, 512, 256, 256, None,
                                     None, None)
    assert rc != 0 and b"groups must be in [1, 16]" in L.sharq_last_error()
    rc = L.sharq_grouped_sparse_residual_quantize_x(None, None, 300, 0, 256, None, 4, None, None, None, None, None, None, None,
                                                    None)
    assert rc != 0 and b"multiple of 256" in L.sharq_last_error()
    import ctypes

    one = ctypes.c_void_p(256)  # any non-null aligned address: the checks below fail before it is used
    rc = L.sharq_add_rmsnorm(one, None, None, one, 1e-6, 4, 8200, one, None)
    assert rc != 0 and b"at most 8192" in L.sharq_last_error()
    rc = L.sharq_add_rmsnorm(one, one, None, one, 1e-6, 4, 4096, one, None)
    assert rc != 0 and b"go together" in L.sharq_last_error()
    assert L.sharq_tp_transition_state_bytes() >= 256 and L.sharq_tp_transition_workspace_bytes(256) == 1024
    assert L.sharq_set_wait_limit_cycles(0) == 0 and L.sharq_set_wait_limit_cycles(-1) != 0


def test_ops_reject_cpu_tensors():
    import torch

    from sharq_b200 import ops

    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.fused_sparse_residual_quantize_x(torch.zeros(4, 128, dtype=torch.bfloat16), 64)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.quantize_w32_shared(torch.zeros(4, 128, dtype=torch.bfloat16))
