"""ctypes binding of the C ABI declared in include/sharq_b200.h.

There is no fallback: if the library is missing or an entry point fails, the
call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_longlong, c_size_t, c_void_p, c_char_p, POINTER
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "lib" / "libsharq_b200.so"
_LIB = None

# name -> (restype, argtypes); mirrors include/sharq_b200.h one to one
_P = c_void_p
SIGNATURES = {
    "sharq_version": (c_int, []),
    "sharq_last_error": (c_char_p, []),
    "sharq_get_sparse_nvfp4_buffer_sizes": (c_int, [c_int, c_int, c_int, POINTER(c_int64)]),
    "sharq_get_fused_sparse_residual_buffer_sizes": (c_int, [c_int, c_int, c_int, POINTER(c_int64)]),
    "sharq_fused_sparse_residual_quantize_x": (c_int, [_P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P]),
    "sharq_fused_sparse_residual_quantize_x_debug": (c_int, [_P, c_int, c_int, c_int, _P, _P, _P, _P, _P]),
    "sharq_prepare_workspace_bytes": (c_size_t, [c_int]),
    "sharq_prepare_timeouts": (c_int, []),
    "sharq_fused_rmsnorm_sparse_residual_quantize_x": (
        c_int, [_P, _P, c_float, c_int, c_int, c_int, _P, c_size_t, _P, _P, _P, _P, _P, _P, _P]),
    "sharq_scaled_sparse_residual_quantize_x": (
        c_int, [_P, c_int, c_int, c_int, _P, c_size_t, _P, _P, _P, _P, _P, _P, _P]),
    "sharq_fused_add_rmsnorm_sparse_residual_quantize_x": (
        c_int, [_P, _P, _P, _P, c_float, c_int, c_int, c_int, _P, c_size_t, _P, _P, _P, _P, _P, _P, _P]),
    "sharq_rope_inplace": (c_int, [_P, c_int, c_int, c_int, c_int, c_int, _P, _P, _P]),
    "sharq_scatter_add_scaled": (c_int, [_P, c_int, _P, _P, _P, c_int, c_int, _P]),
    "sharq_swiglu": (c_int, [_P, c_int, c_int, _P, _P]),
    "sharq_add_rmsnorm": (c_int, [_P, _P, _P, _P, c_float, c_int, c_int, _P, _P]),
    "sharq_swiglu_sparse_residual_quantize_x": (
        c_int, [_P, c_int, c_int, c_int, _P, _P, c_size_t, _P, _P, _P, _P, _P, _P, _P]),
    "sharq_quantize_w32_shared": (c_int, [_P, c_int, c_int, _P, _P, _P, _P]),
    "sharq_duplicate_sfa32_to_sfa16": (c_int, [_P, c_int, c_int, c_int, _P, _P]),
    "sharq_quantize_nvfp4": (c_int, [_P, c_int, c_int, _P, _P, _P]),
    "sharq_compress_sparse_a": (c_int, [_P, c_int, c_int, c_int, _P, _P, _P]),
    "sharq_matmul": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_float, _P, _P, c_float, _P, _P, _P]),
    "sharq_sparse_matmul": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_float, _P, c_float, _P, _P, _P]),
    "sharq_linear_gemm": (
        c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_float, _P, _P, _P, _P, _P]),
    "sharq_gemm_workspace_bytes": (c_size_t, [c_int, c_int]),
    "sharq_matmul_ws": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_float, _P, _P, c_float, _P, _P, c_size_t, _P, _P]),
    "sharq_sparse_matmul_ws": (
        c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_float, _P, c_float, _P, _P, c_size_t, _P, _P]),
    "sharq_linear_gemm_ws": (
        c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_float, _P, _P, _P, _P, c_size_t, _P, _P]),
    "sharq_set_gemm_tile_n": (c_int, [c_int]),
    "sharq_set_wait_limit_cycles": (c_int, [c_longlong]),
    "sharq_allreduce_bf16_multimem": (c_int, [_P, POINTER(c_void_p), c_int, c_int, c_size_t, c_int, _P, _P]),
    "sharq_allreduce_flag_bytes": (c_size_t, []),
    "sharq_allreduce_bf16_peer": (c_int, [POINTER(c_void_p), POINTER(c_void_p), c_int, c_int, c_size_t, c_int, _P, _P]),
    "sharq_grouped_sparse_residual_quantize_x": (c_int, [_P, _P, c_int, c_int, c_int, _P, c_int, _P, _P, _P, _P, _P, _P, _P, _P]),
    "sharq_grouped_swiglu_sparse_residual_quantize_x": (
        c_int, [_P, c_int, c_int, c_int, _P, _P, c_int, _P, _P, _P, _P, _P, _P, _P, _P]),
    "sharq_linear_gemm_grouped": (
        c_int, [_P, _P, _P, _P, _P, c_int, POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p), _P, _P, c_float, c_int,
                c_int, c_int, _P, _P, _P]),
    "sharq_moe_combine": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, _P]),
    "sharq_linear_gemm_scatter": (
        c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_float, _P, POINTER(c_void_p), c_int, c_int, _P, _P]),
    "sharq_tp_transition_state_bytes": (c_size_t, []),
    "sharq_tp_transition_workspace_bytes": (c_size_t, [c_int]),
    "sharq_tp_reduce_rmsnorm_prepare_allgather": (
        c_int, [_P, _P, _P, _P, c_float, c_int, c_int, c_int, _P, c_size_t, _P, _P, _P, _P, _P, c_longlong, _P,
                POINTER(c_void_p), c_int, c_int, _P, _P]),
    "sharq_fused_rmsnorm_sparse_residual_quantize_x_noalloc": (
        c_int, [_P, _P, c_float, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P]),
    "sharq_noalloc_max_rows": (c_int, []),
    "sharq_noalloc_last_error": (c_char_p, []),
}


class SharqError(RuntimeError):
    """An entry point of libsharq_b200 returned a non-zero status."""


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m sharq_b200._build` "
                "(there is no CPU or PyTorch fallback for the SharQ kernels)")
        L = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB


def check(status: int) -> None:
    if status != 0:
        raise SharqError(lib().sharq_last_error().decode())
