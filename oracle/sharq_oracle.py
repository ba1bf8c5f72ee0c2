"""ctypes/numpy front end of the CPU oracle (oracle/sharq_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests, the smoke check and the bench's
cpu_baseline leg.  The product package never imports this module.

bf16 tensors travel as numpy uint16 arrays holding the raw bits; packed FP4,
metadata and scale buffers as uint8.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None


def build(force: bool = False) -> Path:
    """Compile oracle/sharq_oracle.c with gcc (via the Makefile) if needed."""
    so = _HERE / "libsharq_oracle.so"
    src = _HERE / "sharq_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libsharq_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(str(build()))
        L = _LIB
        L.sharq_sf_offset.restype = ctypes.c_size_t
        L.sharq_sf_offset.argtypes = [ctypes.c_int] * 3
        for name in ("sharq_sf_alloc_bytes", "sharq_e_bytes", "sharq_a_comp_bytes"):
            getattr(L, name).restype = ctypes.c_size_t
            getattr(L, name).argtypes = [ctypes.c_int, ctypes.c_int]
        L.sharq_bf16_to_f32.restype = ctypes.c_float
        L.sharq_bf16_to_f32.argtypes = [ctypes.c_uint16]
        L.sharq_f32_to_bf16.restype = ctypes.c_uint16
        L.sharq_f32_to_bf16.argtypes = [ctypes.c_float]
        L.sharq_e2m1_to_f32.restype = ctypes.c_float
        L.sharq_e2m1_to_f32.argtypes = [ctypes.c_uint8]
        L.sharq_f32_to_e2m1.restype = ctypes.c_uint8
        L.sharq_f32_to_e2m1.argtypes = [ctypes.c_float]
        L.sharq_ue4m3_to_f32.restype = ctypes.c_float
        L.sharq_ue4m3_to_f32.argtypes = [ctypes.c_uint8]
        L.sharq_f32_to_ue4m3.restype = ctypes.c_uint8
        L.sharq_f32_to_ue4m3.argtypes = [ctypes.c_float]
        L.sharq_oracle_tensor_scale.restype = ctypes.c_float
        L.sharq_oracle_tensor_scale.argtypes = [ctypes.c_float, ctypes.c_int]
        L.sharq_oracle_absmax_bf16.restype = ctypes.c_float
        L.sharq_oracle_absmax_bf16.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _u16(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint16, a.dtype
    return a


# ---------------------------------------------------------------- sizes / layout

def sf_alloc_bytes(rows: int, k: int) -> int:
    return int(lib().sharq_sf_alloc_bytes(rows, k))


def e_bytes(m: int, k: int) -> int:
    return int(lib().sharq_e_bytes(m, k))


def a_comp_bytes(m: int, k: int) -> int:
    return int(lib().sharq_a_comp_bytes(m, k))


def sf_offsets(rows: int, groups: int) -> np.ndarray:
    """[rows, groups] array of byte offsets into the blocked scale layout."""
    r = np.arange(rows)[:, None]
    g = np.arange(groups)[None, :]
    tiles_k = (groups + 3) // 4
    return ((r // 128) * tiles_k * 512 + (g // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + (g % 4))


# ---------------------------------------------------------------- bf16 helpers

def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------- kernels

def prepare(x_bits: np.ndarray, debug: bool = False):
    """K1: fused sparse + residual prepare of a pre-scaled bf16 activation.

    Returns (a_comp, e, sfa_sparse, q_res, sf_res), or with debug=True
    (q_sparse_dense, sfa_sparse, q_res, sf_res).
    """
    x_bits = _u16(x_bits)
    m, k = x_bits.shape
    assert k % 128 == 0
    sfa = np.empty(sf_alloc_bytes(m, k), np.uint8)
    sfr = np.empty(sf_alloc_bytes(m, k), np.uint8)
    qres = np.empty((m, k // 2), np.uint8)
    if debug:
        qs = np.empty((m, k // 2), np.uint8)
        lib().sharq_oracle_prepare(_p(x_bits), m, k, None, None, _p(qs), _p(sfa), _p(qres), _p(sfr))
        return qs, sfa, qres, sfr
    ac = np.empty(a_comp_bytes(m, k), np.uint8)
    e = np.empty(e_bytes(m, k), np.uint8)
    lib().sharq_oracle_prepare(_p(x_bits), m, k, _p(ac), _p(e), None, _p(sfa), _p(qres), _p(sfr))
    return ac, e, sfa, qres, sfr


def rmsnorm_row_stats(x_bits, gamma_bits, eps: float, inv_rms_in=None):
    """K2.  Returns (inv_rms, row_absmax, sum_sq).  With inv_rms_in the given
    values are used for the normalisation instead of the CPU 1/sqrt."""
    x_bits = _u16(x_bits)
    gamma_bits = _u16(gamma_bits)
    m, k = x_bits.shape
    inv = np.empty(m, np.float32)
    amax = np.empty(m, np.float32)
    ssq = np.empty(m, np.float32)
    inv_in = None if inv_rms_in is None else np.ascontiguousarray(inv_rms_in, dtype=np.float32)
    lib().sharq_oracle_rmsnorm_row_stats(_p(x_bits), _p(gamma_bits), ctypes.c_float(eps), m, k,
                                         _p(inv_in), _p(inv), _p(amax), _p(ssq))
    return inv, amax, ssq


def tensor_scale(amax: float, cuda_mode: bool = True) -> np.float32:
    return np.float32(lib().sharq_oracle_tensor_scale(ctypes.c_float(float(amax)), int(cuda_mode)))


def rmsnorm_prepare(x_bits, gamma_bits, inv_rms, scale: float):
    """K3 given per-row inv_rms and the tensor scale."""
    x_bits = _u16(x_bits)
    gamma_bits = _u16(gamma_bits)
    m, k = x_bits.shape
    inv = np.ascontiguousarray(inv_rms, dtype=np.float32)
    ac = np.empty(a_comp_bytes(m, k), np.uint8)
    e = np.empty(e_bytes(m, k), np.uint8)
    sfa = np.empty(sf_alloc_bytes(m, k), np.uint8)
    sfr = np.empty(sf_alloc_bytes(m, k), np.uint8)
    qres = np.empty((m, k // 2), np.uint8)
    lib().sharq_oracle_rmsnorm_prepare(_p(x_bits), _p(gamma_bits), _p(inv), ctypes.c_float(float(scale)),
                                       m, k, _p(ac), _p(e), None, _p(sfa), _p(qres), _p(sfr))
    return ac, e, sfa, qres, sfr


def absmax_bf16(x_bits) -> np.float32:
    x_bits = _u16(x_bits)
    return np.float32(lib().sharq_oracle_absmax_bf16(_p(x_bits), x_bits.size))


def scale_bf16(x_bits, scale: float, cuda_mode: bool = False) -> np.ndarray:
    """bf16(x / scale) as torch evaluates it for a bf16 tensor and a 0-dim float32 scale: on the CPU by the
    float32 scale, on a CUDA device (cuda_mode) by the scale rounded to bf16."""
    x_bits = _u16(x_bits)
    out = np.empty_like(x_bits)
    lib().sharq_oracle_scale_bf16(_p(x_bits), ctypes.c_float(float(scale)), ctypes.c_size_t(x_bits.size), _p(out),
                                  int(cuda_mode))
    return out


def quantize_w32_shared(w_bits):
    """K4+K5.  Returns (qw [n,k/2], sfw_sparse, sfw_dense)."""
    w_bits = _u16(w_bits)
    n, k = w_bits.shape
    assert k % 32 == 0
    qw = np.empty((n, k // 2), np.uint8)
    sfs = np.empty(sf_alloc_bytes(n, k), np.uint8)
    sfd = np.empty(sf_alloc_bytes(n, k), np.uint8)
    lib().sharq_oracle_quantize_w32_shared(_p(w_bits), n, k, _p(qw), _p(sfs), _p(sfd))
    return qw, sfs, sfd


def duplicate_sf32_to_sf16(sf32, rows: int, k: int) -> np.ndarray:
    sf32 = np.ascontiguousarray(sf32, dtype=np.uint8)
    out = np.empty(sf_alloc_bytes(rows, k), np.uint8)
    lib().sharq_oracle_duplicate_sf32_to_sf16(_p(sf32), rows, k, _p(out))
    return out


def quantize_dense_nvfp4(x_bits, fill: int = 0):
    """K6 (identity reorder, KE=0).  Unwritten scale bytes keep `fill`."""
    x_bits = _u16(x_bits)
    rows, k = x_bits.shape
    assert k % 16 == 0
    q = np.empty((rows, k // 2), np.uint8)
    sf = np.full(sf_alloc_bytes(rows, k), fill, np.uint8)
    lib().sharq_oracle_quantize_dense_nvfp4(_p(x_bits), rows, k, _p(q), _p(sf))
    return q, sf


def compress_sparse_a(a_dense):
    a_dense = np.ascontiguousarray(a_dense, dtype=np.uint8)
    m, kh = a_dense.shape
    k = kh * 2
    ac = np.empty(a_comp_bytes(m, k), np.uint8)
    e = np.empty(e_bytes(m, k), np.uint8)
    lib().sharq_oracle_compress_sparse_a(_p(a_dense), m, k, _p(ac), _p(e))
    return ac, e


def dequant_dense(q, sf, group: int) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    sf = np.ascontiguousarray(sf, dtype=np.uint8)
    rows, kh = q.shape
    out = np.empty((rows, kh * 2), np.float32)
    lib().sharq_oracle_dequant_dense(_p(q), _p(sf), rows, kh * 2, group, _p(out))
    return out


def dequant_sparse(a_comp, e, sfa, m: int, k: int) -> np.ndarray:
    a_comp = np.ascontiguousarray(a_comp, dtype=np.uint8)
    e = np.ascontiguousarray(e, dtype=np.uint8)
    sfa = np.ascontiguousarray(sfa, dtype=np.uint8)
    out = np.empty((m, k), np.float32)
    lib().sharq_oracle_dequant_sparse(_p(a_comp), _p(e), _p(sfa), m, k, _p(out))
    return out


# ---------------------------------------------------------------- GEMM reference

def gemm_reference(a_f32: np.ndarray, b_f32: np.ndarray, alpha: float = 1.0, c=None, beta: float = 0.0):
    """alpha * A @ B^T (+ beta * C) in float64 from dequantised operands
    (epilogue of kernels/src/nvfp4.cu:432-455: D = alpha*acc + beta*C)."""
    y = np.float64(alpha) * (a_f32.astype(np.float64) @ b_f32.astype(np.float64).T)
    if c is not None and beta != 0.0:
        y = y + np.float64(beta) * c.astype(np.float64)
    return y


def sharq_linear_reference(a_comp, e, sfa, q_res, sf_res, qw, sfw_sparse, m, n, k, alpha, bias=None,
                           double_round: bool = True):
    """model/qLinearLayer.py:130-154,177-179: y = G1(Q_res, W; beta=1, C=G2(A_comp, W)) + bias.
    With double_round the sparse result is rounded to bf16 before the dense pass adds
    to it, as the two reference launches do; without it a single rounding at the end."""
    w = dequant_dense(qw, sfw_sparse, 32)
    xs = dequant_sparse(a_comp, e, sfa, m, k)
    xr = dequant_dense(q_res, sf_res, 16)
    ys = np.float64(alpha) * (xs.astype(np.float64) @ w.astype(np.float64).T)
    yr = np.float64(alpha) * (xr.astype(np.float64) @ w.astype(np.float64).T)
    if double_round:
        ys = bf16_bits_to_f32(f32_to_bf16_bits(ys.astype(np.float32))).astype(np.float64)
    y = ys + yr
    if bias is not None:
        y = bf16_bits_to_f32(f32_to_bf16_bits(y.astype(np.float32))).astype(np.float64) + bias.astype(np.float64)
    return y
