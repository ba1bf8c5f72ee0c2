"""The reference's `sharq_ops` operator set on top of the sm_100a C ABI.

Every function has the name, argument meaning, return shapes/dtypes and error
conditions of the op with that name in the reference's extension
(kernels/src/bindings.cpp:705-766 of the reference project): inputs are borrowed
contiguous CUDA tensors, outputs are new tensors from the torch caching allocator,
nothing is mutated, argument errors raise RuntimeError.  Kernels are enqueued on
torch's current stream of the input's device and the call returns without
synchronising.  PyTorch is used only for memory and streams; all arithmetic happens in
libsharq_b200.so.  There is no fallback path: a missing library raises ImportError.

Extra ops that the reference does not have (all optional for a drop-in):
  sharq_linear_forward           the op name the reference's vLLM plugin probes for
  sharq_linear_gemm              fused sparse+residual GEMM on a prepared activation
  scaled_sparse_residual_quantize_x   prepare with the host-side amax/divide folded in
"""
from __future__ import annotations

import contextlib
import ctypes
import os
from typing import Optional, Tuple

import torch

from . import _lib

_ERROR_FLAGS: dict[int, torch.Tensor] = {}
_PREPARE_TIMEOUTS_SEEN = 0


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device: torch.device):
    return torch.cuda.current_stream(device).cuda_stream


def _error_flag(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    flag = _ERROR_FLAGS.get(idx)
    if flag is None:
        flag = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _ERROR_FLAGS[idx] = flag
    return flag


def check_device_errors(device=None) -> None:
    """Synchronising check of the kernels' bounded waits: the GEMM / all-reduce error flag of each
    device and the grid barrier of the one-launch prepare."""
    global _PREPARE_TIMEOUTS_SEEN
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        torch.cuda.synchronize()
        n = int(_lib.lib().sharq_prepare_timeouts())
        if n > _PREPARE_TIMEOUTS_SEEN:
            seen, _PREPARE_TIMEOUTS_SEEN = _PREPARE_TIMEOUTS_SEEN, n
            raise RuntimeError(f"sharq_b200 prepare kernel: {n - seen} grid barrier wait(s) timed out; outputs are undefined")
    for idx, flag in list(_ERROR_FLAGS.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            raise RuntimeError(f"sharq_b200 GEMM kernel reported a timed-out wait (code {code}) on cuda:{idx}")


def _u8(n: int, device) -> torch.Tensor:
    return torch.empty(int(n), dtype=torch.uint8, device=device)


def _sf_bytes(rows: int, k: int) -> int:
    return (rows // 128 + 1) * 128 * k // 16


# --------------------------------------------------------------------------- sizes

def get_sparse_nvfp4_buffer_sizes(M: int, N: int, K: int) -> Tuple[int, int, int, int]:
    out = (ctypes.c_int64 * 4)()
    _lib.check(_lib.lib().sharq_get_sparse_nvfp4_buffer_sizes(M, N, K, out))
    return tuple(int(v) for v in out)


def get_fused_sparse_residual_buffer_sizes(M: int, N: int, K: int) -> Tuple[int, int, int, int, int]:
    out = (ctypes.c_int64 * 5)()
    _lib.check(_lib.lib().sharq_get_fused_sparse_residual_buffer_sizes(M, N, K, out))
    return tuple(int(v) for v in out)


# --------------------------------------------------------------------------- activation prepare

def _check_x(X: torch.Tensor, name: str = "X") -> Tuple[int, int]:
    _check(X.is_cuda, f"{name} must be a CUDA tensor")
    _check(X.is_contiguous(), f"{name} must be contiguous")
    _check(X.dtype == torch.bfloat16, f"{name} must be torch.bfloat16")
    _check(X.dim() == 2, f"{name} must be shaped [M, K]")
    return int(X.shape[0]), int(X.shape[1])


def fused_sparse_residual_quantize_x(X: torch.Tensor, N: int):
    """-> (A_comp, E, SFA_sparse, Q_res [M,K/2], SF_res)."""
    M, K = _check_x(X)
    _check(K % 128 == 0, f"fused_sparse_residual_quantize_x currently requires K to be a multiple of 128, got {K}")
    dev = X.device
    A_comp, E, SFA, Q_res, SF_res, _ = _prepare_buffers(M, K, dev)
    with _on_device(dev):
        _lib.check(_lib.lib().sharq_fused_sparse_residual_quantize_x(
            X.data_ptr(), M, N, K, A_comp.data_ptr(), E.data_ptr(), SFA.data_ptr(), Q_res.data_ptr(),
            SF_res.data_ptr(), _stream(dev)))
    return A_comp, E, SFA, Q_res, SF_res


def fused_sparse_residual_quantize_x_debug(X: torch.Tensor, N: int):
    """-> (Q_sparse dense payload [M,K/2], SFA_sparse, Q_res, SF_res)."""
    M, K = _check_x(X)
    _check(K % 128 == 0,
           f"fused_sparse_residual_quantize_x_debug currently requires K to be a multiple of 128, got {K}")
    dev = X.device
    Q_sparse = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    Q_res = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    SFA, SF_res = _u8(_sf_bytes(M, K), dev), _u8(_sf_bytes(M, K), dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().sharq_fused_sparse_residual_quantize_x_debug(
            _ptr(X), M, N, K, _ptr(Q_sparse), _ptr(SFA), _ptr(Q_res), _ptr(SF_res), _stream(dev)))
    return Q_sparse, SFA, Q_res, SF_res


def _round256(n: int) -> int:
    return (n + 255) & ~255


def _prepare_buffers(M: int, K: int, dev, extra: int = 0):
    """One allocation for the five prepare outputs (+ `extra` trailing bytes), returned as
    256-byte aligned views: (A_comp, E, SFA_sparse, Q_res [M,K/2], SF_res, tail)."""
    k256 = (K + 255) // 256 * 256
    sa = M * k256 // 4
    se = ((M + 127) // 128 * 128) * k256 // 16
    ssf = _sf_bytes(M, K)
    sq = M * (K // 2)
    o1 = _round256(sa)
    o2 = o1 + _round256(se)
    o3 = o2 + _round256(ssf)
    o4 = o3 + _round256(sq)
    o5 = o4 + _round256(ssf)
    buf = torch.empty(o5 + extra, dtype=torch.uint8, device=dev)
    return (buf[:sa], buf[o1:o1 + se], buf[o2:o2 + ssf], buf[o3:o3 + sq].view(M, K // 2), buf[o4:o4 + ssf],
            buf[o5:o5 + extra])


def _on_device(dev):
    """Context that makes `dev` current; free when it already is."""
    idx = dev.index
    if idx is None or idx == torch.cuda.current_device():
        return contextlib.nullcontext()
    return torch.cuda.device(dev)


def _scaled_prepare(X, gamma, eps, N, return_workspace, residual=None):
    M, K = int(X.shape[0]), int(X.shape[1])
    dev = X.device
    ws_bytes = 256 + 4 * M
    A_comp, E, SFA, Q_res, SF_res, tail = _prepare_buffers(M, K, dev, extra=_round256(ws_bytes) + 256)
    ws = tail[:ws_bytes]
    scale = tail[_round256(ws_bytes):_round256(ws_bytes) + 4].view(torch.float32).reshape(())
    L = _lib.lib()
    with _on_device(dev):
        if residual is not None:
            total = torch.empty_like(X)
            _lib.check(L.sharq_fused_add_rmsnorm_sparse_residual_quantize_x(
                X.data_ptr(), residual.data_ptr(), total.data_ptr(), gamma.data_ptr(), float(eps), M, N, K, ws.data_ptr(),
                ws_bytes, A_comp.data_ptr(), E.data_ptr(), SFA.data_ptr(), Q_res.data_ptr(), SF_res.data_ptr(),
                scale.data_ptr(), _stream(dev)))
            return A_comp, E, SFA, Q_res, SF_res, scale, total
        if gamma is not None:
            _lib.check(L.sharq_fused_rmsnorm_sparse_residual_quantize_x(
                X.data_ptr(), gamma.data_ptr(), float(eps), M, N, K, ws.data_ptr(), ws_bytes, A_comp.data_ptr(),
                E.data_ptr(), SFA.data_ptr(), Q_res.data_ptr(), SF_res.data_ptr(), scale.data_ptr(), _stream(dev)))
        else:
            _lib.check(L.sharq_scaled_sparse_residual_quantize_x(
                X.data_ptr(), M, N, K, ws.data_ptr(), ws_bytes, A_comp.data_ptr(), E.data_ptr(), SFA.data_ptr(),
                Q_res.data_ptr(), SF_res.data_ptr(), scale.data_ptr(), _stream(dev)))
    if return_workspace:
        return A_comp, E, SFA, Q_res, SF_res, scale, ws
    return A_comp, E, SFA, Q_res, SF_res, scale


def fused_rmsnorm_sparse_residual_quantize_x(X: torch.Tensor, rmsnorm_weight: torch.Tensor, rmsnorm_eps: float,
                                             N: int, return_workspace: bool = False):
    """-> (A_comp, E, SFA_sparse, Q_res, SF_res, scale [0-dim float32]).

    With return_workspace=True the scratch buffer is appended (bytes [256, 256+4M) hold
    the per-row inv_rms as float32)."""
    M, K = _check_x(X)
    w = rmsnorm_weight
    _check(w.is_cuda, "rmsnorm_weight must be a CUDA tensor")
    _check(w.is_contiguous(), "rmsnorm_weight must be contiguous")
    _check(w.dtype == torch.bfloat16, "rmsnorm_weight must be torch.bfloat16")
    _check(w.dim() == 1, "rmsnorm_weight must be shaped [K]")
    _check(w.device == X.device, "rmsnorm_weight must be on the same device as X")
    _check(w.shape[0] == K, f"rmsnorm_weight size mismatch: expected {K}, got {w.shape[0]}")
    _check(K % 128 == 0,
           f"fused_rmsnorm_sparse_residual_quantize_x currently requires K to be a multiple of 128, got {K}")
    _check(K // 32 <= 1024, f"fused_rmsnorm_sparse_residual_quantize_x requires K/32 <= 1024, got {K // 32}")
    return _scaled_prepare(X, w, rmsnorm_eps, N, return_workspace)


def fused_add_rmsnorm_sparse_residual_quantize_x(X: torch.Tensor, residual: torch.Tensor, rmsnorm_weight: torch.Tensor,
                                                 rmsnorm_eps: float, N: int):
    """-> (A_comp, E, SFA_sparse, Q_res, SF_res, scale, S) with S = X + residual (bf16, as the ATen
    add rounds) and the first six the RMSNorm-fused prepare of S.  The add rides on the row
    statistics pass, so S costs no extra read of X."""
    M, K = _check_x(X)
    _check(residual.is_cuda and residual.dtype == torch.bfloat16 and residual.is_contiguous()
           and tuple(residual.shape) == (M, K) and residual.device == X.device,
           "residual must be a contiguous CUDA bfloat16 tensor shaped like X on the same device")
    w = rmsnorm_weight
    _check(w.is_cuda and w.is_contiguous() and w.dtype == torch.bfloat16 and w.dim() == 1 and w.shape[0] == K
           and w.device == X.device, "rmsnorm_weight must be a contiguous CUDA bfloat16 tensor shaped [K] on X's device")
    _check(K % 128 == 0, f"fused_add_rmsnorm_sparse_residual_quantize_x requires K to be a multiple of 128, got {K}")
    _check(K // 32 <= 1024, f"fused_add_rmsnorm_sparse_residual_quantize_x requires K/32 <= 1024, got {K // 32}")
    return _scaled_prepare(X, w, rmsnorm_eps, N, False, residual=residual)


def rope_inplace_(qkv: torch.Tensor, heads: int, head_dim: int, cos: torch.Tensor, sin: torch.Tensor,
                  seq_len: int) -> torch.Tensor:
    """Rotary embedding in place on the first `heads` heads of every row of qkv [rows, width]
    (bf16, unit column stride); cos/sin bf16 [seq_len, head_dim]; position = row % seq_len.
    Equals `x * cos + rotate_half(x) * sin` of the ATen ops, head by head."""
    _check(qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 2 and qkv.stride(1) == 1,
           "qkv must be a CUDA bfloat16 matrix with unit column stride")
    for t, name in ((cos, "cos"), (sin, "sin")):
        _check(t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous() and tuple(t.shape) == (seq_len, head_dim),
               f"{name} must be a contiguous CUDA bfloat16 tensor shaped [seq_len, head_dim]")
    _check(heads * head_dim <= qkv.shape[1], "heads * head_dim exceeds the row width")
    dev = qkv.device
    with _on_device(dev):
        _lib.check(_lib.lib().sharq_rope_inplace(_ptr(qkv), int(qkv.shape[0]), int(qkv.stride(0)), int(seq_len), int(heads),
                                                 int(head_dim), _ptr(cos), _ptr(sin), _stream(dev)))
    return qkv


def scatter_add_scaled_(out: torch.Tensor, y: torch.Tensor, rows: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[rows[i]] += y[i] * w[i] (bf16, rows int64 and distinct): `out.index_add_(0, rows, y * w[:, None])`
    of the mixture-of-experts loop in one pass.  An index outside out's rows is skipped."""
    _check(out.is_cuda and out.dtype == torch.bfloat16 and out.dim() == 2 and out.is_contiguous(),
           "out must be a contiguous CUDA bfloat16 matrix")
    _check(y.is_cuda and y.dtype == torch.bfloat16 and y.dim() == 2 and y.is_contiguous() and y.shape[1] == out.shape[1],
           "y must be a contiguous CUDA bfloat16 matrix as wide as out")
    _check(rows.is_cuda and rows.dtype == torch.int64 and rows.is_contiguous() and rows.numel() == y.shape[0],
           "rows must be a contiguous CUDA int64 vector with one entry per row of y")
    _check(w.is_cuda and w.dtype == torch.bfloat16 and w.is_contiguous() and w.numel() == y.shape[0],
           "w must be a contiguous CUDA bfloat16 vector with one entry per row of y")
    _check(out.shape[1] % 8 == 0, "width must be a multiple of 8")
    with _on_device(out.device):
        _lib.check(_lib.lib().sharq_scatter_add_scaled(_ptr(out), int(out.shape[0]), _ptr(y), _ptr(rows), _ptr(w),
                                                       int(y.shape[0]), int(out.shape[1]), _stream(out.device)))
    return out


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up of a contiguous bf16 [M, 2F] activation (gate columns first) -> bf16 [M, F]."""
    _check(gate_up.is_cuda and gate_up.dtype == torch.bfloat16 and gate_up.dim() == 2 and gate_up.is_contiguous(),
           "gate_up must be a contiguous CUDA bfloat16 matrix")
    M, F2 = int(gate_up.shape[0]), int(gate_up.shape[1])
    _check(F2 % 16 == 0, f"gate_up width must be a multiple of 16, got {F2}")
    H = torch.empty((M, F2 // 2), dtype=torch.bfloat16, device=gate_up.device)
    with _on_device(gate_up.device):
        _lib.check(_lib.lib().sharq_swiglu(_ptr(gate_up), M, F2 // 2, _ptr(H), _stream(gate_up.device)))
    return H


def add_rmsnorm(X: torch.Tensor, rmsnorm_weight: torch.Tensor, rmsnorm_eps: float, residual: Optional[torch.Tensor] = None):
    """bf16(S * rsqrt(mean(S^2) + eps) * weight) with S = X + residual (bf16, as the ATen add rounds) or
    S = X: one launch (mean and products in float, one rounding per element).
    -> Y, or (Y, S) when a residual is given.  K % 8 == 0, K <= 8192."""
    _check(X.is_cuda and X.dtype == torch.bfloat16 and X.dim() == 2 and X.is_contiguous(),
           "X must be a contiguous CUDA bfloat16 matrix")
    M, K = int(X.shape[0]), int(X.shape[1])
    _check(K % 8 == 0 and K <= 8192, f"add_rmsnorm requires K to be a multiple of 8, at most 8192, got {K}")
    _check(rmsnorm_weight.is_cuda and rmsnorm_weight.dtype == torch.bfloat16 and rmsnorm_weight.is_contiguous()
           and rmsnorm_weight.numel() == K and rmsnorm_weight.device == X.device, "rmsnorm_weight must be bfloat16 [K] on X's device")
    if residual is not None:
        _check(residual.is_cuda and residual.dtype == torch.bfloat16 and residual.is_contiguous()
               and residual.shape == X.shape and residual.device == X.device, "residual must match X")
    Y = torch.empty_like(X)
    S = torch.empty_like(X) if residual is not None else None
    with _on_device(X.device):
        _lib.check(_lib.lib().sharq_add_rmsnorm(_ptr(X), _ptr(residual) if residual is not None else None,
                                                _ptr(S) if S is not None else None, _ptr(rmsnorm_weight), float(rmsnorm_eps),
                                                M, K, _ptr(Y), _stream(X.device)))
    return Y if residual is None else (Y, S)


def swiglu_sparse_residual_quantize_x(gate_up: torch.Tensor, N: int):
    """silu(gate) * up followed by the scaled prepare of the product, for down_proj:
    -> (A_comp, E, SFA_sparse, Q_res, SF_res, scale).  Equals
    scaled_sparse_residual_quantize_x(swiglu(gate_up), N) in two launches: the SwiGLU kernel
    also produces the tensor absmax, so the prepare needs no statistics pass."""
    _check(gate_up.is_cuda and gate_up.dtype == torch.bfloat16 and gate_up.dim() == 2 and gate_up.is_contiguous(),
           "gate_up must be a contiguous CUDA bfloat16 matrix")
    M, F2 = int(gate_up.shape[0]), int(gate_up.shape[1])
    K = F2 // 2
    _check(F2 % 2 == 0 and K % 128 == 0, f"swiglu_sparse_residual_quantize_x requires K to be a multiple of 128, got {K}")
    dev = gate_up.device
    ws_bytes = 256
    h_bytes = M * K * 2
    A_comp, E, SFA, Q_res, SF_res, tail = _prepare_buffers(M, K, dev, extra=512 + h_bytes)
    ws = tail[:ws_bytes]
    scale = tail[256:260].view(torch.float32).reshape(())
    H = tail[512:512 + h_bytes]
    with _on_device(dev):
        _lib.check(_lib.lib().sharq_swiglu_sparse_residual_quantize_x(
            _ptr(gate_up), M, int(N), K, _ptr(H), _ptr(ws), ws_bytes, _ptr(A_comp), _ptr(E), _ptr(SFA), _ptr(Q_res),
            _ptr(SF_res), _ptr(scale), _stream(dev)))
    return A_comp, E, SFA, Q_res, SF_res, scale


def scaled_sparse_residual_quantize_x(X: torch.Tensor, N: int):
    """Unscaled bf16 X -> (A_comp, E, SFA_sparse, Q_res, SF_res, scale): tensor scale,
    division and prepare in two launches (extra op, not in the reference)."""
    M, K = _check_x(X)
    _check(K % 128 == 0, f"scaled_sparse_residual_quantize_x requires K to be a multiple of 128, got {K}")
    return _scaled_prepare(X, None, 0.0, N, False)


# --------------------------------------------------------------------------- weights / dense quant

def quantize_w32_shared(W: torch.Tensor):
    """-> (QW [N,K/2], SFW_sparse, SFW_dense)."""
    _check(W.is_cuda, "W must be a CUDA tensor")
    _check(W.is_contiguous(), "W must be contiguous")
    _check(W.dtype == torch.bfloat16, "W must be torch.bfloat16")
    _check(W.dim() == 2, "W must be shaped [N, K]")
    N, K = int(W.shape[0]), int(W.shape[1])
    _check(K % 32 == 0, f"quantize_w32_shared requires K to be a multiple of 32, got {K}")
    dev = W.device
    QW = torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
    SFS, SFD = _u8(_sf_bytes(N, K), dev), _u8(_sf_bytes(N, K), dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().sharq_quantize_w32_shared(_ptr(W), N, K, _ptr(QW), _ptr(SFS), _ptr(SFD), _stream(dev)))
    return QW, SFS, SFD


def duplicate_sfa32_to_sfa16(SFA_sparse: torch.Tensor, M: int, N: int, K: int) -> torch.Tensor:
    _check(SFA_sparse.is_cuda, "SFA_sparse must be a CUDA tensor")
    _check(SFA_sparse.is_contiguous(), "SFA_sparse must be contiguous")
    _check(SFA_sparse.dtype == torch.uint8, "SFA_sparse must be torch.uint8")
    dev = SFA_sparse.device
    out = _u8(_sf_bytes(M, K), dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().sharq_duplicate_sfa32_to_sfa16(_ptr(SFA_sparse), M, N, K, _ptr(out), _stream(dev)))
    return out


def _quantize_nvfp4(X: torch.Tensor, what: str):
    rows, K = int(X.shape[0]), int(X.shape[1])
    if K % 16 != 0:
        raise RuntimeError(f"Unsupported hidden size in {what}")
    dev = X.device
    Q = torch.empty((rows, K // 2), dtype=torch.uint8, device=dev)
    SF = _u8(_sf_bytes(rows, K), dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().sharq_quantize_nvfp4(_ptr(X.contiguous()), rows, K, _ptr(Q), _ptr(SF), _stream(dev)))
    return Q, SF


def quantize_x_nvfp4(X: torch.Tensor):
    """Dense NVFP4 activation quantisation -> (QX [M,K/2], SFX)."""
    return _quantize_nvfp4(X, "reorder_quantize_x")


def quantize_w_nvfp4(W: torch.Tensor):
    """Dense NVFP4 weight quantisation -> (QW [N,K/2], SFW)."""
    return _quantize_nvfp4(W, "reorder_quantize_w")


def _check_identity(reorder_index: torch.Tensor, K: int, KE: int) -> None:
    _check(int(KE) == 0, "sharq_b200 supports the deprecated reorder ops only with KE == 0")
    _check(reorder_index.numel() == K, "reorder_index must have K entries")
    ident = torch.arange(K, dtype=reorder_index.dtype, device=reorder_index.device)
    _check(bool(torch.equal(reorder_index, ident)), "sharq_b200 supports the deprecated reorder ops only with the identity index")


def reorder_quantize_x(X: torch.Tensor, reorder_index: torch.Tensor, KE: int):
    """Deprecated alias of quantize_x_nvfp4 (identity index, KE == 0 only)."""
    _check_identity(reorder_index, int(X.shape[1]), KE)
    return quantize_x_nvfp4(X)


def reorder_quantize_w(W: torch.Tensor, reorder_index: torch.Tensor, KE: int):
    """Deprecated alias of quantize_w_nvfp4 (identity index, KE == 0 only)."""
    _check_identity(reorder_index, int(W.shape[1]), KE)
    return quantize_w_nvfp4(W)


def compress_sparse_a(A_q_dense: torch.Tensor, N: int):
    """Dense payload with <= 2 non-zero bytes per 4 -> (A_comp, E)."""
    _check(A_q_dense.is_cuda, "A_q_dense must be a CUDA tensor")
    _check(A_q_dense.is_contiguous(), "A_q_dense must be contiguous")
    _check(A_q_dense.dtype == torch.uint8, "A_q_dense must be torch.uint8")
    _check(A_q_dense.dim() == 2, "A_q_dense must be shaped [M, K/2]")
    M, K = int(A_q_dense.shape[0]), int(A_q_dense.shape[1]) * 2
    sa, se, _, _ = get_sparse_nvfp4_buffer_sizes(M, N, K)
    dev = A_q_dense.device
    A_comp, E = _u8(sa, dev), _u8(se, dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().sharq_compress_sparse_a(_ptr(A_q_dense), M, N, K, _ptr(A_comp), _ptr(E), _stream(dev)))
    return A_comp, E


# --------------------------------------------------------------------------- GEMMs

def _scale_ptr(scale: torch.Tensor, reference: torch.Tensor, name: str):
    _check(scale.is_cuda, f"{name} must be a CUDA tensor")
    _check(scale.is_contiguous(), f"{name} must be contiguous")
    _check(scale.dtype == torch.float32, f"{name} must be torch.float32")
    _check(scale.numel() == 1, f"{name} must contain exactly one element")
    _check(scale.device == reference.device, f"{name} must be on the same device as the inputs")
    return _ptr(scale)


def _gemm_scratch(M: int, N: int, dev):
    """Scratch that lets a small-M GEMM split K over the SMs: (tensor or None, bytes)."""
    if M > 128 or os.environ.get("SHARQ_GEMM_SPLIT_K", "1") == "0":
        return None, 0
    nbytes = int(_lib.lib().sharq_gemm_workspace_bytes(M, N))
    return (torch.empty(nbytes, dtype=torch.uint8, device=dev), nbytes) if nbytes else (None, 0)


def _dense_gemm(A, B, SFA, SFB, alpha, alpha_t, C_in, beta, out=None):
    M, N, K = int(A.shape[0]), int(B.shape[0]), int(A.shape[1]) * 2
    dev = A.device
    if out is None:
        D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    else:
        _check(out.is_cuda and out.device == dev and out.dtype == torch.bfloat16 and out.is_contiguous()
               and tuple(out.shape) == (M, N), "out must be a contiguous CUDA bfloat16 tensor shaped [M, N]")
        D = out
    ws, ws_bytes = _gemm_scratch(M, N, dev)
    with _on_device(dev):
        _lib.check(_lib.lib().sharq_matmul_ws(
            _ptr(A), _ptr(B), _ptr(SFA), _ptr(SFB), M, N, K, float(alpha),
            None if alpha_t is None else _scale_ptr(alpha_t, A, "scale"), _ptr(C_in), float(beta), _ptr(D),
            _ptr(ws), ws_bytes, _ptr(_error_flag(dev)), _stream(dev)))
    return D


def _check_c_in(C_in, A, M, N):
    _check(C_in.is_cuda, "C_in must be a CUDA tensor")
    _check(C_in.is_contiguous(), "C_in must be contiguous")
    _check(C_in.dtype == torch.bfloat16, "C_in must be torch.bfloat16")
    _check(C_in.dim() == 2, "C_in must be shaped [M, N]")
    _check(C_in.shape[0] == M and C_in.shape[1] == N,
           f"C_in shape mismatch: expected [{M}, {N}] got [{C_in.shape[0]}, {C_in.shape[1]}]")
    _check(C_in.device == A.device, "C_in must be on the same device as A")


def matmul(A, B, SFA, SFB, scale: float):
    """Dense NVFP4 GEMM -> bf16 [M,N] = scale * A.B^T."""
    return _dense_gemm(A, B, SFA, SFB, scale, None, None, 0.0)


def matmul_tensor_scale(A, B, SFA, SFB, scale: torch.Tensor, out: Optional[torch.Tensor] = None):
    """out (not in the reference's op): optional bf16 [M, N] tensor to write into."""
    return _dense_gemm(A, B, SFA, SFB, 1.0, scale, None, 0.0, out=out)


def matmul_accum(A, B, SFA, SFB, scale: float, C_in, beta: float = 1.0):
    """-> new bf16 [M,N] = scale * A.B^T + beta * C_in."""
    _check_c_in(C_in, A, int(A.shape[0]), int(B.shape[0]))
    return _dense_gemm(A, B, SFA, SFB, scale, None, C_in, beta)


def matmul_accum_tensor_scale(A, B, SFA, SFB, scale: torch.Tensor, C_in, beta: float = 1.0):
    _check_c_in(C_in, A, int(A.shape[0]), int(B.shape[0]))
    return _dense_gemm(A, B, SFA, SFB, 1.0, scale, C_in, beta)


def _sparse_gemm(name, A_comp, B, E, SFA, SFB, M, N, K, alpha, alpha_t, beta):
    _check(M > 0 and N > 0 and K > 0, "M, N, K must be positive")
    _check(beta == 0.0, f"{name} currently requires beta == 0")
    ts = (A_comp, B, E, SFA, SFB)
    _check(all(t.is_cuda for t in ts), f"{name} inputs must be CUDA tensors")
    _check(all(t.is_contiguous() for t in ts), f"{name} inputs must be contiguous")
    for t, nm in zip(ts, ("A_comp", "B", "E", "SFA", "SFB")):
        _check(t.dtype == torch.uint8, f"{nm} must be torch.uint8")
    _check(all(t.device == A_comp.device for t in ts), f"{name} inputs must be on the same device")
    ea, ee, esfa, esfb = get_sparse_nvfp4_buffer_sizes(M, N, K)
    _check(A_comp.numel() == ea, f"A_comp.numel() mismatch: expected {ea}, got {A_comp.numel()}")
    _check(E.numel() == ee, f"E.numel() mismatch: expected {ee}, got {E.numel()}")
    _check(SFA.numel() == esfa, f"SFA.numel() mismatch: expected {esfa}, got {SFA.numel()}")
    _check(SFB.numel() == esfb, f"SFB.numel() mismatch: expected {esfb}, got {SFB.numel()}")
    _check(B.dim() == 2, "B must be a 2D tensor shaped [N, K/2]")
    _check(B.shape[0] == N, f"B.size(0) mismatch: expected {N}, got {B.shape[0]}")
    _check(B.shape[1] == K // 2, f"B.size(1) mismatch: expected {K // 2}, got {B.shape[1]}")
    dev = A_comp.device
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    ws, ws_bytes = _gemm_scratch(M, N, dev)
    with _on_device(dev):
        _lib.check(_lib.lib().sharq_sparse_matmul_ws(
            _ptr(A_comp), _ptr(B), _ptr(E), _ptr(SFA), _ptr(SFB), M, N, K, float(alpha),
            None if alpha_t is None else _scale_ptr(alpha_t, A_comp, "alpha"), float(beta), _ptr(D),
            _ptr(ws), ws_bytes, _ptr(_error_flag(dev)), _stream(dev)))
    return D


def sparse_matmul(A_comp, B, E, SFA, SFB, M: int, N: int, K: int, alpha: float = 1.0, beta: float = 0.0):
    """Sparse NVFP4 GEMM on precompressed A -> bf16 [M,N]."""
    return _sparse_gemm("sparse_matmul", A_comp, B, E, SFA, SFB, M, N, K, alpha, None, beta)


def sparse_matmul_tensor_scale(A_comp, B, E, SFA, SFB, M: int, N: int, K: int, alpha: torch.Tensor,
                               beta: float = 0.0):
    return _sparse_gemm("sparse_matmul_tensor_scale", A_comp, B, E, SFA, SFB, M, N, K, 1.0, alpha, beta)


def sharq_linear_gemm(A_comp, E, SFA_sparse, Q_res, SF_res, QW, SFW_sparse, SFW_dense, alpha,
                      bias: Optional[torch.Tensor] = None, alpha_host: float = 1.0,
                      out: Optional[torch.Tensor] = None, scatter=None) -> Optional[torch.Tensor]:
    """Fused sparse-main + dense-residual GEMM on a prepared activation (one launch).
    alpha: python float or 1-element CUDA float32 tensor; the factor applied is
    alpha * alpha_host.  out: optional contiguous bf16 [M, N] tensor to write into.
    scatter=(rank_ptrs, rank, world): row-parallel output under tensor parallelism; the rows are dealt to the
    collection buffers of their owner GPUs (rank_ptrs: ctypes array of their mappings, see
    sharq_linear_gemm_scatter); nothing is returned."""
    M, K = int(Q_res.shape[0]), int(Q_res.shape[1]) * 2
    N = int(QW.shape[0])
    dev = Q_res.device
    ea, ee, esf, eq, _ = get_fused_sparse_residual_buffer_sizes(M, N, K)
    for t, want, nm in ((A_comp, ea, "A_comp"), (E, ee, "E"), (SFA_sparse, esf, "SFA_sparse"), (Q_res, eq, "Q_res"),
                        (SF_res, esf, "SF_res"), (QW, N * (K // 2), "QW"), (SFW_sparse, _sf_bytes(N, K), "SFW_sparse"),
                        (SFW_dense, _sf_bytes(N, K), "SFW_dense")):
        _check(t.is_cuda and t.device == dev and t.dtype == torch.uint8 and t.is_contiguous(),
               f"{nm} must be a contiguous CUDA uint8 tensor on the device of Q_res")
        _check(t.numel() == want, f"{nm}.numel() mismatch: expected {want}, got {t.numel()}")
    if bias is not None:
        _check(bias.is_cuda and bias.dtype == torch.bfloat16 and bias.numel() == N and bias.is_contiguous(),
               "bias must be a contiguous CUDA bfloat16 tensor with N elements")
    alpha_t = alpha if isinstance(alpha, torch.Tensor) else None
    if scatter is not None:
        _check(bias is None and out is None, "scatter mode takes neither bias nor out")
        rank_ptrs, rank, world = scatter
        with _on_device(dev):
            _lib.check(_lib.lib().sharq_linear_gemm_scatter(
                _ptr(A_comp), _ptr(E), _ptr(SFA_sparse), _ptr(Q_res), _ptr(SF_res), _ptr(QW), _ptr(SFW_sparse),
                _ptr(SFW_dense), M, N, K, float(alpha_host) if alpha_t is not None else float(alpha) * float(alpha_host),
                None if alpha_t is None else _scale_ptr(alpha_t, Q_res, "alpha"), rank_ptrs, int(rank), int(world),
                _ptr(_error_flag(dev)), _stream(dev)))
        return None
    if out is None:
        D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    else:
        _check(out.is_cuda and out.device == dev and out.dtype == torch.bfloat16 and out.is_contiguous()
               and tuple(out.shape) == (M, N), "out must be a contiguous CUDA bfloat16 tensor shaped [M, N]")
        D = out
    ws, ws_bytes = _gemm_scratch(M, N, dev)
    with _on_device(dev):
        _lib.check(_lib.lib().sharq_linear_gemm_ws(
            _ptr(A_comp), _ptr(E), _ptr(SFA_sparse), _ptr(Q_res), _ptr(SF_res), _ptr(QW), _ptr(SFW_sparse),
            _ptr(SFW_dense), M, N, K, float(alpha_host) if alpha_t is not None else float(alpha) * float(alpha_host),
            None if alpha_t is None else _scale_ptr(alpha_t, Q_res, "alpha"), _ptr(bias), _ptr(D),
            _ptr(ws), ws_bytes, _ptr(_error_flag(dev)), _stream(dev)))
    return D


def sharq_linear_forward(x: torch.Tensor, qw: torch.Tensor, sfw_sparse: torch.Tensor, sfw_dense: torch.Tensor,
                         weight_scale: float) -> torch.Tensor:
    """Whole SharQ linear on an unscaled bf16 activation [M,K] -> bf16 [M,N]: the optional
    op the reference's vLLM plugin calls when present (benchmarks/vllm/sharq.py:199-213).
    Two prepare launches and one GEMM launch; the activation scale stays on the device."""
    _check(x.dim() == 2, "x must be shaped [M, K]")
    x = x.contiguous().to(torch.bfloat16)
    N = int(qw.shape[0])
    a_comp, e, sfa, q_res, sf_res, scale = scaled_sparse_residual_quantize_x(x, N)
    return sharq_linear_gemm(a_comp, e, sfa, q_res, sf_res, qw, sfw_sparse, sfw_dense, scale.reshape(1),
                             alpha_host=float(weight_scale))


# --------------------------------------------------------------------------- grouped (mixture-of-experts) launches

def _check_grouped(x: torch.Tensor, unit_group: torch.Tensor, groups: int, name: str):
    _check(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous(),
           f"{name} must be a contiguous CUDA bfloat16 matrix")
    _check(x.shape[0] % 256 == 0 and x.shape[0] > 0, "the grouped activation must have a positive multiple of 256 rows")
    _check(unit_group.is_cuda and unit_group.dtype == torch.int32 and unit_group.is_contiguous()
           and unit_group.numel() == x.shape[0] // 256, "unit_group must be a contiguous CUDA int32 vector with one entry per 256 rows")
    _check(1 <= groups <= 16, "groups must be in [1, 16]")


def grouped_sparse_residual_quantize_x(X: torch.Tensor, unit_group: torch.Tensor, groups: int, N: int = 0,
                                       src_row: Optional[torch.Tensor] = None):
    """Scaled prepare of a grouped activation (rows sorted by group in 256-row units, see
    include/sharq_b200.h): -> (A_comp, E, SFA_sparse, Q_res, SF_res, scales [groups] float32), every group divided by
    its own tensor scale.  With src_row (int32, one entry per grouped row, < 0 = padding) X is the token-major
    activation and grouped row r is X[src_row[r]]."""
    if src_row is None:
        _check_grouped(X, unit_group, groups, "X")
        M = int(X.shape[0])
    else:
        _check(X.is_cuda and X.dtype == torch.bfloat16 and X.dim() == 2 and X.is_contiguous(),
               "X must be a contiguous CUDA bfloat16 matrix")
        _check(src_row.is_cuda and src_row.dtype == torch.int32 and src_row.is_contiguous(), "src_row must be contiguous CUDA int32")
        M = int(src_row.numel())
        _check(M % 256 == 0 and unit_group.numel() == M // 256 and unit_group.dtype == torch.int32,
               "src_row must have a multiple of 256 entries and unit_group one int32 per 256")
    K = int(X.shape[1])
    _check(K % 128 == 0, f"K must be a multiple of 128, got {K}")
    dev = X.device
    A_comp, E, SFA, Q_res, SF_res, tail = _prepare_buffers(M, K, dev, extra=512)
    amax = tail[:64]
    scales = tail[256:256 + 4 * groups].view(torch.float32)
    with _on_device(dev):
        _lib.check(_lib.lib().sharq_grouped_sparse_residual_quantize_x(
            _ptr(X), _ptr(src_row), M, int(N), K, _ptr(unit_group), int(groups), _ptr(amax), _ptr(A_comp), _ptr(E), _ptr(SFA), _ptr(Q_res),
            _ptr(SF_res), _ptr(scales), _stream(dev)))
    return A_comp, E, SFA, Q_res, SF_res, scales


def grouped_swiglu_sparse_residual_quantize_x(gate_up: torch.Tensor, unit_group: torch.Tensor, groups: int, N: int = 0):
    """silu(gate) * up of a grouped merged activation [M, 2K] and the scaled prepare of the product per group:
    -> (A_comp, E, SFA_sparse, Q_res, SF_res, scales [groups])."""
    _check_grouped(gate_up, unit_group, groups, "gate_up")
    M, K = int(gate_up.shape[0]), int(gate_up.shape[1]) // 2
    _check(gate_up.shape[1] % 2 == 0 and K % 128 == 0, f"K must be a multiple of 128, got {K}")
    dev = gate_up.device
    A_comp, E, SFA, Q_res, SF_res, tail = _prepare_buffers(M, K, dev, extra=512 + M * K * 2)
    amax = tail[:64]
    scales = tail[256:256 + 4 * groups].view(torch.float32)
    H = tail[512:512 + M * K * 2]
    with _on_device(dev):
        _lib.check(_lib.lib().sharq_grouped_swiglu_sparse_residual_quantize_x(
            _ptr(gate_up), M, int(N), K, _ptr(H), _ptr(unit_group), int(groups), _ptr(amax), _ptr(A_comp), _ptr(E), _ptr(SFA),
            _ptr(Q_res), _ptr(SF_res), _ptr(scales), _stream(dev)))
    return A_comp, E, SFA, Q_res, SF_res, scales


def linear_gemm_grouped(A_comp, E, SFA_sparse, Q_res, SF_res, weights, unit_group: torch.Tensor, alpha_vec: torch.Tensor,
                        alpha: float = 1.0) -> torch.Tensor:
    """Fused SharQ GEMM of a grouped activation against one weight per group in one launch.  weights: list of
    (QW [N, K/2], SFW_sparse, SFW_dense), all of the same shape; alpha_vec: CUDA float32 [groups]."""
    M, K = int(Q_res.shape[0]), int(Q_res.shape[1]) * 2
    groups = len(weights)
    N = int(weights[0][0].shape[0])
    dev = Q_res.device
    _check(M % 256 == 0, "the grouped activation must have a multiple of 256 rows")
    _check(alpha_vec.is_cuda and alpha_vec.dtype == torch.float32 and alpha_vec.is_contiguous() and alpha_vec.numel() == groups,
           "alpha_vec must be a contiguous CUDA float32 vector with one entry per group")
    for qw, sfs, sfd in weights:
        _check(tuple(qw.shape) == (N, K // 2) and qw.is_contiguous() and qw.device == dev, "weights must share one shape [N, K/2]")
    arr = ctypes.c_void_p * groups
    qws, sfss, sfds = (arr(*[w[i].data_ptr() for w in weights]) for i in range(3))
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    with _on_device(dev):
        _lib.check(_lib.lib().sharq_linear_gemm_grouped(
            _ptr(A_comp), _ptr(E), _ptr(SFA_sparse), _ptr(Q_res), _ptr(SF_res), groups, qws, sfss, sfds, _ptr(unit_group),
            _ptr(alpha_vec), float(alpha), M, N, K, _ptr(D), _ptr(_error_flag(dev)), _stream(dev)))
    return D


def moe_combine(y: torch.Tensor, dest: torch.Tensor, selected: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[t] = sum over the top_k slots of token t, in ascending expert order, of y[dest[t, j]] * w[t, j] (bf16 roundings as
    in the reference's index_add_ loop).  dest int32 [T, top_k], selected int64 [T, top_k], w bf16 [T, top_k]."""
    T, top_k = int(selected.shape[0]), int(selected.shape[1])
    _check(y.is_cuda and y.dtype == torch.bfloat16 and y.dim() == 2 and y.is_contiguous(), "y must be a contiguous CUDA bf16 matrix")
    _check(dest.dtype == torch.int32 and dest.is_contiguous() and dest.numel() == T * top_k, "dest must be int32 [T, top_k]")
    _check(selected.dtype == torch.int64 and selected.is_contiguous(), "selected must be contiguous int64 [T, top_k]")
    _check(w.dtype == torch.bfloat16 and w.is_contiguous() and w.numel() == T * top_k, "w must be contiguous bf16 [T, top_k]")
    out = torch.empty((T, int(y.shape[1])), dtype=torch.bfloat16, device=y.device)
    with _on_device(y.device):
        _lib.check(_lib.lib().sharq_moe_combine(_ptr(out), _ptr(y), _ptr(dest), _ptr(selected), _ptr(w), T, top_k,
                                                int(y.shape[1]), _stream(y.device)))
    return out


def set_gemm_tile_n(tile_n: int) -> None:
    """Force the GEMM tile width (0 = automatic, 128 or 256); test/tuning hook."""
    _lib.check(_lib.lib().sharq_set_gemm_tile_n(int(tile_n)))
