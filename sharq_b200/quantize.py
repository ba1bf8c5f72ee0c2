"""Host-side quantisation helpers with the names and meaning of the reference's
model/quantize.py (lines 43-44, 141-200), running on the sm_100a ops.

Differences in mechanism only: the activation helpers fold the tensor-scale passes
(amax, divide) into the kernels instead of running them as separate PyTorch ops; the
returned tuples are the same.
"""
from __future__ import annotations

import torch

from . import ops


def global_nvfp4_scale(x: torch.Tensor) -> torch.Tensor:
    """clamp(max|x| / (448*6), 1e-9) as a 0-dim float32 tensor (model/quantize.py:43-44)."""
    return torch.clamp(x.abs().max().float() / (448.0 * 6.0), min=1e-9)


@torch.no_grad()
def quantize_weight_shared_nvfp4(weight: torch.Tensor):
    """-> (q_weight, scale_weight_sparse, scale_weight_dense, scale) (model/quantize.py:149-153)."""
    scale = global_nvfp4_scale(weight)
    q, sfs, sfd = ops.quantize_w32_shared((weight / scale).to(torch.bfloat16).contiguous())
    return q, sfs, sfd, scale


@torch.no_grad()
def quantize_weight_nvfp4(weight: torch.Tensor):
    """-> (q_weight, scale_weight, scale) (model/quantize.py:141-145)."""
    scale = global_nvfp4_scale(weight)
    q, sf = ops.quantize_w_nvfp4((weight / scale).to(torch.bfloat16).contiguous())
    return q, sf, scale


@torch.no_grad()
def quantize_activation_nvfp4(x: torch.Tensor):
    """-> (q_x, scale_x, scale) (model/quantize.py:165-169)."""
    scale = global_nvfp4_scale(x)
    q, sf = ops.quantize_x_nvfp4((x / scale).to(torch.bfloat16).contiguous())
    return q, sf, scale


@torch.no_grad()
def quantize_activation_sparse_residual_nvfp4(x: torch.Tensor, out_features: int):
    """-> (a_comp, e, sfa_sparse, q_res, sf_res, scale) (model/quantize.py:179-183)."""
    return ops.scaled_sparse_residual_quantize_x(x.to(torch.bfloat16).contiguous(), out_features)


@torch.no_grad()
def quantize_activation_rmsnorm_sparse_residual_nvfp4(x: torch.Tensor, rmsnorm_weight: torch.Tensor,
                                                      rmsnorm_eps: float, out_features: int):
    """-> (a_comp, e, sfa_sparse, q_res, sf_res, scale) (model/quantize.py:187-200)."""
    return ops.fused_rmsnorm_sparse_residual_quantize_x(
        x.to(torch.bfloat16).contiguous(), rmsnorm_weight.to(torch.bfloat16).contiguous(), float(rmsnorm_eps),
        out_features)


def apply_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Unfused RMSNorm in PyTorch, used only by the dense NVFP4 baseline mode (model/quantize.py:47-51)."""
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * inv * weight.float()).to(torch.bfloat16)
