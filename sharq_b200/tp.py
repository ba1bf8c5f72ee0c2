"""Tensor-parallel SharQ linears: column/row sharding over one process per GPU
(`torch.distributed`, NCCL over NVLink) with an all-reduce after row-parallel layers.

The reference has no tensor parallelism (its model/parallel_utils.py only places whole
layers on GPUs and is never imported); this module is new.  Rules that keep a sharded
layer consistent with the single-GPU layer:

* the weight tensor scale is computed ONCE over the full weight, the full weight is
  divided by it, and only then sliced and quantised per shard.  quantize_w32_shared works
  per row and per 32-element group along K, so a shard's payload and scales equal the
  corresponding slice of the unsharded quantisation when N is cut at multiples of 128 and
  K at multiples of 128;
* column-parallel layers (q/k/v, gate/up) shard N; every rank prepares the same replicated
  activation; no collective;
* row-parallel layers (o_proj, down_proj) shard K; each rank prepares its own K-slice of
  the activation with its own tensor scale and produces a partial sum in bf16; the partial
  sums are all-reduced; the bias is added once, after the reduce.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

K_ALIGN = 128  # the prepare kernels need K % 128 == 0 per shard
N_ALIGN = 128  # scale-factor tiles cover 128 rows


def shard_bounds(total: int, world: int, rank: int, align: int) -> Tuple[int, int]:
    """[begin, end) of `rank`'s slice of `total`, which must split into `world` equal parts
    that are multiples of `align`."""
    if total % world != 0:
        raise ValueError(f"dimension {total} does not divide over {world} ranks; pad it first")
    part = total // world
    if part % align != 0:
        raise ValueError(f"per-rank slice {part} of {total} is not a multiple of {align}; pad it first")
    return rank * part, (rank + 1) * part


def padded_size(total: int, world: int, align: int) -> int:
    """Smallest size >= total that splits into `world` slices that are multiples of `align`
    (e.g. an FFN width of 18944 over 8 ranks becomes 19456)."""
    unit = world * align
    return (total + unit - 1) // unit * unit


def scaled_weight(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Full weight divided by its global tensor scale (bf16), and that scale."""
    scale = torch.clamp(weight.abs().max().float() / (448.0 * 6.0), min=1e-9)
    return (weight / scale).to(torch.bfloat16), scale


class _ShardedBase(nn.Module):
    def __init__(self, group=None):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


class ColumnParallelSharqLinear(_ShardedBase):
    """Shards out_features.  forward returns this rank's [M, N/world] slice."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, group=None, fused_gemm: bool = True):
        super().__init__(group)
        from . import ops
        from .qlinear import QLinearLayer

        n, k = weight.shape
        b, e = shard_bounds(n, self.world, self.rank, N_ALIGN)
        w_scaled, scale = scaled_weight(weight)
        q, sfs, sfd = ops.quantize_w32_shared(w_scaled[b:e].contiguous())
        self.local = QLinearLayer.from_quantized(k, e - b, q, sfs, sfd, scale,
                                                 bias=None if bias is None else bias[b:e], fused_gemm=fused_gemm)

    def prepare_input(self, x_2d, out_features_hint=None):
        return self.local.prepare_input(x_2d, out_features_hint)

    def prepare_input_rmsnorm(self, x_2d, w, eps, out_features_hint=None):
        return self.local.prepare_input_rmsnorm(x_2d, w, eps, out_features_hint)

    def apply_prepared(self, prepared):
        return self.local.apply_prepared(prepared)

    def forward(self, x):
        return self.local(x)


class RowParallelSharqLinear(_ShardedBase):
    """Shards in_features.  forward takes this rank's [M, K/world] slice of the activation
    and returns the all-reduced [M, N] output."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, group=None, fused_gemm: bool = True):
        super().__init__(group)
        from . import ops
        from .qlinear import QLinearLayer

        n, k = weight.shape
        b, e = shard_bounds(k, self.world, self.rank, K_ALIGN)
        w_scaled, scale = scaled_weight(weight)
        q, sfs, sfd = ops.quantize_w32_shared(w_scaled[:, b:e].contiguous())
        self.local = QLinearLayer.from_quantized(e - b, n, q, sfs, sfd, scale, bias=None, fused_gemm=fused_gemm)
        if bias is not None:
            self.register_buffer("bias", bias.to(q.device, torch.bfloat16))
        else:
            self.bias = None

    def reduce(self, y_partial: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(y_partial, op=dist.ReduceOp.SUM, group=self.group)
        if self.bias is not None:
            y_partial = y_partial + self.bias
        return y_partial

    def forward(self, x_local):
        return self.reduce(self.local(x_local))


def all_reduce_sum_(t: torch.Tensor, group=None) -> torch.Tensor:
    """In-place sum over the group (no-op without an initialised process group)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t
