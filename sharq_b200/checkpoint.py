"""SharQ weight checkpoints: conversion of bf16 linear weights to the on-disk tensors the
reference's vLLM plugin loads, and slicing of those tensors for tensor parallelism.

On-disk format (benchmarks/vllm/sharq_quant.py:63-158 of the reference): per linear layer
`<name>.QW` (uint8 [N, K/2], e2m1 pairs), `<name>.SFW_sparse` and `<name>.SFW_dense` (uint8,
blocked UE4M3 scales per 32 and per 16 along K), `<name>.scale_b` (float32 scalar, the tensor
scale the weight was divided by), optional `<name>.bias`; q/k/v are merged into `qkv_proj`
and gate/up into `gate_up_proj`; every other tensor is kept as it is.

Slicing for tensor parallelism needs no re-quantisation: `quantize_w32_shared` works per
row and per 32-element group along K and the tensor scale is global, so the payload and
scale bytes of a shard are a slice of the full tensors when rows are cut at multiples of 128
and K at multiples of 128.  The scale buffers are blocked: 128-row bands, each band a run of
512-byte tiles (4 scales x 128 rows) along K, plus one spare band of zeros at the end.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

NVFP4_DENOM = 448.0 * 6.0
ROW_ALIGN = 128  # scale tiles cover 128 rows
K_ALIGN = 128    # one sparse scale tile covers 128 K (4 groups of 32)


# --------------------------------------------------------------------------- quantisation

def quantize_linear_weight(weight: torch.Tensor) -> Dict[str, torch.Tensor]:
    """bf16 [N, K] -> {QW, SFW_sparse, SFW_dense, scale_b} on the weight's device (CUDA).
    Same steps as quantize_layer_weights (sharq_quant.py:63-78)."""
    from . import ops

    w = weight.to(torch.bfloat16).contiguous()
    scale_b = torch.clamp(w.abs().max().float() / NVFP4_DENOM, min=1e-9)
    qw, sfs, sfd = ops.quantize_w32_shared((w / scale_b).to(torch.bfloat16))
    return {"QW": qw, "SFW_sparse": sfs, "SFW_dense": sfd, "scale_b": scale_b.reshape(1)}


def convert_state_dict(state: Dict[str, torch.Tensor], num_layers: int, device="cuda",
                       prefix: str = "model.layers") -> Dict[str, torch.Tensor]:
    """HuggingFace Llama/Qwen2 state dict -> SharQ checkpoint tensors (CPU), with merged
    `self_attn.qkv_proj` and `mlp.gate_up_proj` (sharq_quant.py:100-150).  Tensors that are
    not decoder linears pass through unchanged."""
    out: Dict[str, torch.Tensor] = {}
    used = set()

    def take(name: str) -> Optional[torch.Tensor]:
        if name in state:
            used.add(name)
            return state[name]
        return None

    def emit(base: str, weights: Sequence[torch.Tensor], biases: Sequence[Optional[torch.Tensor]]):
        w = torch.cat([t.to(device) for t in weights], dim=0) if len(weights) > 1 else weights[0].to(device)
        for key, value in quantize_linear_weight(w).items():
            out[f"{base}.{key}"] = value.cpu()
        if all(b is not None for b in biases):
            out[f"{base}.bias"] = torch.cat([b for b in biases], dim=0).cpu() if len(biases) > 1 else biases[0].cpu()

    for i in range(num_layers):
        p = f"{prefix}.{i}"
        groups = ((f"{p}.self_attn.qkv_proj", [f"{p}.self_attn.{n}" for n in ("q_proj", "k_proj", "v_proj")]),
                  (f"{p}.self_attn.o_proj", [f"{p}.self_attn.o_proj"]),
                  (f"{p}.mlp.gate_up_proj", [f"{p}.mlp.{n}" for n in ("gate_proj", "up_proj")]),
                  (f"{p}.mlp.down_proj", [f"{p}.mlp.down_proj"]))
        for base, parts in groups:
            weights = [take(f"{n}.weight") for n in parts]
            if any(w is None for w in weights):
                raise KeyError(f"missing weight among {parts}")
            emit(base, weights, [take(f"{n}.bias") for n in parts])
    for name, tensor in state.items():
        if name not in used:
            out[name] = tensor
    return out


def save_checkpoint(tensors: Dict[str, torch.Tensor], path: str) -> None:
    """Write `model.safetensors`-style file at `path` (safetensors, as the reference does)."""
    from safetensors.torch import save_file

    save_file({k: v.contiguous() for k, v in tensors.items()}, path)


def load_checkpoint(path: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return load_file(path)


# --------------------------------------------------------------------------- scale-buffer geometry

def sf_bytes(rows: int, k: int) -> int:
    """Allocation of one blocked scale buffer for a [rows, k] matrix (both the 16-group view
    and the 32-group view duplicated into it use this size)."""
    return (rows // 128 + 1) * 128 * k // 16


def _band_bytes(k: int, group: int) -> int:
    return (k // group // 4) * 512


def slice_scale_rows(sf: torch.Tensor, n: int, k: int, group: int, pieces: Iterable[Tuple[int, int]]) -> torch.Tensor:
    """Rows [b, e) of every piece (multiples of 128) of a blocked scale buffer, concatenated,
    in a fresh buffer sized for the result."""
    band = _band_bytes(k, group)
    chunks, rows = [], 0
    for b, e in pieces:
        if b % ROW_ALIGN or e % ROW_ALIGN or not 0 <= b <= e <= n:
            raise ValueError(f"row slice [{b}, {e}) must lie in [0, {n}] at multiples of {ROW_ALIGN}")
        chunks.append(sf[b // 128 * band:e // 128 * band])
        rows += e - b
    out = torch.zeros(sf_bytes(rows, k), dtype=torch.uint8, device=sf.device)
    body = torch.cat(chunks) if chunks else sf[:0]
    out[:body.numel()] = body
    return out


def slice_scale_k(sf: torch.Tensor, n: int, k: int, group: int, kb: int, ke: int) -> torch.Tensor:
    """K range [kb, ke) (multiples of 128) of a blocked scale buffer."""
    if kb % K_ALIGN or ke % K_ALIGN or not 0 <= kb <= ke <= k:
        raise ValueError(f"K slice [{kb}, {ke}) must lie in [0, {k}] at multiples of {K_ALIGN}")
    bands = (n + 127) // 128
    tiles = k // group // 4
    t0, t1 = kb // group // 4, ke // group // 4
    body = sf[:bands * tiles * 512].view(bands, tiles, 512)[:, t0:t1, :].reshape(-1)
    out = torch.zeros(sf_bytes(n, ke - kb), dtype=torch.uint8, device=sf.device)
    out[:body.numel()] = body
    return out


# --------------------------------------------------------------------------- tensor-parallel slicing

def shard_rows(entry: Dict[str, torch.Tensor], pieces: Sequence[Tuple[int, int]]) -> Dict[str, torch.Tensor]:
    """Column-parallel shard: the row ranges `pieces` (each a multiple of 128 rows; several
    for merged layers, e.g. this rank's q, k and v rows) of a quantised layer, concatenated."""
    qw = entry["QW"]
    n, k = int(qw.shape[0]), int(qw.shape[1]) * 2
    out = {"QW": torch.cat([qw[b:e] for b, e in pieces]).contiguous(),
           "SFW_sparse": slice_scale_rows(entry["SFW_sparse"], n, k, 32, pieces),
           "SFW_dense": slice_scale_rows(entry["SFW_dense"], n, k, 16, pieces),
           "scale_b": entry["scale_b"]}
    if "bias" in entry:
        out["bias"] = torch.cat([entry["bias"][b:e] for b, e in pieces])
    return out


def shard_k(entry: Dict[str, torch.Tensor], kb: int, ke: int) -> Dict[str, torch.Tensor]:
    """Row-parallel shard: input features [kb, ke) (multiples of 128).  The bias, if any,
    stays whole: it is added once, after the sum over ranks."""
    qw = entry["QW"]
    n, k = int(qw.shape[0]), int(qw.shape[1]) * 2
    out = {"QW": qw[:, kb // 2:ke // 2].contiguous(),
           "SFW_sparse": slice_scale_k(entry["SFW_sparse"], n, k, 32, kb, ke),
           "SFW_dense": slice_scale_k(entry["SFW_dense"], n, k, 16, kb, ke),
           "scale_b": entry["scale_b"]}
    if "bias" in entry:
        out["bias"] = entry["bias"]
    return out


def merged_row_pieces(partition_sizes: Sequence[int], world: int, rank: int) -> List[Tuple[int, int]]:
    """Row ranges of rank `rank` in a merged column-parallel layer stored UNSHARDED as the
    concatenation of sub-matrices whose PER-RANK sizes are `partition_sizes` (vLLM's
    output_partition_sizes: e.g. [q/world, k/world, v/world])."""
    pieces, start = [], 0
    for part in partition_sizes:
        full = part * world
        pieces.append((start + rank * part, start + (rank + 1) * part))
        start += full
    return pieces


def layer_entry(tensors: Dict[str, torch.Tensor], base: str) -> Dict[str, torch.Tensor]:
    """The tensors of one quantised layer out of a checkpoint dict."""
    entry = {key: tensors[f"{base}.{key}"] for key in ("QW", "SFW_sparse", "SFW_dense", "scale_b")}
    if f"{base}.bias" in tensors:
        entry["bias"] = tensors[f"{base}.bias"]
    return entry
