"""vLLM quantisation method "sharq" on the sharq_b200 kernels.

Stands where the reference's plugin does (benchmarks/vllm/sharq.py:295-402: SHARQConfig,
SHARQLinearMethod, the `sharq_linear_forward` custom op) and loads the same checkpoints
(QW / SFW_sparse / SFW_dense / scale_b per linear, merged qkv_proj and gate_up_proj,
benchmarks/vllm/sharq_quant.py).  Differences, all needed on B200 or for tensor parallelism:

* `get_min_capability` is 100 (sm_100a), not 120;
* `create_weights` sizes the parameters for THIS rank's partition
  (`input_size_per_partition`, `sum(output_partition_sizes)`), and the weight loader cuts the
  unsharded checkpoint tensors down to the partition without re-quantising
  (sharq_b200.checkpoint), so vLLM's own column/row-parallel layers and its all-reduce after
  row-parallel layers work; the reference allocates and loads the full tensors on every rank;
* `apply` is one call of the fused op (scaled prepare + one GEMM launch) on torch's current
  stream, registered as an opaque custom op so that vLLM's graph capture treats it as a leaf.

Importing this module imports vLLM; call `register()` (or import the module) before building the
engine, e.g. from a `vllm.general_plugins` entry point.
"""
from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch
from torch.nn.parameter import Parameter

from . import checkpoint as ckpt

from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase
from vllm.model_executor.layers.quantization import register_quantization_config
from vllm.model_executor.layers.quantization.base_config import QuantizationConfig
from vllm.model_executor.utils import set_weight_attrs

try:  # the helper moved between vLLM releases
    from vllm.utils.torch_utils import direct_register_custom_op
except ImportError:  # pragma: no cover
    from vllm.utils import direct_register_custom_op


def _tp() -> Tuple[int, int]:
    """(rank, world) of vLLM's tensor-parallel group; (0, 1) outside a distributed run."""
    try:
        from vllm.distributed import get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size

        return int(get_tensor_model_parallel_rank()), int(get_tensor_model_parallel_world_size())
    except Exception:
        return 0, 1


# --------------------------------------------------------------------------- the op

def sharq_linear_forward(x: torch.Tensor, qw: torch.Tensor, sfw_sparse: torch.Tensor, sfw_dense: torch.Tensor,
                         weight_scale: float) -> torch.Tensor:
    from . import ops

    return ops.sharq_linear_forward(x, qw, sfw_sparse, sfw_dense, float(weight_scale))


def sharq_linear_forward_fake(x: torch.Tensor, qw: torch.Tensor, sfw_sparse: torch.Tensor, sfw_dense: torch.Tensor,
                              weight_scale: float) -> torch.Tensor:
    return torch.empty((x.shape[0], qw.shape[0]), dtype=torch.bfloat16, device=x.device)


_OP_NAME = "sharq_b200_linear_forward"
_registered = False


def register() -> None:
    """Register the custom op once (the quantisation config registers at import)."""
    global _registered
    if _registered:
        return
    kwargs = {}
    try:
        from vllm.platforms import current_platform

        kwargs["dispatch_key"] = current_platform.dispatch_key
    except Exception:
        pass
    direct_register_custom_op(op_name=_OP_NAME, op_func=sharq_linear_forward, mutates_args=[],
                              fake_impl=sharq_linear_forward_fake, **kwargs)
    _registered = True


# --------------------------------------------------------------------------- partition geometry

def partition_of(layer: torch.nn.Module, input_size_per_partition: int, output_partition_sizes: List[int],
                 input_size: int, output_size: int, rank: int, world: int):
    """What this rank holds of an unsharded [output_size, input_size] weight:
    ("rows", pieces) for column-parallel layers (row ranges, one per merged sub-matrix),
    ("k", (begin, end)) for row-parallel layers, ("all", None) when nothing is cut."""
    if input_size_per_partition != input_size:
        if input_size_per_partition * world != input_size:
            raise ValueError(f"input partition {input_size_per_partition} x {world} != {input_size}")
        return "k", (rank * input_size_per_partition, (rank + 1) * input_size_per_partition)
    local_rows = sum(output_partition_sizes)
    if local_rows != output_size:
        if local_rows * world != output_size:
            raise ValueError(f"output partition {local_rows} x {world} != {output_size}")
        return "rows", ckpt.merged_row_pieces(output_partition_sizes, world, rank)
    return "all", None


def cut_to_partition(name: str, full: torch.Tensor, kind: str, where, output_size: int, input_size: int) -> torch.Tensor:
    """This rank's part of one unsharded checkpoint tensor of a layer."""
    if kind == "all" or name == "scale_b":
        return full
    group = {"SFW_sparse": 32, "SFW_dense": 16}.get(name)
    if kind == "rows":
        if name == "QW" or name == "bias":
            return torch.cat([full[b:e] for b, e in where]).contiguous()
        return ckpt.slice_scale_rows(full.reshape(-1), output_size, input_size, group, where)
    kb, ke = where
    if name == "QW":
        return full[:, kb // 2:ke // 2].contiguous()
    if name == "bias":
        return full
    return ckpt.slice_scale_k(full.reshape(-1), output_size, input_size, group, kb, ke)


# --------------------------------------------------------------------------- vLLM classes

@register_quantization_config("sharq")
class SHARQConfig(QuantizationConfig):
    """Config of the "sharq" method (quantize_config.json / `quantization_config.quant_method`)."""

    def __init__(self, **kwargs) -> None:
        super().__init__()

    @classmethod
    def get_name(cls) -> str:
        return "sharq"

    @classmethod
    def get_supported_act_dtypes(cls) -> list[torch.dtype]:
        return [torch.bfloat16]

    @classmethod
    def get_min_capability(cls) -> int:
        return 100

    @classmethod
    def get_config_filenames(cls) -> list[str]:
        return ["quantize_config.json"]

    @classmethod
    def from_config(cls, config: dict[str, Any]) -> "SHARQConfig":
        return cls(**config)

    def get_quant_method(self, layer: torch.nn.Module, prefix: str) -> Optional[LinearMethodBase]:
        if isinstance(layer, LinearBase):
            return SHARQLinearMethod(self, prefix=prefix)
        return None


class SHARQLinearMethod(LinearMethodBase):
    def __init__(self, quant_config: SHARQConfig, prefix: str = ""):
        self.quant_config = quant_config
        self.prefix = prefix

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int, output_partition_sizes: list[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, **extra_weight_attrs):
        k_local, n_local = int(input_size_per_partition), int(sum(output_partition_sizes))
        if k_local % 128 != 0:
            raise ValueError(f"SHARQ needs the per-rank input size to be a multiple of 128, got {k_local} for {self.prefix}")
        rank, world = _tp()
        kind, where = partition_of(layer, k_local, list(output_partition_sizes), int(input_size), int(output_size), rank,
                                   world)
        if kind == "rows" and any(p % 128 for p in output_partition_sizes):
            raise ValueError(f"SHARQ needs per-rank output partitions that are multiples of 128, got "
                             f"{output_partition_sizes} for {self.prefix}")
        device = "cuda" if torch.cuda.is_available() else "cpu"  # parameters only; the op itself needs CUDA
        layer.input_size = int(input_size)
        layer.output_size = int(output_size)
        layer.scale_b_value = 1.0
        layer.sharq_partition = (kind, where)

        def register_param(name: str, shape, dtype):
            def weight_loader(param: Parameter, loaded_weight: torch.Tensor, *args):
                if param.numel() == 0:
                    return
                part = cut_to_partition(name, loaded_weight, kind, where, int(output_size), int(input_size))
                part = part.to(device=param.device, dtype=param.dtype)
                if part.dim() == 0 and param.numel() == 1:
                    part = part.view(1)
                if part.numel() == param.numel() and part.shape != param.shape:
                    part = part.view(param.shape)
                if part.shape != param.shape:
                    raise ValueError(f"Shape mismatch for {self.prefix}.{name}: expected {tuple(param.shape)}, "
                                     f"got {tuple(part.shape)}")
                param.data.copy_(part)
                if name == "scale_b":
                    layer.scale_b_value = float(part.reshape(-1)[0].float().cpu().item())

            param = Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=False)
            set_weight_attrs(param, {**extra_weight_attrs, "weight_loader": weight_loader})
            layer.register_parameter(name, param)

        sf = ckpt.sf_bytes(n_local, k_local)
        register_param("QW", (n_local, k_local // 2), torch.uint8)
        register_param("SFW_sparse", (sf,), torch.uint8)
        register_param("SFW_dense", (sf,), torch.uint8)
        register_param("scale_b", (1,), torch.float32)

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        register()
        x_2d = x.reshape(-1, x.shape[-1]).contiguous()
        out = getattr(torch.ops.vllm, _OP_NAME)(x_2d, layer.QW, layer.SFW_sparse, layer.SFW_dense, layer.scale_b_value)
        if bias is not None:
            out.add_(bias)
        return out.view(*x.shape[:-1], -1)
