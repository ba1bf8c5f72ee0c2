"""QLinearLayer with the interface of the reference's model/qLinearLayer.py:21-202
for quant_type "SHARQ" and "NVFP4", on the sm_100a kernels.

prepare_input / prepare_input_rmsnorm / apply_prepared / forward keep the reference's
argument meaning and tuple formats, so layer wrappers written against the reference
(one prepared activation shared by q/k/v or by gate/up) work unchanged.  With
fused_gemm=True (default) apply_prepared runs the single-launch sparse+residual GEMM with
the bias folded into its epilogue; with fused_gemm=False it issues the reference's two
GEMM calls (sparse, then dense with beta=1) and a separate bias add.

The reference's pure-PyTorch simulation modes (SHARQ_SIM, HIF4_SIM, ...) are accuracy
tools, not part of the accelerated path; they are not provided here.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import ops
from .quantize import (
    apply_rmsnorm,
    quantize_activation_nvfp4,
    quantize_activation_rmsnorm_sparse_residual_nvfp4,
    quantize_activation_sparse_residual_nvfp4,
    quantize_weight_nvfp4,
    quantize_weight_shared_nvfp4,
)


class QLinearLayer(nn.Module):
    def __init__(self, original_layer: nn.Linear, select_num=None, reorder_index=None, out_reorder_index=None,
                 quant_type: str = "NVFP4", extra_fusion: bool = True, fused_gemm: bool = True,
                 device: Optional[torch.device] = None):
        super().__init__()
        if quant_type not in {"NVFP4", "SHARQ"}:
            raise ValueError(f"Unsupported quant_type: {quant_type}")
        self.in_features = original_layer.in_features
        self.out_features = original_layer.out_features
        self.quant_type = quant_type
        self.enable_quant = True
        self.extra_fusion = extra_fusion
        self.fused_gemm = fused_gemm
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())

        if original_layer.bias is not None:
            self.register_buffer("bias", original_layer.bias.detach().clone().to(dev, torch.bfloat16).contiguous())
        else:
            self.bias = None

        weight_gpu = original_layer.weight.detach().to(device=dev, dtype=torch.bfloat16)
        if quant_type == "SHARQ":
            q, sfs, sfd, scale = quantize_weight_shared_nvfp4(weight_gpu)
            self.register_buffer("weight_q", q)
            self.register_buffer("scale_w_sparse", sfs)
            self.register_buffer("scale_w_dense", sfd)
        else:
            q, sf, scale = quantize_weight_nvfp4(weight_gpu)
            self.register_buffer("weight_q", q)
            self.register_buffer("scale_w", sf)
        self.register_buffer("weight_scale", scale)
        # host copy of the weight tensor scale: lets the GEMM take the activation scale as a
        # device scalar without a separate multiply kernel
        self.weight_scale_host = float(scale.item())

    @classmethod
    def from_quantized(cls, in_features: int, out_features: int, weight_q, scale_w_sparse, scale_w_dense,
                       weight_scale, bias=None, extra_fusion: bool = True, fused_gemm: bool = True):
        """Build a SHARQ layer from an already quantised (possibly sharded) weight."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.in_features, self.out_features = in_features, out_features
        self.quant_type, self.enable_quant = "SHARQ", True
        self.extra_fusion, self.fused_gemm = extra_fusion, fused_gemm
        self.register_buffer("weight_q", weight_q)
        self.register_buffer("scale_w_sparse", scale_w_sparse)
        self.register_buffer("scale_w_dense", scale_w_dense)
        ws = weight_scale if isinstance(weight_scale, torch.Tensor) else torch.tensor(float(weight_scale))
        self.register_buffer("weight_scale", ws.to(weight_q.device, torch.float32))
        self.weight_scale_host = float(ws.item())
        if bias is not None:
            self.register_buffer("bias", bias.to(weight_q.device, torch.bfloat16).contiguous())
        else:
            self.bias = None
        return self

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        # the fused GEMM takes the weight tensor scale as a host scalar: keep it in step with the buffer
        self.weight_scale_host = float(self.weight_scale.item())

    @torch.no_grad()
    def prepare_input(self, x_2d: torch.Tensor, out_features_hint: Optional[int] = None):
        x_2d = x_2d.to(torch.bfloat16)
        if self.quant_type == "SHARQ":
            n = self.out_features if out_features_hint is None else int(out_features_hint)
            a_comp, e, sfa, q_res, sf_res, scale_x = quantize_activation_sparse_residual_nvfp4(x_2d, n)
            return ("SHARQ", a_comp, e, sfa, q_res, sf_res, scale_x)
        qx, scale_x, scale = quantize_activation_nvfp4(x_2d)
        return ("NVFP4", qx, scale_x, scale)

    @torch.no_grad()
    def prepare_input_rmsnorm(self, x_2d: torch.Tensor, rmsnorm_weight: torch.Tensor, rmsnorm_eps: float,
                              out_features_hint: Optional[int] = None):
        if self.quant_type == "SHARQ" and self.extra_fusion:
            n = self.out_features if out_features_hint is None else int(out_features_hint)
            a_comp, e, sfa, q_res, sf_res, scale_x = quantize_activation_rmsnorm_sparse_residual_nvfp4(
                x_2d.to(torch.bfloat16), rmsnorm_weight, rmsnorm_eps, n)
            return ("SHARQ", a_comp, e, sfa, q_res, sf_res, scale_x)
        x_norm = apply_rmsnorm(x_2d.to(torch.bfloat16), rmsnorm_weight, rmsnorm_eps)
        return self.prepare_input(x_norm, out_features_hint=out_features_hint)

    @torch.no_grad()
    def prepare_input_add_rmsnorm(self, x_2d: torch.Tensor, residual_2d: torch.Tensor, rmsnorm_weight: torch.Tensor,
                                  rmsnorm_eps: float, out_features_hint: Optional[int] = None):
        """(prepared activation of rmsnorm(x + residual), x + residual): the residual add of the
        decoder layer rides on the row statistics pass of the RMSNorm-fused prepare."""
        if self.quant_type == "SHARQ" and self.extra_fusion and x_2d.is_cuda:
            n = self.out_features if out_features_hint is None else int(out_features_hint)
            a_comp, e, sfa, q_res, sf_res, scale_x, total = ops.fused_add_rmsnorm_sparse_residual_quantize_x(
                x_2d.to(torch.bfloat16).contiguous(), residual_2d.to(torch.bfloat16).contiguous(), rmsnorm_weight,
                rmsnorm_eps, n)
            return ("SHARQ", a_comp, e, sfa, q_res, sf_res, scale_x), total
        total = x_2d + residual_2d
        return self.prepare_input_rmsnorm(total, rmsnorm_weight, rmsnorm_eps, out_features_hint), total

    @torch.no_grad()
    def prepare_input_swiglu(self, gate_up_2d: torch.Tensor, out_features_hint: Optional[int] = None):
        """Prepared activation of act_fn(gate) * up for this (down_proj) layer from the merged
        gate_up output [M, 2 * in_features]: the three ATen passes of
        model/qLlamaLayer.py:183-185 and the activation quantisation in two launches."""
        if self.quant_type != "SHARQ":
            return self.prepare_input(ops.swiglu(gate_up_2d.to(torch.bfloat16)), out_features_hint)
        n = self.out_features if out_features_hint is None else int(out_features_hint)
        a_comp, e, sfa, q_res, sf_res, scale_x = ops.swiglu_sparse_residual_quantize_x(gate_up_2d, n)
        return ("SHARQ", a_comp, e, sfa, q_res, sf_res, scale_x)

    @torch.no_grad()
    def apply_prepared(self, prepared, out=None, scatter=None):
        """out: optional bf16 [M, N] tensor the fused SharQ GEMM writes into (used by the
        tensor-parallel layers to place partial sums in symmetric memory).  scatter: see
        ops.sharq_linear_gemm (row-parallel output dealt to the owner GPUs; returns None)."""
        tag = prepared[0]
        if scatter is not None:
            if not (tag == "SHARQ" and self.fused_gemm and self.bias is None):
                raise ValueError("scatter= needs the fused SharQ GEMM of a layer without bias")
            _, a_comp, e, sfa, q_res, sf_res, scale_x = prepared
            return ops.sharq_linear_gemm(a_comp, e, sfa, q_res, sf_res, self.weight_q, self.scale_w_sparse,
                                         self.scale_w_dense, scale_x.reshape(1), alpha_host=self.weight_scale_host,
                                         scatter=scatter)
        if out is not None and not ((tag == "SHARQ" and self.fused_gemm) or (tag == "NVFP4" and self.bias is None)):
            raise ValueError("out= is only supported by the fused SharQ GEMM and the bias-free dense NVFP4 GEMM")
        if tag == "SHARQ":
            _, a_comp, e, sfa, q_res, sf_res, scale_x = prepared
            if self.fused_gemm:
                return ops.sharq_linear_gemm(a_comp, e, sfa, q_res, sf_res, self.weight_q, self.scale_w_sparse,
                                             self.scale_w_dense, scale_x.reshape(1), bias=self.bias,
                                             alpha_host=self.weight_scale_host, out=out)
            output_scale = (scale_x * self.weight_scale).reshape(1).contiguous()
            y_sparse = ops.sparse_matmul_tensor_scale(a_comp, self.weight_q, e, sfa, self.scale_w_sparse,
                                                      q_res.shape[0], self.out_features, self.in_features,
                                                      alpha=output_scale)
            if self.extra_fusion:
                y = ops.matmul_accum_tensor_scale(q_res, self.weight_q, sf_res, self.scale_w_dense, output_scale,
                                                  y_sparse, 1.0)
            else:
                y = y_sparse + ops.matmul_tensor_scale(q_res, self.weight_q, sf_res, self.scale_w_dense, output_scale)
        elif tag == "NVFP4":
            _, qx, scale_x, scale = prepared
            y = ops.matmul_tensor_scale(qx, self.weight_q, scale_x, self.scale_w,
                                        (scale * self.weight_scale).reshape(1).contiguous(), out=out)
        else:
            raise ValueError(f"Unsupported prepared input tag: {tag}")
        if self.bias is not None:
            y = y + self.bias
        return y

    @torch.no_grad()
    def forward(self, x):
        if isinstance(x, tuple):
            x_orig, bsz, q_len = x
        else:
            x_orig, bsz, q_len = x, None, x.shape[0]
        x2 = x_orig.reshape(-1, x_orig.shape[-1]).to(torch.bfloat16)
        y = self.apply_prepared(self.prepare_input(x2))
        if bsz is not None:
            return y.reshape(bsz, q_len, -1)
        return y.reshape(q_len, -1)
