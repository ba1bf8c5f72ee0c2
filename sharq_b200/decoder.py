"""Minimal decoder stacks (Llama / Qwen2 shaped) built on the SharQ linears, for prefill.

The reference wraps HuggingFace decoder layers (model/qLlamaLayer.py:50-257,
model/qQwenLayer.py) written against transformers 4.44; those wrappers read attributes
that newer transformers releases no longer have, so this module carries its own small
decoder with the same call pattern on the quantized path:

* one prepared activation is shared by q, k and v (here one merged qkv GEMM) and by
  gate and up (one merged gate_up GEMM)            - model/qLlamaLayer.py:93-106,173-183
* the input and post-attention RMSNorms are fused into the prepare of the following
  linears; the decoder layer never runs them separately - model/qLlamaLayer.py:219-221
* o_proj and down_proj take the plain (non-RMSNorm) prepare
* attention itself is stock `scaled_dot_product_attention` with grouped KV heads; it is not
  part of the accelerated path.  The rotary embedding runs in place on the merged qkv output
  (one kernel, ops.rope_inplace_) and SwiGLU is fused with the prepare of down_proj
  (prepare_input_swiglu); both give the bits of the ATen compositions they replace, which
  `fused_glue=False` still runs.

Tensor parallelism (`world` > 1): attention heads and the FFN width are sharded; qkv and
gate_up are column-parallel, o_proj and down_proj row-parallel with an all-reduce.
Weights are random (N(0, 0.02)): there are no checkpoints in this environment.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .tp import RowParallelSharqLinear, head_layout, padded_size, shard_bounds


@dataclass
class DecoderConfig:
    hidden: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 5e5
    eps: float = 1e-6
    qkv_bias: bool = False
    experts: int = 0  # > 0: sparse mixture-of-experts FFN (Mixtral): `experts` FFNs, `top_k` per token
    top_k: int = 2

    @staticmethod
    def llama3_8b(**kw):
        return DecoderConfig(**kw)

    @staticmethod
    def mixtral_8x7b(**kw):
        return DecoderConfig(**{**dict(hidden=4096, layers=32, heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=32000,
                                       rope_theta=1e6, eps=1e-5, experts=8, top_k=2), **kw})

    @staticmethod
    def qwen25_7b(**kw):
        return DecoderConfig(**{**dict(hidden=3584, layers=28, heads=28, kv_heads=4, head_dim=128, ffn=18944, vocab=152064,
                                       rope_theta=1e6, qkv_bias=True), **kw})


def rope_tables(seq: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, H, S, D]; rotate-half convention."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos + rot * sin


class SharqDecoderLayer(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, gen: torch.Generator, device, world: int = 1, rank: int = 0,
                 keep_reference: bool = False, mode: str = "SHARQ", fused_glue: bool = True, reduce_hook=None):
        super().__init__()
        self.fused_glue = fused_glue
        self.reduce_hook = reduce_hook
        self.grouped_experts = True   # mixture-of-experts FFN: grouped launches (False: the reference's per-expert loop)
        self._expert_weight_scales = None
        if mode not in ("SHARQ", "NVFP4", "BF16"):
            raise ValueError(f"unknown mode {mode}")
        if mode != "SHARQ" and reduce_hook is not None:
            raise ValueError("the NVFP4 and BF16 comparison modes run tensor-parallel only over a process group")
        self.mode = mode
        keep_reference = keep_reference or mode != "SHARQ"
        self.cfg, self.world, self.rank = cfg, world, rank
        self.ref = {} if keep_reference else None  # unquantised bf16 weights (accuracy checks, baselines)
        h, d = cfg.hidden, cfg.head_dim
        # heads of this rank (query ids, -1 = zero padding head; key/value ids), see tp.head_layout
        q_ids, kv_ids = head_layout(cfg.heads, cfg.kv_heads, world)[rank]
        self.local_heads, self.local_kv = len(q_ids), len(kv_ids)

        def rnd(n, k):
            return (0.02 * torch.randn(n, k, generator=gen, device=device)).to(torch.bfloat16)

        def head_rows(w, ids):
            """Rows of the heads `ids` of a [heads * d, *] matrix (or [heads * d] vector); zeros for -1."""
            parts = [w[i * d:(i + 1) * d] if i >= 0 else torch.zeros_like(w[:d]) for i in ids]
            return torch.cat(parts)

        # every rank draws the same full weights (same generator state) and keeps its shard
        wq, wk, wv = rnd(cfg.heads * d, h), rnd(cfg.kv_heads * d, h), rnd(cfg.kv_heads * d, h)
        bias = full_bias = None
        if cfg.qkv_bias:
            bq, bk, bv = ((0.02 * torch.randn(n, generator=gen, device=device)).to(torch.bfloat16) for n in
                          (cfg.heads * d, cfg.kv_heads * d, cfg.kv_heads * d))
            bias = torch.cat((head_rows(bq, q_ids), head_rows(bk, kv_ids), head_rows(bv, kv_ids)))
            full_bias = torch.cat((bq, bk, bv))
        self.qkv = _local_column(torch.cat((head_rows(wq, q_ids), head_rows(wk, kv_ids), head_rows(wv, kv_ids))),
                                 torch.cat((wq, wk, wv)), bias)
        wo = rnd(h, cfg.heads * d)
        wo_local = torch.cat([wo[:, i * d:(i + 1) * d] if i >= 0 else torch.zeros_like(wo[:, :d]) for i in q_ids], dim=1)
        self.o_proj = RowParallelSharqLinear(wo, local_columns=wo_local, world_rank=(world, rank), reduce_hook=reduce_hook)
        # the FFN width is padded with zero rows / columns to world slices that are multiples of 128
        ffn_pad = padded_size(cfg.ffn, world, 128)

        def pad_rows(w):
            return w if ffn_pad == cfg.ffn else torch.cat((w, torch.zeros((ffn_pad - cfg.ffn, w.shape[1]), dtype=w.dtype,
                                                                      device=w.device)))

        fb, fe = shard_bounds(ffn_pad, world, rank, 128)
        if cfg.experts > 0:
            # Mixtral FFN (model/qMixtralLayer.py:166-234): a bf16 router and `experts` SwiGLU FFNs;
            # w1 | w3 share one prepared activation (here one merged GEMM), w2 takes the
            # SwiGLU-fused prepare.  Tensor parallelism shards every expert's FFN width; the
            # partial outputs of all experts are summed over ranks once per layer.
            if mode != "SHARQ":
                raise ValueError("the mixture-of-experts layer has no NVFP4 / BF16 comparison mode")
            self.router = rnd(cfg.experts, h)
            self.experts = []
            ref_experts = []
            for _ in range(cfg.experts):
                wg, wu, wd = rnd(cfg.ffn, h), rnd(cfg.ffn, h), rnd(h, cfg.ffn)
                gate_up = _local_column(torch.cat((pad_rows(wg)[fb:fe], pad_rows(wu)[fb:fe])), torch.cat((wg, wu)), None)
                down = _local_column(pad_rows(wd.T).T[:, fb:fe].contiguous(), wd, None)
                self.experts.append((gate_up, down))
                if keep_reference:
                    ref_experts.append((wg, wu, wd))
                del wg, wu, wd
            self.gate_up = self.down = None
            if keep_reference:
                self.ref = dict(qkv=torch.cat((wq, wk, wv)), qkv_bias=full_bias, o=wo, experts=ref_experts)
            del wq, wk, wv, wo
        else:
            wg, wu = rnd(cfg.ffn, h), rnd(cfg.ffn, h)
            self.gate_up = _local_column(torch.cat((pad_rows(wg)[fb:fe], pad_rows(wu)[fb:fe])), torch.cat((wg, wu)), None)
            wd = rnd(h, cfg.ffn)
            self.down = RowParallelSharqLinear(wd, local_columns=pad_rows(wd.T).T[:, fb:fe], world_rank=(world, rank),
                                               reduce_hook=reduce_hook)
            if keep_reference and (mode == "SHARQ" or world == 1):
                self.ref = dict(qkv=torch.cat((wq, wk, wv)), qkv_bias=full_bias, o=wo, gate=wg, up=wu, down=wd)
            elif keep_reference:
                # comparison modes under tensor parallelism: this rank's shards of the bf16 weights, cut
                # like the SharQ layers (heads / padded FFN width column-parallel, o and down row-parallel)
                self.ref = dict(qkv=torch.cat((head_rows(wq, q_ids), head_rows(wk, kv_ids), head_rows(wv, kv_ids))),
                                qkv_bias=bias, o=wo_local.contiguous(), gate=pad_rows(wg)[fb:fe].contiguous(),
                                up=pad_rows(wu)[fb:fe].contiguous(), down=pad_rows(wd.T).T[:, fb:fe].contiguous())
            del wq, wk, wv, wo, wg, wu, wd
        if mode == "NVFP4":
            # dense NVFP4 baseline: unfused RMSNorm, dense activation quantisation, dense GEMM
            from .qlinear import QLinearLayer

            def dense(w, b=None):
                lin = torch.nn.Linear(w.shape[1], w.shape[0], bias=b is not None, device=device, dtype=torch.bfloat16)
                lin.weight.data.copy_(w)
                if b is not None:
                    lin.bias.data.copy_(b)
                return QLinearLayer(lin, quant_type="NVFP4", device=device)

            r = self.ref
            self.nv = dict(qkv=dense(r["qkv"], r["qkv_bias"]), o=dense(r["o"]),
                           gate_up=dense(torch.cat((r["gate"], r["up"]))), down=dense(r["down"]))
            self.ref = None
            self.qkv = self.o_proj = self.gate_up = self.down = None
        elif mode == "BF16":
            self.qkv = self.o_proj = self.gate_up = self.down = None
            if fused_glue:  # one merged gate_up GEMM, as on the quantised paths
                self.ref["gate_up"] = torch.cat((self.ref.pop("gate"), self.ref.pop("up")))
        self.input_norm = (1 + 0.1 * torch.randn(h, generator=gen, device=device)).to(torch.bfloat16)
        self.post_norm = (1 + 0.1 * torch.randn(h, generator=gen, device=device)).to(torch.bfloat16)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, delta: torch.Tensor = None,
                return_delta: bool = False):
        """x: [B, S, hidden] bf16 -> same shape.  delta: an addend of x that the caller has not
        applied yet (the previous layer's down_proj output); with return_delta the layer returns
        (x_mid, d) whose sum is its output, so that the next layer can fold the add into the
        statistics pass of its first prepare."""
        if self.mode != "SHARQ":
            if delta is not None:
                x = x + delta
            if self.world > 1:
                y = self._forward_comparison_tp(x, cos, sin)
            else:
                y = self.forward_reference(x, cos, sin) if self.mode == "BF16" else self._forward_nvfp4(x, cos, sin)
            return (y, None) if return_delta else y
        cfg = self.cfg
        b, s, h = x.shape
        x2 = x.reshape(b * s, h)
        if delta is not None and self.fused_glue:
            prep, x2 = self.qkv.prepare_input_add_rmsnorm(x2, delta.reshape(b * s, h), self.input_norm, cfg.eps)
        else:
            if delta is not None:
                x2 = x2 + delta.reshape(b * s, h)
            prep = self.qkv.prepare_input_rmsnorm(x2, self.input_norm, cfg.eps)
        qkv = self.qkv.apply_prepared(prep)
        q, k, v = _split_heads(qkv, b, s, self.local_heads, self.local_kv, cfg.head_dim, cos, sin, self.fused_glue)
        attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        attn2 = attn.transpose(1, 2).reshape(b * s, self.local_heads * cfg.head_dim)
        o = self.o_proj(attn2)
        if cfg.experts > 0:
            if self.fused_glue and h <= 8192:
                from . import ops

                # residual add + norm in one launch (the router and the experts read hn)
                hn, x2 = ops.add_rmsnorm(o.contiguous(), self.post_norm, cfg.eps, residual=x2.contiguous())
            else:
                x2 = x2 + o
                hn = _rmsnorm(x2, self.post_norm, cfg.eps)
            d = self._moe(hn)
            if return_delta:
                return x2.view(b, s, h), d.view(b, s, h)
            return (x2 + d).view(b, s, h)
        if self.fused_glue:
            prep, x2 = self.gate_up.prepare_input_add_rmsnorm(x2, o, self.post_norm, cfg.eps)
        else:
            x2 = x2 + o
            prep = self.gate_up.prepare_input_rmsnorm(x2, self.post_norm, cfg.eps)
        gu = self.gate_up.apply_prepared(prep)
        if self.fused_glue:
            d = self.down.apply_prepared_reduced(self.down.local.prepare_input_swiglu(gu))
        else:
            f = gu.shape[1] // 2
            d = self.down(F.silu(gu[:, :f]) * gu[:, f:])
        if return_delta:
            return x2.view(b, s, h), d.view(b, s, h)
        return (x2 + d).view(b, s, h)

    @torch.no_grad()
    def forward_sequence_parallel(self, sp, prepared, x_local: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, b: int,
                                  s: int, next_gamma: torch.Tensor):
        """One layer with the residual stream sharded by rows over the ranks (tp.SequenceParallelContext).
        prepared: the RMSNorm-prepared input of qkv for ALL b*s rows (from the previous transition);
        x_local: this rank's rows of the residual stream.  The two transitions (after o_proj with this
        layer's post-attention norm, after down_proj with the NEXT layer's input norm): the row-parallel GEMM
        deals its output rows to their owner ranks from its epilogue, and one kernel sums them, adds the
        residual, prepares the local rows (RMSNorm fused) and all-gathers the packed activation.  -> (prepared input of the next layer's qkv, x_local)."""
        cfg = self.cfg
        qkv = self.qkv.apply_prepared(prepared)
        q, k, v = _split_heads(qkv, b, s, self.local_heads, self.local_kv, cfg.head_dim, cos, sin, True)
        attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        attn2 = attn.transpose(1, 2).reshape(b * s, self.local_heads * cfg.head_dim)
        self.o_proj.local.apply_prepared(self.o_proj.local.prepare_input(attn2), scatter=sp.scatter)
        prepared, x_local = sp.transition(x_local, self.post_norm, cfg.eps)
        gu = self.gate_up.apply_prepared(prepared)
        self.down.local.apply_prepared(self.down.local.prepare_input_swiglu(gu), scatter=sp.scatter)
        return sp.transition(x_local, next_gamma, cfg.eps)

    @torch.no_grad()
    def _moe(self, hn: torch.Tensor) -> torch.Tensor:
        """Sparse mixture of experts on the normalised hidden state [M, h] (routing as in
        model/qMixtralLayer.py:205-234): softmax over the router logits in float, top-k,
        renormalised weights in bf16; every expert runs on the tokens routed to it."""
        from . import tp

        cfg = self.cfg
        m, h = hn.shape
        routing, selected = _route(hn, self.router, cfg.top_k)
        if self.fused_glue and self.grouped_experts and hn.is_cuda:
            out = self._moe_grouped(hn, routing, selected)
            if self.reduce_hook is not None:
                return self.reduce_hook(out)
            if self.world > 1:
                buf = tp.sum_buffer(None, hn.device, m * h * 2)
                if buf is None:
                    return tp.all_reduce_sum_(out)
                slot, view = buf.take(m, h)
                view.copy_(out)
                buf.sum_(slot, m * h * 2)
                return view
            return out
        buf = tp.sum_buffer(None, hn.device, m * h * 2) if self.world > 1 and self.reduce_hook is None else None
        if buf is not None:
            slot, out = buf.take(m, h)
            out.zero_()
        else:
            out = torch.zeros((m, h), dtype=torch.bfloat16, device=hn.device)
        mask = F.one_hot(selected, num_classes=cfg.experts).permute(2, 1, 0)
        for e, (gate_up, down) in enumerate(self.experts):
            idx, top_x = torch.where(mask[e])
            if top_x.numel() == 0:
                continue
            cur = hn[top_x].contiguous()
            gu = gate_up.apply_prepared(gate_up.prepare_input(cur))
            if self.fused_glue:
                y = down.apply_prepared(down.prepare_input_swiglu(gu))
            else:
                f = gu.shape[1] // 2
                y = down.apply_prepared(down.prepare_input((F.silu(gu[:, :f]) * gu[:, f:]).contiguous()))
            if self.fused_glue:
                from . import ops

                ops.scatter_add_scaled_(out, y, top_x.contiguous(), routing[top_x, idx].contiguous())
            else:
                out.index_add_(0, top_x, y * routing[top_x, idx, None])
        if self.reduce_hook is not None:
            out = self.reduce_hook(out)
        elif self.world > 1:
            if buf is not None:
                buf.sum_(slot, m * h * 2)
            else:
                tp.all_reduce_sum_(out)
        return out

    @torch.no_grad()
    def _moe_grouped(self, hn: torch.Tensor, routing: torch.Tensor, selected: torch.Tensor) -> torch.Tensor:
        """All experts in grouped launches with no host synchronisation (so the layer can be captured in a
        CUDA graph): the token slots are sorted by expert on the device (ATen sort / cumsum: plumbing),
        every expert's segment is padded to 256 rows, and gather -> prepare -> gate_up GEMM -> SwiGLU +
        prepare -> down GEMM -> weighted combine each run once for all experts.  Same arithmetic per
        token as the per-expert loop (each expert's rows get that expert's own tensor scales)."""
        from . import ops

        cfg = self.cfg
        m, h = hn.shape
        e, k = cfg.experts, cfg.top_k
        dev = hn.device
        dest, src_row, unit_group = moe_grouping(selected, e)
        w13 = [(g.weight_q, g.scale_w_sparse, g.scale_w_dense) for g, _ in self.experts]
        w2 = [(d.weight_q, d.scale_w_sparse, d.scale_w_dense) for _, d in self.experts]
        if self._expert_weight_scales is None:
            self._expert_weight_scales = (torch.stack([g.weight_scale.reshape(()) for g, _ in self.experts]).float().contiguous(),
                                          torch.stack([d.weight_scale.reshape(()) for _, d in self.experts]).float().contiguous())
        ws13, ws2 = self._expert_weight_scales
        p1 = ops.grouped_sparse_residual_quantize_x(hn.contiguous(), unit_group, e, src_row=src_row)
        gu = ops.linear_gemm_grouped(*p1[:5], w13, unit_group, (p1[5] * ws13).contiguous())
        p2 = ops.grouped_swiglu_sparse_residual_quantize_x(gu, unit_group, e)
        y = ops.linear_gemm_grouped(*p2[:5], w2, unit_group, (p2[5] * ws2).contiguous())
        return ops.moe_combine(y, dest, selected.contiguous(), routing.contiguous())

    @torch.no_grad()
    def _forward_comparison_tp(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """The dense-NVFP4 or bf16 layer on this rank's weight shards: column-parallel qkv and gate_up,
        row-parallel o_proj and down_proj whose partial outputs are written into symmetric memory and
        summed by the same all-reduce kernel the SharQ layers use (torch.distributed where that is
        not available)."""
        from . import tp

        cfg = self.cfg
        b, s, h = x.shape
        m = b * s
        x2 = x.reshape(m, h)

        def row_parallel(apply, n_out):
            buf = tp.sum_buffer(None, x2.device, m * n_out * 2)
            if buf is None:
                y = apply(None)
                tp.all_reduce_sum_(y)
                return y
            slot, view = buf.take(m, n_out)
            apply(view)
            buf.sum_(slot, m * n_out * 2)
            return view

        if self.mode == "BF16":
            r = self.ref
            qkv = F.linear(_rmsnorm(x2, self.input_norm, cfg.eps), r["qkv"], r["qkv_bias"])
        else:
            nv = self.nv
            qkv = nv["qkv"].apply_prepared(nv["qkv"].prepare_input_rmsnorm(x2, self.input_norm, cfg.eps))
        q, k, v = _split_heads(qkv, b, s, self.local_heads, self.local_kv, cfg.head_dim, cos, sin, self.fused_glue)
        attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        attn2 = attn.transpose(1, 2).reshape(m, self.local_heads * cfg.head_dim)
        if self.mode == "BF16":
            o = row_parallel(lambda out: torch.mm(attn2, r["o"].T, out=out) if out is not None else attn2 @ r["o"].T, h)
        else:
            po = nv["o"].prepare_input(attn2)
            o = row_parallel(lambda out: nv["o"].apply_prepared(po, out=out), h)
        x2 = x2 + o
        if self.mode == "BF16":
            gu = F.linear(_rmsnorm(x2, self.post_norm, cfg.eps), r["gate_up"])
            hmid = _swiglu(gu, self.fused_glue).contiguous()
            d = row_parallel(lambda out: torch.mm(hmid, r["down"].T, out=out) if out is not None else hmid @ r["down"].T, h)
        else:
            gu = nv["gate_up"].apply_prepared(nv["gate_up"].prepare_input_rmsnorm(x2, self.post_norm, cfg.eps))
            pd = nv["down"].prepare_input(_swiglu(gu, self.fused_glue).contiguous())
            d = row_parallel(lambda out: nv["down"].apply_prepared(pd, out=out), h)
        return (x2 + d).view(b, s, h)

    @torch.no_grad()
    def _forward_nvfp4(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        cfg, nv = self.cfg, self.nv
        b, s, h = x.shape
        x2 = x.reshape(b * s, h)
        qkv = nv["qkv"].apply_prepared(nv["qkv"].prepare_input_rmsnorm(x2, self.input_norm, cfg.eps))
        nq = cfg.heads * cfg.head_dim
        q, k, v = _split_heads(qkv, b, s, cfg.heads, cfg.kv_heads, cfg.head_dim, cos, sin, self.fused_glue)
        attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x2 = x2 + nv["o"](attn.transpose(1, 2).reshape(b * s, nq))
        gu = nv["gate_up"].apply_prepared(nv["gate_up"].prepare_input_rmsnorm(x2, self.post_norm, cfg.eps))
        x2 = x2 + nv["down"](_swiglu(gu, self.fused_glue))
        return x2.view(b, s, h)

    @torch.no_grad()
    def forward_reference(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """The same layer with the unquantised bf16 weights (single rank, keep_reference=True)."""
        cfg, r = self.cfg, self.ref
        b, s, h = x.shape

        def norm(t, w):
            tf = t.float()
            return (tf * torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + cfg.eps) * w.float()).to(torch.bfloat16)

        x2 = x.reshape(b * s, h)
        qkv = F.linear(norm(x2, self.input_norm), r["qkv"], r["qkv_bias"])
        nq = cfg.heads * cfg.head_dim
        glue = "gate_up" in r  # BF16 comparison mode; the accuracy reference of a SharQ layer stays pure ATen
        q, k, v = _split_heads(qkv, b, s, cfg.heads, cfg.kv_heads, cfg.head_dim, cos, sin, glue)
        attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x2 = x2 + F.linear(attn.transpose(1, 2).reshape(b * s, nq), r["o"])
        y = norm(x2, self.post_norm)
        if cfg.experts > 0:
            routing, selected = _route(y, self.router, cfg.top_k)
            out = torch.zeros_like(y)
            mask = F.one_hot(selected, num_classes=cfg.experts).permute(2, 1, 0)
            for e, (wg, wu, wd) in enumerate(r["experts"]):
                idx, top_x = torch.where(mask[e])
                if top_x.numel():
                    cur = y[top_x]
                    out.index_add_(0, top_x, F.linear(F.silu(F.linear(cur, wg)) * F.linear(cur, wu), wd)
                                   * routing[top_x, idx, None])
            return (x2 + out).view(b, s, h)
        if glue:
            hmid = _swiglu(F.linear(y, r["gate_up"]), True)
        else:
            hmid = F.silu(F.linear(y, r["gate"])) * F.linear(y, r["up"])
        x2 = x2 + F.linear(hmid, r["down"])
        return x2.view(b, s, h)


def moe_grouping(selected: torch.Tensor, experts: int, unit: int = 256):
    """Device-side plan of a grouped mixture-of-experts step, without host synchronisation.
    selected [tokens, top_k] (expert of every token slot) ->
      dest       int32 [tokens, top_k]: row of every slot in the grouped activation (slots sorted by expert,
                 ascending token order inside an expert, every expert's segment padded to a multiple of `unit` rows)
      src_row    int32 [rows]: token of every grouped row, -1 for padding rows
      unit_group int32 [rows / unit]: expert of every unit, -1 for units without rows
    rows = (ceil(tokens * top_k / unit) + experts) * unit is the static upper bound of the padded total."""
    tokens, k = selected.shape
    dev = selected.device
    slots = tokens * k
    rows = ((slots + unit - 1) // unit + experts) * unit
    flat = selected.reshape(-1)
    order = torch.argsort(flat, stable=True)
    sorted_e = flat[order]
    counts = torch.zeros(experts, dtype=torch.int64, device=dev).scatter_add_(0, flat, torch.ones_like(flat))
    padded = (counts + unit - 1) // unit * unit
    ends = torch.cumsum(padded, 0)
    starts = ends - padded
    first = torch.cumsum(counts, 0) - counts
    dest_sorted = starts[sorted_e] + (torch.arange(slots, device=dev) - first[sorted_e])
    dest = torch.empty(slots, dtype=torch.int32, device=dev)
    dest[order] = dest_sorted.to(torch.int32)
    src_row = torch.full((rows,), -1, dtype=torch.int32, device=dev)
    src_row[dest_sorted] = (order // k).to(torch.int32)
    unit_starts = torch.arange(rows // unit, device=dev) * unit
    unit_group = torch.searchsorted(ends, unit_starts, right=True)
    unit_group = torch.where(unit_group < experts, unit_group, torch.full_like(unit_group, -1)).to(torch.int32)
    return dest.view(tokens, k), src_row, unit_group


def _rmsnorm(t: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    tf = t.float()
    return (tf * torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(torch.bfloat16)


def _route(hn: torch.Tensor, router: torch.Tensor, top_k: int):
    """(weights [M, top_k] bf16, expert ids [M, top_k])."""
    weights = F.softmax(F.linear(hn, router), dim=1, dtype=torch.float)
    weights, selected = torch.topk(weights, top_k, dim=-1)
    weights = weights / weights.sum(dim=-1, keepdim=True)
    return weights.to(hn.dtype), selected


def _split_heads(qkv: torch.Tensor, b: int, s: int, heads: int, kv_heads: int, d: int, cos: torch.Tensor,
                 sin: torch.Tensor, fused: bool):
    """Merged qkv activation [b*s, (heads + 2*kv_heads)*d] -> rotated q, k and v as [b, H, s, d]
    views.  fused: one in-place kernel on the q and k columns; else the ATen composition."""
    nq, nk = heads * d, kv_heads * d
    if fused and qkv.is_cuda:
        from . import ops

        ops.rope_inplace_(qkv, heads + kv_heads, d, cos, sin, s)
    q = qkv[:, :nq].view(b, s, heads, d).transpose(1, 2)
    k = qkv[:, nq:nq + nk].view(b, s, kv_heads, d).transpose(1, 2)
    v = qkv[:, nq + nk:].view(b, s, kv_heads, d).transpose(1, 2)
    if not (fused and qkv.is_cuda):
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    return q, k, v


def _swiglu(gu: torch.Tensor, fused: bool) -> torch.Tensor:
    if fused and gu.is_cuda:
        from . import ops

        return ops.swiglu(gu.contiguous())
    f = gu.shape[1] // 2
    return F.silu(gu[:, :f]) * gu[:, f:]


def _local_column(w_local: torch.Tensor, w_full: torch.Tensor, bias):
    """Column-parallel linear from an already gathered local slice; the weight tensor scale is
    taken over the FULL weight so that shards agree with the unsharded layer."""
    from . import ops
    from .qlinear import QLinearLayer

    scale = torch.clamp(w_full.abs().max().float() / (448.0 * 6.0), min=1e-9)
    q, sfs, sfd = ops.quantize_w32_shared((w_local / scale).to(torch.bfloat16).contiguous())
    return QLinearLayer.from_quantized(w_local.shape[1], w_local.shape[0], q, sfs, sfd, scale, bias=bias)


class SharqDecoder(torch.nn.Module):
    """Embedding -> N decoder layers -> final norm -> (bf16) lm_head on the last token."""

    def __init__(self, cfg: DecoderConfig, device, world: int = 1, rank: int = 0, seed: int = 0,
                 keep_reference: bool = False, mode: str = "SHARQ", fused_glue: bool = True, reduce_hook=None):
        """reduce_hook: callable(partial) -> sum over ranks, used instead of the collectives (lets a
        test run several ranks as threads of one process)."""
        super().__init__()
        self.cfg = cfg
        self.world, self.mode, self.fused_glue, self.reduce_hook = world, mode, fused_glue, reduce_hook
        gen = torch.Generator(device=device).manual_seed(seed)
        self.embed = (0.02 * torch.randn(cfg.vocab, cfg.hidden, generator=gen, device=device)).to(torch.bfloat16)
        self.layers = torch.nn.ModuleList([SharqDecoderLayer(cfg, gen, device, world, rank, keep_reference, mode, fused_glue,
                                                             reduce_hook) for _ in range(cfg.layers)])
        self.final_norm = (1 + 0.1 * torch.randn(cfg.hidden, generator=gen, device=device)).to(torch.bfloat16)
        self.lm_head = (0.02 * torch.randn(cfg.vocab, cfg.hidden, generator=gen, device=device)).to(torch.bfloat16)

    def _sequence_parallel_context(self, m: int):
        """The transition-kernel context for m tokens, or None when this model / shape / system keeps
        the replicated residual stream (single rank, rank threads of a test, mixture of experts,
        comparison modes, biases on row-parallel layers, m not a multiple of 128 * world)."""
        import os

        first = self.layers[0]
        if (self.world == 1 or self.reduce_hook is not None or self.cfg.experts > 0 or self.mode != "SHARQ"
                or not self.fused_glue or os.environ.get("SHARQ_TP_SEQUENCE_PARALLEL", "1") == "0"
                or first.o_proj.bias is not None or first.down.bias is not None):
            return None
        from . import tp

        return tp.sequence_parallel_context(m, self.cfg.hidden, None, self.embed.device)

    @torch.no_grad()
    def prefill(self, token_ids: torch.Tensor, reference: bool = False) -> torch.Tensor:
        """token_ids [B, S] -> logits of the last position [B, vocab] (float32).
        reference=True runs the unquantised bf16 layers (needs keep_reference=True)."""
        b, s = token_ids.shape
        cos, sin = rope_tables(s, self.cfg.head_dim, self.cfg.rope_theta, self.embed.device)
        sp = None if reference else self._sequence_parallel_context(b * s)
        if sp is not None:
            import torch.distributed as dist

            r0, r1 = sp.row_bounds()
            x_local = self.embed[token_ids.reshape(-1)[r0:r1]].contiguous()
            prepared, x_local = sp.transition(x_local, self.layers[0].input_norm, self.cfg.eps, use_partial=False)
            for i, layer in enumerate(self.layers):
                nxt = self.layers[i + 1].input_norm if i + 1 < len(self.layers) else self.final_norm
                prepared, x_local = layer.forward_sequence_parallel(sp, prepared, x_local, cos, sin, b, s, nxt)
            # the last position of every sequence lives on one rank: sum the zero-padded rows over ranks
            last = torch.zeros((b, self.cfg.hidden), dtype=torch.float32, device=x_local.device)
            for bi in range(b):  # python indices only: this runs under stream capture
                row = bi * s + s - 1
                if r0 <= row < r1:
                    last[bi].copy_(x_local[row - r0])
            dist.all_reduce(last, op=dist.ReduceOp.SUM)
        else:
            x = self.embed[token_ids]
            delta = None
            for layer in self.layers:
                if reference:
                    x = layer.forward_reference(x, cos, sin)
                else:
                    x, delta = layer(x, cos, sin, delta=delta, return_delta=True)
            if delta is not None:
                x = x + delta
            last = x[:, -1, :].float()
        last = last * torch.rsqrt(last.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * self.final_norm.float()
        return (last.to(torch.bfloat16) @ self.lm_head.T).float()
