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

The all-reduce of a row-parallel layer on GPUs is this project's own kernel
(csrc/allreduce.cu): the GEMM writes its partial sums straight into a buffer in symmetric
memory (allocated and exchanged through torch.distributed._symmetric_memory, which is
plumbing here) and one kernel per rank reduces them inside the NVSwitch (multimem.ld_reduce
/ multimem.st).  SHARQ_TP_ALLREDUCE=nccl selects torch.distributed's all_reduce instead;
process groups without CUDA multicast support (the gloo groups of the CPU tests) always use
it.
"""
from __future__ import annotations

import ctypes
import os
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


def head_layout(heads: int, kv_heads: int, world: int):
    """Attention heads of every rank: a list of (query head ids, key/value head ids); a query id of
    -1 is a padding head (zero weights).  When both counts divide by `world` the heads are cut
    contiguously.  Otherwise, if `world` is a multiple of `kv_heads`, every KV head is replicated
    on world / kv_heads consecutive ranks and its query group is dealt to them in equal parts,
    padded at the end (Qwen2.5-7B on 8 ranks: 28 query / 4 KV heads -> 4 + 3(+1 pad) query heads
    on the two ranks of each KV head)."""
    if heads % world == 0 and kv_heads % world == 0:
        hq, hk = heads // world, kv_heads // world
        return [(list(range(r * hq, (r + 1) * hq)), list(range(r * hk, (r + 1) * hk))) for r in range(world)]
    if world % kv_heads or heads % kv_heads:
        raise ValueError(f"{heads} query / {kv_heads} KV heads cannot be laid out over {world} ranks")
    rep, group = world // kv_heads, heads // kv_heads
    per_rank = (group + rep - 1) // rep
    out = []
    for r in range(world):
        j, i = r // rep, r % rep
        ids = [j * group + i * per_rank + t if i * per_rank + t < group else -1 for t in range(per_rank)]
        out.append((ids, [j]))
    return out


def scaled_weight(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Full weight divided by its global tensor scale (bf16), and that scale."""
    scale = torch.clamp(weight.abs().max().float() / (448.0 * 6.0), min=1e-9)
    return (weight / scale).to(torch.bfloat16), scale


class SymmetricSumBuffer:
    """bf16 scratch in symmetric memory for the partial sums of row-parallel layers, shared
    by all layers of a process group: SLOTS equal slots used round-robin, so the result of
    one row-parallel layer stays valid until SLOTS more have run.  Construction and growth
    are collective (every rank must do them at the same point, outside stream capture)."""

    SLOTS = 2

    def __init__(self, slot_bytes: int, group, device: torch.device):
        import torch.distributed._symmetric_memory as symm

        from . import _lib

        lib = _lib.lib()
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.slot_bytes = (int(slot_bytes) + 4095) // 4096 * 4096
        flag_bytes = int(lib.sharq_allreduce_flag_bytes())
        self.storage = symm.empty(self.SLOTS * self.slot_bytes + flag_bytes, dtype=torch.uint8, device=device)
        handle = symm.rendezvous(self.storage, group.group_name)
        if not int(handle.multicast_ptr):
            raise RuntimeError("symmetric memory has no NVLink multicast mapping on this system")
        offset = int(getattr(handle, "offset", 0))
        bases = [int(p) + offset for p in handle.buffer_ptrs]
        if bases[self.rank] != self.storage.data_ptr():
            raise RuntimeError("symmetric-memory handle does not describe the tensor it was made from")
        self.multicast = int(handle.multicast_ptr) + offset
        self.storage.zero_()  # the barrier counters in the flag area start at zero
        torch.cuda.synchronize(device)
        dist.barrier(group)
        flags_at = self.SLOTS * self.slot_bytes
        self.flag_ptrs = (ctypes.c_void_p * self.world)(*[b + flags_at for b in bases])
        self.bases = bases
        # two ranks: plain peer loads/stores move fewer bytes per link than the multicast object
        mode = os.environ.get("SHARQ_TP_ALLREDUCE", "auto").lower()
        self.peer_copy = (mode == "peer" and self.world <= 4) or (self.world == 2 and mode != "multimem")
        self.handle = handle
        self._next = 0

    def take(self, m: int, n: int) -> Tuple[int, torch.Tensor]:
        """Next slot and a bf16 [m, n] view of it."""
        slot = self._next
        self._next = (slot + 1) % self.SLOTS
        begin = slot * self.slot_bytes
        return slot, self.storage[begin:begin + m * n * 2].view(torch.bfloat16).view(m, n)

    def sum_(self, slot: int, nbytes: int, max_ctas: int = 0) -> None:
        """Enqueue the in-switch all-reduce of the first nbytes of `slot` on the current stream
        (max_ctas: 0 = the library's default grid limit)."""
        from . import _lib, ops

        flag = ctypes.c_void_p(ops._error_flag(self.device).data_ptr())
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        if self.peer_copy:
            data = (ctypes.c_void_p * self.world)(*[b + slot * self.slot_bytes for b in self.bases])
            with torch.cuda.device(self.device):
                _lib.check(_lib.lib().sharq_allreduce_bf16_peer(data, self.flag_ptrs, self.rank, self.world, nbytes,
                                                                 int(max_ctas), flag, stream))
            return
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().sharq_allreduce_bf16_multimem(
                ctypes.c_void_p(self.multicast + slot * self.slot_bytes), self.flag_ptrs, self.rank, self.world, nbytes,
                int(max_ctas),
                ctypes.c_void_p(ops._error_flag(self.device).data_ptr()),
                ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))


_SUM_BUFFERS = {}


def _multimem_wanted(group) -> bool:
    mode = os.environ.get("SHARQ_TP_ALLREDUCE", "auto").lower()
    if mode not in ("auto", "multimem", "peer", "nccl"):
        raise ValueError("SHARQ_TP_ALLREDUCE must be auto, multimem, peer or nccl")
    if mode == "nccl":
        return False
    usable = torch.cuda.is_available() and dist.get_backend(group) == "nccl"
    if mode == "multimem" and not usable:
        raise RuntimeError("SHARQ_TP_ALLREDUCE=multimem needs CUDA devices and an NCCL process group")
    return usable


def sum_buffer(group, device: torch.device, nbytes: int) -> Optional[SymmetricSumBuffer]:
    """The group's shared SymmetricSumBuffer with slots of at least nbytes (collective when it
    has to be created or grown), or None when the in-switch all-reduce is not in use."""
    group = group if group is not None else dist.group.WORLD
    key = (group.group_name, device.index)
    if key in _SUM_BUFFERS and _SUM_BUFFERS[key] is None:
        return None
    buf = _SUM_BUFFERS.get(key)
    if buf is None or buf.slot_bytes < nbytes:
        if buf is None and not _multimem_wanted(group):
            _SUM_BUFFERS[key] = None
            return None
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the symmetric sum buffer must be created before stream capture: run the layer once first")
        err = None
        try:
            buf = SymmetricSumBuffer(nbytes, group, device)
        except RuntimeError as exc:
            buf, err = None, exc
        # every rank must take the same path: one that failed while the others succeeded would
        # issue a different collective from theirs.  Agree on the outcome before caching it.
        ok = torch.tensor([0 if buf is None else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            buf = None  # no multicast on (some rank of) this system: torch.distributed's all_reduce is used
            if os.environ.get("SHARQ_TP_ALLREDUCE", "auto").lower() == "multimem":
                raise RuntimeError(f"SHARQ_TP_ALLREDUCE=multimem but the symmetric buffer could not be set up: {err}")
        _SUM_BUFFERS[key] = buf
    return buf


def reserve_sum_buffer(group, device: torch.device, nbytes: int) -> Optional[SymmetricSumBuffer]:
    """Create the group's shared buffer once, sized for the largest row-parallel output of the
    model (M x N x 2 bytes), so that no forward pass has to grow it (growth is a collective)."""
    return sum_buffer(group, device, nbytes)


def release_sum_buffers() -> None:
    """Drop the shared symmetric buffers (call before destroying the process group)."""
    _SUM_BUFFERS.clear()
    _SP_CONTEXTS.clear()


class SequenceParallelContext:
    """Symmetric-memory buffers and state of the one-kernel layer transition
    (csrc/sp_transition.cu) for activations of a fixed shape [m, hidden]:

    * the collection buffer [world][m / world, hidden] bf16: block s receives, from rank s's row-parallel
      GEMM (o_proj, down_proj; pass `scatter` as `scatter=` of `QLinearLayer.apply_prepared`), rank s's
      partial products of THIS rank's rows, while that GEMM computes;
    * the prepared activation of all m rows (A_comp, E, both scale buffers, Q_res), which
      `transition` fills on every rank;
    * the state words of the cross-rank hand-shakes.

    The residual stream is sharded by rows: rank r owns rows [r*m/world, (r+1)*m/world).
    Construction is collective (every rank, same arguments, outside stream capture).  Needs
    m % (128 * world) == 0 and NVLink multicast; `supported` says whether a shape qualifies."""

    @staticmethod
    def supported(m: int, hidden: int, world: int) -> bool:
        return world > 1 and m % (128 * world) == 0 and hidden % 128 == 0 and hidden // 32 <= 1024

    def __init__(self, m: int, hidden: int, group, device: torch.device):
        import torch.distributed._symmetric_memory as symm

        from . import _lib, ops

        group = group if group is not None else dist.group.WORLD
        lib = _lib.lib()
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not self.supported(m, hidden, self.world):
            raise ValueError(f"activation [{m}, {hidden}] cannot be sharded by rows over {self.world} ranks")
        self.m, self.hidden, self.rows = m, hidden, m // self.world
        sizes = ops.get_fused_sparse_residual_buffer_sizes(m, hidden, hidden)  # (A_comp, E, SFA_sparse, Q_res, SF_res)

        def up(n):
            return (int(n) + 255) // 256 * 256

        self._off = {}
        cursor = 0
        for name, nbytes in (("partial", m * hidden * 2), ("a_comp", sizes[0]), ("e", sizes[1]), ("sfa", sizes[2]),
                             ("q_res", sizes[3]), ("sf_res", sizes[4]), ("state", int(lib.sharq_tp_transition_state_bytes()))):
            self._off[name] = (cursor, int(nbytes))
            cursor += up(nbytes)
        self.storage = symm.empty(cursor, dtype=torch.uint8, device=device)
        handle = symm.rendezvous(self.storage, group.group_name)
        if not int(handle.multicast_ptr):
            raise RuntimeError("symmetric memory has no NVLink multicast mapping on this system")
        offset = int(getattr(handle, "offset", 0))
        bases = [int(p) + offset for p in handle.buffer_ptrs]
        if bases[self.rank] != self.storage.data_ptr():
            raise RuntimeError("symmetric-memory handle does not describe the tensor it was made from")
        self.handle = handle
        self.multicast_delta = int(handle.multicast_ptr) + offset - bases[self.rank]
        self.storage.zero_()  # the state words start at zero
        torch.cuda.synchronize(device)
        dist.barrier(group)
        state_at = self._off["state"][0]
        self.state_ptrs = (ctypes.c_void_p * self.world)(*[b + state_at for b in bases])
        partial_at = self._off["partial"][0]
        self.blocks = self._view("partial").view(torch.bfloat16).view(self.world, self.rows, hidden)  # block s: from rank s
        self.partial_ptrs = (ctypes.c_void_p * self.world)(*[b + partial_at for b in bases])
        self.scatter = (self.partial_ptrs, self.rank, self.world)  # `scatter=` argument of the row-parallel GEMM
        self.scale = torch.zeros((), dtype=torch.float32, device=device)
        self.workspace = torch.empty(int(lib.sharq_tp_transition_workspace_bytes(self.rows)), dtype=torch.uint8, device=device)

    def _view(self, name: str) -> torch.Tensor:
        begin, nbytes = self._off[name]
        return self.storage[begin:begin + nbytes]

    def row_bounds(self) -> Tuple[int, int]:
        return self.rank * self.rows, (self.rank + 1) * self.rows

    def deliver(self, partial: torch.Tensor) -> None:
        """Deal the rows of a full [m, hidden] bf16 partial product to their owners' collection buffers, as the
        scatter-mode GEMM epilogue does (peer copies; for tests and checks that have the partial product as a tensor).
        Collective in effect: every rank must call it, and a barrier must follow before `transition`."""
        for owner in range(self.world):
            dst = self.handle.get_buffer(owner, (self.world, self.rows, self.hidden), torch.bfloat16,
                                         self._off["partial"][0] // 2)
            dst[self.rank].copy_(partial[owner * self.rows:(owner + 1) * self.rows])

    def transition(self, residual_local: Optional[torch.Tensor], gamma: torch.Tensor, eps: float, use_partial: bool = True,
                   out_features_hint: int = 0):
        """-> (prepared, new_residual_local).  prepared is the reference's ("SHARQ", A_comp, E, SFA_sparse,
        Q_res, SF_res, scale) tuple for ALL m rows (views of this rank's symmetric buffers, valid until
        the next transition); new_residual_local = bf16(residual_local + sum over ranks of the partial
        products) for this rank's rows.  The row-parallel GEMM in scatter mode must precede this call
        on the current stream of every rank."""
        from . import _lib, ops

        if residual_local is None and not use_partial:
            raise ValueError("nothing to normalise: no partial sums and no residual")
        if residual_local is not None and (residual_local.dtype != torch.bfloat16 or not residual_local.is_contiguous()
                                           or tuple(residual_local.shape) != (self.rows, self.hidden)):
            raise ValueError(f"residual_local must be a contiguous bf16 [{self.rows}, {self.hidden}] tensor")
        if gamma.dtype != torch.bfloat16 or not gamma.is_contiguous() or gamma.numel() != self.hidden:
            raise ValueError("gamma must be a contiguous bf16 vector of `hidden` elements")
        new_residual = torch.empty((self.rows, self.hidden), dtype=torch.bfloat16, device=self.device)
        a_comp, e, sfa, q_res, sf_res = (self._view(n) for n in ("a_comp", "e", "sfa", "q_res", "sf_res"))
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().sharq_tp_reduce_rmsnorm_prepare_allgather(
                ctypes.c_void_p(self.blocks.data_ptr()) if use_partial else None,
                None if residual_local is None else ctypes.c_void_p(residual_local.data_ptr()),
                ctypes.c_void_p(new_residual.data_ptr()), ctypes.c_void_p(gamma.data_ptr()), float(eps), self.m,
                int(out_features_hint), self.hidden, ctypes.c_void_p(self.workspace.data_ptr()), self.workspace.numel(),
                ctypes.c_void_p(a_comp.data_ptr()), ctypes.c_void_p(e.data_ptr()), ctypes.c_void_p(sfa.data_ptr()),
                ctypes.c_void_p(q_res.data_ptr()), ctypes.c_void_p(sf_res.data_ptr()), self.multicast_delta,
                ctypes.c_void_p(self.scale.data_ptr()), self.state_ptrs, self.rank, self.world,
                ctypes.c_void_p(ops._error_flag(self.device).data_ptr()),
                ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))
        prepared = ("SHARQ", a_comp, e, sfa, q_res.view(self.m, self.hidden // 2), sf_res, self.scale)
        return prepared, new_residual


_SP_CONTEXTS = {}


def sequence_parallel_context(m: int, hidden: int, group, device: torch.device) -> Optional[SequenceParallelContext]:
    """The group's shared SequenceParallelContext for activations [m, hidden], created on first use
    (collective, outside stream capture); None when the shape or the system does not qualify
    (the ranks agree on that)."""
    group = group if group is not None else dist.group.WORLD
    key = (group.group_name, device.index, m, hidden)
    if key in _SP_CONTEXTS:
        return _SP_CONTEXTS[key]
    world = dist.get_world_size(group)
    ctx = None
    if SequenceParallelContext.supported(m, hidden, world) and _multimem_wanted(group):
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the sequence-parallel context must be created before stream capture")
        err = None
        try:
            ctx = SequenceParallelContext(m, hidden, group, device)
        except RuntimeError as exc:
            ctx, err = None, exc
        ok = torch.tensor([0 if ctx is None else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            ctx = None
            if os.environ.get("SHARQ_TP_ALLREDUCE", "auto").lower() == "multimem":
                raise RuntimeError(f"the sequence-parallel context could not be set up: {err}")
    _SP_CONTEXTS[key] = ctx
    return ctx


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

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, group=None, fused_gemm: bool = True,
                 local_columns: Optional[torch.Tensor] = None, world_rank: Optional[Tuple[int, int]] = None,
                 reduce_hook=None):
        """weight: the full [N, K] matrix (its absmax gives the tensor scale).  local_columns:
        this rank's [N, K_local] part when it is not the contiguous K / world slice (padded or
        regrouped layouts).  world_rank: (world, rank) instead of the process group's.
        reduce_hook: callable(partial) -> sum, used instead of the collective (tests that run
        several ranks in one process)."""
        super().__init__(group)
        from . import ops
        from .qlinear import QLinearLayer

        if world_rank is not None:
            self.world, self.rank = int(world_rank[0]), int(world_rank[1])
        self.reduce_hook = reduce_hook
        n, k = weight.shape
        scale = torch.clamp(weight.abs().max().float() / (448.0 * 6.0), min=1e-9)
        if local_columns is None:
            b, e = shard_bounds(k, self.world, self.rank, K_ALIGN)
            local_columns = weight[:, b:e]
        if local_columns.shape[1] % K_ALIGN:
            raise ValueError(f"per-rank input size {local_columns.shape[1]} is not a multiple of {K_ALIGN}")
        q, sfs, sfd = ops.quantize_w32_shared((local_columns / scale).to(torch.bfloat16).contiguous())
        self.local = QLinearLayer.from_quantized(int(local_columns.shape[1]), n, q, sfs, sfd, scale, bias=None,
                                                 fused_gemm=fused_gemm)
        if bias is not None:
            self.register_buffer("bias", bias.to(q.device, torch.bfloat16))
        else:
            self.bias = None

    def reduce(self, y_partial: torch.Tensor) -> torch.Tensor:
        if self.reduce_hook is not None:
            y_partial = self.reduce_hook(y_partial)
        elif self.world > 1:
            dist.all_reduce(y_partial, op=dist.ReduceOp.SUM, group=self.group)
        if self.bias is not None:
            y_partial = y_partial + self.bias
        return y_partial

    def apply_prepared_reduced(self, prepared) -> torch.Tensor:
        """GEMM on a prepared K-slice and the sum over ranks.  On GPUs with NVLink multicast
        the partial sums go straight into symmetric memory and are reduced in the switch; the
        returned tensor is then a view of a shared slot (valid until SymmetricSumBuffer.SLOTS
        more row-parallel layers of the group have run)."""
        if self.world == 1 or self.reduce_hook is not None:
            return self.reduce(self.local.apply_prepared(prepared))
        m, n = int(prepared[4].shape[0]) if prepared[0] == "SHARQ" else 0, self.local.out_features
        nbytes = m * n * 2
        buf = None
        if prepared[0] == "SHARQ" and self.local.fused_gemm and nbytes > 0 and nbytes % (16 * self.world) == 0:
            buf = sum_buffer(self.group, prepared[4].device, nbytes)
        if buf is None:
            return self.reduce(self.local.apply_prepared(prepared))
        slot, view = buf.take(m, n)
        self.local.apply_prepared(prepared, out=view)
        buf.sum_(slot, nbytes)
        return view + self.bias if self.bias is not None else view

    def forward(self, x_local):
        x2 = x_local.reshape(-1, x_local.shape[-1]).to(torch.bfloat16)
        y = self.apply_prepared_reduced(self.local.prepare_input(x2))
        return y.reshape(*x_local.shape[:-1], y.shape[-1])


def all_reduce_sum_(t: torch.Tensor, group=None) -> torch.Tensor:
    """In-place sum over the group (no-op without an initialised process group)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t
