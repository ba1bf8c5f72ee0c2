"""Host-side logic of the tensor-parallel layers on CPU: shard arithmetic, and a 2-rank
gloo run of the column-parallel / row-parallel + all-reduce data flow with a float matmul
standing in for the local GEMM (the kernels themselves need a GPU)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sharq_b200 import tp


def test_shard_bounds_and_padding():
    assert tp.shard_bounds(4096, 8, 3, 128) == (1536, 2048)
    assert tp.shard_bounds(14336, 8, 7, 128) == (12544, 14336)
    with pytest.raises(ValueError):
        tp.shard_bounds(18944, 8, 0, 128)  # Qwen2.5-7B FFN over 8 ranks: 2368 is not a multiple of 128
    assert tp.padded_size(18944, 8, 128) == 19456
    assert tp.padded_size(4096, 8, 128) == 4096
    with pytest.raises(ValueError):
        tp.shard_bounds(28, 8, 0, 1)


def test_global_weight_scale_is_shared_by_shards():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(256, 512, generator=g).to(torch.bfloat16)
    w_scaled, scale = tp.scaled_weight(w)
    full = torch.clamp(w.abs().max().float() / 2688.0, min=1e-9)
    assert scale == full
    # slices of the scaled weight are what each rank quantises; no per-shard rescaling
    b, e = tp.shard_bounds(512, 2, 1, 128)
    assert torch.equal(w_scaled[:, b:e], (w / full).to(torch.bfloat16)[:, b:e])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        x = torch.randn(16, 256, generator=g)
        w_col = torch.randn(512, 256, generator=g)   # column-parallel: shard N
        w_row = torch.randn(128, 512, generator=g)   # row-parallel: shard K
        nb, ne = tp.shard_bounds(512, world, rank, 128)
        h_local = x @ w_col[nb:ne].T                  # this rank's slice of the hidden activation
        kb, ke = tp.shard_bounds(512, world, rank, 128)
        assert (kb, ke) == (nb, ne)                   # column output slice feeds the row-parallel input
        y = h_local @ w_row[:, kb:ke].T               # partial sum
        tp.all_reduce_sum_(y)
        ref = (x @ w_col.T) @ w_row.T
        out[rank] = float((y - ref).abs().max() / ref.abs().max())
    finally:
        dist.destroy_process_group()


def test_column_then_row_parallel_all_reduce_gloo():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert len(out) == world
    for r in range(world):
        assert out[r] < 1e-5


def test_head_layout_for_non_divisible_models():
    from sharq_b200.tp import head_layout, padded_size

    # Llama-3-8B on 8 ranks: contiguous
    lay = head_layout(32, 8, 8)
    assert lay[3] == ([12, 13, 14, 15], [3])
    # Qwen2.5-7B on 8 ranks: 28 query / 4 KV heads -> KV heads on two ranks each, 4 + 3 (+1 pad) query heads
    lay = head_layout(28, 4, 8)
    assert lay[0] == ([0, 1, 2, 3], [0]) and lay[1] == ([4, 5, 6, -1], [0]) and lay[7] == ([25, 26, 27, -1], [3])
    real = sorted(i for ids, _ in lay for i in ids if i >= 0)
    assert real == list(range(28))  # every query head exactly once
    for ids, kv in lay:  # a rank's query heads all belong to its KV head
        assert all(i // 7 == kv[0] for i in ids if i >= 0)
    assert head_layout(28, 4, 4)[2] == (list(range(14, 21)), [2])
    assert padded_size(18944, 8, 128) == 19456 and padded_size(18944, 4, 128) == 18944
    import pytest
    with pytest.raises(ValueError):
        head_layout(28, 4, 3)


def _leaving_worker(rank, world, port, out):
    """Step 1 runs on every rank; rank 1 then leaves between the steps (no collective in
    flight).  The surviving rank's next all-reduce must end with an error within the
    process-group timeout instead of hanging."""
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    y = torch.ones(8, 8) * (rank + 1)
    tp.all_reduce_sum_(y)
    out[f"step1_{rank}"] = float(y[0, 0])
    if rank == 1:
        os._exit(0)  # leaves between two steps
    t0 = time.time()
    try:
        tp.all_reduce_sum_(torch.ones(8, 8))
        out["survivor"] = "no error"
    except RuntimeError as exc:
        out["survivor"] = f"RuntimeError after {time.time() - t0:.1f}s"
    os._exit(0)


def test_a_rank_that_leaves_ends_the_next_all_reduce_with_an_error():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_leaving_worker, args=(r, world, _free_port_shared(), out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank hung after its peer left"
    assert out["step1_0"] == 3.0 and out["step1_1"] == 3.0
    assert out["survivor"].startswith("RuntimeError"), out["survivor"]


_PORT = {}


def _free_port_shared():
    if "p" not in _PORT:
        _PORT["p"] = _free_port()
    return _PORT["p"]


def _mismatch_worker(rank, world, port, out):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        y = torch.ones(8, 8 if rank == 0 else 16)  # the ranks disagree on the shape of the partial sum
        tp.all_reduce_sum_(y)
        out[rank] = "no error"
    except RuntimeError as exc:
        out[rank] = "RuntimeError"
    os._exit(0)


def test_mismatched_partial_sum_shapes_raise():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_mismatch_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank hung on mismatched shapes"
    assert any(v == "RuntimeError" for v in out.values()), dict(out)


def _sp_flow_worker(rank, world, port, out):
    """The sequence-parallel data flow (reduce-scatter of the partial sums, add to the local rows
    of the residual stream, normalise, all-gather) with gloo collectives and float matmuls in
    place of the kernels: it must reproduce the replicated flow (all-reduce, every rank adds
    and normalises all rows)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1)
        m, h, f = 256 * world, 64, 256
        resid = torch.randn(m, h, generator=g)
        act = torch.randn(m, f, generator=g)
        w_row = torch.randn(h, f, generator=g)
        gamma = 1 + 0.1 * torch.randn(h, generator=g)
        kb, ke = tp.shard_bounds(f, world, rank, 128)
        partial = act[:, kb:ke] @ w_row[:, kb:ke].T

        def norm(t):
            return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma

        # replicated residual stream
        full = partial.clone()
        tp.all_reduce_sum_(full)
        want = norm(resid + full)
        # row-sharded residual stream
        assert tp.SequenceParallelContext.supported(m, 128, world)
        rows = m // world
        mine = full[rank * rows:(rank + 1) * rows]  # gloo has no reduce-scatter: this rank's rows of the sum
        local = norm(resid[rank * rows:(rank + 1) * rows] + mine)
        gathered = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        out[rank] = float((torch.cat(gathered) - want).abs().max())
    finally:
        dist.destroy_process_group()


def test_sequence_parallel_flow_equals_replicated_flow_gloo():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_sp_flow_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert len(out) == world and all(out[r] == 0.0 for r in range(world)), dict(out)
    assert not tp.SequenceParallelContext.supported(2048, 4096, 1)
    assert not tp.SequenceParallelContext.supported(2048 + 64, 4096, 8)
    assert tp.SequenceParallelContext.supported(2048, 4096, 8)


@pytest.mark.parametrize("m,k,world", [(2048, 4096, 8), (2048, 4096, 2), (1024, 3584, 4), (512, 14336, 2), (256, 384, 2)])
def test_transition_all_gather_ranges_cover_exactly_the_ranks_rows(m, k, world):
    """The all-gather phase of the transition kernel (sp_transition.cu), restated: the 16-byte pieces a
    rank pushes to its peers are enumerated as five contiguous runs (Q_res rows, A_comp rows, one run of
    16-byte metadata rows per 256-column tile, the scale-factor bands of both layouts).  Together they
    must be exactly the bytes that the rank's rows occupy in the reference layouts - every byte of
    its rows, and no byte of another rank's rows."""
    import numpy as np

    from oracle import sharq_oracle as oracle

    rows = m // world
    assert rows % 128 == 0
    aligned_m = (m + 127) // 128 * 128
    groups32, groups_padded = k // 32, (k + 255) // 256 * 8
    k_tiles = groups_padded // 8
    for rank in range(world):
        row0 = rank * rows
        pieces = {name: set() for name in ("q_res", "a_comp", "e", "sfa", "sf_res")}
        n_q, n_a, n_e = rows * (k // 2) // 16, rows * (k // 4) // 16, k_tiles * rows
        n_sfa, n_sfr = (rows // 128) * (groups32 // 4) * 32, (rows // 128) * (k // 64) * 32
        for i in range(n_q + n_a + n_e + n_sfa + n_sfr):  # the kernel's piece index -> (buffer, byte offset)
            j = i
            if j < n_q:
                pieces["q_res"].add(row0 * (k // 2) + j * 16)
            elif (j := j - n_q) < n_a:
                pieces["a_comp"].add(row0 * (k // 4) + j * 16)
            elif (j := j - n_a) < n_e:
                kt, r = divmod(j, rows)
                pieces["e"].add((kt * aligned_m + row0 + r) * 16)
            elif (j := j - n_e) < n_sfa:
                pieces["sfa"].add((row0 // 128) * (groups32 // 4) * 512 + j * 16)
            else:
                j -= n_sfa
                pieces["sf_res"].add((row0 // 128) * (k // 64) * 512 + j * 16)
        mine = np.arange(row0, row0 + rows)
        want = {
            "q_res": {int(r) * (k // 2) + c for r in mine for c in range(0, k // 2, 16)},
            "a_comp": {int(r) * (k // 4) + c for r in mine for c in range(0, k // 4, 16)},
            "e": {(kt * aligned_m + int(r)) * 16 for kt in range(k_tiles) for r in mine},
            "sfa": {int(o) // 16 * 16 for o in oracle.sf_offsets(m, groups32)[mine].reshape(-1)},
            "sf_res": {int(o) // 16 * 16 for o in oracle.sf_offsets(m, k // 16)[mine].reshape(-1)},
        }
        for name in pieces:
            assert pieces[name] == want[name], (name, rank)
