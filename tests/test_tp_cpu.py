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
