"""Worker of tests/test_tp_gpu.py: one process per GPU (launched with torch.distributed.run).
Checks the in-switch all-reduce of a row-parallel SharQ linear against the fp32 sum of the
gathered partial outputs, eagerly, repeatedly and replayed from a CUDA graph."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main():
    from sharq_b200 import ops, tp
    from tests import helpers as H

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    g = None
    try:
        # "multimem": the in-switch kernel (fails loudly instead of falling back); "auto": with two
        # ranks the peer-copy kernel
        for mode, (m, n, k) in [(md, shape) for md in ("multimem", "auto")
                                for shape in ((256, 512, 1024), (2048, 4096, 4096), (300, 384, 2048))]:
            if os.environ.get("SHARQ_TP_ALLREDUCE") != mode:
                torch.cuda.synchronize()
                dist.barrier()
                tp.release_sum_buffers()
                os.environ["SHARQ_TP_ALLREDUCE"] = mode
            w = H.config0_w(n, k, 3).to(dev)
            lin = tp.RowParallelSharqLinear(w)
            b, e = tp.shard_bounds(k, world, rank, tp.K_ALIGN)
            x = H.config0_x(m, k, 5)[:, b:e].contiguous().to(dev)
            prep = lin.local.prepare_input(x)
            partial = lin.local.apply_prepared(prep)
            gathered = [torch.empty_like(partial) for _ in range(world)]
            dist.all_gather(gathered, partial)
            want = torch.stack([g.float() for g in gathered]).sum(0)
            for rep in range(3):
                got = lin.apply_prepared_reduced(prep).clone()
                torch.cuda.synchronize()
                ops.check_device_errors()
                # fp32 accumulation inside the switch, one rounding to bf16: within one bf16 ulp of
                # the fp32 sum whatever the order of the additions
                err = (got.float() - want).abs()
                tol = want.abs() * 2.0 ** -7 + 1e-30
                if not bool((err <= tol).all()):
                    ok = False
                    print(f"rank {rank}: mismatch mode={mode} m={m} n={n} k={k} rep={rep} max err {float(err.max())}", flush=True)
            # every rank must hold the same bytes
            mine = lin.apply_prepared_reduced(prep).clone()
            peers = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(peers, mine)
            if not all(torch.equal(p, mine) for p in peers):
                ok = False
                print(f"rank {rank}: ranks disagree m={m} n={n} k={k}", flush=True)
        # replay from a CUDA graph (flags must reset themselves)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            lin.apply_prepared_reduced(prep)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            outs = [lin.apply_prepared_reduced(prep).clone() for _ in range(3)]
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        ops.check_device_errors()
        for o in outs:
            if not bool(((o.float() - want).abs() <= want.abs() * 2.0 ** -7 + 1e-30).all()):
                ok = False
                print(f"rank {rank}: graph replay mismatch", flush=True)
    except Exception as exc:  # no rank may leave while its memory is bound to the multicast object
        ok = False
        print(f"rank {rank}: exception: {exc!r}", flush=True)
    finally:
        try:
            torch.cuda.synchronize()
            flag = torch.tensor([1 if ok else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if rank == 0:
                print("TP_GPU_WORKER_OK" if int(flag.item()) == 1 else "TP_GPU_WORKER_FAILED", flush=True)
            if g is not None:
                g.reset()
            tp.release_sum_buffers()
            torch.cuda.synchronize()
            dist.barrier()
            dist.destroy_process_group()
        finally:
            sys.stdout.flush()
            os._exit(0)


if __name__ == "__main__":
    main()
