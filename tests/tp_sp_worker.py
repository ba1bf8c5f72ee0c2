"""Worker of tests/test_tp_gpu.py: one process per GPU (launched with torch.distributed.run).
Checks the one-kernel tensor-parallel layer transition (reduce-scatter of the partial sums,
residual add, RMSNorm statistics, tensor absmax over all ranks, prepare of the local rows,
all-gather of the packed activation) against the single-GPU RMSNorm prepare of the gathered
rows: every byte of every rank's prepared buffers and the tensor scale must be identical."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def check_case(ctx, m, hidden, rank, world, dev, seed, use_partial, use_residual, say):
    from sharq_b200 import ops
    from tests import helpers as H

    ok = True
    eps = 1e-6
    gamma = H.config0_gamma(hidden, seed).to(dev)
    full_res = H.config0_x(m, hidden, seed + 1).to(dev)                       # same on every rank
    part = (0.3 * H.config0_x(m, hidden, seed + 10 + rank).float()).to(torch.bfloat16).to(dev)  # differs per rank
    b, e = ctx.row_bounds()
    if use_partial:
        ctx.deliver(part)
    res_local = full_res[b:e].contiguous() if use_residual else None
    torch.cuda.synchronize()
    dist.barrier()
    prep, new_res = ctx.transition(res_local, gamma, eps, use_partial=use_partial)
    torch.cuda.synchronize()
    ops.check_device_errors()
    # the rows every rank produced
    rows = [torch.empty_like(new_res) for _ in range(world)]
    dist.all_gather(rows, new_res)
    full_new = torch.cat(rows).contiguous()
    # expected new residual: bf16(residual + bf16(fp32 sum of the partial products in rank order)), exactly
    if use_partial:
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        s32 = parts[0].float()
        for other in parts[1:]:
            s32 = s32 + other.float()
        want = (full_res.float() + s32.to(torch.bfloat16).float()).to(torch.bfloat16) if use_residual else s32.to(torch.bfloat16)
        if not torch.equal(full_new, want):
            ok = False
            say(f"new residual differs from residual + sum: max err {float((full_new.float() - want.float()).abs().max())}")
    elif not torch.equal(full_new, full_res):
        ok = False
        say("new residual differs from the residual although there were no partial sums")
    # the prepared activation of ALL rows must be what one GPU computes for the gathered rows
    ref = ops.fused_rmsnorm_sparse_residual_quantize_x(full_new, gamma, eps, hidden)
    torch.cuda.synchronize()
    for name, got, exp in zip(("a_comp", "e", "sfa_sparse", "q_res", "sf_res"), prep[1:6], ref[:5]):
        if not torch.equal(got.reshape(-1), exp.reshape(-1)):
            ok = False
            bad = int((got.reshape(-1) != exp.reshape(-1)).sum())
            say(f"{name}: {bad} bytes differ from the single-GPU prepare (m={m} hidden={hidden})")
    if not torch.equal(prep[6].reshape(()), ref[5].reshape(())):
        ok = False
        say(f"tensor scale {float(prep[6])} != {float(ref[5])}")
    return ok


def main():
    from sharq_b200 import ops, tp

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    graph = None

    def say(msg):
        print(f"rank {rank}: {msg}", flush=True)

    try:
        for m, hidden in ((128 * world, 256), (512 * world, 1024), (2048, 4096), (8192, 4096)):
            ctx = tp.sequence_parallel_context(m, hidden, None, dev)
            if ctx is None:
                raise RuntimeError("no sequence-parallel context (NVLink multicast missing?)")
            for rep, (use_partial, use_residual) in enumerate(((True, True), (True, True), (False, True), (True, False))):
                ok = check_case(ctx, m, hidden, rank, world, dev, 7 * rep + m % 13, use_partial, use_residual, say) and ok
        # the scatter-mode GEMM deals its output rows to their owners: block s of this rank's collection buffer
        # must hold rank s's plain GEMM output for this rank's rows
        from tests import helpers as H2

        ctx = tp.sequence_parallel_context(2048, 4096, None, dev)
        lin = tp.RowParallelSharqLinear(H2.config0_w(4096, 1024 * world, 3).to(dev))
        kb, ke = tp.shard_bounds(1024 * world, world, rank, tp.K_ALIGN)
        prep = lin.local.prepare_input(H2.config0_x(2048, 1024 * world, 5)[:, kb:ke].contiguous().to(dev))
        plain = lin.local.apply_prepared(prep)
        torch.cuda.synchronize()
        dist.barrier()
        lin.local.apply_prepared(prep, scatter=ctx.scatter)
        torch.cuda.synchronize()
        ops.check_device_errors()
        dist.barrier()
        outs = [torch.empty_like(plain) for _ in range(world)]
        dist.all_gather(outs, plain)
        b0, e0 = ctx.row_bounds()
        for src in range(world):
            if not torch.equal(ctx.blocks[src], outs[src][b0:e0]):
                ok = False
                say(f"scatter GEMM: block {src} differs from rank {src}'s output rows")
        # replay from a CUDA graph: the state words reset themselves
        ctx = tp.sequence_parallel_context(2048, 4096, None, dev)
        from tests import helpers as H

        gamma = H.config0_gamma(4096, 3).to(dev)
        res = H.config0_x(2048, 4096, 4).to(dev)[ctx.row_bounds()[0]:ctx.row_bounds()[1]].contiguous()
        ctx.deliver((0.2 * H.config0_x(2048, 4096, 20 + rank).float()).to(torch.bfloat16).to(dev))
        torch.cuda.synchronize()
        dist.barrier()
        prep, new_res = ctx.transition(res, gamma, 1e-6)
        torch.cuda.synchronize()
        want = [t.clone() for t in prep[1:7]] + [new_res.clone()]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ctx.transition(res, gamma, 1e-6)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(3):
                prep_g, new_g = ctx.transition(res, gamma, 1e-6)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        ops.check_device_errors()
        got = list(prep_g[1:7]) + [new_g]
        for i, (a, b) in enumerate(zip(got, want)):
            if not torch.equal(a.reshape(-1), b.reshape(-1)):
                ok = False
                say(f"graph replay: output {i} differs from the eager call")
        # whole decoder: the sequence-parallel flow against the replicated residual stream (all-reduce)
        from sharq_b200.decoder import DecoderConfig, SharqDecoder

        cfg = DecoderConfig(hidden=512, layers=3, heads=8, kv_heads=4, head_dim=64, ffn=1024, vocab=1000)
        model = SharqDecoder(cfg, dev, world=world, rank=rank, seed=5)
        ids = torch.randint(0, cfg.vocab, (2, 64 * world), generator=torch.Generator().manual_seed(1)).to(dev)
        logits_sp = model.prefill(ids)
        if model._sequence_parallel_context(ids.numel()) is None:
            ok = False
            say("the decoder did not take the sequence-parallel path")
        # reference flow: replicated residual stream with the peer-copy all-reduce, which sums the partial
        # products exactly as the transition kernel does (fp32 in rank order, one rounding), so the logits
        # must be identical
        os.environ["SHARQ_TP_SEQUENCE_PARALLEL"] = "0"
        os.environ["SHARQ_TP_ALLREDUCE"] = "peer"
        logits_ar = model.prefill(ids)
        os.environ["SHARQ_TP_SEQUENCE_PARALLEL"] = "1"
        torch.cuda.synchronize()
        ops.check_device_errors()
        rel = float((logits_sp - logits_ar).norm() / logits_ar.norm())
        say(f"decoder logits: sequence-parallel vs peer-copy all-reduce relative difference {rel:.3e}")
        if not (torch.equal(logits_sp, logits_ar) and bool(torch.isfinite(logits_sp).all())):
            ok = False
            say("decoder logits differ between the sequence-parallel and the all-reduce flow")
    except Exception as exc:  # no rank may leave while its memory is bound to the multicast object
        ok = False
        say(f"exception: {exc!r}")
    finally:
        try:
            torch.cuda.synchronize()
            flag = torch.tensor([1 if ok else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if rank == 0:
                print("TP_SP_WORKER_OK" if int(flag.item()) == 1 else "TP_SP_WORKER_FAILED", flush=True)
            if graph is not None:
                graph.reset()
            tp.release_sum_buffers()
            torch.cuda.synchronize()
            dist.barrier()
            dist.destroy_process_group()
        finally:
            sys.stdout.flush()
            os._exit(0)


if __name__ == "__main__":
    main()
