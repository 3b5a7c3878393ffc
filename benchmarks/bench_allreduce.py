"""Sweep of the fused all-reduce + Adam kernel against NCCL all-reduce followed by a separate torch Adam.

    python -m torch.distributed.run --nproc-per-node N -m benchmarks.bench_allreduce [--max-mb 1024]

fp32 gradient buckets of 4 KB ... 1 GB filled ~ N(0, 1e-2), random Adam state.  Times are CUDA-event durations
on the launching stream, max over ranks, median of the timed iterations; "bus GB/s" uses the all-reduce
convention 2 (n-1)/n * bytes / time.  Rank 0 prints one JSON line per size.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics

import torch


def emulated(args):
    """The fused all-reduce + Adam body with every rank's arena on this GPU: device time per bucket size and the
    local-memory bandwidth it reaches (world reads of the gradients + parameter, moment and bf16 traffic)."""
    from ferrum_b200 import _lib
    from ferrum_b200._lib_dist import DistCtx
    from ferrum_b200.parallel.symm import SymmetricArena
    from ferrum_b200.utils import runtime as rt

    world = args.emulated
    lib = _lib.cuda()
    max_elems = int(args.max_mb * (1 << 20)) // 4 // (4 * world) * (4 * world)
    arenas = SymmetricArena.emulated(max_elems * 10, world)
    ctxs = (DistCtx * world)(*[a.ctx for a in arenas])
    base = arenas[0].data_offset()
    off_p, off_g, off_s = base, base + max_elems * 4, base + max_elems * 8
    for a in arenas:
        a.view(off_p, (max_elems,), torch.float32).normal_()
        a.view(off_g, (max_elems,), torch.float32).normal_(0, 1e-2)
    per = max_elems // world + 4
    ms_ = [torch.zeros(per, device="cuda") for _ in range(world)]
    vs_ = [torch.zeros(per, device="cuda") for _ in range(world)]
    mp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in ms_])
    vp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in vs_])
    stream = torch.cuda.current_stream().cuda_stream
    blocks = max(1, min(args.blocks, 128 // world))  # world x blocks must be co-resident (cooperative launch)
    epoch, n = 1, max_elems
    ts = []
    for i in range(args.iters + 3):
        t = i + 1
        h = _lib.AdamH(3e-4, 0.9, 0.999, 1e-8, 0.0, 1 - 0.9 ** t, 1 - 0.999 ** t, 1.0 / world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = lib.fb_dist_allreduce_emulated(ctxs, world, 2, 0, epoch, off_g, off_p, off_s, n, 0, 1.0,
                                            ctypes.byref(h), None, mp, vp, 1, blocks, args.threads, stream)
        e1.record()
        assert rc == 0, rc
        epoch += 2
        torch.cuda.synchronize()
        if i >= 3:
            ts.append(e0.elapsed_time(e1))
    rt.check_status()
    ms = statistics.median(ts)
    # per element over all virtual ranks: world gradient reads, 1 parameter read, 2 + 2 moment accesses,
    # world parameter writes and world bf16 writes
    moved = n * (4 * world + 4 + 16 + 4 * world + 2 * world)
    print(json.dumps({"kernel": "allreduce_emulated_kernel<adam>", "world": world, "bucket_bytes": n * 4,
                      "blocks_per_rank": blocks, "ms": ms, "local_GBps": moved / 1e9 / (ms / 1e3)}), flush=True)
    for a in arenas:
        a.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=float, default=1024.0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--blocks", type=int, default=128)
    ap.add_argument("--threads", type=int, default=256)
    ap.add_argument("--shard-master", action="store_true", help="publish only the bf16 copy to peers")
    ap.add_argument("--sizes-mb", default="", help="comma-separated bucket sizes in MB instead of the 4 KB .. max sweep")
    ap.add_argument("--out", default="")
    ap.add_argument("--emulated", type=int, default=0, metavar="W",
                    help="one process, one GPU: W ranks emulated by one cooperative launch of the same device code "
                         "(all 'peer' loads stay on this GPU); the form that a profiler may wrap")
    args = ap.parse_args()
    if args.emulated:
        return emulated(args)

    import torch.distributed as dist

    import ferrum_b200 as fb
    from ferrum_b200 import _lib
    from ferrum_b200 import distributed as d
    from ferrum_b200.parallel.symm import SymmetricArena

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    pg = d.init_process_group_from_env("nvlink")
    lib = _lib.cuda()
    max_elems = int(args.max_mb * (1 << 20)) // 4
    arena = SymmetricArena.create(max_elems * 10, rank, world, pg.exchange, pg.config().device_wait_ns())
    base = arena.data_offset()
    off_p, off_g, off_s = base, base + max_elems * 4, base + max_elems * 8
    params = arena.view(off_p, (max_elems,), torch.float32)
    grads = arena.view(off_g, (max_elems,), torch.float32)
    params.normal_()
    grads.normal_(0, 1e-2)
    per_max = (max_elems + world - 1) // world + 4
    m = torch.randn(per_max, device="cuda") * 1e-3
    v = torch.rand(per_max, device="cuda") * 1e-4
    # baseline tensors
    b_grad = torch.randn(max_elems, device="cuda") * 1e-2
    b_param = torch.nn.Parameter(torch.randn(max_elems, device="cuda"))
    stream = torch.cuda.current_stream()
    sizes = []
    nb = 4096
    while nb <= args.max_mb * (1 << 20):
        sizes.append(nb)
        nb *= 4
    if sizes[-1] != int(args.max_mb * (1 << 20)):
        sizes.append(int(args.max_mb * (1 << 20)))
    if args.sizes_mb:
        sizes = [int(float(x) * (1 << 20)) for x in args.sizes_mb.split(",")]
    results = []

    def timed(fn, iters):
        ts = []
        for i in range(iters + 3):
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                ts.append(e0.elapsed_time(e1))
        t = torch.tensor([statistics.median(ts)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    step = [0]
    for nbytes in sizes:
        n = nbytes // 4
        n = max(4 * world, n // (4 * world) * (4 * world))
        use_mc = 1 if arena.has_multicast() else 0

        def ours():
            step[0] += 1
            t = step[0]
            h = _lib.AdamH(3e-4, 0.9, 0.999, 1e-8, 0.0, 1 - 0.9 ** t, 1 - 0.999 ** t, 1.0 / world)
            e = arena.next_epoch(0)
            rc = lib.fb_dist_allreduce(arena.ctx, 2, use_mc, 0, e, off_g, off_p, off_s, n, 0, 1.0, ctypes.byref(h),
                                       None, m.data_ptr(), v.data_ptr(), 0 if args.shard_master else 1,
                                       min(args.blocks, max(1, n // 4096)),
                                       args.threads, stream.cuda_stream)
            assert rc == 0, rc

        bp = torch.nn.Parameter(b_param.data[:n])
        bg = b_grad[:n]
        bopt = torch.optim.Adam([bp], lr=3e-4, fused=True)

        def baseline():
            dist.all_reduce(bg)
            bp.grad = bg
            bg.mul_(1.0 / world)
            bopt.step()

        iters = args.iters if nbytes <= (256 << 20) else max(5, args.iters // 4)
        t_ours = timed(ours, iters)
        t_base = timed(baseline, iters)
        bus = 2 * (world - 1) / world * n * 4 / 1e9
        res = {"bytes": n * 4, "world": world, "fused_ms": t_ours, "nccl_plus_adam_ms": t_base,
               "fused_bus_gbs": bus / (t_ours / 1e3), "baseline_bus_gbs": bus / (t_base / 1e3),
               "speedup": t_base / t_ours, "multicast": bool(use_mc), "blocks": args.blocks,
               "shard_master": bool(args.shard_master)}
        results.append(res)
        if rank == 0:
            print(json.dumps(res), flush=True)
    fb.utils.runtime.check_status()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    dist.barrier()
    arena.close()
    d.destroy_process_group()


if __name__ == "__main__":
    main()
