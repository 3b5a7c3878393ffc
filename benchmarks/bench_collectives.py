"""Latency / bandwidth of the native collectives against their NCCL counterparts.

    python -m torch.distributed.run --nproc-per-node N -m benchmarks.bench_collectives [--max-mb 256]

For fp32 messages of 4 KB ... --max-mb: all_reduce(sum), broadcast, all_gather (message = per-rank chunk),
reduce_scatter (message = full input), plus the barrier; every call goes through the public ``ProcessGroup`` methods
(``nvlink`` backend = this package's kernels on peer-mapped arenas; ``nccl`` backend = torch.distributed).  Times are
CUDA-event durations on the launching stream, max over ranks, median of the timed iterations.  Rank 0 prints one JSON
line per (collective, size).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=float, default=256.0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--registered", action="store_true",
                    help="also time all_reduce / broadcast / all_gather on tensors from ProcessGroup.symmetric_empty "
                         "(in place on the peers' mappings, no staging pass; NCCL gets ordinary tensors)")
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    import torch.distributed as dist

    from ferrum_b200 import distributed as d
    from ferrum_b200.parallel import Backend, ProcessGroup

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    ours = d.init_process_group_from_env("nvlink")
    nccl = ProcessGroup(Backend.Nccl, rank, world, ours.config(), _torch_group=dist.group.WORLD)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(args.iters):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t.item()))
        return statistics.median(ts)

    results = []

    def report(name, nbytes, t_ours, t_nccl, moved):
        res = {"collective": name, "bytes": nbytes, "world": world, "ours_ms": t_ours, "nccl_ms": t_nccl,
               "ours_gbs": moved / t_ours / 1e6 if t_ours > 0 else None,
               "nccl_gbs": moved / t_nccl / 1e6 if t_nccl > 0 else None, "speedup": t_nccl / t_ours}
        results.append(res)
        if rank == 0:
            print(json.dumps(res), flush=True)

    sizes = []
    nb = 4096
    while nb <= args.max_mb * (1 << 20):
        sizes.append(nb)
        nb *= 8
    for nbytes in sizes:
        n = nbytes // 4
        x = torch.randn(n, device="cuda")
        # all_reduce: bus bytes 2 (n-1)/n * size
        report("all_reduce", nbytes, timed(lambda: ours.all_reduce(x, d.ReduceOp.Sum)),
               timed(lambda: nccl.all_reduce(x, d.ReduceOp.Sum)), 2.0 * (world - 1) / world * nbytes)
        report("broadcast", nbytes, timed(lambda: ours.broadcast(x, 0)), timed(lambda: nccl.broadcast(x, 0)),
               float(nbytes))
        outs = [torch.empty(n, device="cuda") for _ in range(world)]
        report("all_gather", nbytes, timed(lambda: ours.all_gather(outs, x)), timed(lambda: nccl.all_gather(outs, x)),
               float((world - 1) * nbytes))
        if args.registered:
            xr = ours.symmetric_empty((n,))
            xr.copy_(x)
            report("all_reduce (registered)", nbytes, timed(lambda: ours.all_reduce(xr, d.ReduceOp.Sum)),
                   timed(lambda: nccl.all_reduce(x, d.ReduceOp.Sum)), 2.0 * (world - 1) / world * nbytes)
            report("broadcast (registered)", nbytes, timed(lambda: ours.broadcast(xr, 0)),
                   timed(lambda: nccl.broadcast(x, 0)), float(nbytes))
            one = torch.empty(world * n, device="cuda")
            outs1 = list(one.view(world, n).unbind(0))
            report("all_gather (registered input)", nbytes, timed(lambda: ours.all_gather(outs1, xr)),
                   timed(lambda: nccl.all_gather(outs1, x)), float((world - 1) * nbytes))
        chunk = max(n // world, 1)
        ins = [torch.randn(chunk, device="cuda") for _ in range(world)]
        o = torch.empty(chunk, device="cuda")
        report("reduce_scatter", chunk * 4 * world,
               timed(lambda: ours.reduce_scatter(o, ins, d.ReduceOp.Sum)),
               timed(lambda: nccl.reduce_scatter(o, ins, d.ReduceOp.Sum)), float((world - 1) * chunk * 4))
    report("barrier", 0, timed(ours.barrier), timed(nccl.barrier), 0.0)
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    d.destroy_process_group()


if __name__ == "__main__":
    main()
