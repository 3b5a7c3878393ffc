"""Where the time of a data-parallel step goes: per-bucket timeline of the fused reduction kernels.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m benchmarks.ddp_timeline [--steps 8] [--comm-blocks B] [--no-shard-master] [--bucket-mb 25]

The headline model (8 x [Linear 4096 - GELU - LayerNorm] + head, per-GPU batch 8192, bf16 autocast, Adam fused into
the bucket kernels) runs with eager launches and ``DistributedDataParallel.comm_profile``: CUDA events give, per
bucket, when its last gradient was enqueued, when its kernel started and ended on the communication stream, and
when the backward pass ended on the compute stream.  Rank 0 prints one JSON line with the per-bucket medians over
the timed steps (max over ranks for the step time) — the table behind "how much of the multi-GPU step is
contention and how much is an exposed tail".  No profiler is involved; nothing here waits on another rank outside
the engine's own bounded handshakes.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--width", type=int, default=4096)
    ap.add_argument("--depth", type=int, default=8)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--comm-blocks", type=int, default=0, help="0 = the engine's default for this world size")
    ap.add_argument("--update-blocks", type=int, default=0, help="blocks of the update kernel (0 = engine default)")
    ap.add_argument("--update-in-backward", action="store_true",
                    help="update kernel per bucket behind its reduce-scatter instead of once after backward")
    ap.add_argument("--no-shard-master", action="store_true")
    ap.add_argument("--single-kernel", action="store_true",
                    help="all-reduce + update + publish in one kernel per bucket inside backward (defer_update(False))")
    a = ap.parse_args()

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    import ferrum_b200 as fb
    from ferrum_b200 import nn, optim
    from ferrum_b200.models import wide_mlp

    dev = fb.Device.Cuda(local)
    fb.distributed.init_process_group_from_env(backend="nvlink")
    torch.manual_seed(1234)
    model = wide_mlp(1024, a.width, a.depth, 1000, device=dev)
    opt = optim.Adam(model.parameters(), optim.AdamConfig(lr=3e-4))
    eng = fb.distributed.DistributedDataParallel(model, fb.distributed.get_world()).bucket_size_mb(a.bucket_mb)
    eng.fuse_optimizer(opt)
    if world > 1 and not a.no_shard_master:
        eng.shard_master_weights(True)
    if a.single_kernel:
        eng.defer_update(False)
    if a.update_in_backward:
        eng.update_in_backward(True)
    if a.update_blocks > 0:
        eng._update_blocks = a.update_blocks
    if a.comm_blocks > 0:
        eng._comm_blocks = a.comm_blocks
    eng.comm_profile(True)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x = torch.randn(a.batch, 1024, device="cuda", generator=g)
    y = torch.randint(0, 1000, (a.batch,), device="cuda", generator=g)

    def step():
        opt.zero_grad()
        with fb.autocast():
            loss = nn.cross_entropy(eng(x), y)
        loss.backward()
        opt.step()

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    recs, step_ms = [], []
    for _ in range(a.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        step_ms.append(e0.elapsed_time(e1))
        recs.append(eng.last_comm_profile())
    fb.utils.runtime.check_status()
    med = statistics.median
    nb = len(recs[0]["buckets"])
    table = []
    for i in range(nb):
        rows = [r["buckets"][i] for r in recs]
        table.append({"bucket": rows[0]["index"], "mb": round(rows[0]["bytes"] / 2 ** 20, 2),
                      "ready_ms": round(med(r["ready_ms"] for r in rows), 3),
                      "start_ms": round(med(r["start_ms"] for r in rows), 3),
                      "end_ms": round(med(r["end_ms"] for r in rows), 3),
                      "kernel_us": round(med(r["kernel_us"] for r in rows), 1),
                      "bus_gbs": round(med(r["bus_gbs"] for r in rows), 1)})
    mine = {"step_ms": med(step_ms), "backward_end_ms": med(r["backward_end_ms"] for r in recs),
            "step_end_ms": med(r["step_end_ms"] for r in recs),
            "exposed_tail_us": med(r["exposed_tail_us"] for r in recs),
            "comm_busy_us": med(r["comm_busy_us"] for r in recs)}
    t = torch.tensor([mine["step_ms"], mine["exposed_tail_us"]], device="cuda")
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    eng.shutdown()
    fb.distributed.destroy_process_group()
    if rank == 0:
        print(json.dumps({"world": world, "comm_blocks": eng._comm_blocks, "shard_master": eng._shard_master,
                          "bucket_mb": a.bucket_mb, "launches": "eager",
                          "reduction": "single kernel per bucket" if a.single_kernel else "reduce-scatter per bucket + one update kernel", "step_ms_max_over_ranks": float(t[0]),
                          "exposed_tail_us_max_over_ranks": float(t[1]), "rank0": mine, "buckets_rank0": table}))


if __name__ == "__main__":
    main()
