"""Headline benchmark: training throughput of the 8-block, 4096-wide MLP (125.8 M parameters).

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference|torch]

Model / config: 8 x [Linear(., 4096) - GELU - LayerNorm(4096)], input 1024 features ~ N(0,1), 1000-way head,
uniform labels, cross-entropy, Adam lr 3e-4, per-GPU batch 8192, fp32 master weights, bf16 tensor-core GEMMs,
25 MB gradient buckets; weak scaling (per-GPU batch fixed).  Synthetic data, random-init weights.

One rank per GPU.  For N > 1 launch with ``python -m torch.distributed.run --nnodes=1 --nproc-per-node N
--master-addr 127.0.0.1 --master-port P bench.py --gpus N ...``.  W untimed warm-up steps, then exactly K steps
timed with CUDA events between barrier + synchronize pairs; the reported time is the max over ranks.  Rank 0
prints one JSON line.

``--impl torch`` runs the stock torch DDP (NCCL + cuBLAS, bf16 autocast, fused Adam) build of the same model:
the comparison baseline.  ``--impl ours`` (the default) runs that baseline too, in the same invocation after its own
arm (same N, steps, warm-up, its own clock samples), and reports ``vs_baseline`` = its samples/s divided by the
baseline's, with the baseline's figures under ``baseline``; ``--no-baseline`` skips it.  ``--impl reference`` is the
arm for the unmodified reference; it is a Rust workspace with no Python package and no toolchain to build it in this
image, so that arm reports itself unavailable.

End-to-end arm (``e2e``): every step's batch is drawn by a seeded ``RandomSampler`` from a dataset of several
batches held in pinned host memory, assembled by the ``DataLoader``'s native worker threads, copied to the GPU
(one step ahead, on a side stream) and the loss is read back to the host every step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

MODEL = dict(in_features=1024, width=4096, depth=8, num_classes=1000)
PER_GPU_BATCH = 8192
LR = 3e-4


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--batch", type=int, default=PER_GPU_BATCH, help="per-GPU batch")
    ap.add_argument("--depth", type=int, default=MODEL["depth"])
    ap.add_argument("--width", type=int, default=MODEL["width"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-baseline", action="store_true",
                    help="skip the torch-DDP baseline arm that --impl ours runs after its own (vs_baseline = null)")
    ap.add_argument("--dataset-batches", type=int, default=8,
                    help="batches in the pinned-host dataset the end-to-end arm samples from")
    ap.add_argument("--loader-workers", type=int, default=6, help="gather threads of the end-to-end DataLoader")
    ap.add_argument("--overlap-optimizer", action="store_true",
                    help="1 GPU: run Adam per bucket behind each weight gradient on a side stream (the engine every "
                         "multi-GPU run uses) instead of one pass after backward; measured slower at one GPU "
                         "(7.22 vs 6.69 ms/step: the update kernels contend with the GEMMs for HBM)")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every kernel of the end-to-end step from Python instead of replaying the step "
                         "recorded in a CUDA graph (multi-GPU: the engine in capturable mode; measured at 2 GPUs: "
                         "2.372 M samples/s replayed vs 2.273 M launched from Python)")
    ap.add_argument("--graph-ddp", action="store_true", help="accepted for compatibility; the graph is the default")
    ap.add_argument("--shard-master", action="store_true",
                    help="DDP: publish only bf16 weights to peers, fp32 master weights stay with the shard owner "
                         "(ZeRO-1 style; the default with several GPUs: 6.97 vs 7.71 ms/step measured at 8 GPUs, 6.83 vs 6.94 at 2)")
    ap.add_argument("--single-kernel-reduction", action="store_true",
                    help="DDP: all-reduce + Adam + publish in one kernel per bucket inside backward instead of a "
                         "reduce-scatter per bucket and one update kernel after backward (the default)")
    ap.add_argument("--update-in-backward", action="store_true",
                    help="DDP: launch the update kernel per bucket behind its reduce-scatter, inside backward")
    ap.add_argument("--no-shard-master", action="store_true",
                    help="DDP: every rank keeps the full fp32 master weights current after every step")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [s for s, p in zip(sm, power) if p > 300.0] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def merge_clocks(mine: dict, world: int):
    """Rank 0 gets its own record plus the slowest median clock and the union of reasons over all ranks' GPUs."""
    if world <= 1:
        return mine
    import torch.distributed as dist

    allc = [None] * world
    dist.all_gather_object(allc, mine)
    out = dict(allc[0])
    meds = [c["sm_mhz"] for c in allc if c and c.get("sm_mhz") is not None]
    out["sm_mhz_min_over_ranks"] = min(meds) if meds else None
    out["sm_mhz_per_rank"] = [c.get("sm_mhz") if c else None for c in allc]
    out["reasons"] = sorted({r for c in allc if c for r in c.get("reasons", [])})
    return out


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def timed_steps(step_fn, steps, world, barrier, finish=None):
    """K calls of ``step_fn`` (and ``finish()``, which collects results still in flight) between two events."""
    import torch

    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step_fn()
    if finish is not None:
        finish()
    e1.record()
    barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def run_ours(args):
    import torch

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    import ferrum_b200 as fb
    from ferrum_b200 import _lib, nn, optim
    from ferrum_b200.models import wide_mlp

    dev = fb.Device.Cuda(local)
    use_engine = world > 1 or args.overlap_optimizer
    if use_engine:
        fb.distributed.init_process_group_from_env(backend="nvlink")
    torch.manual_seed(1234)
    model = wide_mlp(MODEL["in_features"], args.width, args.depth, MODEL["num_classes"], device=dev)
    opt = optim.Adam(model.parameters(), optim.AdamConfig(lr=LR))
    engine = None
    if use_engine:
        engine = fb.distributed.DistributedDataParallel(model, fb.distributed.get_world()).bucket_size_mb(25)
        engine.fuse_optimizer(opt)
        if args.single_kernel_reduction:
            engine.defer_update(False)
        if args.update_in_backward or args.overlap_optimizer:
            engine.update_in_backward(True)
        shard = args.shard_master or (world >= 2 and not args.no_shard_master)
        if shard:
            engine.shard_master_weights(True)
        net = engine
    else:
        net = model
    B = args.batch
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x_dev = torch.randn(B, MODEL["in_features"], device="cuda", generator=g)
    y_dev = torch.randint(0, MODEL["num_classes"], (B,), device="cuda", generator=g)
    # end-to-end input pipeline: a dataset of several batches in pinned host memory, a seeded shuffle per epoch,
    # rows gathered by the loader's native worker threads, device copy one step ahead on a side stream
    nb = max(2, args.dataset_batches)
    gh = torch.Generator().manual_seed(200 + rank)
    x_pin = torch.empty(nb * B, MODEL["in_features"]).pin_memory()
    y_pin = torch.empty(nb * B, dtype=torch.int64).pin_memory()
    x_pin.normal_(generator=gh)
    y_pin.random_(0, MODEL["num_classes"], generator=gh)

    def train_step(x, y):
        opt.zero_grad()
        with fb.autocast():
            logits = net(x)
            loss = nn.cross_entropy(logits, y)
        loss.backward()
        opt.step()
        return loss

    def step_device():
        train_step(x_dev, y_dev)

    losses = []

    loader = (fb.data.DataLoader(fb.data.TensorDataset.from_tensors(x_pin, y_pin)).batch_size(B).shuffle(True)
              .seed(77 + rank).drop_last(True).num_workers(args.loader_workers).pin_memory(True).to(dev).repeat(True))
    feed = iter(loader)
    readback = fb.cuda.HostReadback()

    graph_box = [None]

    def make_graph():
        """The whole step (zero_grad, forward, backward, bucket reductions, Adam) is recorded once in a CUDA graph
        and replayed, so the read-back of the loss at the end of a step does not expose ~70 Python-issued launches
        at the start of the next one.  Falls back to eager launches if the step cannot be captured; with several
        ranks they agree on it first, so that recorded and eager steps never mix."""
        if args.no_graph:
            return
        try:
            graph_box[0] = fb.cuda.GraphedStep(train_step, (x_dev, y_dev), optimizer=opt)
        except Exception as exc:  # noqa: BLE001 - any capture failure means: run eagerly
            print(f"[bench] rank {rank}: CUDA-graph capture unavailable ({type(exc).__name__}: {exc}); eager e2e",
                  file=sys.stderr)
        if world > 1:
            import torch.distributed as dist

            ok = torch.tensor([1 if graph_box[0] is not None else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                graph_box[0] = None

    def step_e2e():
        xb, yb = next(feed)                # host -> device copy of this step's inputs (issued one step ahead)
        x, y = xb._t, yb._t
        loss = graph_box[0](x, y) if graph_box[0] is not None else train_step(x, y)
        readback.push(loss)                # device -> host copy of the step result, enqueued behind the step
        if readback.pending() > 1:         # read the previous step's loss while this step runs
            losses.append(readback.pop())

    def drain_e2e():
        while readback.pending():
            losses.append(readback.pop())

    if world > 1:
        import torch.distributed as dist

        barrier = dist.barrier
    else:
        def barrier():
            return None

    for _ in range(max(args.warmup, 3)):
        step_device()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = _lib.launch_count()
    ms_eager = timed_steps(step_device, args.steps, world, barrier)
    launches = _lib.launch_count() - launches0
    # The same K steps again with the step replayed from a CUDA graph (what a user of GraphedStep runs); the
    # headline value is taken from the replayed steps when the step could be recorded.
    make_graph()
    ms = ms_eager
    if graph_box[0] is not None:
        def step_graph():
            graph_box[0](x_dev, y_dev)

        for _ in range(3):
            step_graph()
        ms = timed_steps(step_graph, args.steps, world, barrier)
    clocks = merge_clocks(sampler.stop(), world)
    e2e = None
    if not args.no_e2e:
        for _ in range(3):
            step_e2e()
        drain_e2e()
        ms_e2e = timed_steps(step_e2e, args.steps, world, barrier, finish=drain_e2e)
        assert len(losses) == args.steps + 3, "every step's loss is read on the host"
        e2e = {"value": args.steps * B * world / (ms_e2e / 1e3), "unit": "samples/s",
               "ms_per_step": ms_e2e / args.steps,
               "h2d_bytes_per_step": B * (x_pin.shape[1] * x_pin.element_size() + y_pin.element_size()),
               "d2h_bytes_per_step": 4, "final_loss": losses[-1] if losses else None,
               "cuda_graph": graph_box[0] is not None,
               "loss_readback": "every step, read on the host one step later (pinned buffer + event)",
               "input_pipeline": f"DataLoader over {nb} batches in pinned host memory, seeded RandomSampler per "
                                 f"epoch, {args.loader_workers} native gather threads, device copy one step ahead "
                                 "on a side stream"}
    feed.close()
    loader.close()
    fb.utils.runtime.check_status()
    multimem = None
    if engine is not None:
        arena = getattr(engine, "_arena", None)
        multimem = arena.has_multicast() if arena is not None else None
        engine.shutdown()
    if use_engine:
        # the torch.distributed rendezvous stays up for the baseline arm that follows in this process
        fb.distributed.destroy_process_group(keep_torch=True)

    if world > 1:
        par = "nvlink-fused-ddp" + ("-sharded-master" if shard else "")
        if multimem is not None:
            par += ", multimem through the NVSwitch" if multimem else ", peer loads"
    else:
        par = "single, optimizer overlapped with backward" if use_engine else "single"
    par += ", step replayed from a CUDA graph" if graph_box[0] is not None else ", eager launches"
    return ms, launches, clocks, e2e, par, ms_eager


def run_torch(args):
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    import torch_ddp_mlp

    return torch_ddp_mlp.run(args, MODEL, LR, dist_env, timed_steps, ClockSampler, merge_clocks)


def main():
    args = parse()
    if args.impl == "reference":
        if dist_env()[0] != 0:
            return 0  # one line per job, from rank 0
        print(json.dumps({"impl": "reference",
                          "unavailable": "reference is a Rust workspace (no Python package: pip install of its "
                                         "source tree fails with 'neither setup.py nor pyproject.toml found') and "
                                         "cargo/rustc are not in this image, so it cannot be built or run here"}))
        return 0
    rank, world, _ = dist_env()
    if world != args.gpus and args.gpus > 1:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")
    ms_eager = None
    base = None
    if args.impl == "ours":
        ms, launches, clocks, e2e, par, ms_eager = run_ours(args)
        if not args.no_baseline:
            import gc

            import torch

            gc.collect()              # the first arm's model, optimizer state and graphs go before the second starts
            torch.cuda.empty_cache()
            bms, _, bclocks, be2e, bpar = run_torch(args)
            base = {"impl": "torch", "engine": bpar, "value": args.steps * args.batch * world / (bms / 1e3),
                    "ms_per_step": bms / args.steps, "e2e_value": be2e["value"] if be2e else None,
                    "clocks": bclocks}
    else:
        ms, launches, clocks, e2e, par = run_torch(args)
    if rank != 0:
        return 0
    steps = args.steps
    value = steps * args.batch * world / (ms / 1e3)
    if base is not None:
        base["ratio"] = value / base["value"]
        base["e2e_ratio"] = (e2e["value"] / base["e2e_value"]) if (e2e and base["e2e_value"]) else None
    out = {
        "metric": "MLP-4096x8 DDP train samples/s", "value": value, "unit": "samples/s", "n_gpus": world,
        "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": base["ratio"] if base is not None else None, "dtype": "bf16", "data": "synthetic", "impl": args.impl,
        "config": {"model": f"MLP {args.depth}x[Linear({args.width})-GELU-LayerNorm] + 1000-way head, 1024 inputs",
                   "global_batch": args.batch * world, "per_gpu_batch": args.batch, "seq_len": 1,
                   "parallelism": f"dp{world}" if world > 1 else "single-gpu", "engine": par,
                   "optimizer": "Adam lr 3e-4 (fp32 master weights)", "loss": "cross_entropy",
                   "l2": "working set per step (>700 MB of weights, activations, optimizer state) exceeds the "
                         "126 MB L2, no explicit flush"},
        "clocks": clocks, "gpu_launches": launches, "e2e": e2e,
        # the stock torch (cuBLAS + NCCL DDP + fused Adam) build of the same model, run after this arm in the same
        # process on the same GPUs; vs_baseline = value / baseline.value
        "baseline": base,
    }
    if ms_eager is not None:
        # same K steps launched kernel by kernel from Python; gpu_launches was counted in that region
        out["ms_per_step_eager_launches"] = ms_eager / steps
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
