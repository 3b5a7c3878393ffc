"""Secondary benchmark configurations (the headline one is bench.py).

    python bench_configs.py --config mnist|embedding [--impl ours|torch] [--steps K] [--warmup W]
    python -m torch.distributed.run --nproc-per-node N bench_configs.py --config embedding ...

mnist      60000 synthetic samples of 784 features ~ U[0,1), labels uniform in 0..9; Linear(784,256)-ReLU-
           LayerNorm(256)-Linear(256,10)-LogSoftmax, nll_loss, Adam lr 1e-3, DataLoader batch 128 shuffled
           (device-resident dataset, one row-gather kernel per batch).
embedding  vocab 50000, dim 1024, 256 token ids ~ Zipf(1.1) per sample, mean-pooled Embedding ->
           Linear(1024,4096)-SiLU-Dropout(0.1)-Linear(4096,512), cross_entropy, SGD momentum 0.9 wd 1e-4 with a
           cosine LR schedule, per-GPU batch 512.

Prints one JSON line (rank 0): samples/s over K timed steps (CUDA events, max over ranks), synthetic seeded data.

    python bench_configs.py --impl cpu_ref --config xor|mnist|wide_mlp [--steps K]

``--impl cpu_ref`` times the reference's CPU arithmetic (no GPU needed): for ``xor`` the reference's own prebuilt
``train_xor`` binary when it is present beside the sources, else the restated loop; for ``mnist`` and ``wide_mlp``
the restated loops of ``csrc/host/cpu_ref.cpp`` (the naive triple-loop matmul of ferrum-core/src/tensor.rs:2487-2558
for the forward, data-gradient and weight-gradient products of every Linear, the row-wise LayerNorm / softmax loops
and the Adam loop of ferrum-optim/src/adam.rs:91-146), single thread, at a stated REDUCED size for ``wide_mlp``
(the full 8 x 4096, batch 8192 step is 6.2 TFLOP: hours per step on these loops).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def cpu_ref(a):
    """Reference-CPU arm: see the module docstring.  Prints one JSON line."""
    import ctypes
    import subprocess
    import time

    import numpy as np

    from ferrum_b200 import _lib

    lib = _lib.host()
    fp = ctypes.POINTER(ctypes.c_float)

    def ptr(x):
        return x.ctypes.data_as(ctypes.c_void_p)

    if a.config == "xor":
        # the reference checkout: FERRUM_REFERENCE_ROOT, else a directory named "reference" beside this repository
        ref_root = os.environ.get("FERRUM_REFERENCE_ROOT") or os.path.join(
            os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "reference")
        exe = os.path.join(ref_root, "target", "release", "examples", "train_xor")
        if os.path.exists(exe):
            ts = []
            for _ in range(10):
                t0 = time.perf_counter()
                subprocess.run([exe], capture_output=True, check=True)
                ts.append(time.perf_counter() - t0)
            ts.sort()
            print(json.dumps({"config": "xor", "impl": "cpu_ref", "what": "the reference's prebuilt train_xor binary, "
                              "whole process, 2000 full-batch epochs of 4 samples", "wall_ms_median": 1e3 * ts[5],
                              "wall_ms_min": 1e3 * ts[0], "samples_per_s": 2000 * 4 / ts[5]}))
            return 0
        H, epochs = 8, 2000
        rng = np.random.default_rng(0)
        w1, b1 = rng.standard_normal((H, 2)).astype(np.float32), np.zeros(H, np.float32)
        w2, b2 = rng.standard_normal((1, H)).astype(np.float32), np.zeros(1, np.float32)
        losses = np.zeros(epochs, np.float32)
        t0 = time.perf_counter()
        lib.fb_ref_train_xor(ptr(w1), ptr(b1), ptr(w2), ptr(b2), H, 1.0, epochs, 0, ptr(losses))
        dt = time.perf_counter() - t0
        print(json.dumps({"config": "xor", "impl": "cpu_ref", "what": "restated train_xor loop (no reference binary "
                          "on this machine)", "wall_ms": 1e3 * dt, "samples_per_s": epochs * 4 / dt,
                          "final_loss": float(losses[-1])}))
        return 0

    # (in, width, depth, classes, batch): mnist is the real size, wide_mlp a reduced one
    cfg = {"mnist": (784, 256, 1, 10, 128), "wide_mlp": (128, 512, 4, 100, 64)}[a.config]
    d_in, width, depth, classes, batch = cfg
    rng = np.random.default_rng(0)
    dims = [d_in] + [width] * depth + [classes]
    Ws = [rng.standard_normal((dims[i + 1], dims[i])).astype(np.float32) * 0.05 for i in range(len(dims) - 1)]
    Bs = [np.zeros(dims[i + 1], np.float32) for i in range(len(dims) - 1)]
    Ms = [np.zeros_like(w) for w in Ws]
    Vs = [np.zeros_like(w) for w in Ws]
    gam, bet = np.ones(width, np.float32), np.zeros(width, np.float32)
    x = rng.standard_normal((batch, d_in)).astype(np.float32)
    steps = max(1, min(a.steps, 5))
    flops = 0

    def step(t):
        nonlocal flops
        acts, h = [x], x
        for i, (w, b) in enumerate(zip(Ws, Bs)):
            y = np.empty((batch, w.shape[0]), np.float32)
            lib.fb_ref_linear(ptr(h), ptr(w), ptr(b), ptr(y), batch, w.shape[1], w.shape[0])
            flops += 2 * batch * w.size
            if i < len(Ws) - 1:
                y = np.maximum(y, 0.0, out=y)           # activation: elementwise, negligible beside the products
                n = np.empty_like(y)
                lib.fb_ref_layernorm_rows(ptr(y), ptr(gam), ptr(bet), ptr(n), batch, width, 1e-5)
                y = n
            acts.append(y)
            h = y
        p = np.empty_like(h)
        lib.fb_ref_softmax_rows(ptr(h), ptr(p), batch, classes, 0)
        g = p / batch                                   # gradient of the mean cross-entropy up to the one-hot term
        for i in reversed(range(len(Ws))):
            w = Ws[i]
            gw = np.empty_like(w)
            gt = np.ascontiguousarray(g.T)
            lib.fb_ref_matmul(ptr(gt), ptr(acts[i]), ptr(gw), w.shape[0], batch, w.shape[1])      # weight gradient
            flops += 2 * batch * w.size
            if i > 0:
                gx = np.empty((batch, w.shape[1]), np.float32)
                lib.fb_ref_matmul(ptr(g), ptr(w), ptr(gx), batch, w.shape[0], w.shape[1])        # data gradient
                flops += 2 * batch * w.size
                g = gx
            lib.fb_ref_adam_step(ptr(w), ptr(gw), ptr(Ms[i]), ptr(Vs[i]), w.size, 1e-3, 0.9, 0.999, 1e-8, 0.0, t)

    step(1)
    flops = 0
    t0 = time.perf_counter()
    for t in range(steps):
        step(t + 2)
    dt = time.perf_counter() - t0
    print(json.dumps({"config": a.config, "impl": "cpu_ref", "what": "restated reference loops (naive matmul x3 per "
                      "Linear, LayerNorm, softmax, Adam), one thread", "model": {"in": d_in, "width": width,
                      "depth": depth, "classes": classes, "batch": batch}, "reduced_size": a.config == "wide_mlp",
                      "steps": steps, "ms_per_step": 1e3 * dt / steps, "samples_per_s": steps * batch / dt,
                      "gflops": flops / dt / 1e9}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["mnist", "embedding", "xor", "wide_mlp"])
    ap.add_argument("--impl", default="ours", choices=["ours", "torch", "cpu_ref"])
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--bf16", action="store_true", help="bf16 tensor-core GEMMs (default for embedding)")
    ap.add_argument("--graph", action="store_true",
                    help="ours (any config, any number of GPUs): record the step (zero_grad, forward, backward, Adam) in a CUDA graph and "
                         "replay it (the batch fetch and the LR schedule stay outside)")
    a = ap.parse_args()
    if a.impl == "cpu_ref":
        if a.config == "embedding":
            raise SystemExit("--impl cpu_ref covers xor, mnist and wide_mlp")
        return cpu_ref(a)
    if a.config in ("xor", "wide_mlp"):
        raise SystemExit(f"--config {a.config} is a --impl cpu_ref configuration (the GPU arms are mnist, embedding; "
                         "the wide MLP is bench.py)")

    import torch

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import ferrum_b200 as fb
    from ferrum_b200 import data, nn, optim
    from ferrum_b200.models import EmbeddingClassifier, mnist_classifier

    if world > 1:
        if a.impl == "ours":
            fb.distributed.init_process_group_from_env("nvlink")
        else:
            torch.distributed.init_process_group("nccl", device_id=dev)
    low = a.bf16 or a.config == "embedding"
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(1 + rank)

    if a.config == "mnist":
        batch = 128
        n = 60000
        x = torch.rand(n, 784, generator=g).to(dev)
        y = torch.randint(0, 10, (n,), generator=g).to(dev)
        if a.impl == "ours":
            model = mnist_classifier(device=fb.Device.Cuda(local))
            opt = optim.Adam(model.parameters(), optim.AdamConfig(lr=1e-3))
            loss_fn = nn.nll_loss
        else:
            model = torch.nn.Sequential(torch.nn.Linear(784, 256), torch.nn.ReLU(), torch.nn.LayerNorm(256),
                                        torch.nn.Linear(256, 10), torch.nn.LogSoftmax(-1)).to(dev)
            opt = torch.optim.Adam(model.parameters(), lr=1e-3, fused=True)
            loss_fn = torch.nn.functional.nll_loss
        sched = None
    else:
        batch = 512
        n = batch * 8
        ids = data.zipf_indices(50000, 1.1, n * 256, seed=7 + rank)
        x = torch.from_numpy(ids).reshape(n, 256).to(dev)
        y = torch.randint(0, 512, (n,), generator=g).to(dev)
        if a.impl == "ours":
            model = EmbeddingClassifier(device=fb.Device.Cuda(local))
            opt = optim.SGD(model.parameters(), optim.SGDConfig(lr=0.1, momentum=0.9, weight_decay=1e-4))
            loss_fn = nn.cross_entropy
            sched = optim.CosineAnnealingLR(0.1, a.steps + a.warmup, 0.0)
        else:
            class Net(torch.nn.Module):
                def __init__(self):
                    super().__init__()
                    self.emb = torch.nn.EmbeddingBag(50000, 1024, mode="mean")
                    self.head = torch.nn.Sequential(torch.nn.Linear(1024, 4096), torch.nn.SiLU(), torch.nn.Dropout(0.1),
                                                    torch.nn.Linear(4096, 512))

                def forward(self, idx):
                    return self.head(self.emb(idx))

            model = Net().to(dev)
            opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
            loss_fn = torch.nn.functional.cross_entropy
            sched = torch.optim.lr_scheduler.CosineAnnealingLR(opt, a.steps + a.warmup)

    net = model
    engine = None
    if world > 1:
        if a.impl == "ours":
            engine = fb.distributed.DistributedDataParallel(model, fb.distributed.get_world()).fuse_optimizer(opt)
            net = engine
        else:
            net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local])

    ds = data.TensorDataset.from_tensors(x, y)
    loader = data.DataLoader(ds, batch_size=batch, shuffle=True, seed=3, drop_last=True)

    def batches():
        while True:
            for xb, yb in loader:
                yield xb.torch(), yb.torch()

    it = batches()
    graphed = None
    if a.graph:
        if a.impl != "ours":
            raise SystemExit("--graph is an option of this framework's arm")

        def train(xb, yb):
            opt.zero_grad()
            with fb.autocast(enabled=low):
                loss = loss_fn(net(xb), yb)
            loss.backward()
            opt.step()
            return loss

        graphed = fb.cuda.GraphedStep(train, next(it), optimizer=opt)

    def step():
        xb, yb = next(it)
        if graphed is not None:
            if sched is not None:  # the learning rate lives in device memory in capturable mode: replays pick it up
                opt.set_learning_rate(sched.get_lr())
                sched.step()
            return graphed(xb, yb)
        if a.impl == "ours":
            if sched is not None:
                opt.set_learning_rate(sched.get_lr())
            opt.zero_grad()
            with fb.autocast(enabled=low):
                loss = loss_fn(net(xb), yb)
            loss.backward()
            opt.step()
            if sched is not None:
                sched.step()
        else:
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16, enabled=low):
                loss = loss_fn(net(xb), yb)
            loss.backward()
            opt.step()
            if sched is not None:
                sched.step()
        return loss

    for _ in range(a.warmup):
        step()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    if a.impl == "ours":
        fb.utils.runtime.check_status()
    if rank == 0:
        print(json.dumps({"config": a.config, "impl": a.impl, "n_gpus": world, "steps": a.steps,
                          "ms_per_step": ms / a.steps, "samples_per_s": a.steps * batch * world / (ms / 1e3),
                          "dtype": "bf16" if low else "fp32", "final_loss": float(loss), "data": "synthetic",
                          "cuda_graph": bool(a.graph)}))
    if engine is not None:
        engine.shutdown()
    if world > 1 and a.impl == "ours":
        fb.distributed.destroy_process_group()
    elif world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
