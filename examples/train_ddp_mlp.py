"""Data-parallel training of a Linear-GELU-LayerNorm MLP with the NVLink engine.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/train_ddp_mlp.py

Every rank owns one GPU.  ``DistributedDataParallel`` lays parameters, gradients and bf16 weight copies into one
peer-mapped arena; during ``backward`` each finished gradient bucket is reduced over NVLink by a kernel that also
applies 1/world and the Adam update to the shard this rank owns and publishes the new weights to every rank, so
``opt.step()`` only waits for those kernels.  ``DistributedSampler`` gives each rank its slice of the data
(reference API: ferrum-distributed/src/ddp.rs:35-123, ferrum-data/src/sampler.rs:286-358).  With one process and no
GPU the script runs the same loop on the CPU over the gloo backend, so it doubles as a smoke test.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import ferrum_b200 as fb  # noqa: E402
from ferrum_b200 import data, nn, optim  # noqa: E402
from ferrum_b200 import distributed as dist  # noqa: E402


def main(steps: int = 20, width: int = 512, batch: int = 256) -> float:
    use_cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", 0))
    if use_cuda:
        torch.cuda.set_device(local)
    pg = dist.init_process_group_from_env("nvlink" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = fb.Device.Cuda(local) if use_cuda else fb.Device.Cpu
    torch.manual_seed(0)  # same initial weights everywhere; the engine broadcasts rank 0's anyway
    model = nn.Sequential(nn.Linear(64, width, device=dev), nn.GELU(), nn.LayerNorm([width], device=dev),
                          nn.Linear(width, width, device=dev), nn.GELU(), nn.LayerNorm([width], device=dev),
                          nn.Linear(width, 10, device=dev))
    opt = optim.Adam(model.parameters(), optim.AdamConfig(lr=1e-3))
    ddp = dist.DistributedDataParallel(model, pg).bucket_size_mb(25)
    if use_cuda:
        ddp.fuse_optimizer(opt)  # reduction + update + publish in one kernel per bucket

    g = torch.Generator().manual_seed(1)
    n = batch * world * 8
    xs = torch.randn(n, 64, generator=g)
    ys = (xs[:, :10].argmax(1)).to(torch.int64)  # a learnable rule
    sampler = data.DistributedSampler(n, world, rank, shuffle=True)
    first = last = None
    step = 0
    for epoch in range(1 + steps * batch * world // n):
        sampler.set_epoch(epoch)
        idx = torch.tensor(list(sampler), dtype=torch.int64)
        for lo in range(0, idx.numel() - batch + 1, batch):
            sel = idx[lo:lo + batch]
            x, y = xs[sel], ys[sel]
            if use_cuda:
                x, y = x.cuda(non_blocking=True), y.cuda(non_blocking=True)
            opt.zero_grad()
            with fb.autocast(enabled=use_cuda):
                loss = nn.cross_entropy(ddp(x), y)
            loss.backward()
            if not use_cuda:
                ddp.sync_gradients()  # CPU ranks: average the gradients over gloo, then a plain optimizer step
            opt.step()
            last = float(loss.item())
            first = last if first is None else first
            step += 1
            if step >= steps:
                break
        if step >= steps:
            break
    if dist.is_main_process():
        print(f"world {world}: loss {first:.4f} -> {last:.4f} after {step} steps")
    ddp.shutdown()
    dist.destroy_process_group()
    return last


if __name__ == "__main__":
    main()
