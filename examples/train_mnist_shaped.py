"""MNIST-shaped classifier on synthetic data: Linear(784,256)-ReLU-LayerNorm(256)-Linear(256,10)-LogSoftmax,
nll_loss, Adam lr 1e-3, DataLoader batch 128 shuffled.  `python examples/train_mnist_shaped.py [--cuda] [--bf16]`;
under torch.distributed.run it trains data-parallel with DistributedSampler + DistributedDataParallel."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ferrum_b200 as fb  # noqa: E402
from ferrum_b200 import data, nn, optim
from ferrum_b200.models import mnist_classifier


def main():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cuda = "--cuda" in sys.argv and fb.cuda_is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = fb.Device.Cuda(torch.cuda.current_device()) if cuda else fb.Device.Cpu
    pg = fb.distributed.init_process_group_from_env("nvlink" if cuda else "gloo") if world > 1 else None
    n = int(os.environ.get("N_SAMPLES", "60000"))
    g = torch.Generator().manual_seed(0)
    x = torch.rand(n, 784, generator=g).to(dev.to_torch())
    y = torch.randint(0, 10, (n,), generator=g).to(dev.to_torch())
    ds = data.TensorDataset.from_tensors(x, y)
    torch.manual_seed(1)
    model = mnist_classifier(device=dev)
    opt = optim.Adam(model.parameters(), optim.AdamConfig(lr=1e-3))
    net = model
    sampler = None
    if pg is not None:
        net = fb.distributed.DistributedDataParallel(model, pg).fuse_optimizer(opt)
        sampler = data.DistributedSampler(n, world, rank, shuffle=True, seed=0)
    loader = data.DataLoader(ds, batch_size=128, shuffle=True, seed=0, sampler=sampler)
    timer = fb.utils.StepTimer(every=100, sink=print if rank == 0 else (lambda s: None))
    for epoch in range(int(os.environ.get("EPOCHS", "1"))):
        if sampler is not None:
            sampler.set_epoch(epoch)
        for xb, yb in loader:
            with timer.step(128 * world):
                opt.zero_grad()
                with fb.autocast(enabled="--bf16" in sys.argv):
                    loss = nn.nll_loss(net(xb), yb)
                loss.backward()
                opt.step()
        if rank == 0:
            print(f"epoch {epoch} last loss {loss.item():.4f}")
    if pg is not None:
        net.shutdown()
        fb.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
