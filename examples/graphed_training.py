"""Launch-bound training made GPU-bound: a small classifier whose whole step (zero_grad, forward, backward, Adam) is
recorded once in a CUDA graph and replayed with one launch per step.  Needs a CUDA device."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import ferrum_b200 as fb  # noqa: E402
from ferrum_b200 import nn, optim  # noqa: E402


def main(steps: int = 300):
    if not fb.cuda_is_available():
        print("no CUDA device: nothing to show")
        return None
    dev = fb.Device.Cuda(0)
    fb.manual_seed(0)
    model = nn.Sequential(nn.Linear(784, 256, device=dev), nn.ReLU(), nn.LayerNorm([256], device=dev),
                          nn.Linear(256, 10, device=dev), nn.LogSoftmax(-1))
    opt = optim.Adam(model.parameters(), optim.AdamConfig(lr=1e-3))
    x = torch.rand(128, 784, device="cuda")
    y = torch.randint(0, 10, (128,), device="cuda")

    def train_step(xb, yb):
        opt.zero_grad()
        loss = nn.nll_loss(model(xb), yb)
        loss.backward()
        opt.step()
        return loss

    def timed(fn):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            loss = fn(x, y)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / steps * 1e3, float(loss)

    for _ in range(10):
        train_step(x, y)
    eager_ms, _ = timed(train_step)
    graphed = fb.cuda.GraphedStep(train_step, (x, y), optimizer=opt)
    graph_ms, loss = timed(graphed)
    print(f"eager {eager_ms:.3f} ms/step, graph replay {graph_ms:.3f} ms/step, loss {loss:.4f}")
    return eager_ms, graph_ms


if __name__ == "__main__":
    main()
