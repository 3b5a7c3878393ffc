"""XOR with raw tensors, autograd and the SGD optimizer (the flow of
ferrum-examples/src/train_xor_autograd.rs; biases are broadcast over the batch the way the maths intends)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ferrum_b200 as fb  # noqa: E402
from ferrum_b200.prelude import *  # noqa: F401,F403,E402


def main():
    dev = fb.Device.Cuda(0) if "--cuda" in sys.argv and fb.cuda_is_available() else fb.Device.Cpu
    fb.manual_seed(1)
    x = Tensor.from_slice([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]], device=dev)
    y = Tensor.from_slice([[0.0], [1.0], [1.0], [0.0]], device=dev)
    w1 = Tensor.randn([2, 4], device=dev).set_requires_grad(True)
    b1 = Tensor.zeros([4], device=dev).set_requires_grad(True)
    w2 = Tensor.randn([4, 1], device=dev).set_requires_grad(True)
    b2 = Tensor.zeros([1], device=dev).set_requires_grad(True)
    opt = SGD([w1, b1, w2, b2], SGDConfig.new(0.5).with_momentum(0.9))
    for epoch in range(1, 1001):
        opt.zero_grad()
        out = x.matmul(w1).add(b1).tanh().matmul(w2).add(b2).sigmoid()
        loss = mse_loss(out, y)
        loss.backward()
        opt.step()
        if epoch % 200 == 0:
            print(f"epoch {epoch:4d}  loss {loss.item():.6f}")
    return loss.item()


if __name__ == "__main__":
    main()
