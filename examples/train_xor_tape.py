"""XOR trained through a GradientTape with a hand-written SGD update (the flow of
ferrum-examples/src/train_xor_simple.rs: 2 -> 4 tanh -> 1 sigmoid, MSE, lr 0.5, 2000 epochs)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ferrum_b200 as fb  # noqa: E402
from ferrum_b200.prelude import *  # noqa: F401,F403,E402


def main():
    dev = fb.Device.Cuda(0) if "--cuda" in sys.argv and fb.cuda_is_available() else fb.Device.Cpu
    fb.manual_seed(0)
    x = Tensor.from_slice([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]], device=dev)
    y = Tensor.from_slice([[0.0], [1.0], [1.0], [0.0]], device=dev)
    w1 = Tensor.randn([2, 4], device=dev).mul_scalar(0.5).detach().set_requires_grad(True)
    b1 = Tensor.zeros([1, 4], device=dev).set_requires_grad(True)
    w2 = Tensor.randn([4, 1], device=dev).mul_scalar(0.5).detach().set_requires_grad(True)
    b2 = Tensor.zeros([1, 1], device=dev).set_requires_grad(True)
    params, lr = [w1, b1, w2, b2], 0.5
    for epoch in range(1, 2001):
        def step(tape):
            h = x.matmul(w1).add(b1).tanh()
            out = h.matmul(w2).add(b2).sigmoid()
            loss = mse_loss(out, y)
            return loss, tape.gradient(loss, params)

        loss, grads = GradientTape.with_tape(step)
        with no_grad():
            for p, g in zip(params, grads):
                p.sub_inplace(g.mul_scalar(lr))
        if epoch % 400 == 0:
            print(f"epoch {epoch:4d}  loss {loss.item():.6f}")
    with no_grad():
        pred = x.matmul(w1).add(b1).tanh().matmul(w2).add(b2).sigmoid().to_vec()
    print("predictions", [round(p, 4) for p in pred])
    return pred


if __name__ == "__main__":
    main()
