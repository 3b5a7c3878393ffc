"""XOR with Sequential + bce_loss + SGD — the README example of the reference, which cannot run there
(ferrum-examples/src/train_xor.rs uses a hand-written backward instead).  Runs on CPU or, with --cuda, on a GPU."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ferrum_b200 as fb  # noqa: E402
from ferrum_b200.prelude import *  # noqa: F401,F403


def main():
    dev = fb.Device.Cuda(0) if "--cuda" in sys.argv and fb.cuda_is_available() else fb.Device.Cpu
    x = Tensor.from_slice([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]], device=dev)
    y = Tensor.from_slice([[0.0], [1.0], [1.0], [0.0]], device=dev)
    model = Sequential(Linear(2, 8, device=dev), Tanh(), Linear(8, 1, device=dev), Sigmoid())
    opt = SGD(model.parameters(), SGDConfig.new(1.0))
    for epoch in range(1, 2001):
        opt.zero_grad()
        loss = bce_loss(model(x), y)
        loss.backward()
        opt.step()
        if epoch % 200 == 0:
            print(f"epoch {epoch:4d}  loss {loss.item():.6f}")
    pred = model(x).to_vec()
    correct = sum(int(round(p) == t) for p, t in zip(pred, [0, 1, 1, 0]))
    print("predictions", [round(p, 4) for p in pred], f"accuracy {correct}/4")


if __name__ == "__main__":
    main()
