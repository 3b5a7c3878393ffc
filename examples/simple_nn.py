"""A small classifier end to end (ferrum-examples/src/simple_nn.rs): Sequential, cross-entropy on logits, Adam,
a cosine schedule, then save / load of the weights in the FERRUM01 container."""
import tempfile
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ferrum_b200 as fb  # noqa: E402
from ferrum_b200.prelude import *  # noqa: F401,F403,E402


def main():
    dev = fb.Device.Cuda(0) if "--cuda" in sys.argv and fb.cuda_is_available() else fb.Device.Cpu
    fb.manual_seed(0)
    n, d, classes = 256, 20, 4
    centers = Tensor.randn([classes, d], device=dev).mul_scalar(3.0)
    labels = Tensor.from_slice([i % classes for i in range(n)], dtype=DType.I64, device=dev)
    onehot = Tensor.eye(classes, device=dev)[labels.to_vec()]          # [n, classes]
    x = Tensor.randn([n, d], device=dev).add(onehot.matmul(centers))
    model = Sequential(Linear(d, 64, device=dev), GELU(), LayerNorm([64], device=dev), Linear(64, classes, device=dev))
    opt = Adam(model.parameters(), AdamConfig.new(1e-2))
    sched = CosineAnnealingLR(1e-2, 200, 1e-4)
    for step in range(200):
        opt.zero_grad()
        loss = fb.nn.cross_entropy(model(x), labels)
        loss.backward()
        opt.step()
        sched.step()
        opt.set_learning_rate(sched.get_lr())
    acc = sum(int(a == b) for a, b in zip(model(x).argmax(1).to_vec(), labels.to_vec())) / n
    print(f"final loss {loss.item():.4f}  accuracy {acc:.3f}  parameters {model.num_parameters()}")
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "model.ferrum")
        save(model.ferrum_state_dict(), path)
        restored = load(path)
        print("checkpoint tensors:", sorted(restored.keys()))
    return acc


if __name__ == "__main__":
    main()
