"""Tour of the secondary layers (ferrum-examples/src/new_features_demo.rs): convolution and pooling, recurrent
layers, attention, embeddings, schedulers, AMP utilities and the data pipeline."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ferrum_b200 as fb  # noqa: E402
from ferrum_b200.prelude import *  # noqa: F401,F403,E402

from ferrum_b200 import nn, optim, data  # noqa: E402


def main():
    dev = fb.Device.Cuda(0) if "--cuda" in sys.argv and fb.cuda_is_available() else fb.Device.Cpu
    fb.manual_seed(0)
    img = Tensor.randn([2, 3, 16, 16], device=dev)
    feat = nn.MaxPool2d.new(2).forward(nn.Conv2d(3, 8, 3, padding=1, device=dev).forward(img))
    print("conv + pool      ", feat.shape)
    seq = Tensor.randn([5, 2, 12], device=dev)
    print("LSTM             ", nn.LSTM(12, 16, 2, device=dev).forward(seq).shape)
    print("GRU              ", nn.GRU(12, 16, 1, device=dev).forward(seq).shape)
    tok = Tensor.randn([2, 10, 32], device=dev)
    print("attention        ", nn.MultiHeadAttention(32, 4, device=dev).forward(tok).shape)
    print("encoder layer    ", nn.TransformerEncoderLayer(32, 4, 64, device=dev).forward(tok).shape)
    emb = nn.Embedding(100, 8, device=dev)
    print("embedding        ", emb.forward_indices(Tensor.from_slice([[1, 2, 3]], dtype=DType.I64, device=dev)).shape)
    sched = optim.OneCycleLR(0.1, 100)
    lrs = []
    for _ in range(100):
        lrs.append(sched.get_lr())
        sched.step()
    print("one-cycle lr     ", f"start {lrs[0]:.4f} peak {max(lrs):.4f} end {lrs[-1]:.6f}")
    scaler = optim.GradScaler.new()
    print("grad scaler      ", scaler.get_scale())
    ds = data.TensorDataset.from_tensors(Tensor.randn([10, 4]), Tensor.arange(0, 10))
    loader = data.DataLoader.new(ds).batch_size(4).shuffle(True)
    print("batch sizes      ", [b[0].shape[0] for b in loader.iter()])
    print(fb.banner())


if __name__ == "__main__":
    main()
