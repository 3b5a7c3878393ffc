"""ResNet-18/34 and VGG-16/19 as laid out in ferrum-nn/src/models.rs:13-244 (no batch norm in the reference's
blocks).  Under bf16 autocast every convolution here — the 7 x 7 stride-2 stem, the 3 x 3 layers, the stride-2
layers and the 1 x 1 stride-2 shortcuts — runs on the implicit-GEMM tensor-core kernels; in fp32 they run as
im2col + GEMM kernels."""
from __future__ import annotations

import torch

from .. import nn
from ..nn.conv import AdaptiveAvgPool2d, Conv2d, MaxPool2d
from ..ops import functional as F


class BasicBlock(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, stride: int = 1, device=None):
        super().__init__()
        self.conv1 = Conv2d(in_channels, out_channels, 3, stride, 1, 1, 1, False, device=device)
        self.conv2 = Conv2d(out_channels, out_channels, 3, 1, 1, 1, 1, False, device=device)
        self.downsample = (Conv2d(in_channels, out_channels, 1, stride, 0, 1, 1, False, device=device)
                           if stride != 1 or in_channels != out_channels else None)

    @classmethod
    def new(cls, in_channels, out_channels, stride):
        return cls(in_channels, out_channels, stride)

    @nn.tensor_io
    def forward(self, x):
        identity = self.downsample(x) if self.downsample is not None else x
        y = self.conv2(F.unary(self.conv1(x), "relu"))
        return F.unary(F.binary(y, identity, "add"), "relu")


class ResNet(nn.Module):
    def __init__(self, layers, num_classes: int = 1000, device=None):
        super().__init__()
        self.conv1 = Conv2d(3, 64, 7, 2, 3, 1, 1, False, device=device)
        self.maxpool = MaxPool2d(3, 2)
        blocks, cin = [], 64
        for i, (n, cout) in enumerate(zip(layers, (64, 128, 256, 512))):
            for j in range(n):
                blocks.append(BasicBlock(cin, cout, 2 if (j == 0 and i > 0) else 1, device=device))
                cin = cout
        self.blocks = nn.Sequential(*blocks)
        self.avgpool = AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(512, num_classes, device=device)

    @classmethod
    def resnet18(cls, num_classes: int = 1000, device=None):
        return cls([2, 2, 2, 2], num_classes, device)

    @classmethod
    def resnet34(cls, num_classes: int = 1000, device=None):
        return cls([3, 4, 6, 3], num_classes, device)

    @nn.tensor_io
    def forward(self, x):
        x = self.maxpool(F.unary(self.conv1(x), "relu"))
        x = self.avgpool(self.blocks(x))
        return self.fc(x.reshape(x.shape[0], -1))


_VGG = {16: [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"],
        19: [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"]}


class VGG(nn.Module):
    def __init__(self, depth: int, num_classes: int = 1000, device=None):
        super().__init__()
        feats, cin = [], 3
        for v in _VGG[depth]:
            if v == "M":
                feats.append(MaxPool2d(2, 2))
            else:
                feats += [Conv2d(cin, v, 3, 1, 1, device=device), nn.ReLU()]
                cin = v
        self.features = nn.Sequential(*feats)
        self.avgpool = AdaptiveAvgPool2d((7, 7))
        self.classifier = nn.Sequential(nn.Linear(512 * 49, 4096, device=device), nn.ReLU(), nn.Dropout(0.5),
                                        nn.Linear(4096, 4096, device=device), nn.ReLU(), nn.Dropout(0.5),
                                        nn.Linear(4096, num_classes, device=device))

    @classmethod
    def vgg16(cls, num_classes: int = 1000, device=None):
        return cls(16, num_classes, device)

    @classmethod
    def vgg19(cls, num_classes: int = 1000, device=None):
        return cls(19, num_classes, device)

    @nn.tensor_io
    def forward(self, x):
        x = self.avgpool(self.features(x))
        return self.classifier(x.reshape(x.shape[0], -1))
