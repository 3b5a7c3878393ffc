"""Convolutions and pooling (ferrum-nn/src/conv.rs:9-497; forward-only host loops there).

Under bf16 autocast an ungrouped convolution runs as an implicit GEMM on the tensor cores in all three directions
(``ops.functional._ConvIgemmFn``: NHWC bf16 activations read through 4-D TMA boxes shifted by the filter tap, no
window matrix in memory; strided convolutions reach the same kernels through a space-to-depth layout,
``_ConvS2dFn``; stride together with dilation takes the explicit path).  Otherwise convolution is lowered to GEMM explicitly: an im2col kernel writes the input windows as a K-major matrix (one row per output
position) and the product with the flattened filters runs on this package's GEMM kernels (tcgen05 under bf16
autocast, fp32 SIMT otherwise); the backward is the dgrad / wgrad GEMMs plus a gather-form col2im kernel.  Groups,
dilation, stride and padding follow the reference; weights ~ U(+-1/sqrt(fan_in)).  Max / average pooling are
their own forward / backward kernels.
"""
from __future__ import annotations

import math

import torch

from ..core import ShapeMismatch, _as_device
from ..ops import functional as F
from .modules import Module, _param, tensor_io


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def _out_hw(x, kernel, stride, padding, dilation):
    Ho = F.conv_out_size(x.shape[2], kernel[0], stride[0], padding[0], dilation[0])
    Wo = F.conv_out_size(x.shape[3], kernel[1], stride[1], padding[1], dilation[1])
    if Ho <= 0 or Wo <= 0:
        raise ShapeMismatch("conv/pool", "input at least as large as the kernel", list(x.shape))
    return Ho, Wo


def conv2d(x, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1):
    B, C, H, W = x.shape
    O, Cg, kh, kw = weight.shape
    if C != Cg * groups or O % groups:
        raise ShapeMismatch("conv2d", f"{Cg * groups} input channels", C)
    Ho, Wo = _out_hw(x, (kh, kw), stride, padding, dilation)
    if F.conv_igemm_ok(x, stride, dilation, padding, (kh, kw), groups):
        return F.conv2d_igemm(x, weight, bias, padding, dilation, stride)  # no window matrix: implicit GEMM
    cols = F.im2col(x, (kh, kw), stride, padding, dilation)              # [B*L, C*kh*kw], K contiguous
    L = Ho * Wo
    outs = []
    og = O // groups
    kg = Cg * kh * kw
    for g in range(groups):
        a = cols if groups == 1 else cols[:, g * kg:(g + 1) * kg].contiguous()
        wg = weight[g * og:(g + 1) * og].reshape(og, kg)                  # [og, K]
        bg = bias[g * og:(g + 1) * og] if bias is not None else None
        outs.append(F.linear(a, wg, bg).reshape(B, L, og))
    y = outs[0] if groups == 1 else torch.cat(outs, 2)
    return y.transpose(1, 2).reshape(B, O, Ho, Wo)


class Conv2d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, device=None):
        super().__init__()
        self.kernel_size, self._stride = _pair(kernel_size), _pair(stride)
        self._padding, self.dilation, self.groups = _pair(padding), _pair(dilation), int(groups)
        self.in_channels, self.out_channels = int(in_channels), int(out_channels)
        dev = _as_device(device).to_torch()
        k = 1.0 / math.sqrt(in_channels * self.kernel_size[0] * self.kernel_size[1])
        self.weight = _param(torch.empty(out_channels, in_channels // groups, *self.kernel_size,
                                         device=dev).uniform_(-k, k))
        if bias:
            self.bias = _param(torch.empty(out_channels, device=dev).uniform_(-k, k))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def new(cls, in_channels, out_channels, kernel_size):
        return cls(in_channels, out_channels, kernel_size)

    @classmethod
    def with_config(cls, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias):
        return cls(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias)

    def stride(self, s):
        self._stride = _pair(s)
        return self

    def padding(self, p):
        self._padding = _pair(p)
        return self

    @tensor_io
    def forward(self, x):
        if x.dim() != 4:
            raise ShapeMismatch("Conv2d.forward", "[B, C, H, W]", list(x.shape))
        return conv2d(x, self.weight, self.bias, self._stride, self._padding, self.dilation, self.groups)


class Conv1d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, device=None):
        super().__init__()
        self.kernel_size, self._stride, self._padding = int(kernel_size), int(stride), int(padding)
        self.dilation, self.groups = int(dilation), int(groups)
        self.in_channels, self.out_channels = int(in_channels), int(out_channels)
        dev = _as_device(device).to_torch()
        k = 1.0 / math.sqrt(in_channels * kernel_size)
        self.weight = _param(torch.empty(out_channels, in_channels // groups, kernel_size, device=dev).uniform_(-k, k))
        if bias:
            self.bias = _param(torch.empty(out_channels, device=dev).uniform_(-k, k))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def new(cls, in_channels, out_channels, kernel_size):
        return cls(in_channels, out_channels, kernel_size)

    @classmethod
    def with_config(cls, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias):
        return cls(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias)

    def stride(self, s):
        self._stride = int(s)
        return self

    def padding(self, p):
        self._padding = int(p)
        return self

    @tensor_io
    def forward(self, x):
        if x.dim() != 3:
            raise ShapeMismatch("Conv1d.forward", "[B, C, L]", list(x.shape))
        y = conv2d(x.unsqueeze(2), self.weight.unsqueeze(2), self.bias, (1, self._stride), (0, self._padding),
                   (1, self.dilation), self.groups)
        return y.squeeze(2)


class _Pool2d(Module):
    op = "max"

    def __init__(self, kernel_size, stride=None):
        super().__init__()
        self.kernel_size = _pair(kernel_size)
        self._stride = _pair(stride if stride is not None else kernel_size)

    @classmethod
    def new(cls, kernel_size):
        return cls(kernel_size)

    @classmethod
    def with_stride(cls, kernel_size, stride):
        return cls(kernel_size, stride)

    @tensor_io
    def forward(self, x):
        if x.dim() != 4:
            raise ShapeMismatch("pool.forward", "[B, C, H, W]", list(x.shape))
        _out_hw(x, self.kernel_size, self._stride, (0, 0), (1, 1))
        return F.pool2d(x, self.kernel_size, self._stride, self.op)


class MaxPool2d(_Pool2d):
    op = "max"


class AvgPool2d(_Pool2d):
    op = "mean"


class AdaptiveAvgPool2d(Module):
    def __init__(self, output_size):
        super().__init__()
        self.output_size = _pair(output_size)

    @classmethod
    def new(cls, output_size):
        return cls(output_size)

    @classmethod
    def square(cls, size):
        return cls((size, size))

    @tensor_io
    def forward(self, x):
        B, C, H, W = x.shape
        oh, ow = self.output_size
        if H % oh == 0 and W % ow == 0:
            kh, kw = H // oh, W // ow
            win = x.reshape(B, C, oh, kh, ow, kw).permute(0, 1, 2, 4, 3, 5).reshape(B, C, oh * ow, kh * kw)
            return F.reduce(win, "mean", 3).reshape(B, C, oh, ow)
        rows = []
        for i in range(oh):
            h0, h1 = (i * H) // oh, -((-(i + 1) * H) // oh)
            cols = []
            for j in range(ow):
                w0, w1 = (j * W) // ow, -((-(j + 1) * W) // ow)
                cols.append(F.reduce(x[:, :, h0:h1, w0:w1].reshape(B, C, -1), "mean", 2))
            rows.append(torch.stack(cols, -1))
        return torch.stack(rows, -2)
