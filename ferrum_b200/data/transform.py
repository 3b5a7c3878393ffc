"""Transforms (ferrum-data/src/transform.rs:6-166).  ``Normalize`` and ``Scale`` are one fused affine
kernel on CUDA; ``GaussianNoise`` and ``ToOneHot`` do what their names say (no-ops in the reference)."""
from __future__ import annotations

import torch

from ..core import Tensor, _unwrap
from ..ops import functional as F


def _apply(x, fn):
    wrapped = isinstance(x, Tensor)
    out = fn(_unwrap(x))
    return Tensor(out) if wrapped else out


class Transform:
    def apply(self, x):
        raise NotImplementedError

    def __call__(self, x):
        return self.apply(x)


class Compose(Transform):
    def __init__(self, transforms):
        self.transforms = list(transforms)

    def apply(self, x):
        for t in self.transforms:
            x = t(x)
        return x


class Normalize(Transform):
    """``(x - mean) / std``"""

    def __init__(self, mean: float, std: float):
        self.mean, self.std = float(mean), float(std)

    @classmethod
    def standard(cls):
        return cls(0.0, 1.0)

    @classmethod
    def imagenet(cls):
        return cls(0.485, 0.229)

    def apply(self, x):
        return _apply(x, lambda t: F.unary(t, "affine", 1.0 / self.std, -self.mean / self.std))


class Scale(Transform):
    """Maps ``[0, 1]`` to ``[min_val, max_val]``."""

    def __init__(self, min_val: float, max_val: float):
        self.min_val, self.max_val = float(min_val), float(max_val)

    @classmethod
    def unit(cls):
        return cls(0.0, 1.0)

    @classmethod
    def symmetric(cls):
        return cls(-1.0, 1.0)

    def apply(self, x):
        return _apply(x, lambda t: F.unary(t, "affine", self.max_val - self.min_val, self.min_val))


class GaussianNoise(Transform):
    def __init__(self, std: float, seed: int | None = None):
        self.std = float(std)
        self._gen = None if seed is None else seed

    def apply(self, x):
        def fn(t):
            g = None
            if self._gen is not None:
                g = torch.Generator(device=t.device).manual_seed(self._gen)
                self._gen += 1
            noise = torch.randn(t.shape, device=t.device, dtype=t.dtype, generator=g)
            return F.binary(t, F.unary(noise, "mul_scalar", self.std), "add")

        return _apply(x, fn)


class Identity(Transform):
    def apply(self, x):
        return x


class ToOneHot(Transform):
    def __init__(self, num_classes: int):
        self.num_classes = int(num_classes)

    def apply(self, x):
        def fn(t):
            idx = t.to(torch.int64)
            out = torch.zeros((*idx.shape, self.num_classes), device=t.device, dtype=torch.float32)
            return out.scatter_(-1, idx.unsqueeze(-1), 1.0)

        return _apply(x, fn)


class Lambda(Transform):
    def __init__(self, func):
        self.func = func

    def apply(self, x):
        return self.func(x)
