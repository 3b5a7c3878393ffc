"""Parameter initialisers (ferrum-nn/src/init.rs:8-72), drawn with torch's seeded generators."""
from __future__ import annotations

import math

import torch


def _dev(device):
    from ..core import Device

    if isinstance(device, Device):
        return device.to_torch()
    return device


def _dt(dtype):
    from ..core import DType

    if isinstance(dtype, DType):
        return dtype.to_torch()
    return dtype or torch.float32


def xavier_uniform(shape, fan_in, fan_out, dtype=None, device=None, generator=None):
    bound = math.sqrt(6.0 / (fan_in + fan_out))
    return torch.empty(tuple(shape), dtype=_dt(dtype), device=_dev(device)).uniform_(-bound, bound,
                                                                                    generator=generator)


def xavier_normal(shape, fan_in, fan_out, dtype=None, device=None, generator=None):
    std = math.sqrt(2.0 / (fan_in + fan_out))
    return torch.empty(tuple(shape), dtype=_dt(dtype), device=_dev(device)).normal_(0.0, std, generator=generator)


def kaiming_uniform(shape, fan_in, dtype=None, device=None, generator=None):
    bound = math.sqrt(6.0 / fan_in)
    return torch.empty(tuple(shape), dtype=_dt(dtype), device=_dev(device)).uniform_(-bound, bound,
                                                                                    generator=generator)


def kaiming_normal(shape, fan_in, dtype=None, device=None, generator=None):
    std = math.sqrt(2.0 / fan_in)
    return torch.empty(tuple(shape), dtype=_dt(dtype), device=_dev(device)).normal_(0.0, std, generator=generator)


def orthogonal(shape, gain=1.0, dtype=None, device=None, generator=None):
    """(Semi-)orthogonal matrix via QR; the reference substitutes ``randn * gain`` (init.rs:52-57)."""
    shape = tuple(shape)
    rows, cols = shape[0], int(math.prod(shape[1:])) if len(shape) > 1 else 1
    a = torch.randn(max(rows, cols), min(rows, cols), generator=generator)
    q, r = torch.linalg.qr(a)
    q = q * torch.sign(torch.diagonal(r)).unsqueeze(0)
    if rows < cols:
        q = q.t()
    return (q[:rows, :cols] * gain).reshape(shape).to(dtype=_dt(dtype), device=_dev(device)).contiguous()


def constant(shape, value, dtype=None, device=None):
    return torch.full(tuple(shape), value, dtype=_dt(dtype), device=_dev(device))


def zeros(shape, dtype=None, device=None):
    return torch.zeros(tuple(shape), dtype=_dt(dtype), device=_dev(device))


def ones(shape, dtype=None, device=None):
    return torch.ones(tuple(shape), dtype=_dt(dtype), device=_dev(device))
