"""Thin Python view of the native CUDA runtime layer (``csrc/runtime/runtime.cpp``)."""
from __future__ import annotations

import ctypes

from .. import _lib

STATUS_NAMES = {0: "ok", 1: "gemm_timeout", 2: "peer_timeout", 3: "bounds_violation", 4: "bad_argument"}

_status_ptrs: dict[int, int] = {}


class DeviceStatusError(RuntimeError):
    """A kernel gave up on a bounded wait or rejected an index; the CUDA context is still usable."""

    def __init__(self, code, where, info0, info1):
        self.code, self.where, self.info0, self.info1 = code, where, info0, info1
        super().__init__(f"device status {STATUS_NAMES.get(code, code)} (site {where}, info {info0}/{info1})")


def status_ptr() -> int:
    """Device address of the host-mapped status block of the current device."""
    lib = _lib.cuda()
    dev = lib.fb_rt_get_device()
    p = _status_ptrs.get(dev)
    if p is None:
        p = lib.fb_rt_status_ptr()
        if not p:
            raise RuntimeError("could not allocate the device status block")
        _status_ptrs[dev] = p
        lib.fb_layernorm_set_status(p)  # kernels without a status argument report here (one device per process)
    return p


def read_status(clear: bool = True):
    """(code, where, info0, info1) recorded by device code since the last clear. Synchronize first."""
    buf = (ctypes.c_int32 * 4)()
    _lib.cuda().fb_rt_status_read(buf, 1 if clear else 0)
    return tuple(buf)


def check_status(synchronize: bool = True) -> None:
    """Synchronize the device and raise :class:`DeviceStatusError` if a kernel reported a failure."""
    import torch

    if synchronize and torch.cuda.is_available():
        torch.cuda.synchronize()
    code, where, i0, i1 = read_status(clear=True)
    if code != 0:
        raise DeviceStatusError(code, where, i0, i1)
