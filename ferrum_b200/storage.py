"""``Storage`` and the allocator traits of ferrum-core (storage.rs:33-442, device.rs:121-184).

Tensors of this package keep their bytes in torch storages (torch's caching allocator on CUDA); ``Storage`` is a thin
handle over one with the reference's methods, including copy-on-write ``make_unique``.  ``CpuAllocator`` hands out
64-byte aligned host buffers; the device allocator is :class:`ferrum_b200.cuda.MemoryPool`.
"""
from __future__ import annotations

import sys

import torch

from .core import AllocationError, DType, Device, NotImplemented_, _as_device, _as_dtype


class DeviceAllocator:
    """``alloc`` / ``dealloc`` / ``copy`` / ``zero`` over raw byte buffers."""

    def alloc(self, nbytes: int):
        raise NotImplementedError

    def dealloc(self, buf) -> None:
        raise NotImplementedError

    def copy(self, dst, src, nbytes: int) -> None:
        dst[:nbytes].copy_(src[:nbytes])

    def zero(self, buf, nbytes: int) -> None:
        buf[:nbytes].zero_()


class CpuAllocator(DeviceAllocator):
    ALIGN = 64

    def alloc(self, nbytes: int) -> torch.Tensor:
        raw = torch.empty(nbytes + self.ALIGN, dtype=torch.uint8)
        off = (-raw.data_ptr()) % self.ALIGN
        return raw[off:off + nbytes]

    def dealloc(self, buf) -> None:
        del buf


class CudaAllocator(DeviceAllocator):
    """Device buffers from the native size-bucketed pool (``csrc/runtime/runtime.cpp``)."""

    def alloc(self, nbytes: int):
        from .cuda import CudaBuffer

        return CudaBuffer(nbytes)

    def dealloc(self, buf) -> None:
        buf.free()

    def copy(self, dst, src, nbytes: int) -> None:
        dst.copy_from_device(src)

    def zero(self, buf, nbytes: int) -> None:
        buf.zero()


class _Box:
    """Bytes shared by several Storage handles, with an explicit holder count."""

    __slots__ = ("t", "refs")

    def __init__(self, t):
        self.t, self.refs = t, 1


class Storage:
    def __init__(self, data: torch.Tensor):
        flat = data.reshape(-1).view(torch.uint8) if data.dtype != torch.uint8 else data.reshape(-1)
        self._box = _Box(flat)

    @property
    def _t(self) -> torch.Tensor:
        return self._box.t

    def __del__(self):
        box = getattr(self, "_box", None)
        if box is not None:
            box.refs -= 1

    @staticmethod
    def uninit(nbytes: int, device=None) -> "Storage":
        dev = _as_device(device)
        if dev.is_metal():
            raise NotImplemented_("Metal storage")
        try:
            return Storage(torch.empty(nbytes, dtype=torch.uint8, device=dev.to_torch()))
        except RuntimeError:
            raise AllocationError(nbytes, dev) from None

    @staticmethod
    def zeros(nbytes: int, device=None) -> "Storage":
        s = Storage.uninit(nbytes, device)
        s._t.zero_()
        return s

    @staticmethod
    def from_bytes(data: bytes, device=None) -> "Storage":
        t = torch.frombuffer(bytearray(data), dtype=torch.uint8).clone()
        return Storage(t.to(_as_device(device).to_torch()))

    @staticmethod
    def from_slice(values, dtype=DType.F32, device=None) -> "Storage":
        t = torch.as_tensor(values, dtype=_as_dtype(dtype).to_torch()).contiguous()
        return Storage(t.to(_as_device(device).to_torch()))

    def size(self) -> int:
        return self._t.numel()

    def device(self) -> Device:
        return Device.from_torch(self._t.device)

    def ref_count(self) -> int:
        return self._box.refs

    def is_unique(self) -> bool:
        return self._box.refs == 1

    def share(self) -> "Storage":
        s = Storage.__new__(Storage)
        s._box = self._box
        self._box.refs += 1
        return s

    clone = share  # Arc-style clone: another handle on the same bytes

    def make_unique(self) -> "Storage":
        """Copy-on-write: detach from other holders of the same bytes."""
        if self._box.refs > 1:
            self._box.refs -= 1
            self._box = _Box(self._box.t.clone())
        return self

    def read_as(self, dtype) -> list:
        return self._t.view(_as_dtype(dtype).to_torch()).tolist()

    def write_as(self, values, dtype, offset: int = 0) -> None:
        src = torch.as_tensor(values, dtype=_as_dtype(dtype).to_torch()).to(self._t.device)
        view = self._t.view(src.dtype)
        view[offset:offset + src.numel()] = src

    def as_ptr(self) -> int:
        return self._t.data_ptr()

    as_mut_ptr = as_ptr

    def as_tensor(self, dtype=DType.F32, shape=None):
        from .core import Tensor

        t = self._t.view(_as_dtype(dtype).to_torch())
        return Tensor(t.reshape(tuple(shape)) if shape is not None else t)
