"""CUDA runtime surface (ferrum-cuda): device queries, memory pool, streams / events, ``CudaTensor``.

In the reference every one of these is a host-memory simulation or a ``todo!()``
(cuda_device.rs:154-200, cuda_memory.rs:161-207, stream.rs:156-388); here they sit
on the native layer in ``csrc/runtime/runtime.cpp``.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .core import AllocationError, Device, DType, FerrumError, Tensor
from .utils.graph import GraphedStep, HostReadback  # noqa: F401
from .utils.runtime import DeviceStatusError, check_status, read_status  # noqa: F401


class CudaError(FerrumError):
    pass


def cuda_available() -> bool:
    return _lib.cuda().fb_rt_device_count() > 0


def device_count() -> int:
    return _lib.cuda().fb_rt_device_count()


get_device_count = device_count


def synchronize() -> None:
    _lib.check(_lib.cuda().fb_rt_synchronize(), "synchronize")


synchronize_device = synchronize


def synchronize_all() -> None:
    lib = _lib.cuda()
    cur = lib.fb_rt_get_device()
    for d in range(lib.fb_rt_device_count()):
        lib.fb_rt_set_device(d)
        lib.fb_rt_synchronize()
    lib.fb_rt_set_device(cur)


def set_device(idx: int) -> None:
    _lib.check(_lib.cuda().fb_rt_set_device(idx), "set_device")
    if torch.cuda.is_available():
        torch.cuda.set_device(idx)


def get_device() -> int:
    return _lib.cuda().fb_rt_get_device()


def init_cuda() -> int:
    return device_count()


class DeviceProperties:
    """Real device attributes (the reference fakes a 10 GB / 68-SM sm_86 part: cuda_device.rs:44-61)."""

    def __init__(self, idx: int = 0):
        raw = _lib.DeviceProps()
        _lib.check(_lib.cuda().fb_rt_device_props(idx, ctypes.byref(raw)), "device_props")
        self.name = raw.name.decode()
        self.total_memory = raw.total_memory
        self.multiprocessor_count = raw.multiprocessor_count
        self.compute_capability_major, self.compute_capability_minor = raw.major, raw.minor
        self.max_threads_per_block = raw.max_threads_per_block
        self.max_block_dims = tuple(raw.max_block_dim)
        self.max_grid_dims = tuple(raw.max_grid_dim)
        self.warp_size = raw.warp_size
        self.shared_memory_per_block = raw.shared_mem_per_block
        self.shared_memory_per_block_optin = raw.shared_mem_per_block_optin
        self.unified_memory = bool(raw.unified_addressing)
        self.l2_cache_bytes = raw.l2_cache_bytes
        self.clock_khz, self.memory_clock_khz = raw.clock_khz, raw.memory_clock_khz
        self.memory_bus_width = raw.memory_bus_width
        self.cluster_launch = bool(raw.cluster_launch)
        # Blackwell (cc 10.x): 256 KB of tensor memory per SM, 5th-generation tensor cores
        self.tensor_memory_per_sm = 256 * 1024 if raw.major >= 10 else 0

    def __repr__(self):
        return (f"DeviceProperties({self.name!r}, {self.total_memory / 2**30:.1f} GiB, "
                f"{self.multiprocessor_count} SMs, cc {self.compute_capability_major}."
                f"{self.compute_capability_minor})")


def get_device_properties(idx: int = 0) -> DeviceProperties:
    return DeviceProperties(idx)


class CudaDevice:
    def __init__(self, idx: int = 0):
        if idx < 0 or idx >= max(device_count(), 0):
            raise CudaError(f"invalid CUDA device {idx} (count {device_count()})")
        self._id = idx
        self._props = None

    @classmethod
    def new(cls, idx):
        return cls(idx)

    def id(self) -> int:
        return self._id

    def properties(self) -> DeviceProperties:
        if self._props is None:
            self._props = DeviceProperties(self._id)
        return self._props

    def name(self) -> str:
        return self.properties().name

    def total_memory(self) -> int:
        return self.properties().total_memory

    def free_memory(self) -> int:
        lib = _lib.cuda()
        cur = lib.fb_rt_get_device()
        lib.fb_rt_set_device(self._id)
        f, t = ctypes.c_ulonglong(), ctypes.c_ulonglong()
        lib.fb_rt_mem_info(ctypes.byref(f), ctypes.byref(t))
        lib.fb_rt_set_device(cur)
        return f.value

    def allocated_memory(self) -> int:
        return self.total_memory() - self.free_memory()

    def set_current(self) -> None:
        set_device(self._id)

    def synchronize(self) -> None:
        lib = _lib.cuda()
        cur = lib.fb_rt_get_device()
        lib.fb_rt_set_device(self._id)
        lib.fb_rt_synchronize()
        lib.fb_rt_set_device(cur)

    def can_access_peer(self, other: int) -> bool:
        return bool(_lib.cuda().fb_rt_can_access_peer(self._id, other))


class CudaDeviceManager:
    _inst = None

    def __init__(self):
        self._devices = {}

    @classmethod
    def initialize(cls):
        if cls._inst is None:
            cls._inst = cls()
        return cls._inst

    def device_count(self) -> int:
        return device_count()

    def set_device(self, idx: int) -> None:
        set_device(idx)

    def current_device(self) -> int:
        return get_device()

    def synchronize(self) -> None:
        synchronize()

    def get_device(self, idx: int) -> CudaDevice:
        if idx not in self._devices:
            self._devices[idx] = CudaDevice(idx)
        return self._devices[idx]


class CudaBuffer:
    """Owning device allocation from the native pool (cuda_memory.rs:11-154)."""

    def __init__(self, size: int, device: int | None = None, _ptr: int | None = None, _owned: bool = True):
        self._size, self._owned = int(size), _owned
        lib = _lib.cuda()
        if device is not None:
            lib.fb_rt_set_device(device)
        self._device = lib.fb_rt_get_device()
        if _ptr is None:
            _ptr = lib.fb_rt_pool_alloc(self._size)
            if not _ptr:
                raise AllocationError(self._size, Device.Cuda(self._device))
        self._ptr = _ptr

    @classmethod
    def new(cls, size, device=None):
        return cls(size, device)

    @classmethod
    def from_ptr(cls, ptr: int, size: int, device: int | None = None):
        return cls(size, device, _ptr=ptr, _owned=False)

    def ptr(self) -> int:
        return self._ptr

    def size(self) -> int:
        return self._size

    def device(self) -> int:
        return self._device

    def copy_from_host(self, data: bytes | bytearray | memoryview) -> None:
        mv = memoryview(data).cast("B")
        if len(mv) > self._size:
            raise CudaError("host buffer larger than device buffer")
        buf = (ctypes.c_char * len(mv)).from_buffer_copy(mv)
        _lib.check(_lib.cuda().fb_rt_memcpy_h2d(self._ptr, ctypes.addressof(buf), len(mv), None), "memcpy_h2d")
        synchronize()

    def copy_to_host(self) -> bytes:
        buf = (ctypes.c_char * self._size)()
        _lib.check(_lib.cuda().fb_rt_memcpy_d2h(ctypes.addressof(buf), self._ptr, self._size, None), "memcpy_d2h")
        synchronize()
        return bytes(buf)

    def copy_from_device(self, other: "CudaBuffer") -> None:
        n = min(self._size, other._size)
        _lib.check(_lib.cuda().fb_rt_memcpy_d2d(self._ptr, other._ptr, n, None), "memcpy_d2d")

    def zero(self) -> None:
        _lib.check(_lib.cuda().fb_rt_memset(self._ptr, 0, self._size, None), "memset")

    def clone(self) -> "CudaBuffer":
        b = CudaBuffer(self._size, self._device)
        b.copy_from_device(self)
        return b

    def free(self) -> None:
        if self._owned and self._ptr:
            _lib.cuda().fb_rt_pool_free(self._ptr, self._size)
        self._ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class MemoryPool:
    """Size-bucketed caching allocator: 21 power-of-two buckets from 256 B to 256 MiB (cuda_memory.rs:327-393)."""

    def alloc(self, size: int) -> CudaBuffer:
        return CudaBuffer(size)

    def free(self, buf: CudaBuffer) -> None:
        buf.free()

    def clear(self) -> None:
        _lib.cuda().fb_rt_pool_clear()

    def allocated_bytes(self) -> int:
        return _lib.cuda().fb_rt_pool_allocated()

    def cached_bytes(self) -> int:
        return _lib.cuda().fb_rt_pool_cached()

    @staticmethod
    def round_size(size: int) -> int:
        return _lib.cuda().fb_rt_pool_round(size)


class CudaEvent:
    def __init__(self, timing: bool = False):
        self._h = _lib.cuda().fb_rt_event_create(1 if timing else 0)
        if not self._h:
            raise CudaError("event creation failed")
        self._timing = timing

    @classmethod
    def new(cls):
        return cls(False)

    @classmethod
    def with_timing(cls):
        return cls(True)

    def handle(self) -> int:
        return self._h

    def record(self, stream: "CudaStream | None" = None) -> None:
        _lib.check(_lib.cuda().fb_rt_event_record(self._h, stream.handle() if stream else None), "event_record")

    def query(self) -> bool:
        return _lib.cuda().fb_rt_event_query(self._h) == 1

    def synchronize(self) -> None:
        _lib.check(_lib.cuda().fb_rt_event_synchronize(self._h), "event_synchronize")

    def elapsed_time(self, end: "CudaEvent") -> float:
        """Milliseconds between this event and ``end`` (both recorded with timing)."""
        ms = _lib.cuda().fb_rt_event_elapsed_ms(self._h, end._h)
        if ms < 0:
            raise CudaError("elapsed_time needs two completed timing events")
        return ms

    def __del__(self):
        try:
            if self._h:
                _lib.cuda().fb_rt_event_destroy(self._h)
        except Exception:
            pass


class CudaStream:
    def __init__(self, high_priority: bool = False, _handle: int | None = None):
        self._owned = _handle is None
        self._h = _lib.cuda().fb_rt_stream_create(1 if high_priority else 0) if _handle is None else _handle
        if self._owned and not self._h:
            raise CudaError("stream creation failed")

    @classmethod
    def new(cls):
        return cls()

    @classmethod
    def default_stream(cls):
        return cls(_handle=0)

    def handle(self) -> int:
        return self._h or 0

    def device(self) -> int:
        return get_device()

    def synchronize(self) -> None:
        _lib.check(_lib.cuda().fb_rt_stream_synchronize(self._h or None), "stream_synchronize")

    def query(self) -> bool:
        return _lib.cuda().fb_rt_stream_query(self._h or None) == 1

    def record_event(self, event: CudaEvent | None = None) -> CudaEvent:
        event = event or CudaEvent()
        event.record(self)
        return event

    def wait_event(self, event: CudaEvent) -> None:
        _lib.check(_lib.cuda().fb_rt_stream_wait_event(self._h or None, event.handle()), "stream_wait_event")

    def as_torch(self) -> "torch.cuda.ExternalStream":
        return torch.cuda.ExternalStream(self._h)

    def __del__(self):
        try:
            if self._owned and self._h:
                _lib.cuda().fb_rt_stream_destroy(self._h)
        except Exception:
            pass


class StreamPool:
    def __init__(self):
        self._free = []

    def get(self) -> CudaStream:
        return self._free.pop() if self._free else CudaStream()

    def put(self, s: CudaStream) -> None:
        self._free.append(s)


class CudaTensor(Tensor):
    """A :class:`Tensor` that lives on ``Device.Cuda``; the reference's separate type (ferrum-cuda/src/tensor.rs)
    collapses into the one tensor class, these constructors keep its names."""

    @classmethod
    def from_host(cls, data, shape=None, device: int = 0):
        return Tensor.from_slice(data, shape, Device.Cuda(device))

    from_f32 = from_host

    @classmethod
    def from_f64(cls, data, shape=None, device: int = 0):
        return Tensor.from_slice(data, shape, Device.Cuda(device), dtype=DType.F64)

    @classmethod
    def new(cls, shape, dtype=DType.F32, device: int = 0):
        return Tensor.uninit(shape, dtype, Device.Cuda(device))

    @classmethod
    def zeros_on(cls, shape, dtype=DType.F32, device: int = 0):
        return Tensor.zeros(shape, dtype, Device.Cuda(device))


def to_host(t: Tensor):
    return t.cpu().to_vec()
