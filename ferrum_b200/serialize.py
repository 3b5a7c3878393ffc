"""``save`` / ``load`` of named tensors in the FERRUM01 container (ferrum-serialize/src/io.rs:13-202).

The file layout is byte-compatible with the reference (magic, u64 header length,
bincode-1.3 header, raw little-endian tensor bytes); parsing and writing are done
by the native host library (``csrc/host/ferrum_format.cpp``).  Differences from the
reference: all eight dtypes round-trip (it materialises F32/F64/I32/I64 only),
CUDA tensors are staged through pinned host memory on save and can be loaded
straight onto a device, and ``save_checkpoint`` / ``load_checkpoint`` put model,
optimizer and scheduler state into the same container as additional named
tensors (``optim.m.<i>``, ``optim.step``, ...) so that a plain reader still opens it.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from .core import DType, SerializationError, Tensor, _as_device, _unwrap

MAGIC = b"FERRUM01"
VERSION = 1


def _to_host(t: torch.Tensor) -> torch.Tensor:
    t = t.detach()
    if t.is_cuda:
        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        host.copy_(t.contiguous(), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return host
    return t.contiguous()


def save(tensors: dict, path) -> None:
    """Write ``{name: tensor}`` to ``path``.  Offsets follow the mapping's iteration order."""
    path = os.fspath(path)
    names, hosts = [], []
    for k, v in tensors.items():
        if not isinstance(k, str):
            raise SerializationError(f"tensor names must be strings, got {type(k)}")
        t = _unwrap(v)
        if not isinstance(t, torch.Tensor):
            t = torch.as_tensor(t)
        try:
            DType.from_torch(t.dtype)
        except Exception:
            raise SerializationError(f"Unsupported dtype for serialization: {t.dtype}") from None
        names.append(k)
        hosts.append(_to_host(t))
    n = len(names)
    c_names = (ctypes.c_char_p * n)(*[s.encode("utf-8") for s in names])
    ndims = (ctypes.c_int * n)(*[h.dim() for h in hosts])
    flat = [d for h in hosts for d in h.shape]
    dims = (ctypes.c_longlong * max(len(flat), 1))(*flat)
    dtypes = (ctypes.c_int * n)(*[int(DType.from_torch(h.dtype)) for h in hosts])
    ptrs = (ctypes.c_void_p * n)(*[h.data_ptr() if h.numel() else None for h in hosts])
    sizes = (ctypes.c_ulonglong * n)(*[h.numel() * h.element_size() for h in hosts])
    err = ctypes.create_string_buffer(512)
    rc = _lib.host().fb_ser_save(path.encode(), n, c_names, ndims, dims, dtypes, ptrs, sizes, err, 512)
    if rc != 0:
        raise SerializationError(err.value.decode() or f"save failed ({rc})")


def load(path, device=None) -> dict:
    """Read every tensor of a FERRUM01 file; ``device`` (default CPU) may be ``Device.Cuda(i)``."""
    path = os.fspath(path)
    lib = _lib.host()
    err = ctypes.create_string_buffer(512)
    h = lib.fb_ser_open(path.encode(), err, 512)
    if not h:
        raise SerializationError(err.value.decode() or "load failed")
    dev = _as_device(device).to_torch()
    out = {}
    try:
        count = lib.fb_ser_count(h)
        dims = (ctypes.c_longlong * 64)()
        for i in range(count):
            nlen = lib.fb_ser_name_len(h, i)
            name = ctypes.create_string_buffer(nlen + 1)
            ndim, dt = ctypes.c_int(), ctypes.c_int()
            off, size = ctypes.c_ulonglong(), ctypes.c_ulonglong()
            rc = lib.fb_ser_meta(h, i, name, nlen + 1, ctypes.byref(ndim), dims, 64, ctypes.byref(dt),
                                 ctypes.byref(off), ctypes.byref(size))
            if rc != 0:
                raise SerializationError(f"corrupt tensor table entry {i}")
            dtype = DType(dt.value)
            shape = [dims[d] for d in range(ndim.value)]
            numel = 1
            for d in shape:
                numel *= d
            if numel * dtype.size_of() != size.value:
                raise SerializationError(f"tensor '{name.value.decode()}': size {size.value} does not match shape")
            pin = dev.type == "cuda"
            t = torch.empty(shape, dtype=dtype.to_torch(), pin_memory=pin)
            if numel and lib.fb_ser_read(h, i, t.data_ptr()) != 0:
                raise SerializationError(f"Failed to read data of tensor '{name.value.decode()}'")
            if pin:
                t = t.to(dev, non_blocking=True)
            out[name.value.decode("utf-8")] = Tensor(t)
        if dev.type == "cuda":
            torch.cuda.current_stream().synchronize()
    finally:
        lib.fb_ser_close(h)
    return out


def save_checkpoint(path, model=None, optimizer=None, scheduler=None, extra: dict | None = None) -> None:
    """Model parameters / buffers, optimizer state and scheduler scalars in one FERRUM01 file."""
    tensors = {}
    if model is not None:
        for k, v in model.state_dict().items():
            tensors[f"model.{k}"] = v
    if optimizer is not None:
        tensors.update(optimizer.state_tensors())
        tensors["optim.lr"] = torch.tensor(optimizer.learning_rate(), dtype=torch.float64)
    if scheduler is not None:
        for k, v in scheduler.state_dict().items():
            if isinstance(v, bool):
                tensors[f"sched.{k}"] = torch.tensor(v, dtype=torch.bool)
            elif isinstance(v, int):
                tensors[f"sched.{k}"] = torch.tensor(v, dtype=torch.int64)
            elif isinstance(v, float):
                tensors[f"sched.{k}"] = torch.tensor(v, dtype=torch.float64)
    for k, v in (extra or {}).items():
        tensors[f"extra.{k}"] = _unwrap(v) if isinstance(_unwrap(v), torch.Tensor) else torch.as_tensor(v)
    save(tensors, path)


def load_checkpoint(path, model=None, optimizer=None, scheduler=None, device=None) -> dict:
    """Inverse of :func:`save_checkpoint`; returns the ``extra`` entries."""
    raw = {k: v._t for k, v in load(path, device).items()}
    if model is not None:
        sd = {k[len("model."):]: v for k, v in raw.items() if k.startswith("model.")}
        model.load_state_dict(sd)
    if optimizer is not None:
        optimizer.load_state_tensors({k: v for k, v in raw.items() if k.startswith("optim.")})
        if "optim.lr" in raw:
            optimizer.set_learning_rate(float(raw["optim.lr"].item()))
    if scheduler is not None:
        scheduler.load_state_dict({k[len("sched."):]: v.item() for k, v in raw.items() if k.startswith("sched.")})
    return {k[len("extra."):]: Tensor(v) for k, v in raw.items() if k.startswith("extra.")}
