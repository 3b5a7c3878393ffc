"""Symmetric arenas: per-rank device buffers with the same layout, mapped into every peer.

Two transports give the peer mappings the kernels need:

``ipc``    the native allocator (``csrc/dist/symm_mem.cpp``): cudaMalloc + CUDA IPC handles exchanged over
           the process group's store.  Peer loads / stores only.
``torch``  ``torch.distributed._symmetric_memory`` (CUDA VMM): additionally yields the NVSwitch multicast
           alias used by the ``multimem`` code path.  Optional; selected with ``FERRUM_SYMM=torch``.

``emulated`` arenas live in one process on one GPU and stand in for the ranks of a job in tests that run
all ranks as one cooperative kernel launch.

Layout of an arena: ``[flag region: fb_dist_query_flag_bytes()] [data ...]``; offsets handed to kernels are
relative to the arena base.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _lib
from .._lib_dist import DistCtx
from ..utils import runtime as _rt
from .backend import CommunicationError

_TYPESTR = {torch.float32: "<f4", torch.bfloat16: None, torch.uint8: "|u1", torch.int64: "<i8", torch.int32: "<i4",
            torch.float16: "<f2", torch.float64: "<f8"}


class _RawView:
    """Exposes a region of device memory through ``__cuda_array_interface__`` (keeps its owner alive)."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class SymmetricArena:
    def __init__(self, rank: int, world: int, local_ptr: int, peer_ptrs, nbytes: int, mc_ptr: int = 0,
                 wait_ns: int = 10_000_000_000, owner=None, device: int | None = None, emulated: bool = False):
        self.rank, self.world, self.nbytes = rank, world, nbytes
        self.local_ptr, self.peer_ptrs, self.mc_ptr = local_ptr, list(peer_ptrs), mc_ptr
        self._owner, self._emulated = owner, emulated
        self.device = torch.cuda.current_device() if device is None else device
        self.flag_bytes = _lib.cuda().fb_dist_query_flag_bytes()
        ctx = DistCtx()
        ctx.rank, ctx.world = rank, world
        for r in range(world):
            ctx.arena[r] = self.peer_ptrs[r]
        ctx.mc_arena = mc_ptr or None
        ctx.status = _rt.status_ptr()
        ctx.timeout_ns = int(wait_ns)
        self.ctx = ctx
        self._epochs = [1] * _lib.cuda().fb_dist_query_channels()
        self._closed = False

    # ------------------------------------------------------------------ construction
    @classmethod
    def create(cls, nbytes_data: int, rank: int, world: int, exchange, wait_ns: int, transport: str | None = None):
        """Collective: every rank of the group calls this with the same size.

        ``exchange(obj) -> list`` gathers one picklable object from every rank (rank order).
        """
        lib = _lib.cuda()
        total = lib.fb_dist_query_flag_bytes() + int(nbytes_data)
        total = (total + 2 * 1024 * 1024 - 1) // (2 * 1024 * 1024) * (2 * 1024 * 1024)
        transport = (transport or os.environ.get("FERRUM_SYMM", "ipc")).lower()
        if transport == "torch":
            try:
                return cls._create_torch(total, rank, world, wait_ns)
            except Exception as exc:  # fall back to the native allocator
                if rank == 0:
                    import warnings

                    warnings.warn(f"torch symmetric memory unavailable ({exc}); using CUDA IPC arenas")
        ptr = lib.fb_symm_alloc(total)
        if not ptr:
            raise CommunicationError(f"could not allocate a {total} byte symmetric arena")
        hbytes = lib.fb_symm_handle_bytes()
        buf = ctypes.create_string_buffer(hbytes)
        rc = lib.fb_symm_export(ptr, buf)
        if rc != 0:
            raise CommunicationError(f"cudaIpcGetMemHandle failed ({rc})")
        handles = exchange(bytes(buf.raw))
        peers = []
        for r, h in enumerate(handles):
            if r == rank:
                peers.append(ptr)
                continue
            err = ctypes.c_int(0)
            p = lib.fb_symm_import(ctypes.create_string_buffer(h, hbytes), ctypes.byref(err))
            if not p:
                raise CommunicationError(f"cudaIpcOpenMemHandle for rank {r} failed ({err.value})")
            peers.append(p)
        return cls(rank, world, ptr, peers, total, 0, wait_ns, owner=("ipc", ptr))

    @classmethod
    def _create_torch(cls, total: int, rank: int, world: int, wait_ns: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        name = dist.group.WORLD.group_name
        try:  # needed by some torch versions, a deprecated no-op in others
            import warnings

            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                symm.enable_symm_mem_for_group(name)
        except Exception:
            pass
        t = symm.empty(total, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        hdl = symm.rendezvous(t, name)
        t.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        ptrs = list(hdl.buffer_ptrs)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        if os.environ.get("FERRUM_NVLS", "1") == "0":
            mc = 0
        return cls(rank, world, ptrs[rank], ptrs, total, mc, wait_ns, owner=("torch", t, hdl))

    @classmethod
    def emulated(cls, nbytes_data: int, world: int, wait_ns: int = 2_000_000_000):
        """``world`` arenas on the current GPU, one object per virtual rank."""
        lib = _lib.cuda()
        total = lib.fb_dist_query_flag_bytes() + int(nbytes_data)
        ptrs = []
        for _ in range(world):
            p = lib.fb_symm_alloc(total)
            if not p:
                raise CommunicationError("arena allocation failed")
            ptrs.append(p)
        return [cls(r, world, ptrs[r], ptrs, total, 0, wait_ns, owner=("ipc", ptrs[r]), emulated=True)
                for r in range(world)]

    # ------------------------------------------------------------------ access
    def view(self, byte_offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        """A tensor over this rank's own arena memory at ``byte_offset`` (relative to the arena base)."""
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        if byte_offset < 0 or byte_offset + nbytes > self.nbytes:
            raise ValueError("view outside the arena")
        raw = torch.as_tensor(_RawView(self.local_ptr + byte_offset, max(nbytes, 1), self),
                              device=torch.device("cuda", self.device))
        return raw[:nbytes].view(dtype).reshape(tuple(shape))

    def data_offset(self) -> int:
        return self.flag_bytes

    def next_epoch(self, channel: int) -> int:
        """Reserve the two epochs (entry, exit) a collective consumes on ``channel``.  Epochs live modulo 2^32,
        the modulus of the device-side counter and of the kernels' wrap-safe comparison
        ``(int32)(flag - epoch) >= 0``."""
        e = self._epochs[channel]
        self._epochs[channel] = (e + 2) & 0xFFFFFFFF
        return e

    def has_multicast(self) -> bool:
        return bool(self.mc_ptr)

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        lib = _lib.cuda()
        kind = self._owner[0] if self._owner else None
        if kind == "ipc":
            if not self._emulated:
                for r, p in enumerate(self.peer_ptrs):
                    if r != self.rank and p:
                        lib.fb_symm_close(p)
            lib.fb_symm_free(self._owner[1])
        self._owner = None
