"""Process groups and collectives (ferrum-distributed/src/{lib,process_group,collectives}.rs).

One process per GPU.  ``torch.distributed`` provides the rendezvous (TCP store at ``MASTER_ADDR:MASTER_PORT``)
and the CPU / NCCL baselines; with ``Backend.Nvlink`` every collective on CUDA tensors is one of this package's
kernels (``csrc/dist/collectives.cu``) acting on peer-mapped symmetric arenas: the tensor is staged into the
arena, the kernel handshakes with the peers through flags in the arenas, moves / reduces the data over NVLink,
and the result is copied back out.  A group of world size 1 needs no rendezvous and its collectives are
identities — the behaviour of the reference's ``SimulatedCollectives`` for any world size.
"""
from __future__ import annotations

import datetime
import os
import threading

import torch

from .. import _lib
from ..core import Tensor, _unwrap
from ..utils import runtime as _rt
from .backend import (AlreadyInitialized, Backend, BackendConfig, CommunicationError, InvalidConfiguration,
                      InvalidRank, NotInitialized, ReduceOp, TensorError, Timeout, UnsupportedBackend)
from .symm import SymmetricArena

_lock = threading.Lock()
_default_group: "ProcessGroup | None" = None

_OP_CODE = {ReduceOp.Sum: 0, ReduceOp.Product: 1, ReduceOp.Min: 2, ReduceOp.Max: 3, ReduceOp.Average: 4}


def _torch_op(op: ReduceOp):
    import torch.distributed as dist

    return {ReduceOp.Sum: dist.ReduceOp.SUM, ReduceOp.Product: dist.ReduceOp.PRODUCT, ReduceOp.Min: dist.ReduceOp.MIN,
            ReduceOp.Max: dist.ReduceOp.MAX, ReduceOp.Average: dist.ReduceOp.SUM}[op]


class ProcessGroup:
    def __init__(self, backend: Backend, rank: int, world_size: int, config: BackendConfig | None = None,
                 _torch_group=None, _ranks=None):
        if world_size < 1 or not 0 <= rank < world_size:
            raise InvalidRank(rank, world_size)
        if not backend.is_available() and world_size > 1:
            raise UnsupportedBackend(backend.value)
        self._backend, self._rank, self._world = backend, rank, world_size
        self._config = config or BackendConfig.from_env()
        self._tg = _torch_group
        self._ranks = list(_ranks) if _ranks is not None else list(range(world_size))
        self._arena: SymmetricArena | None = None
        self._sync_arena: SymmetricArena | None = None
        self._chunk = int(float(os.environ.get("FERRUM_COMM_CHUNK_MB", "32")) * (1 << 20))
        self._seq = 0  # collective sequence number, identical on all ranks of a correct program
        self._last_peer_check = 0.0
        self._left = False
        self._symm = {}  # data_ptr -> (arena, offset, bytes) of tensors handed out by symmetric_empty

    # ------------------------------------------------------------------ accessors
    @classmethod
    def new(cls, backend, rank, world_size):
        return cls(backend, rank, world_size)

    @classmethod
    def with_config(cls, backend, rank, world_size, config):
        return cls(backend, rank, world_size, config)

    def backend(self) -> Backend:
        return self._backend

    def rank(self) -> int:
        return self._rank

    def world_size(self) -> int:
        return self._world

    def is_main(self) -> bool:
        return self._rank == 0

    def config(self) -> BackendConfig:
        return self._config

    def torch_group(self):
        return self._tg

    # ------------------------------------------------------------------ liveness (error.rs:20-26, backend.rs:84-88)
    # A rank that stops taking part between two steps says so in the rendezvous store before it goes
    # (``leave()``); every collective of the others looks there first, so they fail with CommunicationError on
    # the host instead of launching a kernel or a library call that would wait for the missing rank.  A rank
    # that dies without a word is caught by the bounded waits: the process-group timeout on host collectives,
    # the device-side wait limit on the NVLink kernels (Timeout).
    _LEFT_KEY = "ferrum/left/"

    def _store(self):
        import torch.distributed as dist

        if self._world == 1 or not dist.is_initialized():
            return None
        return dist.distributed_c10d._get_default_store()

    def departed(self) -> list:
        """Group ranks that announced their departure."""
        st = self._store()
        if st is None:
            return []
        return [r for r, g in enumerate(self._ranks) if g != self._ranks[self._rank] and st.check([f"{self._LEFT_KEY}{g}"])]

    def check_peers(self, min_interval: float = 0.0) -> None:
        """Raises ``CommunicationError`` if a rank of the group has left.  ``min_interval`` (seconds) skips the
        look-up when the last one is younger (the per-step call of the data-parallel engine)."""
        import time

        now = time.monotonic()
        if min_interval > 0.0 and now - self._last_peer_check < min_interval:
            return
        self._last_peer_check = now
        gone = self.departed()
        if gone:
            raise CommunicationError(f"rank(s) {gone} left the job; destroy the process group and continue with "
                                     f"the {self._world - len(gone)} remaining ranks from the last checkpoint")

    def leave(self) -> None:
        """Announce that this rank takes no further part (call it between steps, with no collective in flight),
        then release this rank's arenas.  The other ranks learn of it at their next collective."""
        st = self._store()
        if st is not None and not self._left:
            st.set(f"{self._LEFT_KEY}{self._ranks[self._rank]}", "1")
        self._left = True
        self.close()

    def _begin(self) -> None:
        """Start of every collective: count it, and do not start it if a peer is known to be gone."""
        self._seq += 1
        if self._world > 1:
            # the look-up is a round trip to the store: always before a host collective (milliseconds anyway),
            # at most five times a second in front of the NVLink kernels, whose waits are bounded on the device
            self.check_peers(0.2 if self._backend is Backend.Nvlink else 0.0)

    @staticmethod
    def _host_call(what: str, fn, *args, **kw):
        """A torch.distributed call with its failures mapped to this package's errors."""
        try:
            return fn(*args, **kw)
        except RuntimeError as exc:  # includes DistBackendError / DistNetworkError
            msg = str(exc)
            if "imeout" in msg or "timed out" in msg:
                raise Timeout(f"{what} ({msg.splitlines()[0]})") from None
            raise CommunicationError(f"{what}: {msg.splitlines()[0] if msg else type(exc).__name__}") from None

    # ------------------------------------------------------------------ plumbing
    def exchange(self, obj) -> list:
        """Gather one picklable object from every rank (host side, rank order)."""
        if self._world == 1:
            return [obj]
        import torch.distributed as dist

        out = [None] * self._world
        dist.all_gather_object(out, obj, group=self._tg)
        return out

    def _native(self, t: torch.Tensor) -> bool:
        return self._backend is Backend.Nvlink and self._world > 1 and t.is_cuda

    def comm_arena(self) -> SymmetricArena:
        """The staging arena of this group (allocated collectively on first use)."""
        if self._arena is None:
            need = self._chunk * (1 + self._world) + 2 * self._ONESHOT_BYTES  # + the two one-shot slots
            self._arena = SymmetricArena.create(need, self._rank, self._world, self.exchange,
                                                self._config.device_wait_ns())
        return self._arena

    # ------------------------------------------------------------------ registered tensors
    def symmetric_empty(self, shape, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """A tensor in peer-mapped symmetric memory (collective: every rank calls it with the same arguments, in
        the same order).  ``all_reduce`` and ``broadcast`` on it, and ``all_gather`` from it, run directly on the
        peers' mappings, without the pass that stages an ordinary tensor into the group's arena and back.  The
        tensor stays valid until the group is closed.  With one rank (or off the NVLink backend) it is an
        ordinary tensor."""
        shape = tuple(int(d) for d in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
        numel = 1
        for d in shape:
            numel *= d
        if not (self._backend is Backend.Nvlink and self._world > 1 and torch.cuda.is_available()):
            return torch.empty(shape, dtype=dtype, device="cuda" if torch.cuda.is_available() else "cpu")
        esz = torch.empty((), dtype=dtype).element_size()
        unit = 16 * self._world                                  # every rank's shard starts on a 16-byte boundary
        nbytes = max(unit, (numel * esz + unit - 1) // unit * unit)
        arena = SymmetricArena.create(nbytes, self._rank, self._world, self.exchange, self._config.device_wait_ns())
        off = arena.data_offset()
        arena.view(off, (nbytes,), torch.uint8).zero_()
        t = arena.view(off, (numel,), dtype).view(shape)
        self._symm[t.data_ptr()] = (arena, off, nbytes)
        torch.cuda.current_stream().synchronize()
        self.barrier()                                           # every rank's padding is zero before anyone reads it
        return t

    def _registered(self, t: torch.Tensor):
        """(arena, byte offset, region bytes) when ``t`` is a whole tensor from ``symmetric_empty``."""
        ent = self._symm.get(t.data_ptr()) if t.is_cuda and t.is_contiguous() else None
        if ent is not None and t.numel() * t.element_size() <= ent[2]:
            return ent
        return None

    # Messages up to this size are all-reduced by the one-shot kernel (one handshake, every rank reduces for
    # itself); its two alternating slots sit behind the staging regions of the other collectives.
    _ONESHOT_BYTES = 256 * 1024

    def _check_device_status(self, what: str) -> None:
        code, where, i0, i1 = _rt.read_status(clear=True)
        if code == 2:
            raise Timeout(f"{what} (rank {self._rank} waited for rank {i0}, epoch {i1}, site {where})")
        if code != 0:
            raise CommunicationError(f"{what}: device status {code} at site {where} ({i0}, {i1})")

    def _stream(self) -> int:
        return torch.cuda.current_stream().cuda_stream

    def _blocks(self, nbytes: int) -> int:
        # one block per 32 KiB up to 128: mid-sized messages are latency-bound, so they want many short loops
        return max(1, min(128, nbytes // (32 * 1024) + 1))

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, tensor, op: ReduceOp = ReduceOp.Sum):
        """In-place reduction over all ranks; ``Average`` divides by the world size."""
        t = _unwrap(tensor)
        self._begin()
        if self._world == 1:
            return tensor
        if self._native(t):
            self._native_allreduce(t, op)
            return tensor
        import torch.distributed as dist

        self._host_call("all_reduce", dist.all_reduce, t, op=_torch_op(op), group=self._tg)
        if op is ReduceOp.Average:
            t.div_(self._world)
        return tensor

    def _native_allreduce(self, t: torch.Tensor, op: ReduceOp) -> None:
        from ..ops import functional as F

        if not t.is_floating_point():
            raise TensorError("native all_reduce supports floating-point tensors")
        lib = _lib.cuda()
        reg = self._registered(t) if t.dtype == torch.float32 else None
        if reg is not None:
            # in place on the peers' mappings: two-shot over the (zero-padded) region, no staging pass
            arena, roff, rbytes = reg
            e = arena.next_epoch(0)
            scale = 1.0 / self._world if op is ReduceOp.Average else 1.0
            use_mc = 1 if (arena.has_multicast() and op in (ReduceOp.Sum, ReduceOp.Average)) else 0
            _lib.check(lib.fb_dist_allreduce(arena.ctx, 0, use_mc, 0, e, roff, 0, -1, rbytes // 4, _OP_CODE[op],
                                             scale, None, None, None, None, 1, self._blocks(rbytes), 256,
                                             self._stream()), "fb_dist_allreduce")
            return
        arena = self.comm_arena()
        flat = t.contiguous().view(-1)
        work = flat if flat.dtype == torch.float32 else F.raw_cast(flat, torch.float32) if flat.dtype == torch.bfloat16 \
            else flat.float()
        n = work.numel()
        per = self._chunk // 4
        off = arena.data_offset()
        scale = 1.0 / self._world if op is ReduceOp.Average else 1.0
        if n * 4 <= self._ONESHOT_BYTES and work.data_ptr() % 4 == 0:
            self._oneshot_parity = 1 - getattr(self, "_oneshot_parity", 1)
            slot = off + self._chunk * (1 + self._world) + self._oneshot_parity * self._ONESHOT_BYTES
            e = arena.next_epoch(0)
            _lib.check(lib.fb_dist_allreduce_oneshot(arena.ctx, 0, e, slot, n, _OP_CODE[op], scale, work.data_ptr(),
                                                     work.data_ptr(), max(1, min(128, (n + 1023) // 1024)), 256,
                                                     self._stream()), "fb_dist_allreduce_oneshot")
            if work.data_ptr() != flat.data_ptr():
                flat.copy_(work)
            if flat.data_ptr() != t.data_ptr():
                t.copy_(flat.view(t.shape))
            return
        use_mc = 1 if (arena.has_multicast() and op in (ReduceOp.Sum, ReduceOp.Average)) else 0
        for lo in range(0, n, per):
            cnt = min(per, n - lo)
            padded = (cnt + 4 * self._world - 1) // (4 * self._world) * (4 * self._world)
            e = arena.next_epoch(0)
            # staging into and out of the arena happens inside the kernel (each block moves the positions it
            # handshakes for), so an all-reduce of any fp32 tensor is ONE launch
            ptr = work.data_ptr() + lo * 4
            _lib.check(lib.fb_dist_allreduce_staged(arena.ctx, use_mc, 0, e, off, padded, _OP_CODE[op], scale, ptr,
                                                    ptr, cnt, self._blocks(padded * 4), 256, self._stream()),
                       "fb_dist_allreduce_staged")
        if work.data_ptr() != flat.data_ptr():
            flat.copy_(work)
        if flat.data_ptr() != t.data_ptr():
            t.copy_(flat.view(t.shape))

    def _staged(self, mode: int, root: int, src: torch.Tensor | None, dst: torch.Tensor | None, nbytes_chunk: int,
                op: ReduceOp = ReduceOp.Sum) -> None:
        """One pull-collective launch on tensors outside the arena: the kernel stages ``src`` (contiguous, or None
        where this rank contributes nothing) into the arena's input region itself and writes this rank's result
        straight into ``dst`` (contiguous, or None where it receives nothing)."""
        arena = self.comm_arena()
        e = arena.next_epoch(0)
        scale = 1.0 / self._world if op is ReduceOp.Average else 1.0
        _lib.check(_lib.cuda().fb_dist_collective_staged(
            arena.ctx, mode, 0, e, root, arena.data_offset(), nbytes_chunk, _OP_CODE[op], scale,
            src.data_ptr() if src is not None else None, dst.data_ptr() if dst is not None else None,
            self._blocks(nbytes_chunk), self._stream()), "fb_dist_collective_staged")

    @staticmethod
    def _as_one_buffer(tensors, nbytes: int):
        """The tensors as ONE contiguous buffer when they already are consecutive slices of one (the usual
        ``buf.chunk(world)`` case), else None."""
        base = tensors[0].data_ptr()
        for r, t in enumerate(tensors):
            if not t.is_contiguous() or t.data_ptr() != base + r * nbytes:
                return None
        return tensors[0]

    def broadcast(self, tensor, root: int = 0):
        t = _unwrap(tensor)
        self._begin()
        if not 0 <= root < self._world:
            raise InvalidRank(root, self._world)
        if self._world == 1:
            return tensor
        reg = self._registered(t) if self._native(t) else None
        if reg is not None:  # every rank pulls the root's region into its own, in place
            arena, roff, rbytes = reg
            e = arena.next_epoch(0)
            _lib.check(_lib.cuda().fb_dist_collective(arena.ctx, 0, 0, e, root, roff, roff, rbytes, 0, 1.0,
                                                      self._blocks(rbytes), self._stream()), "fb_dist_collective")
            return tensor
        if self._native(t):
            flat = t.contiguous().view(-1).view(torch.uint8)
            for lo in range(0, flat.numel(), self._chunk):
                part = flat[lo:lo + min(self._chunk, flat.numel() - lo)]
                is_root = self._rank == root
                self._staged(0, root, part if is_root else None, None if is_root else part, part.numel())
            if flat.data_ptr() != t.data_ptr():
                t.copy_(flat.view(t.dtype).view(t.shape))
            return tensor
        import torch.distributed as dist

        self._host_call("broadcast", dist.broadcast, t, src=self._ranks[root], group=self._tg)
        return tensor

    def reduce(self, tensor, dst: int = 0, op: ReduceOp = ReduceOp.Sum):
        t = _unwrap(tensor)
        self._begin()
        if not 0 <= dst < self._world:
            raise InvalidRank(dst, self._world)
        if self._world == 1:
            return tensor
        if self._native(t) and t.dtype == torch.float32 and t.numel() * 4 <= self._chunk:
            work = t if t.is_contiguous() else t.contiguous()
            self._staged(5, dst, work, work if self._rank == dst else None, t.numel() * 4, op)
            if self._rank == dst and work.data_ptr() != t.data_ptr():
                t.copy_(work)
            return tensor
        import torch.distributed as dist

        self._host_call("reduce", dist.reduce, t, dst=self._ranks[dst], op=_torch_op(op), group=self._tg)
        if op is ReduceOp.Average and self._rank == dst:
            t.div_(self._world)
        return tensor

    def _gather_like(self, mode: int, root: int, x: torch.Tensor, outs, nbytes: int) -> None:
        receives = mode == 1 or self._rank == root
        buf = None
        if receives:
            buf = self._as_one_buffer(outs, nbytes)
            direct = buf is not None
            if not direct:
                buf = torch.empty(nbytes * self._world, device=x.device, dtype=torch.uint8)
        self._staged(mode, root, x.contiguous(), buf, nbytes)
        if receives and not direct:
            for r, o in enumerate(outs):
                o.copy_(buf[r * nbytes:(r + 1) * nbytes].view(x.dtype).view(o.shape))

    def all_gather(self, output, input):
        """``output[r]`` receives rank ``r``'s ``input``."""
        x = _unwrap(input)
        outs = [_unwrap(o) for o in output]
        self._begin()
        if len(outs) != self._world:
            raise InvalidConfiguration(f"all_gather needs {self._world} output tensors, got {len(outs)}")
        if self._world == 1:
            outs[0].copy_(x)
            return output
        nbytes = x.numel() * x.element_size()
        reg = self._registered(x) if self._native(x) else None
        if reg is not None and nbytes % 16 == 0:
            # the peers read this tensor where it lies; the results go straight into the output tensors
            arena, roff, _ = reg
            one = self._as_one_buffer(outs, nbytes)
            dst = one if one is not None else torch.empty(self._world * nbytes, dtype=torch.uint8, device=x.device)
            e = arena.next_epoch(0)
            _lib.check(_lib.cuda().fb_dist_collective_staged(arena.ctx, 1, 0, e, 0, roff, nbytes, 0, 1.0, None,
                                                             dst.data_ptr(), self._blocks(nbytes), self._stream()),
                       "fb_dist_collective_staged")
            if one is None:
                for r, o in enumerate(outs):
                    o.copy_(dst[r * nbytes:(r + 1) * nbytes].view(o.dtype).view(o.shape))
            return output
        if self._native(x) and nbytes <= self._chunk:
            self._gather_like(1, 0, x, outs, nbytes)
            return output
        import torch.distributed as dist

        self._host_call("all_gather", dist.all_gather, outs, x, group=self._tg)
        return output

    def gather(self, output, input, dst: int = 0):
        x = _unwrap(input)
        self._begin()
        if not 0 <= dst < self._world:
            raise InvalidRank(dst, self._world)
        outs = [_unwrap(o) for o in output] if output is not None else None
        if self._rank == dst and (outs is None or len(outs) != self._world):
            raise InvalidConfiguration("gather needs one output tensor per rank on the destination")
        if self._world == 1:
            outs[0].copy_(x)
            return output
        nbytes = x.numel() * x.element_size()
        if self._native(x) and nbytes <= self._chunk:
            self._gather_like(2, dst, x, outs, nbytes)
            return output
        import torch.distributed as dist

        self._host_call("gather", dist.gather, x, outs if self._rank == dst else None, dst=self._ranks[dst], group=self._tg)
        return output

    def _scatter_like(self, mode: int, root: int, ins, o: torch.Tensor, nbytes: int, op: ReduceOp) -> None:
        src = None
        if ins is not None:
            src = self._as_one_buffer(ins, nbytes)
            if src is None:
                src = torch.cat([i.contiguous().view(-1) for i in ins])
        dst = o if o.is_contiguous() else torch.empty_like(o, memory_format=torch.contiguous_format)
        self._staged(mode, root, src, dst, nbytes, op)
        if dst.data_ptr() != o.data_ptr():
            o.copy_(dst)

    def scatter(self, output, input, src: int = 0):
        o = _unwrap(output)
        self._begin()
        if not 0 <= src < self._world:
            raise InvalidRank(src, self._world)
        ins = [_unwrap(i) for i in input] if input is not None else None
        if self._rank == src and (ins is None or len(ins) != self._world):
            raise InvalidConfiguration("scatter needs one input tensor per rank on the source")
        if self._world == 1:
            o.copy_(ins[0])
            return output
        nbytes = o.numel() * o.element_size()
        if self._native(o) and nbytes * self._world <= self._chunk:
            self._scatter_like(3, src, ins if self._rank == src else None, o, nbytes, ReduceOp.Sum)
            return output
        import torch.distributed as dist

        self._host_call("scatter", dist.scatter, o, ins if self._rank == src else None, src=self._ranks[src], group=self._tg)
        return output

    def reduce_scatter(self, output, input, op: ReduceOp = ReduceOp.Sum):
        """``output`` receives the reduction over ranks of ``input[rank]``."""
        o = _unwrap(output)
        ins = [_unwrap(i) for i in input]
        self._begin()
        if len(ins) != self._world:
            raise InvalidConfiguration(f"reduce_scatter needs {self._world} input tensors, got {len(ins)}")
        if self._world == 1:
            o.copy_(ins[0])
            return output
        nbytes = o.numel() * 4
        if self._native(o) and o.dtype == torch.float32 and nbytes * self._world <= self._chunk:
            self._scatter_like(4, 0, ins, o, nbytes, op)
            return output
        import torch.distributed as dist

        self._host_call("reduce_scatter", dist.reduce_scatter, o, ins, op=_torch_op(op), group=self._tg)
        if op is ReduceOp.Average:
            o.div_(self._world)
        return output

    def barrier(self) -> None:
        self._begin()
        if self._world == 1:
            return
        if self._backend is Backend.Nvlink and torch.cuda.is_available():
            if self._sync_arena is None:  # a flags-only arena: the barrier moves no data
                self._sync_arena = SymmetricArena.create(4096, self._rank, self._world, self.exchange,
                                                         self._config.device_wait_ns())
            arena = self._sync_arena
            e = arena.next_epoch(1)
            _lib.check(_lib.cuda().fb_dist_barrier(arena.ctx, 1, e, self._stream()), "fb_dist_barrier")
            torch.cuda.current_stream().synchronize()
            self._check_device_status("barrier")
            return
        import torch.distributed as dist

        try:
            dist.barrier(group=self._tg)
        except RuntimeError as exc:
            raise Timeout(f"barrier ({exc})") from None

    def sequence_number(self) -> int:
        """How many collectives this rank has issued on the group (for mismatch detection on the host)."""
        return self._seq

    def verify_in_step(self) -> None:
        """Host-side check that all ranks issued the same number of collectives; raises on mismatch."""
        seqs = self.exchange(self._seq)
        if len(set(seqs)) != 1:
            raise CommunicationError(f"ranks disagree on the collective sequence number: {seqs}")

    def close(self) -> None:
        for arena, _, _ in self._symm.values():
            arena.close()
        self._symm = {}
        for name in ("_arena", "_sync_arena"):
            a = getattr(self, name)
            if a is not None:
                a.close()
                setattr(self, name, None)


# ---------------------------------------------------------------------- module-level API (lib.rs:46-130)
def _init_torch(backend: Backend, rank: int, world: int, cfg: BackendConfig) -> None:
    import torch.distributed as dist

    if dist.is_initialized():
        return
    tb = "gloo" if backend is Backend.Gloo else "cpu:gloo,cuda:nccl"
    if backend is Backend.Mpi:
        raise UnsupportedBackend("mpi")
    os.environ.setdefault("MASTER_ADDR", cfg.master_addr)
    os.environ.setdefault("MASTER_PORT", str(cfg.master_port))
    try:
        dist.init_process_group(tb, init_method=f"tcp://{cfg.master_addr}:{cfg.master_port}", rank=rank,
                                world_size=world, timeout=datetime.timedelta(seconds=cfg.timeout_seconds))
    except Exception as exc:  # rendezvous failed: a rank never joined, wrong address, ...
        msg = str(exc)
        if "imeout" in msg or "timed out" in msg:
            raise Timeout(f"rendezvous at {cfg.master_addr}:{cfg.master_port} ({msg})") from None
        raise CommunicationError(msg) from None


def init_process_group(backend=Backend.Nvlink, rank: int = 0, world_size: int = 1,
                       config: BackendConfig | None = None) -> ProcessGroup:
    global _default_group
    if isinstance(backend, str):
        backend = Backend.from_str(backend)
    with _lock:
        if _default_group is not None:
            raise AlreadyInitialized()
        if world_size < 1 or not 0 <= rank < world_size:
            raise InvalidRank(rank, world_size)
        cfg = config or BackendConfig.from_env()
        if world_size > 1:
            if not backend.is_available():
                raise UnsupportedBackend(backend.value)
            _init_torch(backend, rank, world_size, cfg)
        _default_group = ProcessGroup(backend, rank, world_size, cfg)
        return _default_group


def init_process_group_from_env(backend=None) -> ProcessGroup:
    """``RANK`` (0), ``WORLD_SIZE`` (1), ``DIST_BACKEND`` (gloo), plus ``LOCAL_RANK`` to pick the GPU."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if backend is None:
        backend = os.environ.get("DIST_BACKEND", "gloo")
    if isinstance(backend, str):
        backend = Backend.from_str(backend)
    if backend in (Backend.Nvlink, Backend.Nccl) and torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", str(rank))) % max(torch.cuda.device_count(), 1))
    return init_process_group(backend, rank, world)


def get_world():
    return _default_group


def is_initialized() -> bool:
    return _default_group is not None


def destroy_process_group(keep_torch: bool = False) -> None:
    """Closes the default group and its arenas.  ``keep_torch`` leaves the ``torch.distributed`` rendezvous up for
    code that runs afterwards in the same process (a later ``init_process_group`` reuses it)."""
    global _default_group
    with _lock:
        g, _default_group = _default_group, None
    if g is not None:
        g.close()
        import torch.distributed as dist

        if g.world_size() > 1 and dist.is_initialized() and not keep_torch:
            dist.destroy_process_group()


def leave_process_group() -> None:
    """This rank stops taking part: it announces its departure in the rendezvous store (the remaining ranks get a
    ``CommunicationError`` from their next collective instead of waiting for it) and closes its group.  Call it
    between steps, with no collective of this rank in flight."""
    global _default_group
    with _lock:
        g, _default_group = _default_group, None
    if g is not None:
        g.leave()


def get_rank() -> int:
    return _default_group.rank() if _default_group is not None else 0


def get_world_size() -> int:
    return _default_group.world_size() if _default_group is not None else 1


def is_main_process() -> bool:
    return get_rank() == 0


def barrier() -> None:
    if _default_group is not None:
        _default_group.barrier()


def new_group(ranks) -> ProcessGroup:
    """A sub-group of the default group containing ``ranks`` (collective over the default group)."""
    if _default_group is None:
        raise NotInitialized()
    ranks = sorted(int(r) for r in ranks)
    world = _default_group.world_size()
    if not ranks or any(r < 0 or r >= world for r in ranks):
        raise InvalidRank(ranks[0] if ranks else -1, world)
    me = _default_group.rank()
    tg = None
    if world > 1:
        import torch.distributed as dist

        tg = dist.new_group(ranks)
    backend = _default_group.backend()
    if backend is Backend.Nvlink and len(ranks) != world:
        backend = Backend.Nccl  # arenas are mapped for the full world; sub-groups use the library transport
    if me not in ranks:
        return ProcessGroup(backend, 0, 1, _default_group.config())
    return ProcessGroup(backend, ranks.index(me), len(ranks), _default_group.config(), _torch_group=tg, _ranks=ranks)
