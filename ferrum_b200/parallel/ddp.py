"""``DistributedDataParallel`` (ferrum-distributed/src/ddp.rs:35-237), for real.

The reference wraps a module and offers ``sync_gradients`` / ``broadcast_parameters`` that loop over no-op
collectives; its 25 MB ``bucket_size_mb`` and ``GradientBucket`` are never used.  Here:

* parameters, gradients and the bf16 weight copies live in ONE peer-mapped symmetric arena per rank, laid out
  by the native bucket planner (reverse registration order, ``bucket_size_mb`` buckets);
* during ``backward`` each Linear's weight-gradient GEMM writes straight into its arena slot; when the last
  gradient of a bucket is enqueued, the bucket's reduction kernel is launched on a separate high-priority
  stream, so the reduction of layer *l* overlaps the backward GEMMs of layer *l-1*;
* with ``fuse_optimizer(opt)`` the reduction is split where the optimizer's memory traffic would otherwise land
  on the backward GEMMs: per bucket a small reduce-scatter kernel (``fb_dist_reduce_scatter_shard``: each rank sums
  its shard over the peers, 1/world folded in) runs beside the rest of backward, and after backward ONE kernel
  (``fb_dist_shard_update``) applies SGD-momentum / Adam to the rank's shards and stores the new weights into
  every rank's arena, i.e. the all-gather half of the all-reduce fused with the optimizer; ``opt.step()`` then only
  joins the streams.  ``defer_update(False)`` selects the single-kernel form instead (all-reduce + update +
  publish per bucket inside backward, ``fb_dist_allreduce``).  Optimizer moments are kept only by the rank that
  owns a shard (1/world of the state per GPU);
* without a fused optimizer the same kernel averages the gradients in place and ``opt.step()`` runs the usual
  multi-tensor update;
* ``broadcast_parameters`` copies rank 0's arena to every rank with the pull-broadcast kernel.

With ``Backend.Nccl`` / ``Backend.Gloo`` (baseline and CPU tests) gradients are averaged per bucket with the
library's all-reduce on flat buffers and the optimizer runs unfused.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _lib, config
from ..core import Tensor, _unwrap
from ..nn.modules import Embedding, Linear, Module, tensor_io
from ..ops import gemm as _gemm
from ..ops.functional import GradSink
from ..utils import runtime as _rt
from .backend import Backend, CommunicationError, InternalError, ReduceOp, Timeout
from .process_group import ProcessGroup, get_world
from .symm import SymmetricArena

_GUARD_BYTES = 65536   # keeps every region on the 64 KiB alignment it has without the bands
_GUARD_PATTERN = 0xA5


class GradientBucket:
    """A contiguous run of gradient slots reduced together (ddp.rs:126-180)."""

    def __init__(self, index: int = 0, start: int = 0, length: int = 0):
        self.index, self.start, self.length = index, start, length
        self.param_indices: list[int] = []
        self.sizes: list[int] = []
        self.buffer: list[float] = []  # host-side staging used only by add_gradient()
        self.ready = False
        self._pending = 0

    @classmethod
    def new(cls):
        return cls()

    def add_gradient(self, param_idx: int, grad) -> None:
        vals = list(_unwrap(grad).reshape(-1).tolist()) if isinstance(_unwrap(grad), torch.Tensor) else list(grad)
        self.param_indices.append(param_idx)
        self.sizes.append(len(vals))
        self.buffer.extend(vals)

    def mark_ready(self) -> None:
        self.ready = True

    def is_ready(self) -> bool:
        return self.ready

    def size_bytes(self) -> int:
        return (self.length or len(self.buffer)) * 4

    def __repr__(self):
        return f"GradientBucket(index={self.index}, params={self.param_indices}, bytes={self.size_bytes()})"


class GradientHook:
    """Bucket bookkeeping handle (ddp.rs:182-198)."""

    def __init__(self, process_group, num_buckets: int):
        self.process_group = process_group
        self.buckets = [GradientBucket(i) for i in range(num_buckets)]

    @classmethod
    def new(cls, process_group, num_buckets):
        return cls(process_group, num_buckets)

    def all_ready(self) -> bool:
        return all(b.is_ready() for b in self.buckets)


def _plan(sizes, cap_elems: int, align: int, param_align: int, kinds=None):
    n = len(sizes)
    LL, I = ctypes.c_longlong, ctypes.c_int
    szs = (LL * n)(*sizes)
    offs, bof = (LL * n)(), (I * n)()
    bstart, blen = (LL * max(n, 1))(), (LL * max(n, 1))()
    nb = I(0)
    kd = (I * n)(*kinds) if kinds is not None else None
    total = _lib.host().fb_plan_buckets_kinds(n, szs, kd, cap_elems, align, param_align, offs, bof, bstart, blen,
                                              ctypes.byref(nb))
    if total < 0:
        raise ValueError("bucket planning failed")
    return total, list(offs), list(bof), list(bstart)[:nb.value], list(blen)[:nb.value]


class DistributedDataParallel(Module, GradSink):
    def __init__(self, module: torch.nn.Module, process_group: ProcessGroup | None = None, optimizer=None):
        super().__init__()
        self.inner = module
        self._pg = process_group or get_world() or ProcessGroup(Backend.Gloo, 0, 1)
        self._bucket_mb = 25.0
        self._broadcast_buffers = True
        self._find_unused = False
        self._built = False
        self._opt = None
        self._capturable = False
        self._dev_epoch = None        # uint32 device counter of the bucket kernels' handshake epochs (capturable mode)
        self._advanced = False        # the optimizer's device scalars were advanced in this step
        self._shard_master = os.environ.get("FERRUM_SHARD_MASTER", "0") == "1"
        self._master_stale = False
        # Push mode: the weight-gradient GEMMs store their results straight into the shard owners' memory.
        self._push = os.environ.get("FERRUM_GEMM_PUSH", "0") == "1"
        self._pushed = []
        self._pushed_params = set()
        # Blocks of a bucket kernel.  The per-bucket reduce-scatter kernel is light (at most 80 registers, it sits
        # beside a persistent GEMM CTA), and 128 blocks measured best at 2 and at 8 ranks (8 ranks: a 64 MB bucket
        # takes 128 us with 128 blocks and 216 - 308 us with 48, step 7.1 against 7.6 ms with eager launches).  The
        # single-kernel form (defer_update(False)) carries the optimizer and wanted 48 at 4 and 8 ranks.
        env_blocks = os.environ.get("FERRUM_COMM_BLOCKS")
        self._comm_blocks = int(env_blocks) if env_blocks else 128
        self._comm_threads = int(os.environ.get("FERRUM_COMM_THREADS", "256"))
        # Deferred update (default): reduce-scatter per bucket inside backward, one optimizer + publish kernel after
        # it.  Measured at 2 GPUs on the 8 x 4096 MLP: the single-kernel form keeps 128 blocks of 200+ registers
        # busy for 230 us per 64 MB bucket; they do not fit beside a persistent GEMM CTA and stream half of the
        # optimizer state through the L2 the GEMMs live on (7.4 ms/step against 6.3 on one GPU).
        self._defer = True
        self._update_in_backward = False  # two-kernel form with the update launched per bucket inside backward
        self._update_blocks = 592     # blocks of the update kernel: four per SM, it runs alone (measured best of 444 / 592 / 888)
        self._dev_epoch_up = None
        self._table = None
        self._prof = None             # per-step timing events of the bucket kernels (comm_profile)
        self._prof_last = None
        if optimizer is not None:
            self.fuse_optimizer(optimizer)

    # ------------------------------------------------------------------ reference API
    @classmethod
    def new(cls, module, process_group):
        return cls(module, process_group)

    def bucket_size_mb(self, size: float) -> "DistributedDataParallel":
        self._bucket_mb = float(size)
        return self

    def broadcast_buffers(self, flag: bool) -> "DistributedDataParallel":
        self._broadcast_buffers = bool(flag)
        return self

    def find_unused_parameters(self, flag: bool) -> "DistributedDataParallel":
        self._find_unused = bool(flag)
        return self

    def module(self):
        return self.inner

    module_mut = module

    def process_group(self) -> ProcessGroup:
        return self._pg

    def into_inner(self):
        self.shutdown()
        return self.inner

    def shard_master_weights(self, flag: bool = True) -> "DistributedDataParallel":
        """Keep the fp32 master copy of a parameter current only on the rank that owns its shard.

        The fused reduction then publishes just the bf16 copies (2 instead of 6 bytes per parameter per peer),
        which is all that bf16 forward / backward passes read.  The fp32 tensors of the other ranks are brought
        up to date by ``sync_master_weights()`` (called automatically by ``shutdown`` and ``state_dict``-style
        accessors of this wrapper); use it only together with ``autocast``.
        """
        self._shard_master = bool(flag)
        self._table = None  # the per-bucket publish flags follow
        return self

    def defer_update(self, flag: bool = True) -> "DistributedDataParallel":
        """``True`` (default): reduce-scatter per bucket during backward, one optimizer + publish kernel after it.
        ``False``: all-reduce, optimizer and publish in one kernel per bucket, inside backward."""
        self._defer = bool(flag)
        if not os.environ.get("FERRUM_COMM_BLOCKS"):
            self._comm_blocks = 128 if (self._defer or self._pg.world_size() <= 2) else 48
        return self

    def update_in_backward(self, flag: bool = True) -> "DistributedDataParallel":
        """Two-kernel form with the update kernel launched per bucket right behind its reduce-scatter instead of
        once after backward: both kernels are small enough to share an SM with a persistent GEMM CTA, so the
        optimizer's memory traffic is spread over the backward pass."""
        self._update_in_backward = bool(flag)
        if flag:
            self._defer = True
        return self

    def push_gradients(self, flag: bool = True) -> "DistributedDataParallel":
        """Fuse the gradient reduce-scatter into the weight-gradient GEMMs: the epilogue of each (bf16, CTA-pair
        sized) wgrad GEMM stores every 16-byte piece of dW over NVLink into the bucket region of the rank that owns
        it, so the transfer overlaps the following tiles and the bucket kernel reads only local memory for those
        ranges.  In this mode ``param.grad`` of such a weight holds no usable values on any rank (the owner's
        region contains one slot per source rank), so gradient clipping or inspection of those tensors is not
        available; a weight used twice in one step is not supported.  Off by default (``FERRUM_GEMM_PUSH=1``)."""
        self._push = bool(flag)
        return self

    def comm_profile(self, flag: bool = True) -> "DistributedDataParallel":
        """Time every bucket kernel with CUDA events (eager steps only, not while a step is recorded in or
        replayed from a CUDA graph): when its last gradient was enqueued, when the kernel started and ended on the
        communication stream, and when the backward pass itself ended.  ``last_comm_profile()`` returns the
        record of the most recent finished step."""
        self._prof = {} if flag else None
        return self

    def last_comm_profile(self) -> dict | None:
        """``{"buckets": [{index, bytes, ready_ms, start_ms, end_ms, kernel_us, bus_gbs}], "backward_end_ms",
        "step_end_ms", "exposed_tail_us", "comm_busy_us"}``: times relative to the step's ``zero_grad``;
        ``bus_gbs`` = bytes x 2 (world - 1) / world / kernel time, the usual all-reduce bus bandwidth;
        ``exposed_tail_us`` = how long after the last backward kernel the last bucket kernel ended."""
        rec = self._prof_last
        if rec is None:
            return None
        rec["done"].synchronize()
        t0 = rec["t0"]
        world = self._pg.world_size()
        out = {"buckets": []}
        busy = 0.0
        # bytes x (world - 1) / world cross the link per half of an all-reduce; the single-kernel form does both
        halves = 1.0 if (self._defer and self._opt is not None and not self._push) else 2.0
        for b, (ready, start, end, nbytes) in sorted(rec["buckets"].items(), key=lambda kv: t0.elapsed_time(kv[1][1])):
            us = start.elapsed_time(end) * 1e3
            busy += us
            out["buckets"].append({"index": b, "bytes": nbytes, "ready_ms": t0.elapsed_time(ready),
                                   "start_ms": t0.elapsed_time(start), "end_ms": t0.elapsed_time(end),
                                   "kernel_us": us,
                                   "bus_gbs": (nbytes * halves * (world - 1) / world / (us * 1e-6) / 1e9) if us > 0
                                   else 0.0})
        out["backward_end_ms"] = t0.elapsed_time(rec["bwd_end"])
        out["step_end_ms"] = t0.elapsed_time(rec["done"])
        last_end = max((x["end_ms"] for x in out["buckets"]), default=out["backward_end_ms"])
        out["exposed_tail_us"] = max(0.0, (last_end - out["backward_end_ms"]) * 1e3)
        out["comm_busy_us"] = busy
        return out

    def try_push(self, param, a: torch.Tensor, b: torch.Tensor) -> bool:
        """GradSink extension used by the Linear backward: run ``dW = a @ b^T`` with the pushing epilogue if this
        parameter's gradient may be delivered that way.  Returns False when the ordinary path must be taken."""
        # Needs the fused optimizer: a plain all-reduce writes its results back into the gradient region, where the
        # other ranks' contribution slots live.
        if not (self._push and getattr(self, "_use_native", False) and self._sync_enabled and self._opt is not None):
            return False
        world = self._pg.world_size()
        if world < 2 or not _gemm.push_operands_ok(a, b):
            return False
        i = self._index[id(param)]
        if self._written[i] or tuple(param.shape) != (a.shape[0], b.shape[0]):
            return False
        bi = self._bucket_of[i]
        bk = self.buckets[bi]
        # Only a bucket that holds this one tensor: the slot a source rank writes in the owner's region would
        # otherwise alias the ordinarily laid-out gradients of the bucket's other tensors.
        if bk.length % (4 * world) or len(bk.param_indices) != 1 or self._pushed[bi]:
            return False
        rel = self._offs[i] - bk.start
        if rel % 4 or rel < 0 or rel + param.numel() > bk.length:
            return False
        if not _gemm.gemm_bf16_push(a, b, self._arena.ctx, self._off_grad + bk.start * 4, rel, bk.length // world,
                                    bk.length):
            return False
        self._written[i] = True
        self._pushed_params.add(i)
        ranges = self._pushed[bi]
        if ranges and ranges[-1][1] == rel:       # extends the previous range
            ranges[-1] = (ranges[-1][0], rel + param.numel())
        elif ranges and ranges[-1][0] == rel + param.numel():
            ranges[-1] = (rel, ranges[-1][1])
        else:
            ranges.append((rel, rel + param.numel()))
        return True

    def sync_master_weights(self) -> None:
        """All-gather the fp32 parameter shards so that every rank holds the full, current master weights."""
        if not (getattr(self, "_use_native", False) and self._master_stale):
            return
        a = self._arena
        world = self._pg.world_size()
        self._done_event.record(self._comm_stream)
        torch.cuda.current_stream().wait_event(self._done_event)
        st = torch.cuda.current_stream().cuda_stream
        for bk in self.buckets:
            per = bk.length // world
            # channel 3: its epochs are only ever advanced from the host.  The bucket kernels' channel (2) is
            # advanced on the device when a recorded step is replayed, so a host-side epoch for it can be stale.
            e = a.next_epoch(3)
            _lib.check(_lib.cuda().fb_dist_collective(a.ctx, 6, 3, e, 0, self._off_param + bk.start * 4, 0,
                                                      per * 4, 0, 1.0, 32, st), "fb_dist_collective")
        self._master_stale = False

    def capturable(self, flag: bool = True) -> "DistributedDataParallel":
        """Make the step recordable in a CUDA graph: the handshake epochs of the bucket kernels and the optimizer's
        step-dependent factors are then read from device memory and advanced by kernels on the communication stream
        (a graph would freeze the by-value arguments).  Needs a fused optimizer in capturable mode.  One-way: after
        the switch every step, recorded or not, uses the device-side counters."""
        if flag and self._opt is None:
            raise CommunicationError("capturable() needs fuse_optimizer() first")
        self._capturable = bool(flag)
        if flag and self._opt._dyn is None:
            self._opt.capturable(True)
        return self

    def fuse_optimizer(self, optimizer) -> "DistributedDataParallel":
        """Apply ``optimizer``'s update inside the bucket reduction kernels (SGD or Adam)."""
        self._opt = optimizer
        optimizer._engine = self
        return self

    # ------------------------------------------------------------------ build
    def _native(self) -> bool:
        # A single rank also takes the native path once an optimizer is fused: the "reduction" then has nothing to
        # fetch, and what remains is the per-bucket optimizer update launched behind each weight gradient on the
        # side stream, i.e. the update overlapped with the rest of backward instead of a separate pass after it.
        world = self._pg.world_size()
        return (self._pg.backend() is Backend.Nvlink and (world > 1 or (world == 1 and self._opt is not None)) and
                all(p.is_cuda for p in torch.nn.Module.parameters(self.inner)))

    def _build(self) -> None:
        if self._built:
            return
        self._built = True
        self._params = [p for p in torch.nn.Module.parameters(self.inner) if p.requires_grad]
        if any(p.dtype != torch.float32 for p in self._params):
            raise CommunicationError("DistributedDataParallel expects fp32 master parameters")
        world, rank = self._pg.world_size(), self._pg.rank()
        cap = max(1, int(self._bucket_mb * (1 << 20)) // 4)
        sizes = [p.numel() for p in self._params]
        self._index = {id(p): i for i, p in enumerate(self._params)}
        # Linear / Embedding weights: their gradients are written into the arena by the producing kernel (a "sink").
        # Under bf16 autocast forward and backward read Linear weights through their bf16 copies; everything else
        # (biases, normalisation scales and shifts, embedding tables) is read in fp32.  A bucket holds one kind.
        self._use_native = self._native()
        sink_ids, sink_mods, bf16_ids = set(), [], set()
        for mod in self.inner.modules():
            if (type(mod) is Linear or isinstance(mod, Embedding)) and id(mod.weight) in self._index:
                sink_ids.add(id(mod.weight))
                sink_mods.append(mod)
                if type(mod) is Linear:  # an embedding table is gathered from its fp32 values
                    bf16_ids.add(id(mod.weight))
        kinds = [1 if id(p) in bf16_ids else 0 for p in self._params]
        total, offs, bof, bstart, blen = _plan(sizes, cap, 4 * world, 32, kinds)
        self._total, self._offs, self._bucket_of = total, offs, bof
        self.buckets = [GradientBucket(i, bstart[i], blen[i]) for i in range(len(bstart))]
        for i, b in enumerate(bof):
            self.buckets[b].param_indices.append(i)
            self.buckets[b].sizes.append(sizes[i])
        # fp32 values of a bucket go to the peers unless every parameter in it is consumed through its bf16 copy
        self._bucket_bf16_only = [all(kinds[i] == 1 for i in bk.param_indices) for bk in self.buckets]
        self._written = [False] * len(self._params)
        self._launched = [False] * len(self.buckets)
        dev = self._params[0].device if self._params else torch.device("cpu")
        if self._use_native:
            self._build_native(total, dev)
        else:
            self._flat_grads = torch.zeros(total, device=dev, dtype=torch.float32)
            for i, p in enumerate(self._params):
                p.grad = self._flat_grads[offs[i]:offs[i] + sizes[i]].view(p.shape)
        # sinks and hooks
        self._small_runs = []  # (start, length) runs of non-GEMM gradients, zeroed every step
        self._hook_handles, self._sink_modules = [], []
        if not self._use_native:
            sink_ids = set()  # gradients arrive through autograd hooks
        for mod in sink_mods if self._use_native else []:
            # through __dict__: a plain attribute assignment would register the engine as a SUBMODULE of the
            # layer and close a cycle (engine -> inner -> layer -> engine) under state_dict() / apply()
            mod.__dict__["grad_sink"] = self
            self._sink_modules.append(mod)
        run = None
        order = sorted(range(len(self._params)), key=lambda i: offs[i])
        for i in order:
            p = self._params[i]
            if id(p) in sink_ids:
                if run:
                    self._small_runs.append(tuple(run))
                    run = None
                continue
            if run and run[0] + run[1] <= offs[i] <= run[0] + run[1] + 64:
                run[1] = offs[i] + sizes[i] - run[0]
            else:
                if run:
                    self._small_runs.append(tuple(run))
                run = [offs[i], sizes[i]]
            self._hook_handles.append(p.register_post_accumulate_grad_hook(self._make_hook(i)))
        if run:
            self._small_runs.append(tuple(run))
        self._sink_ids = sink_ids
        self.broadcast_parameters()
        self._reset_step_state()

    def _build_native(self, total: int, dev) -> None:
        world, rank = self._pg.world_size(), self._pg.rank()
        lib = _lib.cuda()
        fb = lib.fb_dist_query_flag_bytes()
        # FERRUM_GUARD_BANDS=1 (debug): 64 KiB of a fixed byte pattern before, between and after the three regions;
        # check_guard_bands() tells whether any kernel, local or a peer's, wrote outside its region.
        gb = _GUARD_BYTES if os.environ.get("FERRUM_GUARD_BANDS") == "1" else 0
        self._off_param = fb + gb
        self._off_grad = self._off_param + total * 4 + gb
        self._off_shadow = self._off_grad + total * 4 + gb
        self._arena = SymmetricArena.create(total * 10 + 4 * gb, rank, world, self._pg.exchange,
                                            self._pg.config().device_wait_ns())
        a = self._arena
        self._guards = []
        if gb:
            for name, off in (("before the parameters", fb), ("parameters | gradients", self._off_grad - gb),
                              ("gradients | bf16 copies", self._off_shadow - gb),
                              ("after the bf16 copies", self._off_shadow + total * 2)):
                band = a.view(off, (gb,), torch.uint8)
                band.fill_(_GUARD_PATTERN)
                self._guards.append((name, band))
        self._flat_params = a.view(self._off_param, (total,), torch.float32)
        self._flat_grads = a.view(self._off_grad, (total,), torch.float32)
        self._flat_shadow = a.view(self._off_shadow, (total,), torch.bfloat16)
        for i, p in enumerate(self._params):
            o, n = self._offs[i], p.numel()
            slot = self._flat_params[o:o + n].view(p.shape)
            slot.copy_(p.detach())
            p.data = slot
            p.grad = self._flat_grads[o:o + n].view(p.shape)
            p.__dict__["_fb_shadow"] = self._flat_shadow[o:o + n].view(p.shape)
            p.__dict__["_fb_shadow_key"] = None
        # per-shard optimizer state (owner only) — allocated lazily in _launch_bucket
        self._state_m = None
        self._state_v = None
        self._comm_stream = torch.cuda.Stream(device=dev, priority=int(os.environ.get("FERRUM_COMM_PRIORITY", "-1")))
        self._ready_event = torch.cuda.Event()
        self._done_event = torch.cuda.Event()
        # A reduction block (256 threads, no shared memory) fits on an SM beside a persistent GEMM CTA, so the
        # GEMM grid is not shrunk by default; FERRUM_GEMM_CTA_LIMIT reserves SMs for experiments.
        self._gemm_limit = int(os.environ.get("FERRUM_GEMM_CTA_LIMIT", "0"))

    def _refresh_shadow(self) -> None:
        """Recompute every bf16 weight copy from the fp32 arena with one cast kernel."""
        lib = _lib.cuda()
        _lib.check(lib.fb_cast(self._flat_params.data_ptr(), self._flat_shadow.data_ptr(), self._total, 0, 3,
                               torch.cuda.current_stream().cuda_stream), "fb_cast")
        for p in self._params:
            p.__dict__["_fb_shadow_key"] = (p._version, p.data_ptr())

    # ------------------------------------------------------------------ GradSink (called from Linear backward)
    def acquire(self, param):
        i = self._index[id(param)]
        if i in self._pushed_params:
            raise CommunicationError("a weight whose gradient was pushed to its shard owners cannot receive a "
                                     "second gradient in the same step (push_gradients(False) for such models)")
        o, n = self._offs[i], param.numel()
        acc = self._written[i]
        self._written[i] = True
        return self._flat_grads[o:o + n].view(param.shape), acc

    def ready(self, param) -> None:
        self._mark_ready(self._index[id(param)])

    def _make_hook(self, i: int):
        def hook(p):
            self._mark_ready(i)

        return hook

    def _mark_ready(self, i: int) -> None:
        if not self._sync_enabled:
            return
        b = self._bucket_of[i]
        bk = self.buckets[b]
        if i in self._pending[b]:
            self._pending[b].discard(i)
            if not self._pending[b] and not self._launched[b]:
                self._launch_bucket(b)

    def _reset_step_state(self) -> None:
        self._pending = [set(b.param_indices) for b in self.buckets]
        self._launched = [False] * len(self.buckets)
        self._written = [False] * len(self._params)
        self._pushed = [[] for _ in self.buckets]
        self._pushed_params = set()
        self._advanced = False
        self._deferred = False
        self._sync_enabled = True
        for b in self.buckets:
            b.ready = False

    # ------------------------------------------------------------------ bucket reduction
    def _launch_bucket(self, b: int) -> None:
        self._launched[b] = True
        bk = self.buckets[b]
        bk.ready = True
        world = self._pg.world_size()
        if not self._use_native:
            if world > 1:
                seg = self._flat_grads[bk.start:bk.start + bk.length]
                self._pg.all_reduce(seg, ReduceOp.Average)
            return
        lib = _lib.cuda()
        a = self._arena
        cur = torch.cuda.current_stream()
        # A Linear / Embedding weight whose GEMM did not run in this step still holds the previous step's gradient
        # (those slots are overwritten, never zeroed): it takes part as a zero gradient, as in torch.
        for i in bk.param_indices:
            if not self._written[i] and id(self._params[i]) in self._sink_ids:
                o = self._offs[i]
                self._flat_grads[o:o + self._params[i].numel()].zero_()
        self._ready_event.record(cur)
        self._comm_stream.wait_event(self._ready_event)
        prof = self._prof if (self._prof is not None and not torch.cuda.is_current_stream_capturing()) else None
        if prof is not None:
            if "t0" not in prof:  # no zero_grad() seen: the step starts here
                prof["t0"] = torch.cuda.Event(enable_timing=True)
                prof["t0"].record(cur)
                prof["buckets"] = {}
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record(cur)
            ev[1].record(self._comm_stream)
            prof["buckets"][b] = (ev[0], ev[1], ev[2], bk.length * 4)
        opt = self._opt
        fuse, adam_h, sgd_h, m_ptr, v_ptr = 0, None, None, None, None
        per = ((bk.length + world - 1) // world + 3) // 4 * 4
        lo = min(bk.length, per * self._pg.rank())
        if opt is not None:
            from ..optim.optimizers import SGD, Adam

            self._ensure_state()
            so = self._state_off[b]
            if isinstance(opt, Adam):
                fuse = 2
                adam_h = ctypes.pointer(opt.hparams(opt.step_count + 1, 1.0 / world))
                m_ptr = self._state_m.data_ptr() + so * 4
                v_ptr = self._state_v.data_ptr() + so * 4
            elif isinstance(opt, SGD):
                fuse = 1
                sgd_h = ctypes.pointer(opt.hparams(1.0 / world))
                if opt.config.momentum != 0.0:
                    m_ptr = self._state_m.data_ptr() + so * 4
            else:
                raise CommunicationError(f"cannot fuse optimizer of type {type(opt).__name__}")
        e = a.next_epoch(2)
        use_mc = 1 if a.has_multicast() else 0
        if fuse and self._defer and not self._push:
            # reduce-scatter only; the update of all shards follows in _flush
            dev_e = None
            if self._capturable:
                if self._dev_epoch is None:
                    self._dev_epoch = torch.tensor([e - (1 << 32) if e >= (1 << 31) else e], dtype=torch.int32,
                                                   device=self._flat_params.device)
                dev_e = self._dev_epoch.data_ptr()
            rc = 0
            if world > 1:
                rc = lib.fb_dist_reduce_scatter_shard(a.ctx, use_mc, 2, e, dev_e, self._off_grad + bk.start * 4,
                                                      bk.length, 1.0 / world, self._comm_blocks, self._comm_threads,
                                                      self._comm_stream.cuda_stream)
            _lib.check(rc, "fb_dist_reduce_scatter_shard")
            if self._update_in_backward:
                self._launch_update(None, bucket=b)
            else:
                self._deferred = True
            if prof is not None:
                prof["buckets"][b][2].record(self._comm_stream)
            return
        if self._pushed[b]:  # consumed by the launch below: these ranges are already complete in local memory
            rng = self._pushed[b]
            LLn = ctypes.c_longlong * len(rng)
            _lib.check(lib.fb_dist_set_pushed_ranges(len(rng), LLn(*[r[0] for r in rng]), LLn(*[r[1] for r in rng])),
                       "fb_dist_set_pushed_ranges")
        if self._capturable and fuse:
            if self._dev_epoch is None:  # continue the host-side sequence on the device
                self._dev_epoch = torch.tensor([e - (1 << 32) if e >= (1 << 31) else e], dtype=torch.int32,
                                               device=self._flat_params.device)
            dyn = opt._dyn
            if not self._advanced:
                self._advanced = True
                if fuse == 2:  # Adam: one advance of beta^t / bias corrections per step, before the first bucket
                    _lib.check(lib.fb_optim_advance(dyn.data_ptr(), opt.config.beta1, opt.config.beta2,
                                                    self._comm_stream.cuda_stream), "fb_optim_advance")
            rc = lib.fb_dist_allreduce_dyn(a.ctx, fuse, use_mc, 2, self._dev_epoch.data_ptr(),
                                           self._off_grad + bk.start * 4, self._off_param + bk.start * 4,
                                           self._off_shadow + bk.start * 2, bk.length, 4, 1.0 / world, adam_h, sgd_h,
                                           m_ptr, v_ptr, 0 if (self._shard_master and fuse and self._bucket_bf16_only[b]) else 1,
                                           self._comm_blocks, self._comm_threads, dyn.data_ptr(),
                                           self._comm_stream.cuda_stream)
        else:
            rc = lib.fb_dist_allreduce(a.ctx, fuse, use_mc, 2, e, self._off_grad + bk.start * 4,
                                       self._off_param + bk.start * 4, self._off_shadow + bk.start * 2, bk.length,
                                       4, 1.0 / world, adam_h, sgd_h, m_ptr, v_ptr,
                                       0 if (self._shard_master and fuse and self._bucket_bf16_only[b]) else 1, self._comm_blocks,
                                       self._comm_threads, self._comm_stream.cuda_stream)
        if self._shard_master and fuse:
            self._master_stale = True
        if prof is not None:
            prof["buckets"][b][2].record(self._comm_stream)
        _lib.check(rc, "fb_dist_allreduce")

    def _launch_update(self, prof, bucket: int | None = None) -> None:
        """Optimizer update of this rank's shards + publication of the new weights on the communication stream:
        one kernel over every bucket behind everything the backward pass enqueued, or (``bucket`` given) the
        kernel for that one bucket behind its reduce-scatter."""
        from ..optim.optimizers import Adam

        lib, a, opt = _lib.cuda(), self._arena, self._opt
        world = self._pg.world_size()
        cur = torch.cuda.current_stream()
        if bucket is None:
            self._deferred = False
            self._ready_event.record(cur)          # the new weights must not land under a GEMM that still reads them
            self._comm_stream.wait_event(self._ready_event)
        self._ensure_state()
        if self._table is None:
            rows = [[bk.start, bk.length, self._state_off[i],
                     0 if (self._shard_master and self._bucket_bf16_only[i]) else 1]
                    for i, bk in enumerate(self.buckets)]
            self._table = torch.tensor(rows, dtype=torch.int64, device=self._flat_params.device)
        adam = isinstance(opt, Adam)
        adam_h = ctypes.pointer(opt.hparams(opt.step_count + 1, 1.0)) if adam else None
        sgd_h = None if adam else ctypes.pointer(opt.hparams(1.0))
        m_ptr = self._state_m.data_ptr() if (adam or opt.config.momentum != 0.0) else None
        v_ptr = self._state_v.data_ptr() if adam else None
        e = a.next_epoch(4)
        dev_e = dyn = None
        st = self._comm_stream.cuda_stream
        if self._capturable:
            if self._dev_epoch_up is None:
                self._dev_epoch_up = torch.tensor([e], dtype=torch.int32, device=self._flat_params.device)
            dev_e = self._dev_epoch_up.data_ptr()
            dyn = opt._dyn.data_ptr()
            if adam and not self._advanced:  # once per step, before the first update kernel
                self._advanced = True
                _lib.check(lib.fb_optim_advance(dyn, opt.config.beta1, opt.config.beta2, st), "fb_optim_advance")
        ev = None
        if prof is not None and "buckets" in prof:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record(cur)
            ev[1].record(self._comm_stream)
        first, count, blocks = (0, len(self.buckets), self._update_blocks) if bucket is None else (
            bucket, 1, self._comm_blocks)
        rc = lib.fb_dist_shard_update(a.ctx, 2 if adam else 1, 1 if a.has_multicast() else 0, 4, e, dev_e,
                                      self._off_grad, self._off_param, self._off_shadow,
                                      self._table.data_ptr() + 32 * first, count, adam_h, sgd_h, m_ptr, v_ptr,
                                      blocks, 256, dyn, st)
        if ev is not None:
            ev[2].record(self._comm_stream)
            prof["buckets"]["update"] = (ev[0], ev[1], ev[2], self._total * 4)
        if self._shard_master:
            self._master_stale = True
        _lib.check(rc, "fb_dist_shard_update")

    def _shard_len(self, bk) -> int:
        world = self._pg.world_size()
        return ((bk.length + world - 1) // world + 3) // 4 * 4

    def _ensure_state(self) -> None:
        """Optimizer moments of this rank's shards (1 / world of every bucket), allocated on first use."""
        if self._state_m is not None:
            return
        from ..optim.optimizers import Adam

        dev = self._flat_params.device
        acc, self._state_off = 0, []
        for x in self.buckets:
            self._state_off.append(acc)
            acc += self._shard_len(x)
        self._state_m = torch.zeros(acc, device=dev, dtype=torch.float32)
        self._state_v = torch.zeros(acc, device=dev, dtype=torch.float32) if isinstance(self._opt, Adam) else None

    def _flush(self) -> None:
        """Launch every bucket that has not been reduced in this step (unused parameters, explicit sync)."""
        prof = self._prof if (self._prof is not None and self._use_native
                              and not torch.cuda.is_current_stream_capturing()) else None
        if prof is not None and "t0" in prof:
            prof["bwd_end"] = torch.cuda.Event(enable_timing=True)
            prof["bwd_end"].record(torch.cuda.current_stream())
        for b in range(len(self.buckets)):
            if not self._launched[b]:
                self._launch_bucket(b)
        if self._use_native and getattr(self, "_deferred", False):
            self._launch_update(prof)
        if self._use_native:
            self._done_event.record(self._comm_stream)
            torch.cuda.current_stream().wait_event(self._done_event)
        if prof is not None and "bwd_end" in prof and prof.get("buckets"):
            prof["done"] = torch.cuda.Event(enable_timing=True)
            prof["done"].record(torch.cuda.current_stream())
            self._prof_last, self._prof = prof, {}

    # ------------------------------------------------------------------ step protocol
    def zero_grad(self) -> None:
        self._build()
        if self._pg.world_size() > 1:
            self._pg.check_peers(0.2)  # a rank that left between steps ends the step here, on the host
        for start, length in self._small_runs:
            self._flat_grads[start:start + length].zero_()
        if not self._use_native:
            self._flat_grads.zero_()
        self._reset_step_state()
        if self._prof is not None and self._use_native and not torch.cuda.is_current_stream_capturing():
            self._prof = {"t0": torch.cuda.Event(enable_timing=True), "buckets": {}}
            self._prof["t0"].record(torch.cuda.current_stream())

    def finish_step(self, optimizer) -> None:
        """Called by ``optimizer.step()`` when the update is fused into the reduction."""
        self._build()
        self._flush()
        if self._use_native and self._opt is optimizer:
            optimizer.step_count += 1
            for p in self._params:  # the kernels refreshed the bf16 copies together with the fp32 weights
                p.__dict__["_fb_shadow_key"] = (p._version, p.data_ptr())
        else:
            optimizer._step_local()
        self._check_status()
        self._reset_step_state()

    def sync_gradients(self, gradients=None) -> None:
        """Average gradients over the group.  With arena-backed gradients this flushes the pending buckets;
        explicit ``gradients`` (the reference's calling convention) are all-reduced one by one."""
        if gradients is not None:
            for g in gradients:
                self._pg.all_reduce(g, ReduceOp.Average)
            return
        self._build()
        self._flush()
        self._check_status()

    def broadcast_parameters(self, parameters=None) -> None:
        """Make every rank's parameters (and buffers) equal to rank 0's."""
        if parameters is not None:
            for p in parameters:
                self._pg.broadcast(p, 0)
            return
        self._build()
        world = self._pg.world_size()
        if self._use_native:
            a = self._arena
            torch.cuda.current_stream().synchronize()
            e = a.next_epoch(3)  # host-advanced channel (see sync_master_weights)
            _lib.check(_lib.cuda().fb_dist_collective(a.ctx, 0, 3, e, 0, self._off_param, self._off_param,
                                                      self._total * 4, 0, 1.0, 32,
                                                      torch.cuda.current_stream().cuda_stream), "fb_dist_collective")
            self._refresh_shadow()
            torch.cuda.current_stream().synchronize()
            self._check_status()
        elif world > 1:
            with torch.no_grad():
                for p in self._params:
                    self._pg.broadcast(p.data, 0)
        if self._broadcast_buffers and world > 1:
            with torch.no_grad():
                for buf in self.inner.buffers():
                    self._pg.broadcast(buf, 0)

    def no_sync(self):
        """Context manager: accumulate gradients locally without reducing (gradient accumulation)."""
        engine = self

        class _NoSync:
            def __enter__(self):
                engine._build()
                engine._sync_enabled = False

            def __exit__(self, *exc):
                engine._sync_enabled = True

        return _NoSync()

    def _check_status(self) -> None:
        if not self._use_native:
            return
        code, where, i0, i1 = _rt.read_status(clear=False)
        if code == 0:
            return
        _rt.read_status(clear=True)
        if code == 2:
            raise Timeout(f"gradient reduction (rank {self._pg.rank()} waited for rank {i0}, epoch {i1})")
        raise CommunicationError(f"device status {code} at site {where} ({i0}, {i1})")

    # ------------------------------------------------------------------ forward
    @tensor_io
    def forward(self, *args, **kw):
        self._build()
        if self._use_native:
            _gemm.set_gemm_cta_limit(self._gemm_limit)
        return self.inner(*args, **kw)

    def gather_optimizer_state(self) -> dict:
        """Full-length optimizer moments assembled from the shard owners (for checkpoints)."""
        if not (self._use_native and self._state_m is not None):
            return {}
        world = self._pg.world_size()
        out = {}
        for name, st in (("m", self._state_m), ("v", self._state_v)):
            if st is None:
                continue
            parts = [torch.empty_like(st) for _ in range(world)]
            self._pg.all_gather(parts, st)
            full = torch.zeros(self._total, device=st.device, dtype=torch.float32)
            for b, bk in enumerate(self.buckets):
                per = ((bk.length + world - 1) // world + 3) // 4 * 4
                for r in range(world):
                    lo = min(bk.length, per * r)
                    hi = min(bk.length, lo + per)
                    if hi > lo:
                        full[bk.start + lo:bk.start + hi] = parts[r][self._state_off[b]:self._state_off[b] + hi - lo]
            out[name] = full
        return out

    def owns_optimizer_state(self) -> bool:
        """True when the moments of the fused optimizer live in this engine's shards, not in the optimizer."""
        self._build()
        return bool(self._use_native and self._opt is not None)

    def export_optimizer_state(self, optimizer) -> dict:
        """The fused optimizer's moments as one full tensor per parameter, named as the optimizer itself names
        them (``optim.m.<i>`` / ``optim.v.<i>`` for Adam, ``optim.velocity.<i>`` for SGD).  Collective: every
        rank calls it (the shards are gathered from their owners), every rank gets the full state."""
        from ..optim.optimizers import Adam

        self._build()
        full = self.gather_optimizer_state()
        out = {}
        if not full:
            return out
        adam = isinstance(optimizer, Adam)
        for j, p in enumerate(optimizer.params):
            i = self._index.get(id(p))
            if i is None:
                continue
            o, n = self._offs[i], p.numel()
            if adam:
                out[f"optim.m.{j}"] = full["m"][o:o + n].view(p.shape).clone()
                out[f"optim.v.{j}"] = full["v"][o:o + n].view(p.shape).clone()
            elif optimizer.config.momentum != 0.0:
                out[f"optim.velocity.{j}"] = full["m"][o:o + n].view(p.shape).clone()
        return out

    def import_optimizer_state(self, optimizer, tensors: dict) -> None:
        """Inverse of :meth:`export_optimizer_state`: every rank keeps the slices of its own shards."""
        from ..optim.optimizers import Adam

        self._build()
        if not self._use_native:
            return
        self._ensure_state()
        adam = isinstance(optimizer, Adam)
        dev = self._flat_params.device
        names = (("m", "optim.m."), ("v", "optim.v.")) if adam else (("m", "optim.velocity."),)
        world, rank = self._pg.world_size(), self._pg.rank()
        for key, prefix in names:
            st = self._state_m if key == "m" else self._state_v
            if st is None:
                continue
            full = torch.zeros(self._total, device=dev, dtype=torch.float32)
            for j, p in enumerate(optimizer.params):
                i, t = self._index.get(id(p)), tensors.get(f"{prefix}{j}")
                if i is not None and t is not None:
                    o = self._offs[i]
                    full[o:o + p.numel()] = t.to(dev, torch.float32).reshape(-1)
            for b, bk in enumerate(self.buckets):
                per = self._shard_len(bk)
                lo = min(bk.length, per * rank)
                hi = min(bk.length, lo + per)
                if hi > lo:
                    st[self._state_off[b]:self._state_off[b] + hi - lo] = full[bk.start + lo:bk.start + hi]

    def state_dict(self, *args, **kw):
        """Parameters and buffers of the wrapped module under ``inner.``; with sharded master weights the fp32
        shards are gathered from their owners first (collective: every rank calls it)."""
        self.sync_master_weights()
        return super().state_dict(*args, **kw)

    def load_state_dict(self, state_dict, *args, **kw):
        out = super().load_state_dict(state_dict, *args, **kw)
        if getattr(self, "_use_native", False):
            self._refresh_shadow()      # the bf16 copies follow the loaded fp32 weights
            self._master_stale = False
        return out

    def check_guard_bands(self) -> int:
        """Debug aid (``FERRUM_GUARD_BANDS=1`` when the engine is built): verify that the pattern-filled bands
        around the parameter, gradient and bf16 regions of the arena are intact.  Returns the number of bands
        checked (0 when the feature is off); raises ``InternalError`` naming the band and the first damaged byte."""
        guards = getattr(self, "_guards", None) or []
        if guards:
            torch.cuda.synchronize()
        for name, band in guards:
            bad = (band != _GUARD_PATTERN).nonzero()
            if bad.numel():
                raise InternalError(f"guard band '{name}' of the gradient arena was overwritten at byte "
                                    f"{int(bad[0])} (value {int(band[int(bad[0])])}) on rank {self._pg.rank()}")
        return len(guards)

    def shutdown(self) -> None:
        """Release the arena (collective: every rank should call it after its last step) and hand the wrapped
        module back in a state in which it trains on its own: gradient sinks and hooks are removed."""
        for mod in getattr(self, "_sink_modules", []):
            mod.__dict__["grad_sink"] = None
        for h in getattr(self, "_hook_handles", []):
            h.remove()
        self._sink_modules, self._hook_handles = [], []
        opt = self._opt
        native = getattr(self, "_use_native", False) and getattr(self, "_arena", None) is not None
        if opt is not None and getattr(opt, "_engine", None) is self:
            state = None
            if native and self._state_m is not None:
                try:  # the moments return to the optimizer, which carries on unfused
                    state = self.export_optimizer_state(opt)
                except Exception:  # noqa: BLE001 - a peer is gone: the shards of the others cannot be fetched
                    state = None
            opt._engine = None
            if state:
                opt.load_state_tensors(state)
        if native:
            self.sync_master_weights()
            torch.cuda.synchronize()
            self.check_guard_bands()
            self._guards = []
            _gemm.set_gemm_cta_limit(0)
            try:
                self._pg.barrier()
            except Exception:
                pass
            for p in self._params:  # detach parameters from the arena before it is unmapped
                p.data = p.data.clone()
                p.grad = None
                p.__dict__.pop("_fb_shadow", None)
                p.__dict__.pop("_fb_shadow_key", None)
            self._flat_params = self._flat_grads = self._flat_shadow = None
            self._arena.close()
            self._arena = None
            self._use_native = False
