"""``DataLoader`` (ferrum-data/src/dataloader.rs:13-190).

Builder-style configuration as in the reference (``batch_size`` / ``shuffle`` / ``drop_last`` /
``num_workers``).  A batch is, by default, the pair of stacked tensors the reference's README shows;
``collate(False)`` yields the reference's actual ``Vec<Sample>`` (a list).  For a dataset built from
stacked tensors the batch is fetched with one row-gather kernel on the device that holds the data;
``num_workers > 0`` fetches samples of map-style datasets on a thread pool.  ``pin_memory(True)``
together with ``to(device)`` stages batches in pinned host memory and copies them asynchronously.

A dataset of stacked HOST tensors with ``num_workers > 0`` takes the native path: the worker threads of the host
library (``csrc/host/loader.cpp``) gather the sampled rows into a ring of staging buffers a few batches ahead,
and with ``to(device)`` the loader itself copies batch ``i + 1`` to the GPU on a side stream while the caller
computes on batch ``i``.  ``repeat(True)`` runs epoch after epoch without draining that pipeline.
"""
from __future__ import annotations

import ctypes
from collections import deque
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch

from ..core import Tensor, _as_device, _unwrap
from .dataset import Dataset, TensorDataset
from .sampler import BatchSampler, RandomSampler, Sampler, SequentialSampler


def default_collate(samples):
    """Stack a list of samples field by field."""
    first = samples[0]
    if isinstance(first, (tuple, list)):
        return tuple(default_collate([s[i] for s in samples]) for i in range(len(first)))
    if isinstance(first, (Tensor, torch.Tensor)):
        return Tensor(torch.stack([_unwrap(s) for s in samples], 0))
    return Tensor(torch.as_tensor(samples))


class DataLoader:
    def __init__(self, dataset: Dataset, batch_size: int = 1, shuffle: bool = False, drop_last: bool = False,
                 num_workers: int = 0, sampler: Sampler | None = None, seed: int | None = None):
        self._dataset = dataset
        self._batch_size, self._shuffle, self._drop_last = int(batch_size), bool(shuffle), bool(drop_last)
        self._num_workers, self._sampler, self._seed = int(num_workers), sampler, seed
        self._collate = default_collate
        self._pin, self._device = False, None
        self._epoch = 0
        self._pool = None
        self._repeat = False
        self._native = None  # (handle, slot tensors, copy stream) of the native batch assembler, built on first use

    @classmethod
    def new(cls, dataset):
        return cls(dataset)

    # builder methods (each returns self)
    def batch_size(self, n: int) -> "DataLoader":
        self._batch_size = int(n)
        return self

    def shuffle(self, flag: bool) -> "DataLoader":
        self._shuffle = bool(flag)
        return self

    def drop_last(self, flag: bool) -> "DataLoader":
        self._drop_last = bool(flag)
        return self

    def num_workers(self, n: int) -> "DataLoader":
        self._num_workers = int(n)
        return self

    def sampler(self, s: Sampler) -> "DataLoader":
        self._sampler = s
        return self

    def seed(self, s: int) -> "DataLoader":
        self._seed = int(s)
        return self

    def collate(self, fn) -> "DataLoader":
        """``False``/``None`` = list of samples (the reference's behaviour); a callable = custom collation."""
        self._collate = fn if fn else None
        return self

    def pin_memory(self, flag: bool = True) -> "DataLoader":
        self._pin = bool(flag)
        return self

    def to(self, device) -> "DataLoader":
        self._device = _as_device(device).to_torch()
        return self

    def repeat(self, flag: bool = True) -> "DataLoader":
        """Iterate epoch after epoch without end (a new shuffle per epoch); batches keep being prepared across
        the epoch boundary."""
        self._repeat = bool(flag)
        return self

    def dataset(self) -> Dataset:
        return self._dataset

    def len(self) -> int:
        n = self._sampler.len() if self._sampler is not None else self._dataset.len()
        return n // self._batch_size if self._drop_last else -(-n // self._batch_size)

    __len__ = len

    def is_empty(self) -> bool:
        return self.len() == 0

    def _make_sampler(self) -> Sampler:
        if self._sampler is not None:
            self._sampler.reset()
            return self._sampler
        n = self._dataset.len()
        if self._shuffle:
            s = RandomSampler(n, None if self._seed is None else self._seed + self._epoch)
        else:
            s = SequentialSampler(n)
        return s

    def _move(self, t):
        if isinstance(t, tuple):
            return tuple(self._move(x) for x in t)
        if isinstance(t, Tensor) and self._device is not None and t._t.device != self._device:
            src = t._t
            if self._pin and not src.is_cuda and not src.is_pinned():
                src = src.pin_memory()
            return Tensor(src.to(self._device, non_blocking=True))
        return t

    # ------------------------------------------------------------------ native batch assembler
    _DEPTH = 3  # staging slots: one being copied to the device, one complete, one being gathered

    def _native_ok(self, ds) -> bool:
        return (self._num_workers > 0 and isinstance(ds, TensorDataset) and ds.stacked
                and self._collate is default_collate and not ds.inputs.is_cuda and not ds.targets.is_cuda
                and ds.inputs.is_contiguous() and ds.targets.is_contiguous() and ds.len() > 0)

    def _native_state(self, ds):
        if self._native is None:
            from .. import _lib

            to_gpu = self._device is not None and self._device.type == "cuda"
            pin = (self._pin or to_gpu) and torch.cuda.is_available()
            fields = (ds.inputs, ds.targets)
            slots = [[torch.empty((self._batch_size,) + tuple(f.shape[1:]), dtype=f.dtype, pin_memory=pin)
                      for f in fields] for _ in range(self._DEPTH)]
            src = (ctypes.c_void_p * 2)(*(f.data_ptr() for f in fields))
            rb = (ctypes.c_longlong * 2)(*(f.stride(0) * f.element_size() if f.dim() > 1 else f.element_size()
                                           for f in fields))
            ptrs = (ctypes.c_void_p * (2 * self._DEPTH))(*(t.data_ptr() for s in slots for t in s))
            h = _lib.host().fb_loader_create(2, src, rb, ds.len(), self._DEPTH, ptrs, self._num_workers)
            if not h:
                raise RuntimeError("fb_loader_create failed")
            stream = torch.cuda.Stream(device=self._device) if to_gpu else None
            self._native = (h, slots, stream)
        return self._native

    def close(self) -> None:
        """Stops the worker threads of the native batch assembler (also done when the loader is collected)."""
        if self._native is not None:
            from .. import _lib

            h, self._native = self._native[0], None
            _lib.host().fb_loader_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass

    def _iter_native(self, ds):
        from .. import _lib

        lib = _lib.host()
        h, slots, stream = self._native_state(ds)
        to_gpu = stream is not None
        state = {"bs": BatchSampler(self._make_sampler(), self._batch_size, self._drop_last)}
        self._epoch += 1
        pending = deque()                 # (slot, rows) handed to the workers, in order
        copied = [None] * self._DEPTH     # event after the device copy that last read the slot
        free = deque(range(self._DEPTH))

        def next_indices():
            idx = state["bs"].next_batch()
            if idx is None and self._repeat:
                state["bs"] = BatchSampler(self._make_sampler(), self._batch_size, self._drop_last)
                self._epoch += 1
                idx = state["bs"].next_batch()
            return idx

        def refill():
            while free:
                idx = next_indices()
                if idx is None:
                    return
                slot = free.popleft()
                if copied[slot] is not None:
                    copied[slot].synchronize()    # the copy that read this slot has finished (long ago, normally)
                    copied[slot] = None
                idx = np.ascontiguousarray(idx, dtype=np.int64)
                rc = lib.fb_loader_submit(h, slot, idx.ctypes.data, len(idx))
                if rc != 0:
                    raise RuntimeError(f"fb_loader_submit failed ({rc})")
                pending.append((slot, len(idx)))

        def stage():
            """The next finished slot as a batch: on the GPU path its copy is enqueued on the side stream."""
            if self._native is None or self._native[0] != h:
                raise RuntimeError("the DataLoader was closed while it was being iterated")
            refill()
            if not pending:
                return None
            slot, n = pending.popleft()
            rc = lib.fb_loader_wait(h, slot)
            if rc == -2:
                raise IndexError("sampler produced an index outside the dataset")
            views = [t[:n] for t in slots[slot]]
            if to_gpu:
                with torch.cuda.stream(stream):
                    dev = [v.to(self._device, non_blocking=True) for v in views]
                    ev = torch.cuda.Event()
                    ev.record(stream)
                copied[slot] = ev
                free.append(slot)
                return dev, ev
            out = [v.clone() for v in views]      # the slot is rewritten a few batches later
            free.append(slot)
            return out, None

        try:
            staged = stage()
            while staged is not None:
                cur, ev = staged
                staged = stage()                   # batch i + 1 is on its way before batch i is consumed
                if ev is not None:
                    consumer = torch.cuda.current_stream(self._device)
                    consumer.wait_event(ev)
                    for t in cur:
                        t.record_stream(consumer)
                yield Tensor(cur[0]), Tensor(cur[1])
        finally:
            # an abandoned iteration leaves slots in flight: wait for them so the ring can be reused
            # (not after close(): the workers and the handle are gone then)
            while pending and self._native is not None and self._native[0] == h:
                slot, _ = pending.popleft()
                lib.fb_loader_wait(h, slot)

    def iter(self):
        ds = self._dataset
        if self._native_ok(ds):
            yield from self._iter_native(ds)
            return
        bs = BatchSampler(self._make_sampler(), self._batch_size, self._drop_last)
        self._epoch += 1
        fast = isinstance(ds, TensorDataset) and ds.stacked and self._collate is default_collate
        while True:
            idx = bs.next_batch()
            if idx is None and self._repeat:
                bs = BatchSampler(self._make_sampler(), self._batch_size, self._drop_last)
                self._epoch += 1
                idx = bs.next_batch()
            if idx is None:
                return
            if fast:
                batch = ds.get_batch(idx)
            else:
                if self._num_workers > 0:
                    if self._pool is None:
                        self._pool = ThreadPoolExecutor(self._num_workers)
                    samples = list(self._pool.map(ds.get, idx.tolist()))
                else:
                    samples = [ds.get(int(i)) for i in idx]
                batch = self._collate(samples) if self._collate is not None else samples
            yield self._move(batch) if self._collate is not None else batch

    __iter__ = iter


class CollatedDataLoader:
    """Wraps a loader that yields sample lists with a collate function (dataloader.rs:169-190)."""

    def __init__(self, loader: DataLoader, collate_fn):
        self.loader, self.collate_fn = loader, collate_fn

    @classmethod
    def new(cls, loader, collate_fn):
        return cls(loader, collate_fn)

    def iter(self):
        prev = self.loader._collate
        self.loader._collate = None
        try:
            for samples in self.loader.iter():
                yield self.collate_fn(samples)
        finally:
            self.loader._collate = prev

    __iter__ = iter

    def len(self):
        return self.loader.len()


class DevicePrefetcher:
    """Wraps any iterable of batches (tensors or tuples / lists of tensors, ideally in pinned host memory) and hands
    them out on the GPU one step ahead: while the caller computes on batch ``i``, batch ``i + 1`` is already being
    copied on a side stream, so the host-to-device copy is off the critical path of the step.

    The reference's loader fetches a batch synchronously when it is asked for it
    (ferrum-data/src/dataloader.rs:144-165); on a GPU that serialises a PCIe copy with every step.
    """

    def __init__(self, batches, device=None):
        self._it = iter(batches)
        self._device = _as_device(device if device is not None else "cuda").to_torch()
        self._stream = torch.cuda.Stream(device=self._device)
        self._next = None
        self._preload()

    def _to_device(self, obj):
        if isinstance(obj, Tensor):
            return Tensor(obj._t.to(self._device, non_blocking=True))
        if isinstance(obj, torch.Tensor):
            return obj.to(self._device, non_blocking=True)
        if isinstance(obj, (tuple, list)):
            return type(obj)(self._to_device(o) for o in obj)
        return obj

    def _preload(self) -> None:
        try:
            batch = next(self._it)
        except StopIteration:
            self._next = None
            return
        with torch.cuda.stream(self._stream):
            self._next = self._to_device(batch)

    @staticmethod
    def _record(obj, stream) -> None:
        if isinstance(obj, Tensor):
            obj = obj._t
        if isinstance(obj, torch.Tensor):
            if obj.is_cuda:
                obj.record_stream(stream)
        elif isinstance(obj, (tuple, list)):
            for o in obj:
                DevicePrefetcher._record(o, stream)

    def __iter__(self):
        return self

    def __next__(self):
        if self._next is None:
            raise StopIteration
        cur = torch.cuda.current_stream(self._device)
        cur.wait_stream(self._stream)      # the copy of this batch is complete before the step reads it
        batch = self._next
        self._record(batch, cur)           # its memory is not reused while the step is still running
        self._preload()                    # start copying the following batch
        return batch
