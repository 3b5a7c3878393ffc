"""Whole-step CUDA graphs: capture ``zero_grad -> forward -> backward -> optimizer.step`` once, replay it with one
launch per step.

Small models are bound by launch latency, not by the GPU (a 784-256-10 MLP step is a dozen kernels of a few
microseconds each); every launcher of this package enqueues on the current stream and takes its step-dependent
scalars either by value (constant over replays) or, for the optimizers in capturable mode, from device memory, so a
step can be recorded in a graph and replayed.  No tracing compiler is involved: the graph is the recorded launches.
"""
from __future__ import annotations

import torch

from ..core import Tensor, _unwrap


class GraphedStep:
    """``step = GraphedStep(fn, example_inputs, optimizer)``; ``loss = step(x, y)``.

    ``fn(*inputs)`` runs one full training step on device tensors and returns a tensor (typically the loss).  The
    inputs of every later call are copied into the static buffers the graph reads; the returned tensor is the
    graph's static output (read it, or copy it, before the next call).  ``optimizer`` is switched to capturable mode
    (device-side learning rate and bias corrections); ``optimizer.set_learning_rate`` keeps working between calls.
    Dropout draws its mask offset from a device-side counter from now on, so replays differ as they should.
    With the distributed engine (optimizer fused into the bucket reduction) the engine is switched to capturable
    mode too: handshake epochs come from a device counter, and every rank must record / replay the same steps.
    """

    def __init__(self, fn, example_inputs, optimizer=None, warmup: int = 3):
        if not torch.cuda.is_available():
            raise RuntimeError("GraphedStep needs a CUDA device")
        self._fn, self._opt = fn, optimizer
        if optimizer is not None:
            optimizer.capturable(True)
            engine = getattr(optimizer, "_engine", None)
            if engine is not None:  # fused into the distributed engine: its epochs move to the device as well
                engine.capturable(True)
        from ..ops import functional as _F

        _F.set_capturable_rng(True)  # dropout masks: device-side counter, a new mask at every replay
        self._wrapped = [isinstance(t, Tensor) for t in example_inputs]
        self._static_in = [_unwrap(t).detach().clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # eager warm-up: lazy state, scratch buffers and attributes get created here
            for _ in range(max(1, warmup)):
                self._call_fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self._steps_before = int(getattr(optimizer, "step_count", 0)) if optimizer is not None else 0
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            out = self._call_fn()
        self._out_wrapped = isinstance(out, Tensor)
        self._static_out = _unwrap(out)
        if optimizer is not None and hasattr(optimizer, "step_count"):
            optimizer.step_count = self._steps_before  # recording ran the Python of a step, not its kernels

    def _call_fn(self):
        args = [Tensor(t) if w else t for t, w in zip(self._static_in, self._wrapped)]
        return self._fn(*args)

    def __call__(self, *inputs):
        if len(inputs) != len(self._static_in):
            raise ValueError(f"expected {len(self._static_in)} inputs, got {len(inputs)}")
        for s, t in zip(self._static_in, inputs):
            s.copy_(_unwrap(t), non_blocking=True)
        self._graph.replay()
        if self._opt is not None and hasattr(self._opt, "step_count"):
            self._opt.step_count += 1  # host-side bookkeeping (checkpoints); the kernels use the device counter
        return Tensor(self._static_out) if self._out_wrapped else self._static_out

    @property
    def graph(self):
        return self._graph


class HostReadback:
    """Reads one small device tensor per step on the host without draining the GPU's queue.

    ``loss.item()`` right after a step waits for that step and leaves the GPU idle while the host prepares the
    next one.  ``push(t)`` instead enqueues a copy of ``t`` into pinned host memory behind the step that produced
    it; ``pop()`` returns the oldest value once its copy has landed.  Popping the value of step ``i - 1`` after
    step ``i`` has been launched keeps one step in the queue at all times; every step's value is still read.
    """

    def __init__(self, depth: int = 2, dtype: torch.dtype = torch.float32):
        self._slots = [torch.empty((), dtype=dtype).pin_memory() for _ in range(depth + 1)]
        self._events = [torch.cuda.Event() for _ in range(depth + 1)]
        self._head = self._count = 0

    def pending(self) -> int:
        return self._count

    def push(self, value) -> None:
        if self._count == len(self._slots):
            raise RuntimeError("HostReadback is full: pop() before pushing more")
        i = (self._head + self._count) % len(self._slots)
        self._slots[i].copy_(_unwrap(value).detach().reshape(()), non_blocking=True)
        self._events[i].record()
        self._count += 1

    def pop(self) -> float:
        if self._count == 0:
            raise RuntimeError("HostReadback is empty")
        i = self._head
        self._events[i].synchronize()
        self._head = (self._head + 1) % len(self._slots)
        self._count -= 1
        return float(self._slots[i])
