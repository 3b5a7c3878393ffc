"""Tracing and metrics (the reference has none: a search of its sources shows only ``name()`` strings and a simulated
``CudaEvent::elapsed_time``).

``profile()``    context manager that times every native kernel launcher with CUDA events on the launching stream
                 and wraps it in an NVTX range named after the entry point; ``report()`` aggregates per kernel.
``StepTimer``    per-step throughput meter emitting JSON lines: samples/s, ms/step, optional achieved TFLOP/s and
                 roofline fractions against the measured peaks file when it exists.
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from collections import defaultdict

import torch

from .. import _lib


class _TimedLib:
    def __init__(self, inner, records, use_nvtx):
        self._inner, self._records, self._nvtx = inner, records, use_nvtx

    def __getattr__(self, name):
        fn = getattr(self._inner, name)
        if name.startswith(("fb_rt_", "fb_reduce_scratch", "fb_layernorm_bwd_blocks", "fb_dist_query", "fb_symm_")):
            return fn

        def timed(*args):
            if self._nvtx:
                torch.cuda.nvtx.range_push(name)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(*args)
            e1.record()
            if self._nvtx:
                torch.cuda.nvtx.range_pop()
            self._records.append((name, e0, e1))
            return rc

        return timed


class Profile:
    def __init__(self):
        self.records = []

    def report(self) -> dict:
        """{entry point: {"calls", "total_ms", "mean_us"}} sorted by total time (synchronizes)."""
        torch.cuda.synchronize()
        agg = defaultdict(lambda: [0, 0.0])
        for name, e0, e1 in self.records:
            agg[name][0] += 1
            agg[name][1] += e0.elapsed_time(e1)
        out = {k: {"calls": c, "total_ms": t, "mean_us": 1e3 * t / c} for k, (c, t) in agg.items()}
        return dict(sorted(out.items(), key=lambda kv: -kv[1]["total_ms"]))

    def table(self) -> str:
        rep = self.report()
        tot = sum(v["total_ms"] for v in rep.values()) or 1.0
        lines = [f"{'kernel entry point':34s} {'calls':>6s} {'total ms':>10s} {'mean us':>9s} {'share':>6s}"]
        for k, v in rep.items():
            lines.append(f"{k:34s} {v['calls']:6d} {v['total_ms']:10.3f} {v['mean_us']:9.1f} "
                         f"{100 * v['total_ms'] / tot:5.1f}%")
        return "\n".join(lines)


@contextlib.contextmanager
def profile(nvtx: bool = True):
    """Time every kernel launcher called inside the block."""
    prof = Profile()
    real = _lib.cuda()
    _lib._cuda = _TimedLib(real, prof.records, nvtx)
    try:
        yield prof
    finally:
        _lib._cuda = real


def measured_peaks() -> dict | None:
    """The driver-written hardware peaks (HBM GB/s, bf16 TFLOP/s) when the file exists at the repository root."""
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                     "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f)
    return None


class StepTimer:
    """``with timer.step(batch): ...`` — emits one JSON line every ``every`` steps: samples/s, ms/step, with
    ``flops_per_sample`` the TFLOP/s and the fraction of the measured sustained tensor-core rate, and with
    ``engine`` (a ``DistributedDataParallel`` in ``comm_profile`` mode) the communication record of the last
    step: bucket count, kernel time per bucket, achieved all-reduce bus GB/s and the exposed tail after backward."""

    def __init__(self, every: int = 10, flops_per_sample: float | None = None, sink=print, engine=None):
        self.every, self.flops, self.sink = every, flops_per_sample, sink
        self.engine = engine
        if engine is not None:
            engine.comm_profile(True)
        self._n = self._samples = 0
        self._t0 = None
        self.history = []

    @contextlib.contextmanager
    def step(self, batch_size: int):
        if self._t0 is None:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self._t0 = time.perf_counter()
        yield
        self._n += 1
        self._samples += batch_size
        if self._n % self.every == 0:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            dt = time.perf_counter() - self._t0
            rec = {"steps": self._n, "samples_per_s": self._samples / dt, "ms_per_step": 1e3 * dt / self.every}
            if self.flops:
                rec["tflops"] = self.flops * self._samples / dt / 1e12
                pk = measured_peaks()
                if pk:
                    rec["frac_of_measured_bf16_sustained"] = rec["tflops"] / pk["bf16_tflops_sustained"]
            comm = self.engine.last_comm_profile() if self.engine is not None else None
            if comm and comm["buckets"]:
                us = [b["kernel_us"] for b in comm["buckets"]]
                nbytes = sum(b["bytes"] for b in comm["buckets"])
                rec["comm"] = {"buckets": len(us), "bucket_kernel_us": [round(u, 1) for u in us],
                               "comm_busy_us": round(comm["comm_busy_us"], 1),
                               "bus_gbs": round(sum(b["bus_gbs"] * b["bytes"] for b in comm["buckets"]) / nbytes, 1),
                               "exposed_tail_us": round(comm["exposed_tail_us"], 1)}
            self.history.append(rec)
            self.sink(json.dumps(rec))
            self._samples, self._t0 = 0, time.perf_counter()
