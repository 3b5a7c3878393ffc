"""Reverse-mode automatic differentiation API (ferrum-autograd).

The reference records a thread-local tape of backward callbacks (tape.rs:51-220,
graph.rs:18-208) and walks it in ``backward`` (backward.rs:35-118).  Here the
graph is torch's: every op of :mod:`ferrum_b200.ops.functional` is a
``torch.autograd.Function`` whose backward launches this package's kernels, and
the engine's topological walk replaces the hand-rolled DFS.  The tape object is
kept as the user-facing handle: it scopes recording, counts the operations that
were recorded and answers ``gradient(output, inputs)``.

Gradient formulas are the mathematically correct ones; the routing defects of the
reference's tape (wrong cells for leaf gradients, dropped gradients after scalar
ops) are not reproduced.
"""
from __future__ import annotations

import contextlib
import threading

import torch

from .core import AutogradError, Tensor, _unwrap

_tls = threading.local()


def is_grad_enabled() -> bool:
    return torch.is_grad_enabled()


def set_grad_enabled(flag: bool) -> None:
    torch.set_grad_enabled(flag)


# Names of the core hook layer (autograd_ops.rs:95-183).  The reference wires its tensor type to the tape through a
# thread-local pair of callbacks; with torch's engine underneath there is nothing to wire, so registration only
# keeps the callables (they are invoked by ``record_operation`` / ``execute_backward`` for code that drives the
# hooks by hand) and the enable switch maps onto torch's grad mode.
is_autograd_enabled = is_grad_enabled
set_autograd_enabled = set_grad_enabled
_id_lock = threading.Lock()
_next_tensor_id = [1]


def new_tensor_id() -> int:
    """Process-wide monotonically increasing tensor id (autograd_ops.rs:133-138)."""
    with _id_lock:
        v = _next_tensor_id[0]
        _next_tensor_id[0] += 1
        return v


class NodeId(int):
    """Identifier of a graph node (graph.rs:18-30); allocated from a global counter."""

    _counter = [0]

    @classmethod
    def new(cls) -> "NodeId":
        with _id_lock:
            cls._counter[0] += 1
            return cls(cls._counter[0])


def register_autograd_callbacks(record_fn, backward_fn) -> None:
    _tls.callbacks = (record_fn, backward_fn)


def unregister_autograd_callbacks() -> None:
    _tls.callbacks = None


def record_operation(*args, **kwargs):
    """Forward to the registered record callback, if any (autograd_ops.rs:140-161)."""
    cb = getattr(_tls, "callbacks", None)
    return cb[0](*args, **kwargs) if cb and cb[0] is not None and torch.is_grad_enabled() else None


def execute_backward(output):
    """Run the registered backward callback, or the engine's backward (autograd_ops.rs:163-183)."""
    cb = getattr(_tls, "callbacks", None)
    if cb and cb[1] is not None:
        return cb[1](output)
    return backward(output)


class NoGradGuard:
    """RAII-style guard: gradients are not recorded while it is alive (autograd_ops.rs:189-212)."""

    def __init__(self):
        self._prev = torch.is_grad_enabled()
        torch.set_grad_enabled(False)

    def release(self):
        if self._prev is not None:
            torch.set_grad_enabled(self._prev)
            self._prev = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()

    def __del__(self):
        self.release()


@contextlib.contextmanager
def _no_grad_cm():
    with torch.no_grad():
        yield


def no_grad(fn=None):
    """``with no_grad(): ...`` or ``no_grad(lambda: ...)`` (autograd_ops.rs:214-221)."""
    if fn is None:
        return _no_grad_cm()
    with torch.no_grad():
        return fn()


def _graph_nodes(root):
    seen, stack, order = set(), [root], []
    while stack:
        fn = stack.pop()
        if fn is None or fn in seen:
            continue
        seen.add(fn)
        order.append(fn)
        stack.extend(f for f, _ in fn.next_functions)
    return order


class Node:
    """Introspection view of one recorded operation (graph.rs:18-83)."""

    def __init__(self, grad_fn):
        self.grad_fn = grad_fn

    def name(self) -> str:
        return type(self.grad_fn).__name__.replace("Backward0", "Backward").lstrip("_")

    def inputs(self):
        return [Node(f) for f, _ in self.grad_fn.next_functions if f is not None]

    def __repr__(self):
        return f"Node({self.name()})"


class ComputationGraph:
    """The operations reachable from an output tensor (graph.rs:86-208)."""

    def __init__(self, output=None):
        self._root = None if output is None else _unwrap(output).grad_fn

    def nodes(self):
        return [Node(f) for f in _graph_nodes(self._root)] if self._root is not None else []

    def len(self) -> int:
        return len(self.nodes())

    __len__ = len

    def is_empty(self) -> bool:
        return self.len() == 0

    def clear(self) -> None:
        self._root = None


class GradientTape:
    """Recording scope (tape.rs:51-220): ``with_tape``, ``gradient``, ``stop`` / ``start``, ``no_grad``."""

    def __init__(self):
        self._recording = True
        self._outputs = []

    @classmethod
    def new(cls):
        return cls()

    def is_recording(self) -> bool:
        return self._recording

    def stop(self) -> None:
        self._recording = False
        torch.set_grad_enabled(False)

    def start(self) -> None:
        self._recording = True
        torch.set_grad_enabled(True)

    def no_grad(self, fn):
        with torch.no_grad():
            return fn()

    def watch(self, tensor: Tensor) -> Tensor:
        return tensor.set_requires_grad(True)

    def record(self, output) -> None:
        self._outputs.append(_unwrap(output))

    def gradient(self, output, inputs):
        """d(output)/d(input) for each input (None where there is no dependence)."""
        out = _unwrap(output)
        if out.numel() != 1:
            raise AutogradError(f"gradient() requires a scalar output, got shape {list(out.shape)}")
        ins = [_unwrap(t) for t in inputs]
        grads = torch.autograd.grad(out, ins, allow_unused=True, retain_graph=True)
        return [None if g is None else Tensor(g) for g in grads]

    def backward(self, output) -> None:
        backward(output)

    def len(self) -> int:
        n = 0
        for o in self._outputs:
            if o.grad_fn is not None:
                n += len(_graph_nodes(o.grad_fn))
        return n

    __len__ = len

    def is_empty(self) -> bool:
        return self.len() == 0

    def clear(self) -> None:
        self._outputs.clear()

    @staticmethod
    def current():
        return getattr(_tls, "tape", None)

    @staticmethod
    def with_tape(fn):
        """Run ``fn(tape)`` with recording enabled and this tape installed as the current one."""
        tape = GradientTape()
        prev = getattr(_tls, "tape", None)
        _tls.tape = tape
        try:
            with torch.enable_grad():
                return fn(tape)
        finally:
            _tls.tape = prev

    def __enter__(self):
        self._prev = getattr(_tls, "tape", None)
        self._cm = torch.enable_grad()
        self._cm.__enter__()
        _tls.tape = self
        return self

    def __exit__(self, *exc):
        _tls.tape = self._prev
        return self._cm.__exit__(*exc)

    def __repr__(self):
        return f"GradientTape(recording={self._recording}, ops={self.len()})"


def backward(output, graph: ComputationGraph | None = None) -> None:
    """Back-propagate from a scalar ``output`` into the ``.grad`` of every leaf that requires grad."""
    out = _unwrap(output)
    if out.numel() != 1:
        raise AutogradError(f"backward() requires a scalar output, got shape {list(out.shape)}")
    if not out.requires_grad:
        raise AutogradError("backward() called on a tensor that does not require grad")
    out.backward()


Function = torch.autograd.Function


class GradChecker:
    """Central-difference gradient check (backward.rs:185-280: eps 1e-5, rtol 1e-3, atol 1e-5)."""

    def __init__(self, eps: float = 1e-5, rtol: float = 1e-3, atol: float = 1e-5):
        self.eps, self.rtol, self.atol = eps, rtol, atol

    def numerical_gradient(self, fn, x):
        xt = _unwrap(x).detach().double().clone()
        g = torch.zeros_like(xt)
        flat, gf = xt.reshape(-1), g.reshape(-1)
        for i in range(flat.numel()):
            orig = flat[i].item()
            flat[i] = orig + self.eps
            fp = float(_unwrap(fn(Tensor(xt.clone()))).double().sum())
            flat[i] = orig - self.eps
            fm = float(_unwrap(fn(Tensor(xt.clone()))).double().sum())
            flat[i] = orig
            gf[i] = (fp - fm) / (2 * self.eps)
        return g

    def check(self, fn, x) -> bool:
        xt = _unwrap(x).detach().double().clone().requires_grad_(True)
        out = _unwrap(fn(Tensor(xt))).sum()
        (analytic,) = torch.autograd.grad(out, xt)
        numeric = self.numerical_gradient(fn, x)
        return bool(torch.allclose(analytic, numeric, rtol=self.rtol, atol=self.atol))


def check_gradients(fn, inputs, eps: float = 1e-4, rtol: float = 0.01, atol: float = 0.01, verbose: bool = False):
    """Compare analytic and numeric gradients for the first 100 elements (gradcheck.rs:45-158)."""
    ok = True
    report = []
    for x in inputs:
        xt = _unwrap(x).detach().double().clone().requires_grad_(True)
        out = _unwrap(fn(Tensor(xt))).sum()
        (an,) = torch.autograd.grad(out, xt)
        flat = xt.detach().reshape(-1)
        n = min(flat.numel(), 100)
        for i in range(n):
            orig = flat[i].item()
            flat[i] = orig + eps
            fp = float(_unwrap(fn(Tensor(flat.reshape(xt.shape).clone()))).sum())
            flat[i] = orig - eps
            fm = float(_unwrap(fn(Tensor(flat.reshape(xt.shape).clone()))).sum())
            flat[i] = orig
            num = (fp - fm) / (2 * eps)
            a = an.reshape(-1)[i].item()
            good = abs(a - num) <= atol + rtol * abs(num)
            ok &= good
            if verbose or not good:
                report.append((i, a, num, good))
    if verbose:
        for r in report:
            print("  elem %d analytic %.6f numeric %.6f %s" % (r[0], r[1], r[2], "ok" if r[3] else "MISMATCH"))
    return ok


def quick_gradcheck(fn, x) -> bool:
    return check_gradients(fn, [x])
