"""Process-wide numeric policy.

The reference trains in fp32 everywhere.  On a B200 the product path runs the
GEMMs on the bf16 tensor cores with fp32 accumulation and fp32 master weights;
that is opt-in so that parity runs keep exact fp32 arithmetic:

* ``matmul_precision("fp32")`` (default) — fp32 SIMT GEMM, bit-for-bit fp32 math.
* ``matmul_precision("tf32")`` — tensors stay fp32 but GEMMs run on the tensor cores as TF32 (tcgen05 kind::tf32:
  10-bit mantissa operands, fp32 accumulation), several times the SIMT rate at ~1e-3 relative error.
* ``matmul_precision("bf16")`` or ``with autocast():`` — tcgen05 GEMMs on bf16
  operands; activations flow in bf16, normalisation / softmax / loss statistics
  stay in fp32 inside the kernels.

Environment overrides: ``FERRUM_MATMUL_PRECISION`` (``fp32`` | ``tf32`` | ``bf16``).
"""
from __future__ import annotations

import contextlib
import os
import threading

import torch

_state = threading.local()
_default_precision = os.environ.get("FERRUM_MATMUL_PRECISION", "fp32").lower()


def matmul_precision(value: str | None = None) -> str:
    """Get or set the default GEMM precision (``"fp32"``, ``"tf32"`` or ``"bf16"``)."""
    global _default_precision
    if value is not None:
        value = value.lower()
        if value not in ("fp32", "tf32", "bf16"):
            raise ValueError("matmul precision must be 'fp32', 'tf32' or 'bf16'")
        _default_precision = value
    return _default_precision


def compute_dtype() -> torch.dtype:
    """The dtype GEMM-shaped ops should compute in right now."""
    stack = getattr(_state, "autocast", None)
    if stack:
        return stack[-1]
    return torch.bfloat16 if _default_precision == "bf16" else torch.float32


def low_precision_active() -> bool:
    return compute_dtype() == torch.bfloat16


def tf32_active() -> bool:
    """fp32 tensors, TF32 tensor-core GEMMs (only when no autocast block overrides the default)."""
    return _default_precision == "tf32" and not getattr(_state, "autocast", None)


@contextlib.contextmanager
def autocast(dtype=torch.bfloat16, enabled: bool = True):
    """Run GEMM-shaped ops in ``dtype`` (bf16) inside the block; fp32 elsewhere."""
    from .core import DType

    if isinstance(dtype, DType):
        dtype = dtype.to_torch()
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("autocast supports bf16 (or fp32 to switch it off)")
    stack = getattr(_state, "autocast", None)
    if stack is None:
        stack = _state.autocast = []
    stack.append(dtype if enabled else torch.float32)
    try:
        yield
    finally:
        stack.pop()
