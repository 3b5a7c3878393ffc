"""ferrum_b200 — a Blackwell-native (NVIDIA B200, sm_100a) deep-learning framework with FERRUM's API surface.

Sub-packages mirror the reference's crates (facade: ferrum/src/lib.rs:67-134):
``core`` (Tensor / DType / Device / Shape / errors), ``autograd``, ``ops``, ``nn``, ``optim``, ``data``,
``distributed`` (= ``parallel``), ``serialize``, ``cuda`` and ``models``.  ``from ferrum_b200.prelude import *``
brings in the same names as ``ferrum::prelude``.
"""
from __future__ import annotations

__version__ = "0.1.0"

from . import config
from .config import autocast, matmul_precision
from .core import (AllocationError, ArithmeticError_, AutogradError, BroadcastError, Device, DeviceMismatch, DType,
                   DTypeMismatch, FerrumError, IndexOutOfBounds, InternalError, InvalidAxis, InvalidShape,
                   NonContiguous, NotImplemented_, ReshapeError, SerializationError, Shape, ShapeMismatch, Tensor,
                   UnsupportedDType, cuda_device_count, cuda_is_available)

from . import utils  # noqa: E402
from . import ops  # noqa: E402
from . import nn  # noqa: E402
from . import optim  # noqa: E402
from . import models  # noqa: E402
from . import autograd  # noqa: E402
from . import data  # noqa: E402
from . import serialize  # noqa: E402
from . import cuda  # noqa: E402
from . import kernels  # noqa: E402
from . import autograd_functions  # noqa: E402
from .storage import CpuAllocator, CudaAllocator, DeviceAllocator, Storage  # noqa: E402
from . import parallel  # noqa: E402
from . import parallel as distributed  # noqa: E402
from .autograd import GradientTape, NoGradGuard, backward, is_grad_enabled, no_grad  # noqa: E402
from .serialize import load, save  # noqa: E402



def manual_seed(seed: int) -> None:
    """Seed every random source the package draws from (the reference is unseeded: ferrum-core/src/tensor.rs:216):
    tensor factories, parameter initialisers and dropout take their streams from the torch generators."""
    import torch

    torch.manual_seed(int(seed))
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(int(seed))


Result = object  # Rust's Result<T> maps to "returns T or raises FerrumError"


def banner() -> str:
    """One-line description (ferrum/src/lib.rs:136-153)."""
    return (f"ferrum_b200 {__version__} — Blackwell-native deep learning framework "
            f"(CUDA available: {cuda_is_available()}, devices: {cuda_device_count()})")
