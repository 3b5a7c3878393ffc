"""Core value types: ``DType``, ``Device``, ``Shape``, the error hierarchy and ``Tensor``.

API parity with ferrum-core (dtype.rs:31-114, device.rs:32-115, shape.rs:51-442,
error.rs:21-140, tensor.rs:72-2656).  ``Tensor`` is a thin handle around a
``torch.Tensor``; every differentiable method forwards to
:mod:`ferrum_b200.ops.functional`, which runs this package's sm_100a kernels
for CUDA tensors and plain torch ops on the CPU.  Unlike the reference,
``Device.Cuda(i)`` really holds data, and there is one tensor type for both
devices.
"""
from __future__ import annotations

import enum
import math
from typing import Iterable, Sequence

import torch


# --------------------------------------------------------------------------- errors
class FerrumError(Exception):
    """Base class; subclasses mirror the variants of ferrum-core/src/error.rs:21-110."""


class ShapeMismatch(FerrumError):
    def __init__(self, operation, expected, actual):
        super().__init__(f"Shape mismatch: {operation} expects {expected}, got {actual}")


class BroadcastError(FerrumError):
    def __init__(self, lhs, rhs):
        super().__init__(f"Cannot broadcast shapes {list(lhs)} and {list(rhs)}")


class DTypeMismatch(FerrumError):
    def __init__(self, operation, expected, actual):
        super().__init__(f"DType mismatch: {operation} expects {expected}, got {actual}")


class UnsupportedDType(FerrumError):
    def __init__(self, operation, dtype):
        super().__init__(f"Operation '{operation}' not supported for dtype {dtype}")


class DeviceMismatch(FerrumError):
    def __init__(self, operation, d1, d2):
        super().__init__(f"Device mismatch: {operation} requires tensors on same device, got {d1} and {d2}")


class InvalidAxis(FerrumError):
    def __init__(self, axis, ndim):
        super().__init__(f"Invalid axis {axis} for tensor with {ndim} dimensions")


class IndexOutOfBounds(FerrumError):
    def __init__(self, index, dim, size):
        super().__init__(f"Index {index} out of bounds for dimension {dim} with size {size}")


class InvalidShape(FerrumError):
    def __init__(self, message):
        super().__init__(f"Invalid shape: {message}")


class ReshapeError(FerrumError):
    def __init__(self, src_numel, target, target_numel):
        super().__init__(
            f"Cannot reshape tensor with {src_numel} elements to shape {list(target)} ({target_numel} elements)")


class NonContiguous(FerrumError):
    def __init__(self, operation):
        super().__init__(f"Operation '{operation}' requires contiguous storage")


class ArithmeticError_(FerrumError):
    def __init__(self, operation, message):
        super().__init__(f"Arithmetic error in '{operation}': {message}")


class AllocationError(FerrumError):
    def __init__(self, nbytes, device):
        super().__init__(f"Failed to allocate {nbytes} bytes on {device}")


class InternalError(FerrumError):
    def __init__(self, message):
        super().__init__(f"Internal error: {message}. This is a bug, please report it.")


class NotImplemented_(FerrumError):
    def __init__(self, feature):
        super().__init__(f"Not implemented: {feature}")


class AutogradError(FerrumError):
    def __init__(self, message):
        super().__init__(f"Autograd error: {message}")


class SerializationError(FerrumError):
    def __init__(self, message):
        super().__init__(f"Serialization error: {message}")


# --------------------------------------------------------------------------- dtype
class DType(enum.IntEnum):
    """Element types; the integer values are part of the checkpoint format (dtype.rs:31-40)."""

    F32 = 0
    F64 = 1
    F16 = 2
    BF16 = 3
    I32 = 4
    I64 = 5
    U8 = 6
    Bool = 7

    def size_of(self) -> int:
        return _DTYPE_SIZE[self]

    def supports_grad(self) -> bool:
        return self.is_float()

    def is_float(self) -> bool:
        return self in (DType.F32, DType.F64, DType.F16, DType.BF16)

    def is_integer(self) -> bool:
        return self in (DType.I32, DType.I64, DType.U8)

    def is_signed(self) -> bool:
        return self not in (DType.U8, DType.Bool)

    @staticmethod
    def default_float() -> "DType":
        return DType.F32

    @staticmethod
    def default_int() -> "DType":
        return DType.I64

    def to_torch(self) -> torch.dtype:
        return _TO_TORCH[self]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DType":
        try:
            return _FROM_TORCH[dt]
        except KeyError:
            raise UnsupportedDType("from_torch", dt) from None

    def __str__(self) -> str:
        return self.name.lower()

    def __call__(self):  # lets ``tensor.dtype()`` work like the reference's method
        return self


_DTYPE_SIZE = {DType.F32: 4, DType.F64: 8, DType.F16: 2, DType.BF16: 2, DType.I32: 4, DType.I64: 8, DType.U8: 1,
               DType.Bool: 1}
_TO_TORCH = {DType.F32: torch.float32, DType.F64: torch.float64, DType.F16: torch.float16,
             DType.BF16: torch.bfloat16, DType.I32: torch.int32, DType.I64: torch.int64, DType.U8: torch.uint8,
             DType.Bool: torch.bool}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


def _as_dtype(d) -> DType:
    if isinstance(d, DType):
        return d
    if isinstance(d, torch.dtype):
        return DType.from_torch(d)
    if d is None:
        return DType.F32
    raise TypeError(f"not a dtype: {d!r}")


# --------------------------------------------------------------------------- device
class Device:
    """``Device.Cpu``, ``Device.Cuda(i)``, ``Device.Metal(i)`` (device.rs:32-115)."""

    __slots__ = ("kind", "idx")
    Cpu: "Device"

    def __init__(self, kind: str = "cpu", idx: int = 0):
        if kind not in ("cpu", "cuda", "metal"):
            raise ValueError(kind)
        self.kind, self.idx = kind, int(idx)

    @staticmethod
    def Cuda(idx: int = 0) -> "Device":
        return Device("cuda", idx)

    @staticmethod
    def Metal(idx: int = 0) -> "Device":
        return Device("metal", idx)

    @staticmethod
    def default() -> "Device":
        return Device.Cpu

    def is_cpu(self) -> bool:
        return self.kind == "cpu"

    def is_cuda(self) -> bool:
        return self.kind == "cuda"

    def is_metal(self) -> bool:
        return self.kind == "metal"

    def is_gpu(self) -> bool:
        return self.kind != "cpu"

    def index(self):
        return None if self.kind == "cpu" else self.idx

    def to_torch(self) -> torch.device:
        if self.kind == "cpu":
            return torch.device("cpu")
        if self.kind == "cuda":
            return torch.device("cuda", self.idx)
        raise NotImplemented_("Metal devices")

    @staticmethod
    def from_torch(d) -> "Device":
        d = torch.device(d)
        if d.type == "cpu":
            return Device.Cpu
        if d.type == "cuda":
            return Device("cuda", d.index or 0)
        raise NotImplemented_(f"device {d}")

    def __eq__(self, other):
        return isinstance(other, Device) and (self.kind, self.idx if self.kind != "cpu" else 0) == (
            other.kind, other.idx if other.kind != "cpu" else 0)

    def __hash__(self):
        return hash((self.kind, self.idx if self.kind != "cpu" else 0))

    def __str__(self):
        return "cpu" if self.kind == "cpu" else f"{self.kind}:{self.idx}"

    __repr__ = __str__

    def __call__(self):
        return self


Device.Cpu = Device("cpu")


def cuda_is_available() -> bool:
    return torch.cuda.is_available()


def cuda_device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _as_device(d) -> Device:
    if isinstance(d, Device):
        return d
    if d is None:
        return Device.Cpu
    return Device.from_torch(d)


# --------------------------------------------------------------------------- shape
class Shape(tuple):
    """Immutable dimension list with the helpers of shape.rs:51-442.

    It is a tuple (so it compares equal to tuples and unpacks), and calling it
    returns itself so both ``t.shape`` and the reference's ``t.shape()`` work.
    """

    def __new__(cls, dims: Iterable[int] = ()):
        if isinstance(dims, int):
            dims = (dims,)
        dims = tuple(int(d) for d in dims)
        if any(d < 0 for d in dims):
            raise InvalidShape(f"negative dimension in {list(dims)}")
        return super().__new__(cls, dims)

    @staticmethod
    def scalar() -> "Shape":
        return Shape(())

    @staticmethod
    def from_slice(dims) -> "Shape":
        return Shape(dims)

    def __call__(self):
        return self

    def dims(self):
        return list(self)

    def ndim(self) -> int:
        return len(self)

    def is_scalar(self) -> bool:
        return len(self) == 0

    def numel(self) -> int:
        return math.prod(self)

    def normalize_dim(self, dim: int) -> int:
        n = len(self)
        if dim < -n or dim >= n:
            raise InvalidAxis(dim, n)
        return dim + n if dim < 0 else dim

    def dim(self, i: int) -> int:
        return self[self.normalize_dim(i)]

    def strides_contiguous(self):
        s, acc = [], 1
        for d in reversed(self):
            s.append(acc)
            acc *= d
        return list(reversed(s))

    def is_contiguous(self, strides: Sequence[int]) -> bool:
        return list(strides) == self.strides_contiguous()

    def broadcast(self, other) -> "Shape":
        a, b = list(self), list(other)
        n = max(len(a), len(b))
        a = [1] * (n - len(a)) + a
        b = [1] * (n - len(b)) + b
        out = []
        for x, y in zip(a, b):
            if x == y or y == 1:
                out.append(x)
            elif x == 1:
                out.append(y)
            else:
                raise BroadcastError(self, other)
        return Shape(out)

    def broadcast_strides(self, strides: Sequence[int], target) -> list:
        """Strides that view this shape as ``target`` (0 on broadcast dimensions)."""
        t = list(target)
        pad = len(t) - len(self)
        if pad < 0:
            raise BroadcastError(self, target)
        out = [0] * pad
        for d, s, td in zip(self, strides, t[pad:]):
            if d == td:
                out.append(s)
            elif d == 1:
                out.append(0)
            else:
                raise BroadcastError(self, target)
        return out

    def can_reshape_to(self, other) -> bool:
        return self.numel() == Shape(other).numel()

    def transpose(self, perm: Sequence[int]) -> "Shape":
        if sorted(perm) != list(range(len(self))):
            raise InvalidShape(f"invalid permutation {list(perm)} for {len(self)} dimensions")
        return Shape(self[p] for p in perm)

    def unsqueeze(self, dim: int) -> "Shape":
        n = len(self)
        if dim < -(n + 1) or dim > n:
            raise InvalidAxis(dim, n)
        if dim < 0:
            dim += n + 1
        d = list(self)
        d.insert(dim, 1)
        return Shape(d)

    def squeeze(self, dim: int | None = None) -> "Shape":
        if dim is None:
            return Shape(d for d in self if d != 1)
        i = self.normalize_dim(dim)
        d = list(self)
        if d[i] == 1:
            d.pop(i)
        return Shape(d)

    def __str__(self):
        return "[" + ", ".join(str(d) for d in self) + "]"

    def __repr__(self):
        return f"Shape({list(self)})"


def _as_shape(s) -> Shape:
    if isinstance(s, Shape):
        return s
    if isinstance(s, int):
        return Shape((s,))
    if s is None:
        return Shape(())
    return Shape(s)


# --------------------------------------------------------------------------- tensor
_tensor_id_counter = 0


def new_tensor_id() -> int:
    global _tensor_id_counter
    _tensor_id_counter += 1
    return _tensor_id_counter


def _unwrap(x):
    return x._t if isinstance(x, Tensor) else x


class Tensor:
    """N-dimensional array on ``Device.Cpu`` or ``Device.Cuda(i)`` (ferrum-core/src/tensor.rs)."""

    __slots__ = ("_t", "tensor_id", "__weakref__")
    __array_priority__ = 100

    def __init__(self, t: torch.Tensor, tensor_id: int | None = None):
        if isinstance(t, Tensor):
            t = t._t
        if not isinstance(t, torch.Tensor):
            t = torch.as_tensor(t)
        self._t = t
        self.tensor_id = new_tensor_id() if tensor_id is None else tensor_id

    # ------------------------------------------------------------ constructors (tensor.rs:100-643)
    @staticmethod
    def _factory(fn, shape, dtype, device, **kw):
        return Tensor(fn(tuple(_as_shape(shape)), dtype=_as_dtype(dtype).to_torch(),
                         device=_as_device(device).to_torch(), **kw))

    @staticmethod
    def zeros(shape, dtype=DType.F32, device=None):
        return Tensor._factory(torch.zeros, shape, dtype, device)

    @staticmethod
    def ones(shape, dtype=DType.F32, device=None):
        return Tensor._factory(torch.ones, shape, dtype, device)

    @staticmethod
    def full(shape, value, dtype=DType.F32, device=None):
        return Tensor(torch.full(tuple(_as_shape(shape)), value, dtype=_as_dtype(dtype).to_torch(),
                                 device=_as_device(device).to_torch()))

    @staticmethod
    def uninit(shape, dtype=DType.F32, device=None):
        return Tensor._factory(torch.empty, shape, dtype, device)

    @staticmethod
    def from_slice(data, shape=None, device=None, dtype=None):
        t = torch.as_tensor(data)
        if dtype is not None:
            t = t.to(_as_dtype(dtype).to_torch())
        elif t.dtype == torch.float64 and not isinstance(data, torch.Tensor):
            t = t.to(torch.float32)  # Python floats are f32 data in the reference's examples
        if shape is not None:
            shp = _as_shape(shape)
            if shp.numel() != t.numel():
                raise ShapeMismatch("from_slice", f"{shp.numel()} elements", f"{t.numel()} elements")
            t = t.reshape(tuple(shp))
        return Tensor(t.to(_as_device(device).to_torch()).contiguous())

    from_vec = from_slice

    @staticmethod
    def randn(shape, dtype=DType.F32, device=None, generator=None):
        return Tensor(torch.randn(tuple(_as_shape(shape)), dtype=_as_dtype(dtype).to_torch(),
                                  device=_as_device(device).to_torch(), generator=generator))

    @staticmethod
    def normal(shape, mean=0.0, std=1.0, dtype=DType.F32, device=None, generator=None):
        t = Tensor.randn(shape, dtype, device, generator)._t
        return Tensor(t.mul_(std).add_(mean))

    @staticmethod
    def uniform(shape, low=0.0, high=1.0, dtype=DType.F32, device=None, generator=None):
        t = torch.rand(tuple(_as_shape(shape)), dtype=_as_dtype(dtype).to_torch(),
                       device=_as_device(device).to_torch(), generator=generator)
        return Tensor(t.mul_(high - low).add_(low))

    @staticmethod
    def eye(n, dtype=DType.F32, device=None):
        return Tensor(torch.eye(n, dtype=_as_dtype(dtype).to_torch(), device=_as_device(device).to_torch()))

    @staticmethod
    def arange(start, end=None, step=1, dtype=DType.F32, device=None):
        if end is None:
            start, end = 0, start
        if step == 0:
            raise InvalidShape("arange step must be non-zero")
        return Tensor(torch.arange(start, end, step, dtype=_as_dtype(dtype).to_torch(),
                                   device=_as_device(device).to_torch()))

    @staticmethod
    def linspace(start, end, steps, dtype=DType.F32, device=None):
        return Tensor(torch.linspace(start, end, steps, dtype=_as_dtype(dtype).to_torch(),
                                     device=_as_device(device).to_torch()))

    @staticmethod
    def cat(tensors, dim=0):
        from .ops import functional as F

        if not tensors:
            raise InvalidShape("cat of an empty list")
        return Tensor(F.cat([_unwrap(t) for t in tensors], dim))

    @staticmethod
    def stack(tensors, dim=0):
        from .ops import functional as F

        if not tensors:
            raise InvalidShape("stack of an empty list")
        return Tensor(F.cat([_unwrap(t).unsqueeze(dim) for t in tensors], dim))

    # ------------------------------------------------------------ properties (tensor.rs:649-716)
    @property
    def shape(self) -> Shape:
        return Shape(self._t.shape)

    def shape_obj(self) -> Shape:
        return self.shape

    def ndim(self) -> int:
        return self._t.dim()

    def numel(self) -> int:
        return self._t.numel()

    def strides(self):
        return list(self._t.stride())

    @property
    def dtype(self) -> DType:
        return DType.from_torch(self._t.dtype)

    @property
    def device(self) -> Device:
        return Device.from_torch(self._t.device)

    def requires_grad(self) -> bool:
        return self._t.requires_grad

    def size(self, dim: int) -> int:
        return self.shape.dim(dim)

    def is_contiguous(self) -> bool:
        return self._t.is_contiguous()

    def is_scalar(self) -> bool:
        return self._t.dim() == 0

    def storage_ref_count(self) -> int:
        import sys

        return max(1, sys.getrefcount(self._t.untyped_storage()) - 1)

    def torch(self) -> torch.Tensor:
        """The underlying ``torch.Tensor`` (shares storage)."""
        return self._t

    # ------------------------------------------------------------ grad API (tensor.rs:722-786)
    def set_requires_grad(self, flag: bool = True) -> "Tensor":
        if flag and not self.dtype.is_float():
            raise UnsupportedDType("set_requires_grad", self.dtype)
        if self._t.is_leaf:
            self._t.requires_grad_(flag)
        elif flag != self._t.requires_grad:
            self._t = self._t.detach().requires_grad_(flag)
        return self

    def with_requires_grad(self, flag: bool = True) -> "Tensor":
        return self.set_requires_grad(flag)

    requires_grad_ = set_requires_grad

    def grad(self):
        g = self._t.grad
        return None if g is None else Tensor(g)

    def set_grad(self, grad) -> None:
        self._t.grad = None if grad is None else _unwrap(grad)

    def zero_grad(self) -> None:
        self._t.grad = None

    def accumulate_grad(self, grad) -> None:
        g = _unwrap(grad)
        if self._t.grad is None:
            self._t.grad = g.detach().clone()
        else:
            self._t.grad.add_(g)

    def detach(self) -> "Tensor":
        return Tensor(self._t.detach())

    def backward(self, gradient=None, retain_graph: bool = False) -> None:
        """Reverse-mode differentiation from a scalar (autograd_ops.rs:227-249)."""
        if gradient is None and self._t.numel() != 1:
            raise AutogradError(f"backward() requires a scalar output, got shape {self.shape}")
        if not self._t.requires_grad:
            raise AutogradError("backward() called on a tensor that does not require grad")
        self._t.backward(_unwrap(gradient) if gradient is not None else None, retain_graph=retain_graph)

    # ------------------------------------------------------------ views (tensor.rs:793-1083)
    def _view(self, t: torch.Tensor) -> "Tensor":
        return Tensor(t, self.tensor_id)

    def reshape(self, *shape) -> "Tensor":
        if len(shape) == 1 and not isinstance(shape[0], int):
            shape = tuple(shape[0])
        shape = list(shape)
        if -1 in shape:
            known = math.prod(d for d in shape if d != -1)
            if shape.count(-1) > 1 or known == 0 or self.numel() % known:
                raise ReshapeError(self.numel(), shape, known)
            shape[shape.index(-1)] = self.numel() // known
        if math.prod(shape) != self.numel():
            raise ReshapeError(self.numel(), shape, math.prod(shape))
        return self._view(self._t.reshape(shape))

    view = reshape

    def flatten(self) -> "Tensor":
        return self._view(self._t.reshape(-1))

    def contiguous(self) -> "Tensor":
        return self if self._t.is_contiguous() else Tensor(self._t.contiguous())

    def transpose(self, dim0: int, dim1: int) -> "Tensor":
        s = self.shape
        return self._view(self._t.transpose(s.normalize_dim(dim0), s.normalize_dim(dim1)))

    def t(self) -> "Tensor":
        if self._t.dim() != 2:
            raise InvalidShape(f"t() expects a 2-D tensor, got {self._t.dim()} dimensions")
        return self._view(self._t.t())

    def permute(self, *dims) -> "Tensor":
        if len(dims) == 1 and not isinstance(dims[0], int):
            dims = tuple(dims[0])
        self.shape.transpose([self.shape.normalize_dim(d) for d in dims])
        return self._view(self._t.permute(*dims))

    def unsqueeze(self, dim: int) -> "Tensor":
        self.shape.unsqueeze(dim)
        return self._view(self._t.unsqueeze(dim))

    def squeeze(self, dim: int | None = None) -> "Tensor":
        if dim is None:
            return self._view(self._t.squeeze())
        return self._view(self._t.squeeze(self.shape.normalize_dim(dim)))

    def expand(self, *shape) -> "Tensor":
        if len(shape) == 1 and not isinstance(shape[0], int):
            shape = tuple(shape[0])
        try:
            return self._view(self._t.expand(*shape))
        except RuntimeError:
            raise BroadcastError(self.shape, shape) from None

    def narrow(self, dim: int, start: int, length: int) -> "Tensor":
        d = self.shape.normalize_dim(dim)
        if start < 0 or start + length > self.shape[d]:
            raise IndexOutOfBounds(start + length, d, self.shape[d])
        return Tensor(self._t.narrow(d, start, length))

    def __getitem__(self, idx):
        return Tensor(self._t[_unwrap(idx)])

    # ------------------------------------------------------------ data access (tensor.rs:1089-1240)
    def item(self):
        if self._t.numel() != 1:
            raise InvalidShape(f"item() requires a single-element tensor, got shape {self.shape}")
        return self._t.item()

    def to_vec(self):
        return self._t.detach().reshape(-1).tolist()

    # raw access in the vocabulary of the reference's GPU tensor (ferrum-cuda/src/tensor.rs:120-159)
    def ptr(self) -> int:
        """Address of the first element (device address for a tensor on ``Device.Cuda``)."""
        return self._t.data_ptr()

    def size_bytes(self) -> int:
        return self._t.numel() * self._t.element_size()

    def to_host(self) -> bytes:
        """The elements, in logical order, as raw bytes in host memory."""
        return self._t.detach().contiguous().cpu().reshape(-1).view(torch.uint8).numpy().tobytes()

    def to_f32(self) -> list:
        """The elements converted to fp32, as a host list."""
        return self._t.detach().to(torch.float32).reshape(-1).tolist()

    def to_f64(self) -> list:
        return self._t.detach().to(torch.float64).reshape(-1).tolist()

    tolist = to_vec

    def numpy(self):
        return self._t.detach().cpu().numpy()

    def to_dtype(self, dtype) -> "Tensor":
        from .ops import functional as F

        return Tensor(F.cast(self._t, _as_dtype(dtype).to_torch()))

    def to_device(self, device) -> "Tensor":
        dev = _as_device(device)
        if dev.is_metal():
            raise NotImplemented_("Metal devices")
        if dev.is_cuda() and not torch.cuda.is_available():
            raise AllocationError(self.numel() * self.dtype.size_of(), dev)
        return Tensor(self._t.to(dev.to_torch()))

    to = to_device

    def cuda(self, idx: int = 0) -> "Tensor":
        return self.to_device(Device.Cuda(idx))

    def cpu(self) -> "Tensor":
        return self.to_device(Device.Cpu)

    def clone(self) -> "Tensor":
        return Tensor(self._t.clone())

    # ------------------------------------------------------------ arithmetic (tensor.rs:1247-1466)
    def _bin(self, other, op: str) -> "Tensor":
        from .ops import functional as F

        o = _unwrap(other)
        if not isinstance(o, torch.Tensor):
            return Tensor(F.scalar_op(self._t, op, float(o)))
        if o.device != self._t.device:
            raise DeviceMismatch(op, self.device, Device.from_torch(o.device))
        try:
            self.shape.broadcast(o.shape)
        except BroadcastError:
            raise
        return Tensor(F.binary(self._t, o, op))

    def add(self, other):
        return self._bin(other, "add")

    def sub(self, other):
        return self._bin(other, "sub")

    def mul(self, other):
        return self._bin(other, "mul")

    def div(self, other):
        return self._bin(other, "div")

    def maximum(self, other):
        return self._bin(other, "max")

    def minimum(self, other):
        return self._bin(other, "min")

    def add_scalar(self, s: float):
        from .ops import functional as F

        return Tensor(F.scalar_op(self._t, "add", float(s)))

    def mul_scalar(self, s: float):
        from .ops import functional as F

        return Tensor(F.scalar_op(self._t, "mul", float(s)))

    def sub_scalar(self, s: float):
        return self.add_scalar(-float(s))

    def div_scalar(self, s: float):
        return self.mul_scalar(1.0 / float(s))

    __add__ = add
    __sub__ = sub
    __mul__ = mul
    __truediv__ = div

    def __radd__(self, other):
        return self.add(other)

    def __rmul__(self, other):
        return self.mul(other)

    def __rsub__(self, other):
        from .ops import functional as F

        return Tensor(F.scalar_op(self._t, "rsub", float(other)))

    def __rtruediv__(self, other):
        from .ops import functional as F

        return Tensor(F.scalar_op(self._t, "rdiv", float(other)))

    def __neg__(self):
        return self.neg()

    def __matmul__(self, other):
        return self.matmul(other)

    # in-place, no autograd (tensor.rs:1340-1466) — used by hand-written update loops
    def sub_inplace(self, other) -> "Tensor":
        o = _unwrap(other)
        if tuple(o.shape) != tuple(self._t.shape):
            raise ShapeMismatch("sub_inplace", self.shape, Shape(o.shape))
        with torch.no_grad():
            self._t.sub_(o)
        return self

    def add_inplace(self, other) -> "Tensor":
        o = _unwrap(other)
        if tuple(o.shape) != tuple(self._t.shape):
            raise ShapeMismatch("add_inplace", self.shape, Shape(o.shape))
        with torch.no_grad():
            self._t.add_(o)
        return self

    def mul_scalar_inplace(self, s: float) -> "Tensor":
        with torch.no_grad():
            self._t.mul_(float(s))
        return self

    # ------------------------------------------------------------ unary (tensor.rs:1594-1605, 2246-2422)
    def _un(self, op: str, alpha: float = 0.0, beta: float = 0.0) -> "Tensor":
        from .ops import functional as F

        return Tensor(F.unary(self._t, op, alpha, beta))

    def neg(self):
        return self._un("neg")

    def pow(self, e: float):
        return self._un("pow", float(e))

    def sqrt(self):
        return self._un("sqrt")

    def exp(self):
        return self._un("exp")

    def log(self):
        return self._un("log")

    def abs(self):
        return self._un("abs")

    def sin(self):
        return self._un("sin")

    def cos(self):
        return self._un("cos")

    def relu(self):
        return self._un("relu")

    def sigmoid(self):
        return self._un("sigmoid")

    def tanh(self):
        return self._un("tanh")

    def gelu(self):
        return self._un("gelu")

    def silu(self):
        return self._un("silu")

    def leaky_relu(self, slope: float = 0.01):
        return self._un("leaky_relu", slope)

    def elu(self, alpha: float = 1.0):
        return self._un("elu", alpha)

    def clamp(self, lo: float, hi: float):
        return self._un("clamp", float(lo), float(hi))

    # ------------------------------------------------------------ reductions (tensor.rs:1611-2243)
    def _red(self, op: str, dim=None, keepdim: bool = False) -> "Tensor":
        from .ops import functional as F

        if dim is not None:
            dim = self.shape.normalize_dim(dim)
        return Tensor(F.reduce(self._t, op, dim, keepdim))

    def sum(self):
        return self._red("sum")

    def mean(self):
        return self._red("mean")

    def prod(self):
        return self._red("prod")

    def max(self):
        return self._red("max")

    def min(self):
        return self._red("min")

    def sum_dim(self, dim: int, keepdim: bool = False):
        return self._red("sum", dim, keepdim)

    def mean_dim(self, dim: int, keepdim: bool = False):
        return self._red("mean", dim, keepdim)

    def max_dim(self, dim: int, keepdim: bool = False):
        return self._red("max", dim, keepdim)

    # names of the reference's GPU tensor (ferrum-cuda/src/tensor.rs:266-279): reduce one axis away
    def sum_axis(self, axis: int):
        return self._red("sum", axis, False)

    def mean_axis(self, axis: int):
        return self._red("mean", axis, False)

    def min_dim(self, dim: int, keepdim: bool = False):
        return self._red("min", dim, keepdim)

    def argmax(self, dim: int | None = None, keepdim: bool = False):
        from .ops import functional as F

        return Tensor(F.arg_reduce(self._t, True, None if dim is None else self.shape.normalize_dim(dim), keepdim))

    def argmin(self, dim: int | None = None, keepdim: bool = False):
        from .ops import functional as F

        return Tensor(F.arg_reduce(self._t, False, None if dim is None else self.shape.normalize_dim(dim), keepdim))

    # ------------------------------------------------------------ matmul (tensor.rs:2433-2558)
    def matmul(self, other) -> "Tensor":
        from .ops import functional as F

        o = _unwrap(other)
        a = self._t
        if a.dim() == 0 or o.dim() == 0:
            raise InvalidShape("matmul needs at least 1-D operands")
        ka = a.shape[-1]
        kb = o.shape[0] if o.dim() == 1 else o.shape[-2]
        if ka != kb:
            raise ShapeMismatch("matmul", f"inner dimension {ka}", f"{kb}")
        if a.device != o.device:
            raise DeviceMismatch("matmul", self.device, Device.from_torch(o.device))
        return Tensor(F.matmul(a, o))

    def bmm(self, other) -> "Tensor":
        return self.matmul(other)

    def softmax(self, dim: int = -1):
        from .ops import functional as F

        return Tensor(F.softmax(self._t, dim))

    def log_softmax(self, dim: int = -1):
        from .ops import functional as F

        return Tensor(F.log_softmax(self._t, dim))

    # ------------------------------------------------------------ display (tensor.rs:2605-2656)
    def __repr__(self) -> str:
        flat = self._t.detach().reshape(-1)
        n = flat.numel()
        vals = flat[:10].tolist()
        if self.dtype.is_float():
            body = ", ".join(f"{v:.4f}" for v in vals)
        else:
            body = ", ".join(str(v) for v in vals)
        if n > 10:
            body += ", ..."
        return f"Tensor(shape={self.shape}, dtype={self.dtype}, data=[{body}])"

    __str__ = __repr__

    def __len__(self):
        if self._t.dim() == 0:
            raise TypeError("len() of a 0-d tensor")
        return self._t.shape[0]

    def __eq__(self, other):  # identity semantics keep tensors hashable
        return self is other

    def __hash__(self):
        return id(self)
