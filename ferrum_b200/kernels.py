"""The eight kernel entry points of ferrum-cuda/src/kernels.rs:10-697 with their op enums, taking
:class:`ferrum_b200.Tensor` operands on ``Device.Cuda``.  There they are CPU simulations / ``todo!()``; here each
call launches one sm_100a kernel (non-differentiable, like the reference's)."""
from __future__ import annotations

import enum

import torch

from .core import Tensor, _unwrap
from .ops import functional as F
from .ops import gemm as _gemm


class BinaryOp(enum.Enum):
    Add = "add"
    Sub = "sub"
    Mul = "mul"
    Div = "div"
    Pow = "pow"
    Max = "max"
    Min = "min"


class UnaryOp(enum.Enum):
    Neg = "neg"
    Exp = "exp"
    Log = "log"
    Sqrt = "sqrt"
    Abs = "abs"
    Sin = "sin"
    Cos = "cos"
    Tanh = "tanh"
    Sigmoid = "sigmoid"
    Relu = "relu"
    LeakyRelu = "leaky_relu"
    Gelu = "gelu"
    Silu = "silu"


class ScalarOp(enum.Enum):
    Add = "add"
    Sub = "sub"
    Mul = "mul"
    Div = "div"
    Pow = "pow"


class ReduceKind(enum.Enum):
    Sum = "sum"
    Mean = "mean"
    Max = "max"
    Min = "min"
    Prod = "prod"


def _cuda(t) -> torch.Tensor:
    t = _unwrap(t)
    if not t.is_cuda:
        raise ValueError("kernel entry points take tensors on Device.Cuda")
    return t


def binary_op(a, b, op: BinaryOp) -> Tensor:
    """c = a (op) b with real broadcasting (the reference's simulation cycles b)."""
    with torch.no_grad():
        return Tensor(F.raw_binary(F._f32(_cuda(a)), F._f32(_cuda(b)), op.value))


def unary_op(x, op: UnaryOp, alpha: float = 0.01) -> Tensor:
    with torch.no_grad():
        return Tensor(F.raw_unary(_cuda(x), op.value, alpha if op is UnaryOp.LeakyRelu else 0.0))


def scalar_op(x, scalar: float, op: ScalarOp) -> Tensor:
    with torch.no_grad():
        return Tensor(F.scalar_op(_cuda(x), op.value, float(scalar)))


def reduce_op(x, op: ReduceKind, axis: int | None = None, keepdim: bool = False) -> Tensor:
    t = _cuda(x)
    with torch.no_grad():
        return Tensor(F.raw_reduce(F._f32(t), op.value, None if axis is None else axis % t.dim(), keepdim))


def matmul(a, b) -> Tensor:
    """C[M,N] = A[M,K] B[K,N]: tcgen05 kernel for bf16 operands, fp32 SIMT kernel otherwise."""
    ta, tb = _cuda(a), _cuda(b)
    with torch.no_grad():
        if ta.dtype == torch.bfloat16 and tb.dtype == torch.bfloat16 and _gemm.bf16_operand_ok(ta) and \
                _gemm.bf16_operand_ok(tb.t()):
            return Tensor(_gemm.gemm_bf16(ta, tb.t()))
        return Tensor(_gemm.gemm_f32(F._f32(ta), F._f32(tb).transpose(-1, -2)))


def transpose(x) -> Tensor:
    """Materialised transpose of the last two dimensions."""
    t = _cuda(x)
    with torch.no_grad():
        if t.dim() == 2:
            return Tensor(F.transpose_2d(t))
        lead = t.shape[:-2]
        flat = t.reshape(-1, *t.shape[-2:])
        return Tensor(torch.stack([F.transpose_2d(m) for m in flat]).reshape(*lead, t.shape[-1], t.shape[-2]))


def softmax(x) -> Tensor:
    with torch.no_grad():
        return Tensor(F.softmax(_cuda(x), -1))


def log_softmax(x) -> Tensor:
    with torch.no_grad():
        return Tensor(F.log_softmax(_cuda(x), -1))
