"""The named backward formulas of ferrum-core/src/autograd_ops.rs:257-586 and ferrum-autograd/src/function.rs:29-571
as callable objects: ``XBackward(saved...).backward(grad_output) -> [grads]``, ``name()``.

The engine does not use them (each op of :mod:`ferrum_b200.ops.functional` carries its own backward kernel); they
exist for API parity and as directly testable statements of the formulas, computed with this package's ops."""
from __future__ import annotations

from .core import Tensor, _unwrap
from .ops import functional as F


def _t(x):
    return _unwrap(x)


class Function:
    """``backward(grad_output)`` and ``name()`` (function.rs:29-40)."""

    def name(self) -> str:
        return type(self).__name__

    def backward(self, grad_output):
        raise NotImplementedError


def reduce_gradient(grad, shape):
    """Sum a broadcast gradient down to ``shape`` (function.rs:437-506)."""
    return Tensor(F.reduce_to_shape(_t(grad), tuple(shape)))


class _Binary(Function):
    def __init__(self, a, b):
        self.a, self.b = _t(a), _t(b)

    def _fit(self, ga, gb):
        return [Tensor(F.reduce_to_shape(ga, self.a.shape)), Tensor(F.reduce_to_shape(gb, self.b.shape))]


class AddBackward(_Binary):
    def backward(self, g):
        g = _t(g)
        return self._fit(g, g)


class SubBackward(_Binary):
    def backward(self, g):
        g = _t(g)
        return self._fit(g, F.unary(g, "neg"))


class MulBackward(_Binary):
    def backward(self, g):
        g = _t(g)
        return self._fit(F.binary(g, self.b, "mul"), F.binary(g, self.a, "mul"))


class DivBackward(_Binary):
    def backward(self, g):
        g = _t(g)
        ga = F.binary(g, self.b, "div")
        gb = F.unary(F.binary(F.binary(g, self.a, "mul"), F.binary(self.b, self.b, "mul"), "div"), "neg")
        return self._fit(ga, gb)


class MatMulBackward(Function):
    def __init__(self, a, b):
        self.a, self.b = _t(a), _t(b)

    def backward(self, g):
        g = _t(g)
        return [Tensor(F.matmul(g, self.b.t())), Tensor(F.matmul(self.a.t(), g))]


class _Unary(Function):
    op, saves_output = "none", False

    def __init__(self, saved, alpha: float = 0.0):
        self.saved, self.alpha = _t(saved), alpha

    def backward(self, g):
        g, s = _t(g), self.saved
        if s.is_cuda:
            return [Tensor(F.raw_unary_bwd(g, s, self.op, self.alpha))]
        return [Tensor(self._cpu(g, s))]


class NegBackward(Function):
    def backward(self, g):
        return [Tensor(F.unary(_t(g), "neg"))]


class ReLUBackward(_Unary):
    op = "relu"

    def _cpu(self, g, x):
        return g * (x > 0).to(g.dtype)


class SigmoidBackward(_Unary):
    op, saves_output = "sigmoid", True

    def _cpu(self, g, y):
        return g * y * (1 - y)


class TanhBackward(_Unary):
    op, saves_output = "tanh", True

    def _cpu(self, g, y):
        return g * (1 - y * y)


class ExpBackward(_Unary):
    op, saves_output = "exp", True

    def _cpu(self, g, y):
        return g * y


class LogBackward(_Unary):
    op = "log"

    def _cpu(self, g, x):
        return g / x


class SqrtBackward(_Unary):
    op, saves_output = "sqrt", True

    def _cpu(self, g, y):
        return g / (2 * y)


class PowBackward(_Unary):
    op = "pow"

    def __init__(self, x, exponent: float):
        super().__init__(x, float(exponent))

    def _cpu(self, g, x):
        return g * self.alpha * x ** (self.alpha - 1)


class SumBackward(Function):
    def __init__(self, input_shape):
        self.shape = tuple(input_shape)

    def backward(self, g):
        return [Tensor(_t(g).reshape([1] * len(self.shape)).expand(self.shape).contiguous())]


class MeanBackward(SumBackward):
    def backward(self, g):
        n = 1
        for d in self.shape:
            n *= d
        return [Tensor(F.scalar_op(_t(g), "mul", 1.0 / max(n, 1)).reshape([1] * len(self.shape)).expand(
            self.shape).contiguous())]


class SumDimBackward(Function):
    def __init__(self, input_shape, dim: int, keepdim: bool = False):
        self.shape, self.dim, self.keepdim = tuple(input_shape), dim % len(input_shape), keepdim

    def backward(self, g):
        g = _t(g)
        if not self.keepdim:
            g = g.unsqueeze(self.dim)
        return [Tensor(g.expand(self.shape).contiguous())]


class CatBackward(Function):
    def __init__(self, sizes, dim: int):
        self.sizes, self.dim = list(sizes), dim

    def backward(self, g):
        return [Tensor(p.contiguous()) for p in _t(g).split(self.sizes, self.dim)]
