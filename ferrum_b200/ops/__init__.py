"""Functional op namespace (ferrum-ops/src/lib.rs:8-19) plus the kernel launchers.

``add sub mul div`` / ``relu sigmoid tanh exp log sqrt neg`` / ``sum mean sum_dim mean_dim argmax argmin max_dim
min_dim cat stack`` / ``matmul matmul_optimized matmul_tiled matmul_parallel matmul_blas bmm`` take and return
:class:`ferrum_b200.Tensor`.  All matmul variants of the reference (tiled, rayon-parallel, BLAS) resolve to the one
GEMM path of this package: the tcgen05 kernel under bf16 precision, the fp32 SIMT kernel otherwise.
"""
from __future__ import annotations


def _T():
    from ..core import Tensor

    return Tensor


def add(a, b):
    return a.add(b)


def sub(a, b):
    return a.sub(b)


def mul(a, b):
    return a.mul(b)


def div(a, b):
    return a.div(b)


def relu(x):
    return x.relu()


def sigmoid(x):
    return x.sigmoid()


def tanh(x):
    return x.tanh()


def exp(x):
    return x.exp()


def log(x):
    return x.log()


def sqrt(x):
    return x.sqrt()


def neg(x):
    return x.neg()


def sum(x):  # noqa: A001 - mirrors the reference's name
    return x.sum()


def mean(x):
    return x.mean()


def sum_dim(x, dim, keepdim=False):
    return x.sum_dim(dim, keepdim)


def mean_dim(x, dim, keepdim=False):
    return x.mean_dim(dim, keepdim)


def argmax(x, dim=None):
    return x.argmax(dim)


def argmin(x, dim=None):
    return x.argmin(dim)


def max_dim(x, dim, keepdim=False):
    return x.max_dim(dim, keepdim)


def min_dim(x, dim, keepdim=False):
    return x.min_dim(dim, keepdim)


def cat(tensors, dim=0):
    return _T().cat(tensors, dim)


def stack(tensors, dim=0):
    return _T().stack(tensors, dim)


def matmul(a, b):
    return a.matmul(b)


matmul_optimized = matmul_tiled = matmul_parallel = matmul_blas = matmul


def bmm(a, b):
    return a.matmul(b)
