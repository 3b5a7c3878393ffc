"""Loss functions and functional softmax (ferrum-nn/src/loss.rs:24-183).

``cross_entropy_loss(log_probs, one_hot)`` keeps the reference's normalisation
(mean over all B*C elements).  ``nll_loss`` accepts either one-hot targets (the
reference's alias behaviour) or integer class indices (what its docstring
promises: mean over the batch).  ``cross_entropy`` is the fused logits +
integer-label form used by the training configurations.  ``l1_loss`` and
``smooth_l1_loss`` are true |d| and Huber(1) rather than sqrt(d^2)
(loss.rs:79-105).
"""
from __future__ import annotations

import functools

import torch

from ..core import ShapeMismatch, Tensor, _unwrap
from ..ops import functional as F


def _io(fn):
    @functools.wraps(fn)
    def wrapper(*args, **kw):
        wrapped = any(isinstance(a, Tensor) for a in args)
        out = fn(*[_unwrap(a) for a in args], **kw)
        return Tensor(out) if wrapped else out

    return wrapper


def _check(p, t, what):
    if tuple(p.shape) != tuple(t.shape):
        try:
            torch.broadcast_shapes(p.shape, t.shape)
        except RuntimeError:
            raise ShapeMismatch(what, list(p.shape), list(t.shape)) from None


def _is_index_target(log_probs, targets) -> bool:
    return (not targets.is_floating_point()) and targets.dim() == log_probs.dim() - 1


def _ce_onehot(log_probs, targets):
    _check(log_probs, targets, "cross_entropy_loss")
    t = targets if targets.is_floating_point() else targets.to(log_probs.dtype)
    return F.unary(F.reduce(F.binary(t, log_probs, "mul"), "mean"), "neg")


def _nll_index(log_probs, targets):
    C = log_probs.shape[-1]
    lp2 = log_probs.reshape(-1, C)
    onehot = torch.zeros(lp2.shape, device=lp2.device, dtype=lp2.dtype)
    onehot.scatter_(1, targets.reshape(-1, 1).to(torch.int64), 1.0)
    return F.unary(F.reduce(F.binary(onehot, lp2, "mul"), "sum"), "mul_scalar", -1.0 / lp2.shape[0])


@_io
def mse_loss(predictions, targets):
    """mean((p - t)^2)"""
    _check(predictions, targets, "mse_loss")
    return F.elementwise_loss(predictions, targets, "mse")


@_io
def bce_loss(predictions, targets):
    """-mean(t ln(p + 1e-7) + (1 - t) ln((1 + 1e-7) - (p + 1e-7))), the reference's epsilon placement"""
    _check(predictions, targets, "bce_loss")
    return F.elementwise_loss(predictions, targets, "bce")


@_io
def l1_loss(predictions, targets):
    """mean(|p - t|)"""
    _check(predictions, targets, "l1_loss")
    return F.elementwise_loss(predictions, targets, "l1")


@_io
def smooth_l1_loss(predictions, targets):
    """Huber loss with delta = 1"""
    _check(predictions, targets, "smooth_l1_loss")
    return F.elementwise_loss(predictions, targets, "smooth_l1")


@_io
def cross_entropy_loss(log_probs, targets):
    """``-mean(targets * log_probs)`` over all elements (log-probabilities and one-hot targets)."""
    if _is_index_target(log_probs, targets):
        return _nll_index(log_probs, targets)
    return _ce_onehot(log_probs, targets)


@_io
def nll_loss(log_probs, targets):
    """Negative log-likelihood of log-probabilities; integer targets give the mean over the batch."""
    if _is_index_target(log_probs, targets):
        return _nll_index(log_probs, targets)
    return _ce_onehot(log_probs, targets)


@_io
def cross_entropy(logits, labels):
    """Fused ``log_softmax`` + NLL on raw logits with integer labels (mean over the batch)."""
    return F.cross_entropy_logits(logits, labels)


@_io
def softmax(x, dim=-1):
    return F.softmax(x, dim)


@_io
def log_softmax(x, dim=-1):
    return F.log_softmax(x, dim)
