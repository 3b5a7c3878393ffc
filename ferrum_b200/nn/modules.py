"""``Module`` base class and the core layers.

Parity with ferrum-nn: module.rs:13-46 (Module trait), linear.rs:16-114,
container.rs:17-99, activation.rs:9-227, norm.rs:13-219, embedding.rs:21-227.
Layers hold ``torch.nn.Parameter`` objects (fp32 master weights); ``forward``
accepts either :class:`ferrum_b200.Tensor` or ``torch.Tensor`` and returns the
same kind.  On CUDA, ``Sequential`` fuses adjacent layers into single kernels
(bias / ReLU / Tanh / Sigmoid into the GEMM epilogue, GELU into LayerNorm).
"""
from __future__ import annotations

import functools
import math
from collections import OrderedDict

import torch

from .. import config
from ..core import DType, Device, FerrumError, IndexOutOfBounds, InvalidShape, ShapeMismatch, Tensor, _as_device
from ..ops import functional as F
from . import init as _init


def _wrap_out(out, wrapped: bool):
    if not wrapped:
        return out
    if isinstance(out, torch.Tensor):
        return Tensor(out)
    if isinstance(out, (tuple, list)):
        return type(out)(_wrap_out(o, True) for o in out)
    return out


def tensor_io(fn):
    """Let a torch-level ``forward`` accept and return :class:`Tensor` handles."""

    @functools.wraps(fn)
    def wrapper(self, *args, **kw):
        wrapped = any(isinstance(a, Tensor) for a in args)
        args = [a._t if isinstance(a, Tensor) else a for a in args]
        return _wrap_out(fn(self, *args, **kw), wrapped)

    return wrapper


class Module(torch.nn.Module):
    """Base class of all layers (ferrum-nn/src/module.rs:13-46).

    ``parameters()`` returns a list of :class:`Tensor` handles that alias the
    layer's ``torch.nn.Parameter`` objects (updates and ``.grad()`` are shared),
    mirroring the reference's ``Vec<Tensor>``; ``torch_parameters()`` yields the
    raw parameters.
    """

    def parameters(self, recurse: bool = True):  # type: ignore[override]
        out = []
        for p in super().parameters(recurse):
            w = p.__dict__.get("_ferrum_handle")
            if w is None or w._t is not p:
                w = Tensor(p)
                p.__dict__["_ferrum_handle"] = w
            out.append(w)
        return out

    def torch_parameters(self, recurse: bool = True):
        return super().parameters(recurse)

    def zero_grad(self, set_to_none: bool = True) -> None:  # type: ignore[override]
        for p in super().parameters():
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.detach_().zero_()

    def requires_grad_(self, flag: bool = True):  # type: ignore[override]
        for p in super().parameters():
            p.requires_grad_(flag)
        return self

    def is_training(self) -> bool:
        return self.training

    def name(self) -> str:
        return type(self).__name__

    def num_parameters(self) -> int:
        return sum(p.numel() for p in super().parameters())

    def to_device(self, device) -> "Module":
        return self.to(_as_device(device).to_torch())

    # state_dict / load_state_dict come from torch.nn.Module; keys are "<idx>.weight" etc.
    def ferrum_state_dict(self) -> dict:
        """``{name: Tensor}`` ready for :func:`ferrum_b200.serialize.save`."""
        return {k: Tensor(v.detach()) for k, v in self.state_dict().items()}

    def load_ferrum_state_dict(self, tensors: dict, strict: bool = True):
        sd = {k: (v._t if isinstance(v, Tensor) else v) for k, v in tensors.items()}
        return self.load_state_dict(sd, strict=strict)


def _param(t: torch.Tensor, requires_grad: bool = True) -> torch.nn.Parameter:
    return torch.nn.Parameter(t, requires_grad=requires_grad)


def low_precision_weight(p: torch.nn.Parameter):
    """An up-to-date bf16 copy of ``p`` (cached on the parameter), or None outside bf16 mode.

    The fused optimizer kernels rewrite the copy in the same pass that updates the
    fp32 master weight, so in steady state no cast kernel runs.  Any other
    modification of the parameter (torch in-place op, ``.data`` swap) is detected
    through the version counter / data pointer and triggers one re-cast.
    """
    if not (p.is_cuda and p.dtype == torch.float32 and config.low_precision_active()):
        return None
    d = p.__dict__
    sh = d.get("_fb_shadow")
    key = (p._version, p.data_ptr())
    if sh is None or sh.shape != p.shape or sh.device != p.device:
        sh = torch.empty_like(p, dtype=torch.bfloat16)
        d["_fb_shadow"] = sh
        d["_fb_shadow_key"] = None
    if d.get("_fb_shadow_key") != key:
        from .. import _lib

        src = p.detach().contiguous()
        _lib.check(_lib.cuda().fb_cast(src.data_ptr(), sh.data_ptr(), p.numel(), F.F32, F.BF16, F._stream()),
                   "fb_cast")
        d["_fb_shadow_key"] = key
    return sh


class Linear(Module):
    """``y = x W^T + b`` with ``W [out, in]`` (ferrum-nn/src/linear.rs:16-114).

    Init: ``W ~ U(+-sqrt(6 / in))`` (init.rs:36-39), ``b ~ U(+-1 / sqrt(in))``.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None):
        super().__init__()
        self._in, self._out = int(in_features), int(out_features)
        dev = _as_device(device).to_torch()
        self.weight = _param(_init.kaiming_uniform((out_features, in_features), in_features, device=dev))
        if bias:
            bound = 1.0 / math.sqrt(in_features)
            self.bias = _param(torch.empty(out_features, device=dev).uniform_(-bound, bound))
        else:
            self.register_parameter("bias", None)
        self.grad_sink = None  # set by the DDP engine

    @classmethod
    def new(cls, in_features, out_features):
        return cls(in_features, out_features, True)

    @classmethod
    def with_bias(cls, in_features, out_features, bias):
        return cls(in_features, out_features, bias)

    def in_features(self) -> int:
        return self._in

    def out_features(self) -> int:
        return self._out

    def _forward_act(self, x: torch.Tensor, act):
        if x.shape[-1] != self._in:
            raise ShapeMismatch("Linear.forward", f"[*, {self._in}]", list(x.shape))
        return F.linear(x, self.weight, self.bias, act=act, w_low=low_precision_weight(self.weight),
                        sink=self.grad_sink)

    @tensor_io
    def forward(self, x):
        return self._forward_act(x, None)

    def extra_repr(self):
        return f"in_features={self._in}, out_features={self._out}, bias={self.bias is not None}"


# ------------------------------------------------------------------ activations
class _Act(Module):
    op = "none"
    alpha = 0.0

    @tensor_io
    def forward(self, x):
        return F.unary(x, self.op, self.alpha)


class ReLU(_Act):
    op = "relu"


class Sigmoid(_Act):
    op = "sigmoid"


class Tanh(_Act):
    op = "tanh"


class GELU(_Act):
    """tanh approximation with the reference's constants (activation.rs:254-262)."""
    op = "gelu"


class SiLU(_Act):
    op = "silu"


class LeakyReLU(_Act):
    op = "leaky_relu"

    def __init__(self, negative_slope: float = 0.01):
        super().__init__()
        self.alpha = float(negative_slope)


class ELU(_Act):
    op = "elu"

    def __init__(self, alpha: float = 1.0):
        super().__init__()
        self.alpha = float(alpha)


class Softmax(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    @tensor_io
    def forward(self, x):
        return F.softmax(x, self.dim)


class LogSoftmax(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    @tensor_io
    def forward(self, x):
        return F.log_softmax(x, self.dim)


# ------------------------------------------------------------------ normalisation / dropout
class LayerNorm(Module):
    """Normalises over ``normalized_shape`` (trailing dims); gamma = 1, beta = 0, both trainable.

    The reference's version uses the statistics of the whole tensor and frozen
    parameters (norm.rs:13-68); this one is per row with trainable affine terms.
    """

    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True, device=None):
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = [normalized_shape]
        self.normalized_shape = tuple(int(d) for d in normalized_shape)
        self.eps = float(eps)
        dev = _as_device(device).to_torch()
        if elementwise_affine:
            self.weight = _param(torch.ones(self.normalized_shape, device=dev))
            self.bias = _param(torch.zeros(self.normalized_shape, device=dev))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    def _forward_pre(self, x, pre_act):
        n = len(self.normalized_shape)
        if tuple(x.shape[-n:]) != self.normalized_shape:
            raise ShapeMismatch("LayerNorm.forward", f"[*, {list(self.normalized_shape)}]", list(x.shape))
        return F.layer_norm(x, self.weight, self.bias, self.eps, pre_act, n)

    @tensor_io
    def forward(self, x):
        return self._forward_pre(x, None)


class BatchNorm1d(Module):
    """Per-feature batch norm over ``[B, F]`` with running statistics (norm.rs:75-165, fixed per D7/D11)."""

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, device=None):
        super().__init__()
        dev = _as_device(device).to_torch()
        self.num_features, self.eps, self.momentum = int(num_features), float(eps), float(momentum)
        self.weight = _param(torch.ones(num_features, device=dev))
        self.bias = _param(torch.zeros(num_features, device=dev))
        self.register_buffer("running_mean", torch.zeros(num_features, device=dev))
        self.register_buffer("running_var", torch.ones(num_features, device=dev))

    @tensor_io
    def forward(self, x):
        if x.dim() != 2 or x.shape[1] != self.num_features:
            raise ShapeMismatch("BatchNorm1d.forward", f"[B, {self.num_features}]", list(x.shape))
        return F.batch_norm(x, self.weight, self.bias, self.running_mean, self.running_var, self.training,
                            self.momentum, self.eps)


class Dropout(Module):
    """Inverted dropout (the reference scales by (1-p) with no mask: norm.rs:192-202)."""

    def __init__(self, p: float = 0.5):
        super().__init__()
        if not 0.0 <= p <= 1.0:
            raise FerrumError(f"dropout probability must be in [0, 1], got {p}")
        self.p = float(p)

    @tensor_io
    def forward(self, x):
        return F.dropout(x, self.p, self.training)


# ------------------------------------------------------------------ embedding
class Embedding(Module):
    """Lookup table ``[V, D]`` ~ N(0, 1) (embedding.rs:21-227) with a real scatter-add backward."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: int | None = None, dtype=DType.F32,
                 device=None, _weight=None, freeze: bool = False):
        super().__init__()
        self.num_embeddings, self.embedding_dim = int(num_embeddings), int(embedding_dim)
        self.padding_idx = padding_idx
        dev = _as_device(device).to_torch()
        if _weight is None:
            _weight = torch.randn(num_embeddings, embedding_dim, device=dev, dtype=dtype.to_torch())
            if padding_idx is not None:
                _weight[padding_idx].zero_()
        self.weight = _param(_weight, requires_grad=not freeze)
        self.grad_sink = None  # set by the DDP engine

    @classmethod
    def new(cls, num_embeddings, embedding_dim):
        return cls(num_embeddings, embedding_dim)

    @classmethod
    def new_with_dtype(cls, num_embeddings, embedding_dim, dtype):
        return cls(num_embeddings, embedding_dim, dtype=dtype)

    def with_padding_idx(self, idx: int) -> "Embedding":
        if not 0 <= idx < self.num_embeddings:
            raise IndexOutOfBounds(idx, 0, self.num_embeddings)
        self.padding_idx = idx
        with torch.no_grad():
            self.weight[idx].zero_()
        return self

    @classmethod
    def from_pretrained(cls, weight, freeze: bool = True):
        w = weight._t if isinstance(weight, Tensor) else weight
        if w.dim() != 2:
            raise InvalidShape("from_pretrained expects a [V, D] weight")
        return cls(w.shape[0], w.shape[1], _weight=w.detach().clone(), freeze=freeze)

    def _check(self, idx):
        if idx.dtype not in (torch.int64, torch.int32):
            raise FerrumError(f"Embedding indices must be I64, got {idx.dtype}")
        if not idx.is_cuda and idx.numel():
            lo, hi = int(idx.min()), int(idx.max())
            if lo < 0 or hi >= self.num_embeddings:
                raise IndexOutOfBounds(hi if hi >= self.num_embeddings else lo, 0, self.num_embeddings)

    @tensor_io
    def forward(self, idx):
        self._check(idx)
        return F.embedding(self.weight, idx, self.padding_idx, sink=self.grad_sink)

    forward_indices = forward

    @tensor_io
    def forward_mean(self, idx):
        """Mean-pooled lookup ``[B, S] -> [B, D]`` in one kernel."""
        self._check(idx)
        out_dtype = torch.bfloat16 if config.low_precision_active() and self.weight.is_cuda else None
        return F.embedding_mean_pool(self.weight, idx, out_dtype, self.grad_sink)


class MeanPoolEmbedding(Embedding):
    """``Embedding`` whose ``forward`` is the fused mean-pooled lookup (bag of tokens)."""

    @tensor_io
    def forward(self, idx):
        self._check(idx)
        out_dtype = torch.bfloat16 if config.low_precision_active() and self.weight.is_cuda else None
        return F.embedding_mean_pool(self.weight, idx, out_dtype, self.grad_sink)


# ------------------------------------------------------------------ container
_EPILOGUE_ACTS = {ReLU: "relu", Tanh: "tanh", Sigmoid: "sigmoid"}


class Sequential(Module):
    """Ordered container (container.rs:17-99): ``add`` / ``add_boxed`` / ``len`` / ``is_empty``."""

    def __init__(self, *layers):
        super().__init__()
        if len(layers) == 1 and isinstance(layers[0], (list, tuple, OrderedDict)):
            layers = tuple(layers[0].values()) if isinstance(layers[0], OrderedDict) else tuple(layers[0])
        for l in layers:
            self.add(l)

    @classmethod
    def new(cls):
        return cls()

    def add(self, layer: torch.nn.Module) -> "Sequential":
        self.add_module(str(len(self._modules)), layer)
        return self

    add_boxed = add

    def len(self) -> int:
        return len(self._modules)

    __len__ = len

    def is_empty(self) -> bool:
        return len(self._modules) == 0

    def __getitem__(self, i):
        return list(self._modules.values())[i]

    def __iter__(self):
        return iter(self._modules.values())

    @tensor_io
    def forward(self, x):
        layers = list(self._modules.values())
        i, n = 0, len(layers)
        fuse = isinstance(x, torch.Tensor) and x.is_cuda
        while i < n:
            l = layers[i]
            nxt = layers[i + 1] if i + 1 < n else None
            nxt2 = layers[i + 2] if i + 2 < n else None
            if (fuse and type(l) is Linear and type(nxt) is GELU and type(nxt2) is LayerNorm
                    and len(nxt2.normalized_shape) == 1 and nxt2.weight is not None
                    and nxt2.normalized_shape[0] == l._out):
                x = F.linear_act_layernorm(x, l.weight, l.bias, nxt2.weight, nxt2.bias, nxt2.eps, "gelu",
                                           low_precision_weight(l.weight), l.grad_sink)
                i += 3
            elif fuse and type(l) is Linear and type(nxt) in _EPILOGUE_ACTS:
                x = l._forward_act(x, _EPILOGUE_ACTS[type(nxt)])
                i += 2
            elif fuse and type(l) is GELU and type(nxt) is LayerNorm and len(nxt.normalized_shape) == 1:
                x = nxt._forward_pre(x, "gelu")
                i += 2
            else:
                x = l(x)
                i += 1
        return x
