"""``Optimizer``, ``SGD`` and ``Adam`` (ferrum-optim/src/{optimizer,sgd,adam}.rs).

Update rules are the reference's: SGD adds ``wd * p`` to the gradient, keeps a
momentum buffer whose first value is the gradient itself, optional Nesterov;
Adam applies decoupled decay ``p -= lr * wd * p`` before the moment updates,
uses one global step count and ``1 - beta^t`` bias corrections.

On CUDA a step is ONE multi-tensor kernel launch (``csrc/optim/fused_optim.cu``)
that also refreshes the bf16 copy of each weight used by the tensor-core GEMMs.
On CPU the same arithmetic runs as in-place torch ops.  When an optimizer is
attached to a ``DistributedDataParallel`` engine in fused mode, ``step()`` only
waits for the reduction kernels, which have already applied the update.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, replace

import torch

from .. import _lib
from ..core import Tensor


@dataclass
class SGDConfig:
    lr: float = 0.01
    momentum: float = 0.0
    weight_decay: float = 0.0
    nesterov: bool = False

    @classmethod
    def new(cls, lr: float) -> "SGDConfig":
        return cls(lr=lr)

    def with_momentum(self, momentum: float) -> "SGDConfig":
        return replace(self, momentum=momentum)

    def with_weight_decay(self, weight_decay: float) -> "SGDConfig":
        return replace(self, weight_decay=weight_decay)

    def with_nesterov(self, nesterov: bool) -> "SGDConfig":
        return replace(self, nesterov=nesterov)


@dataclass
class AdamConfig:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0

    def __init__(self, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                 weight_decay: float = 0.0, betas=None):
        if betas is not None:  # the README spelling
            beta1, beta2 = betas
        self.lr, self.beta1, self.beta2, self.eps, self.weight_decay = lr, beta1, beta2, eps, weight_decay

    @classmethod
    def new(cls, lr: float) -> "AdamConfig":
        return cls(lr=lr)

    def with_betas(self, beta1: float, beta2: float) -> "AdamConfig":
        return replace(self, beta1=beta1, beta2=beta2)

    def with_weight_decay(self, weight_decay: float) -> "AdamConfig":
        return replace(self, weight_decay=weight_decay)

    def with_eps(self, eps: float) -> "AdamConfig":
        return replace(self, eps=eps)

    @property
    def betas(self):
        return (self.beta1, self.beta2)


def _collect(params) -> list:
    if isinstance(params, torch.nn.Module):
        params = list(torch.nn.Module.parameters(params))
    out = []
    for p in params:
        if isinstance(p, Tensor):
            p = p._t
        if not isinstance(p, torch.Tensor):
            raise TypeError(f"optimizer parameters must be tensors, got {type(p)}")
        out.append(p)
    return out


class Optimizer:
    """``step`` / ``zero_grad`` / ``learning_rate`` / ``set_learning_rate`` / ``param_groups`` (optimizer.rs:6-21)."""

    def __init__(self, params):
        self.params = _collect(params)
        self._engine = None  # a DDP engine that applies the update inside its reduction kernel
        self._dyn = None     # device scalars {lr, bias_corr1, bias_corr2, beta1^t, beta2^t, t} (capturable mode)

    # -- reference API
    def learning_rate(self) -> float:
        return self.config.lr

    def set_learning_rate(self, lr: float) -> None:
        self.config.lr = float(lr)
        if self._dyn is not None:
            self._dyn[0:1].fill_(float(lr))  # picked up by the next launch or graph replay

    def capturable(self, flag: bool = True) -> "Optimizer":
        """Keep the step-dependent factors (learning rate, Adam's bias corrections) in device memory and advance
        them with a kernel, so that a step captured in a CUDA graph replays with the right values.  The update
        rule is unchanged; ``set_learning_rate`` keeps working between replays."""
        if not flag:
            self._dyn = None
            return self
        dev = next((p.device for p in self.params if p.is_cuda), None)
        if dev is None:
            raise ValueError("capturable mode needs parameters on a CUDA device")
        vals = self._dyn_values()
        if self._dyn is None:
            self._dyn = torch.tensor(vals, dtype=torch.float32, device=dev)
        else:  # in place: a recorded graph keeps reading the same device memory
            self._dyn.copy_(torch.tensor(vals, dtype=torch.float32))
        return self

    def _dyn_values(self) -> list:
        t = int(getattr(self, "step_count", 0))
        b1 = float(getattr(self.config, "beta1", 1.0))
        b2 = float(getattr(self.config, "beta2", 1.0))
        return [self.config.lr, 1.0 - b1 ** t, 1.0 - b2 ** t, b1 ** t, b2 ** t, float(t)]

    def _engine_owns_state(self) -> bool:
        e = self._engine
        return e is not None and hasattr(e, "owns_optimizer_state") and e.owns_optimizer_state()

    def _after_state_load(self) -> None:
        """The device-side step factors follow a restored step count (capturable mode)."""
        if self._dyn is not None:
            self.capturable(True)

    def zero_grad(self, set_to_none: bool = True) -> None:
        if self._engine is not None:
            self._engine.zero_grad()
            return
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.detach_().zero_()

    def param_groups(self):
        return [{"params": [Tensor(p) for p in self.params], **self.config.__dict__}]

    def step(self) -> None:
        if self._engine is not None:
            self._engine.finish_step(self)
            return
        self._step_local()

    # -- helpers
    def _split(self):
        cuda, cpu = [], []
        for i, p in enumerate(self.params):
            if p.grad is None:
                continue
            (cuda if (p.is_cuda and p.dtype == torch.float32 and p.grad.dtype == torch.float32
                      and p.is_contiguous() and p.grad.is_contiguous()) else cpu).append(i)
        return cuda, cpu

    @staticmethod
    def _ptr_array(vals):
        arr = (ctypes.c_void_p * len(vals))()
        for i, v in enumerate(vals):
            arr[i] = v
        return arr

    @staticmethod
    def _shadow_ptr(p):
        sh = p.__dict__.get("_fb_shadow")
        if sh is None or sh.shape != p.shape or p.__dict__.get("_fb_shadow_key") != (p._version, p.data_ptr()):
            return None  # absent or stale: the owning layer re-casts on its next forward
        return sh.data_ptr()


class SGD(Optimizer):
    """Stochastic gradient descent with momentum / Nesterov / L2 decay (sgd.rs:61-139)."""

    def __init__(self, params, config: SGDConfig | None = None, **kw):
        super().__init__(params)
        self.config = replace(config) if config is not None else SGDConfig(**kw)
        self.velocity = [None] * len(self.params)
        self.step_count = 0

    @classmethod
    def new(cls, params, config):
        return cls(params, config)

    def hparams(self, grad_scale: float = 1.0) -> _lib.SgdH:
        c = self.config
        return _lib.SgdH(c.lr, c.momentum, c.weight_decay, grad_scale, 1 if c.nesterov else 0,
                         1 if self.step_count == 0 else 0)

    def _step_local(self) -> None:
        c = self.config
        cuda_idx, cpu_idx = self._split()
        if cuda_idx:
            ps, gs, bs, shs, ns = [], [], [], [], []
            for i in cuda_idx:
                p = self.params[i]
                first = self.velocity[i] is None
                if c.momentum != 0.0 and first:
                    self.velocity[i] = torch.zeros_like(p)
                ps.append(p.data_ptr())
                gs.append(p.grad.data_ptr())
                bs.append(self.velocity[i].data_ptr() if c.momentum != 0.0 else None)
                shs.append(self._shadow_ptr(p))
                ns.append(p.numel())
            # buffers start at zero, so mu * 0 + g == g reproduces the reference's first step (sgd.rs:95-104)
            h = self.hparams()
            n = len(ps)
            st = torch.cuda.current_stream().cuda_stream
            if self._dyn is not None:
                _lib.check(_lib.cuda().fb_sgd_multi_dyn(self._ptr_array(ps), self._ptr_array(gs), self._ptr_array(bs),
                                                        self._ptr_array(shs), (ctypes.c_longlong * n)(*ns), n, h,
                                                        self._dyn.data_ptr(), st), "fb_sgd_multi_dyn")
            else:
                _lib.check(_lib.cuda().fb_sgd_multi(self._ptr_array(ps), self._ptr_array(gs), self._ptr_array(bs),
                                                    self._ptr_array(shs), (ctypes.c_longlong * n)(*ns), n, h, st),
                           "fb_sgd_multi")
        with torch.no_grad():
            for i in cpu_idx:
                p = self.params[i]
                g = p.grad
                if c.weight_decay != 0.0:
                    g = g + c.weight_decay * p
                if c.momentum != 0.0:
                    v = self.velocity[i]
                    v = g.clone() if v is None else v * c.momentum + g
                    self.velocity[i] = v
                    g = g + c.momentum * v if c.nesterov else v
                p.sub_(c.lr * g)
        self.step_count += 1

    def state_tensors(self) -> dict:
        """Momentum buffers and the step count.  With a fused data-parallel engine the buffers live in the
        engine's shards and are gathered from their owners (collective: every rank calls it)."""
        if self._engine_owns_state():
            out = self._engine.export_optimizer_state(self)
        else:
            out = {f"optim.velocity.{i}": v for i, v in enumerate(self.velocity) if v is not None}
        out["optim.step"] = torch.tensor(self.step_count, dtype=torch.int64)
        return out

    def load_state_tensors(self, tensors: dict) -> None:
        if self._engine_owns_state():
            self._engine.import_optimizer_state(self, tensors)
        else:
            for i, p in enumerate(self.params):
                v = tensors.get(f"optim.velocity.{i}")
                if v is not None:
                    self.velocity[i] = v.to(p.device, p.dtype).clone()
        if "optim.step" in tensors:
            self.step_count = int(tensors["optim.step"].item())
        self._after_state_load()


class Adam(Optimizer):
    """Adam with decoupled weight decay applied before the moments (adam.rs:65-165)."""

    def __init__(self, params, config: AdamConfig | None = None, **kw):
        super().__init__(params)
        self.config = replace(config) if config is not None else AdamConfig(**kw)
        self.m = [None] * len(self.params)
        self.v = [None] * len(self.params)
        self.step_count = 0

    @classmethod
    def new(cls, params, config):
        return cls(params, config)

    def hparams(self, step: int | None = None, grad_scale: float = 1.0) -> _lib.AdamH:
        c = self.config
        t = self.step_count + 1 if step is None else step
        return _lib.AdamH(c.lr, c.beta1, c.beta2, c.eps, c.weight_decay, 1.0 - c.beta1 ** t, 1.0 - c.beta2 ** t,
                          grad_scale)

    def _step_local(self) -> None:
        c = self.config
        self.step_count += 1
        t = self.step_count
        bc1, bc2 = 1.0 - c.beta1 ** t, 1.0 - c.beta2 ** t
        cuda_idx, cpu_idx = self._split()
        if cuda_idx:
            ps, gs, ms, vs, shs, ns = [], [], [], [], [], []
            for i in cuda_idx:
                p = self.params[i]
                if self.m[i] is None:
                    self.m[i] = torch.zeros_like(p)
                    self.v[i] = torch.zeros_like(p)
                ps.append(p.data_ptr())
                gs.append(p.grad.data_ptr())
                ms.append(self.m[i].data_ptr())
                vs.append(self.v[i].data_ptr())
                shs.append(self._shadow_ptr(p))
                ns.append(p.numel())
            n = len(ps)
            st = torch.cuda.current_stream().cuda_stream
            if self._dyn is not None:
                lib = _lib.cuda()
                _lib.check(lib.fb_optim_advance(self._dyn.data_ptr(), c.beta1, c.beta2, st), "fb_optim_advance")
                _lib.check(lib.fb_adam_multi_dyn(self._ptr_array(ps), self._ptr_array(gs), self._ptr_array(ms),
                                                 self._ptr_array(vs), self._ptr_array(shs),
                                                 (ctypes.c_longlong * n)(*ns), n, self.hparams(t),
                                                 self._dyn.data_ptr(), st), "fb_adam_multi_dyn")
            else:
                _lib.check(_lib.cuda().fb_adam_multi(self._ptr_array(ps), self._ptr_array(gs), self._ptr_array(ms),
                                                     self._ptr_array(vs), self._ptr_array(shs),
                                                     (ctypes.c_longlong * n)(*ns), n, self.hparams(t), st),
                           "fb_adam_multi")
        with torch.no_grad():
            for i in cpu_idx:
                p = self.params[i]
                g = p.grad
                if self.m[i] is None:
                    self.m[i] = torch.zeros_like(p)
                    self.v[i] = torch.zeros_like(p)
                if c.weight_decay != 0.0:
                    p.sub_(c.lr * c.weight_decay * p)
                self.m[i].mul_(c.beta1).add_(g, alpha=1.0 - c.beta1)
                self.v[i].mul_(c.beta2).addcmul_(g, g, value=1.0 - c.beta2)
                mh = self.m[i] / bc1
                vh = self.v[i] / bc2
                p.sub_(c.lr * mh / (vh.sqrt() + c.eps))

    def state_tensors(self) -> dict:
        """Both moments per parameter and the step count.  With a fused data-parallel engine the moments live in
        the engine's shards and are gathered from their owners (collective: every rank calls it)."""
        out = {}
        if self._engine_owns_state():
            out = self._engine.export_optimizer_state(self)
        else:
            for i in range(len(self.params)):
                if self.m[i] is not None:
                    out[f"optim.m.{i}"] = self.m[i]
                    out[f"optim.v.{i}"] = self.v[i]
        out["optim.step"] = torch.tensor(self.step_count, dtype=torch.int64)
        return out

    def load_state_tensors(self, tensors: dict) -> None:
        if self._engine_owns_state():
            self._engine.import_optimizer_state(self, tensors)
        else:
            for i, p in enumerate(self.params):
                m, v = tensors.get(f"optim.m.{i}"), tensors.get(f"optim.v.{i}")
                if m is not None and v is not None:
                    self.m[i] = m.to(p.device, p.dtype).clone()
                    self.v[i] = v.to(p.device, p.dtype).clone()
        if "optim.step" in tensors:
            self.step_count = int(tensors["optim.step"].item())
        self._after_state_load()
