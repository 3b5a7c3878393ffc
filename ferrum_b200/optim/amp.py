"""Mixed-precision utilities (ferrum-optim/src/amp.rs:12-238).

``GradScaler`` keeps the reference's schedule (scale 65536, x2 every 2000 clean
steps, x0.5 on overflow).  With bf16 tensor-core GEMMs and fp32 accumulation the
loss scale is optional; it is kept for API parity and for fp16 experiments.
On CUDA, unscale + inf/nan detection and global-norm clipping are multi-tensor
kernels (``csrc/optim/fused_optim.cu``) — one launch each for all gradients.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib, config
from ..core import DType, Tensor, _unwrap
from ..ops import functional as F


def _grad_targets(tensors):
    """The tensors to modify: a parameter's ``.grad`` when it has one, else the tensor itself."""
    out = []
    for t in tensors:
        t = _unwrap(t)
        if t.requires_grad and t.grad is not None:
            out.append(t.grad)
        elif not t.requires_grad:
            out.append(t)
    return out


def _tables(gs):
    n = len(gs)
    ptrs = (ctypes.c_void_p * n)(*[g.data_ptr() for g in gs])
    sizes = (ctypes.c_longlong * n)(*[g.numel() for g in gs])
    return ptrs, sizes, n


def _cuda_f32(gs):
    return bool(gs) and all(g.is_cuda and g.dtype == torch.float32 and g.is_contiguous() for g in gs)


class GradScaler:
    def __init__(self, init_scale: float = 65536.0, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, enabled: bool = True):
        self._scale = float(init_scale)
        self.growth_factor, self.backoff_factor = float(growth_factor), float(backoff_factor)
        self.growth_interval, self.enabled = int(growth_interval), bool(enabled)
        self.step_count = 0

    @classmethod
    def new(cls):
        return cls()

    @classmethod
    def with_scale(cls, init_scale: float):
        return cls(init_scale=init_scale)

    def get_scale(self) -> float:
        return self._scale

    def is_enabled(self) -> bool:
        return self.enabled

    def scale(self, loss):
        if not self.enabled:
            return loss
        if isinstance(loss, Tensor):
            return loss.mul_scalar(self._scale)
        return F.scalar_op(loss, "mul", self._scale)

    def unscale_gradients(self, gradients) -> bool:
        """Divide by the scale in place; returns True when every value is finite."""
        if not self.enabled:
            return True
        gs = _grad_targets(gradients)
        if not gs:
            return True
        inv = 1.0 / self._scale
        if _cuda_f32(gs):
            flag = torch.zeros(1, device=gs[0].device, dtype=torch.float32)
            ptrs, sizes, n = _tables(gs)
            _lib.check(_lib.cuda().fb_unscale_check(ptrs, sizes, n, inv, flag.data_ptr(),
                                                    torch.cuda.current_stream().cuda_stream), "fb_unscale_check")
            return flag.item() == 0.0
        ok = True
        with torch.no_grad():
            for g in gs:
                if not torch.isfinite(g).all():
                    ok = False
                    break
                g.mul_(inv)
        return ok

    def update(self, found_inf: bool) -> None:
        if not self.enabled:
            return
        if found_inf:
            self._scale *= self.backoff_factor
        else:
            self.step_count += 1
            if self.step_count % self.growth_interval == 0:
                self._scale *= self.growth_factor

    def step(self, gradients) -> bool:
        valid = self.unscale_gradients(gradients)
        self.update(not valid)
        return valid


class Autocast:
    """Context / helper selecting the GEMM compute dtype (amp.rs:129-176; a placeholder there).

    ``with Autocast.with_dtype(DType.BF16): ...`` runs Linear / matmul on the bf16
    tensor cores with fp32 accumulation; ``cast`` / ``cast_back`` convert a tensor.
    """

    def __init__(self, dtype: DType = DType.BF16, enabled: bool = True):
        self.dtype, self.enabled = dtype, enabled
        self._cm = None

    @classmethod
    def new(cls):
        return cls()

    @classmethod
    def with_dtype(cls, dtype: DType):
        return cls(dtype)

    def is_enabled(self) -> bool:
        return self.enabled

    def cast(self, tensor):
        if not self.enabled:
            return tensor
        return tensor.to_dtype(self.dtype) if isinstance(tensor, Tensor) else F.cast(tensor, self.dtype.to_torch())

    def cast_back(self, tensor):
        return tensor.to_dtype(DType.F32) if isinstance(tensor, Tensor) else F.cast(tensor, torch.float32)

    def __enter__(self):
        dt = self.dtype.to_torch() if self.dtype in (DType.BF16, DType.F32) else torch.bfloat16
        self._cm = config.autocast(dt, self.enabled)
        self._cm.__enter__()
        return self

    def __exit__(self, *exc):
        cm, self._cm = self._cm, None
        return cm.__exit__(*exc)


def _conv(tensor, dt):
    if isinstance(tensor, Tensor):
        return tensor.to_dtype(dt)
    return F.cast(tensor, DType(dt).to_torch())


def to_half(tensor):
    return _conv(tensor, DType.F16)


def to_bfloat16(tensor):
    return _conv(tensor, DType.BF16)


def to_float(tensor):
    return _conv(tensor, DType.F32)


def has_inf_or_nan(tensor) -> bool:
    t = _unwrap(tensor)
    return not bool(torch.isfinite(t).all().item())


def clip_grad_norm(parameters, max_norm: float) -> float:
    """Scale gradients so their global L2 norm is at most ``max_norm``; returns the norm before clipping."""
    gs = _grad_targets(parameters)
    if not gs:
        return 0.0
    if _cuda_f32(gs):
        total = torch.zeros(1, device=gs[0].device, dtype=torch.float32)
        ptrs, sizes, n = _tables(gs)
        st = torch.cuda.current_stream().cuda_stream
        lib = _lib.cuda()
        _lib.check(lib.fb_sumsq_multi(ptrs, sizes, n, total.data_ptr(), st), "fb_sumsq_multi")
        _lib.check(lib.fb_scale_multi(ptrs, sizes, n, total.data_ptr(), float(max_norm), 0.0, 0, st),
                   "fb_scale_multi")
        return float(total.sqrt().item())
    with torch.no_grad():
        total = float(torch.sqrt(sum((g.float() ** 2).sum() for g in gs)))
        if total > max_norm:
            coef = max_norm / (total + 1e-6)
            for g in gs:
                g.mul_(coef)
    return total


def clip_grad_value(parameters, clip_value: float) -> None:
    gs = _grad_targets(parameters)
    if not gs:
        return
    if _cuda_f32(gs):
        ptrs, sizes, n = _tables(gs)
        _lib.check(_lib.cuda().fb_scale_multi(ptrs, sizes, n, None, 0.0, float(clip_value), 1,
                                              torch.cuda.current_stream().cuda_stream), "fb_scale_multi")
        return
    with torch.no_grad():
        for g in gs:
            g.clamp_(-clip_value, clip_value)
