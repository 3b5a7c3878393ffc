"""Differentiable ops on ``torch.Tensor`` values.

Every function here takes and returns plain torch tensors.  For CUDA tensors
(fp32 / bf16) the forward and the backward both run this package's sm_100a
kernels through ``torch.autograd.Function`` subclasses; for CPU tensors the
same mathematics is expressed with torch CPU ops so that the torch autograd
engine differentiates it.  There is no second GPU implementation: if the
native library is missing on a GPU machine the launchers raise.

Formulas follow the reference where it is sound (GELU tanh constants of
ferrum-nn/src/activation.rs:254-262, BCE epsilon of ferrum-nn/src/loss.rs:51-71,
mean over B*C in cross_entropy_loss, loss.rs:119-123) and are mathematically
correct where the reference's tape is not (per-row softmax / LayerNorm,
gradients through scalar ops, embedding backward).
"""
from __future__ import annotations

import math

import torch
from torch.autograd import Function

from .. import _lib, config
from ..utils import runtime as _rt
from . import gemm as _gemm

F32, BF16 = 0, 3

UNARY = {
    "none": 0, "relu": 1, "gelu": 2, "silu": 3, "tanh": 4, "sigmoid": 5, "leaky_relu": 6, "elu": 7, "neg": 8,
    "exp": 9, "log": 10, "sqrt": 11, "abs": 12, "sin": 13, "cos": 14, "pow": 15, "add_scalar": 16,
    "mul_scalar": 17, "rsub_scalar": 18, "rdiv_scalar": 19, "affine": 20, "clamp": 21,
}
_SAVES_OUTPUT = {"tanh", "sigmoid", "exp", "sqrt"}
_SAVES_NOTHING = {"neg", "add_scalar", "mul_scalar", "rsub_scalar", "affine", "none"}
BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "pow": 4, "max": 5, "min": 6}
REDUCE = {"sum": 0, "mean": 1, "max": 2, "min": 3, "prod": 4}
LOSS = {"mse": 0, "bce": 1, "l1": 2, "smooth_l1": 3}

GELU_C = 0.7978845608028654
GELU_A = 0.044715


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"kernel supports fp32 / bf16, got {t.dtype}")


def _native(t: torch.Tensor) -> bool:
    """True when `t` is handled by this package's CUDA kernels."""
    return t.is_cuda and t.dtype in (torch.float32, torch.bfloat16)


def _ptr(t):
    return None if t is None else t.data_ptr()


# =============================================================================== raw launchers
def raw_cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    if x.is_cuda and {x.dtype, dtype} == {torch.float32, torch.bfloat16}:
        x = x.contiguous()
        out = torch.empty_like(x, dtype=dtype)
        _lib.check(_lib.cuda().fb_cast(x.data_ptr(), out.data_ptr(), x.numel(), _dt(x), _dt(out), _stream()),
                   "fb_cast")
        return out
    return x.to(dtype)


def raw_unary(x: torch.Tensor, op: str, alpha: float = 0.0, beta: float = 0.0) -> torch.Tensor:
    x = x.contiguous()
    y = torch.empty_like(x)
    _lib.check(_lib.cuda().fb_unary_fwd(x.data_ptr(), y.data_ptr(), x.numel(), UNARY[op], alpha, beta, _dt(x),
                                        _stream()), "fb_unary_fwd")
    return y


def raw_unary_bwd(dy: torch.Tensor, saved, op: str, alpha: float = 0.0, beta: float = 0.0) -> torch.Tensor:
    dy = dy.contiguous()
    if saved is not None:
        saved = saved.contiguous()
        if saved.dtype != dy.dtype:
            saved = raw_cast(saved, dy.dtype)
    dx = torch.empty_like(dy)
    _lib.check(_lib.cuda().fb_unary_bwd(dy.data_ptr(), _ptr(saved), dx.data_ptr(), dy.numel(), UNARY[op], alpha,
                                        beta, _dt(dy), _stream()), "fb_unary_bwd")
    return dx


def raw_binary(a: torch.Tensor, b: torch.Tensor, op: str) -> torch.Tensor:
    """Broadcasting fp32 binary op; operands may be strided / expanded views."""
    import ctypes

    shape = torch.broadcast_shapes(a.shape, b.shape)
    if len(shape) > 6:
        a, b = a.expand(shape).reshape(-1), b.expand(shape).reshape(-1)
        shape = a.shape
    ae, be = a.expand(shape), b.expand(shape)
    out = torch.empty(shape, device=a.device, dtype=torch.float32)
    n = len(shape)
    LL = ctypes.c_longlong * max(n, 1)
    _lib.check(_lib.cuda().fb_binary_fwd(ae.data_ptr(), be.data_ptr(), out.data_ptr(), BINARY[op], n,
                                         LL(*shape) if n else LL(1), LL(*ae.stride()) if n else LL(0),
                                         LL(*be.stride()) if n else LL(0), _stream()), "fb_binary_fwd")
    return out


_scratch_cache: dict = {}


def _scratch(device, nfloats: int) -> torch.Tensor:
    """A per-device fp32 workspace reused by reductions (grown on demand)."""
    key = (device.type, device.index)
    buf = _scratch_cache.get(key)
    if buf is None or buf.numel() < nfloats:
        buf = torch.empty(max(nfloats, 1 << 16), device=device, dtype=torch.float32)
        _scratch_cache[key] = buf
    return buf


def raw_reduce(x: torch.Tensor, op: str, dim: int | None, keepdim: bool = False) -> torch.Tensor:
    x = x.contiguous()
    if dim is None:
        outer, R, inner = 1, x.numel(), 1
        oshape = [1] * x.dim() if keepdim else []
    else:
        shp = list(x.shape)
        outer = math.prod(shp[:dim])
        R = shp[dim]
        inner = math.prod(shp[dim + 1:])
        oshape = shp[:dim] + ([1] if keepdim else []) + shp[dim + 1:]
    out = torch.empty(oshape, device=x.device, dtype=torch.float32)
    if out.numel() == 0:
        return out
    lib = _lib.cuda()
    want = lib.fb_reduce_scratch_elems(outer, R, inner)
    scr = _scratch(x.device, want) if want > 0 else None
    _lib.check(lib.fb_reduce(x.data_ptr(), out.data_ptr(), outer, R, inner, REDUCE[op], _ptr(scr),
                             scr.numel() if scr is not None else 0, _stream()), "fb_reduce")
    return out


def raw_colsum(x2d: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    x2d = x2d.contiguous()
    rows, cols = x2d.shape
    if out is None:
        out = torch.empty(cols, device=x2d.device, dtype=torch.float32)
        accumulate = False
    _lib.check(_lib.cuda().fb_colsum(x2d.data_ptr(), out.data_ptr(), rows, cols, _dt(x2d), 1 if accumulate else 0,
                                     _stream()), "fb_colsum")
    return out


def _f32(x: torch.Tensor) -> torch.Tensor:
    return raw_cast(x, torch.float32) if x.is_cuda else x.float()


def reduce_to_shape(g: torch.Tensor, shape) -> torch.Tensor:
    """Sum a broadcast gradient back to the operand's shape (autograd_ops.rs:589-640)."""
    shape = tuple(shape)
    if tuple(g.shape) == shape:
        return g
    if not g.is_cuda:
        return g.sum_to_size(shape) if shape else g.sum()
    out = _f32(g)
    while out.dim() > len(shape):
        out = raw_reduce(out, "sum", 0)
    for i, s in enumerate(shape):
        if s == 1 and out.shape[i] != 1:
            out = raw_reduce(out, "sum", i, keepdim=True)
    return out


# =============================================================================== elementwise
def _unary_cpu(x, op, a, b):
    if op == "relu":
        return torch.relu(x)
    if op == "gelu":
        return 0.5 * x * (1.0 + torch.tanh(GELU_C * (x + GELU_A * x * x * x)))
    if op == "silu":
        return x * torch.sigmoid(x)
    if op == "tanh":
        return torch.tanh(x)
    if op == "sigmoid":
        return torch.sigmoid(x)
    if op == "leaky_relu":
        return torch.where(x > 0, x, x * a)
    if op == "elu":
        return torch.where(x > 0, x, a * (torch.exp(x) - 1.0))
    if op == "neg":
        return -x
    if op == "exp":
        return torch.exp(x)
    if op == "log":
        return torch.log(x)
    if op == "sqrt":
        return torch.sqrt(x)
    if op == "abs":
        return torch.abs(x)
    if op == "sin":
        return torch.sin(x)
    if op == "cos":
        return torch.cos(x)
    if op == "pow":
        return torch.pow(x, a)
    if op == "add_scalar":
        return x + a
    if op == "mul_scalar":
        return x * a
    if op == "rsub_scalar":
        return a - x
    if op == "rdiv_scalar":
        return a / x
    if op == "affine":
        return x * a + b
    if op == "clamp":
        return torch.clamp(x, a, b)
    if op == "none":
        return x
    raise ValueError(op)


class _UnaryFn(Function):
    @staticmethod
    def forward(ctx, x, op, alpha, beta):
        y = raw_unary(x, op, alpha, beta)
        ctx.op, ctx.alpha, ctx.beta = op, alpha, beta
        if op in _SAVES_NOTHING:
            ctx.save_for_backward()
        elif op in _SAVES_OUTPUT:
            ctx.save_for_backward(y)
        else:
            ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, g):
        saved = ctx.saved_tensors[0] if ctx.saved_tensors else None
        return raw_unary_bwd(g, saved, ctx.op, ctx.alpha, ctx.beta), None, None, None


def unary(x: torch.Tensor, op: str, alpha: float = 0.0, beta: float = 0.0) -> torch.Tensor:
    if _native(x):
        return _UnaryFn.apply(x, op, float(alpha), float(beta))
    return _unary_cpu(x, op, alpha, beta)


_SCALAR_TO_UNARY = {"add": "add_scalar", "mul": "mul_scalar", "rsub": "rsub_scalar", "rdiv": "rdiv_scalar"}


def scalar_op(x: torch.Tensor, op: str, s: float) -> torch.Tensor:
    """x (op) s for op in add / sub / mul / div / pow / rsub / rdiv — differentiable (unlike tensor.rs:1551-1591)."""
    if op == "sub":
        op, s = "add", -s
    elif op == "div":
        op, s = "mul", 1.0 / s
    if op == "pow":
        return unary(x, "pow", s)
    if op in ("max", "min"):
        return unary(x, "clamp", s if op == "max" else -3.0e38, 3.0e38 if op == "max" else s)
    return unary(x, _SCALAR_TO_UNARY[op], s)


class _BinaryFn(Function):
    @staticmethod
    def forward(ctx, a, b, op):
        af, bf = _f32(a), _f32(b)
        out = raw_binary(af, bf, op)
        ctx.op = op
        ctx.dtypes = (a.dtype, b.dtype)
        ctx.shapes = (a.shape, b.shape)
        if op in ("add", "sub"):
            ctx.save_for_backward()
        elif op in ("pow",):
            ctx.save_for_backward(af, bf, out)
        else:
            ctx.save_for_backward(af, bf)
        rd = torch.promote_types(a.dtype, b.dtype)
        return raw_cast(out, rd)

    @staticmethod
    def backward(ctx, g):
        op = ctx.op
        g = _f32(g.contiguous())
        need_a, need_b = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        ga = gb = None
        if op in ("add", "sub"):
            if need_a:
                ga = g
            if need_b:
                gb = g if op == "add" else raw_unary(g, "neg")
        else:
            a, b = ctx.saved_tensors[0], ctx.saved_tensors[1]
            if op == "mul":
                ga = raw_binary(g, b, "mul") if need_a else None
                gb = raw_binary(g, a, "mul") if need_b else None
            elif op == "div":
                ga = raw_binary(g, b, "div") if need_a else None
                if need_b:
                    q = raw_binary(raw_binary(g, a, "mul"), raw_binary(b, b, "mul"), "div")
                    gb = raw_unary(q, "neg")
            elif op == "pow":
                out = ctx.saved_tensors[2]
                if need_a:  # b * a^(b-1) = b * out / a
                    ga = raw_binary(g, raw_binary(raw_binary(b, out, "mul"), a, "div"), "mul")
                if need_b:
                    gb = raw_binary(g, raw_binary(out, raw_unary(a, "log"), "mul"), "mul")
            else:  # max / min: gradient goes to the selected operand (ties -> a)
                sel = (a >= b) if op == "max" else (a <= b)
                self_mask = sel.to(torch.float32)
                if need_a:
                    ga = raw_binary(g, self_mask, "mul")
                if need_b:
                    gb = raw_binary(g, raw_unary(self_mask, "rsub_scalar", 1.0), "mul")
        if ga is not None:
            ga = raw_cast(reduce_to_shape(ga, ctx.shapes[0]), ctx.dtypes[0])
        if gb is not None:
            gb = raw_cast(reduce_to_shape(gb, ctx.shapes[1]), ctx.dtypes[1])
        return ga, gb, None


def _binary_cpu(a, b, op):
    if op == "add":
        return a + b
    if op == "sub":
        return a - b
    if op == "mul":
        return a * b
    if op == "div":
        return a / b
    if op == "pow":
        return torch.pow(a, b)
    if op == "max":
        return torch.maximum(a, b)
    if op == "min":
        return torch.minimum(a, b)
    raise ValueError(op)


def binary(a: torch.Tensor, b: torch.Tensor, op: str) -> torch.Tensor:
    if _native(a) and _native(b):
        return _BinaryFn.apply(a, b, op)
    return _binary_cpu(a, b, op)


class _CastFn(Function):
    @staticmethod
    def forward(ctx, x, dtype):
        ctx.src = x.dtype
        return raw_cast(x, dtype)

    @staticmethod
    def backward(ctx, g):
        return raw_cast(g, ctx.src), None


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    if x.is_cuda and {x.dtype, dtype} == {torch.float32, torch.bfloat16}:
        return _CastFn.apply(x, dtype)
    return x.to(dtype)


def cat(tensors, dim: int = 0) -> torch.Tensor:
    """Concatenation is pure data movement (async device copies); torch provides the CatBackward split."""
    return torch.cat(list(tensors), dim)


# =============================================================================== reductions
class _ReduceFn(Function):
    @staticmethod
    def forward(ctx, x, op, dim, keepdim):
        xf = _f32(x)
        y = raw_reduce(xf, op, dim, True)
        ctx.op, ctx.dim, ctx.keepdim, ctx.src_dtype = op, dim, keepdim, x.dtype
        ctx.xshape = x.shape
        if op in ("max", "min", "prod"):
            ctx.save_for_backward(xf, y)
        else:
            ctx.save_for_backward()
        out = y if keepdim else (y.reshape(()) if dim is None else y.squeeze(dim))
        return raw_cast(out, x.dtype)

    @staticmethod
    def backward(ctx, g):
        op, dim = ctx.op, ctx.dim
        g = _f32(g)
        kshape = [1] * len(ctx.xshape) if dim is None else [
            1 if i == dim else s for i, s in enumerate(ctx.xshape)]
        gk = g.reshape(kshape)
        if op == "sum":
            gx = gk.expand(ctx.xshape)
        elif op == "mean":
            R = math.prod(ctx.xshape) if dim is None else ctx.xshape[dim]
            gx = raw_unary(gk, "mul_scalar", 1.0 / max(R, 1)).expand(ctx.xshape)
        elif op in ("max", "min"):
            x, y = ctx.saved_tensors
            mask = (x == y).to(torch.float32)
            gx = raw_binary(gk, mask, "mul")
        else:  # prod: d/dx_i = prod / x_i
            x, y = ctx.saved_tensors
            gx = raw_binary(raw_binary(gk, y, "mul"), x, "div")
        if gx.dtype != ctx.src_dtype:
            gx = raw_cast(gx.contiguous(), ctx.src_dtype)
        return gx, None, None, None


def reduce(x: torch.Tensor, op: str, dim: int | None = None, keepdim: bool = False) -> torch.Tensor:
    if _native(x) and x.numel() > 0:
        return _ReduceFn.apply(x, op, dim, keepdim)
    if dim is None:
        fn = {"sum": torch.sum, "mean": torch.mean, "max": torch.max, "min": torch.min, "prod": torch.prod}[op]
        out = fn(x)
        return out.reshape([1] * x.dim()) if keepdim else out
    if op in ("max", "min"):
        return getattr(torch, op)(x, dim=dim, keepdim=keepdim).values
    return getattr(torch, op)(x, dim=dim, keepdim=keepdim)


def arg_reduce(x: torch.Tensor, is_max: bool, dim: int | None = None, keepdim: bool = False) -> torch.Tensor:
    """Index of the first maximum / minimum (tensor.rs:1838-2036)."""
    if _native(x) and x.numel() > 0:
        xf = _f32(x).contiguous()
        if dim is None:
            outer, R, inner, oshape = 1, xf.numel(), 1, []
        else:
            shp = list(xf.shape)
            outer, R, inner = math.prod(shp[:dim]), shp[dim], math.prod(shp[dim + 1:])
            oshape = shp[:dim] + ([1] if keepdim else []) + shp[dim + 1:]
        idx = torch.empty(oshape, device=x.device, dtype=torch.int64)
        _lib.check(_lib.cuda().fb_arg_reduce(xf.data_ptr(), idx.data_ptr(), None, outer, R, inner,
                                             1 if is_max else 0, _stream()), "fb_arg_reduce")
        return idx
    fn = torch.argmax if is_max else torch.argmin
    return fn(x) if dim is None else fn(x, dim=dim, keepdim=keepdim)


# =============================================================================== GEMM-shaped ops
def _gemm_nt(a: torch.Tensor, b_nt: torch.Tensor, bias=None, act=None, low: bool = False, out=None,
             out_dtype=None, accumulate=False) -> torch.Tensor:
    """out = act(a @ b_nt^T + bias) with a [M,K], b_nt [N,K] (any strides)."""
    if low:
        ab = a if a.dtype == torch.bfloat16 else raw_cast(a.contiguous(), torch.bfloat16)
        bb = b_nt if b_nt.dtype == torch.bfloat16 else raw_cast(b_nt.contiguous(), torch.bfloat16)
        if not _gemm.bf16_operand_ok(ab):
            ab = ab.contiguous()
        if not _gemm.bf16_operand_ok(bb):
            bb = bb.contiguous()
        if _gemm.bf16_operand_ok(ab) and _gemm.bf16_operand_ok(bb):
            return _gemm.gemm_bf16(ab, bb, bias=bias, act=act, out=out,
                                   out_dtype=out_dtype or torch.bfloat16, accumulate=accumulate)
        # row pitch not a multiple of 16 bytes: exact SIMT kernel on fp32 copies
        res = _gemm.gemm_f32(_f32(ab), _f32(bb), bias=bias, act=act, out=out if out is not None and
                             out.dtype == torch.float32 else None, accumulate=accumulate and out is not None)
        if out is not None and out.dtype != torch.float32:
            out.copy_(res)
            return out
        return raw_cast(res, out_dtype or torch.bfloat16)
    af, bf = _f32(a), _f32(b_nt)
    if (config.tf32_active() and _gemm.tf32_operand_ok(af) and _gemm.tf32_operand_ok(bf)
            and (out is None or (out.dtype == torch.float32 and out.stride(-1) == 1))
            and (bias is None or bias.dtype == torch.float32)):
        return _gemm.gemm_tf32(af, bf, bias=bias, act=act, out=out, accumulate=accumulate)
    res = _gemm.gemm_f32(af, bf, bias=bias, act=act, out=out, accumulate=accumulate)
    return res


class _MatmulFn(Function):
    @staticmethod
    def forward(ctx, a, b, low):
        ctx.low = low
        ctx.dtypes = (a.dtype, b.dtype)
        if low:
            a = raw_cast(a.contiguous(), torch.bfloat16)
            b = raw_cast(b.contiguous(), torch.bfloat16)
        ctx.save_for_backward(a, b)
        out = _gemm_nt(a, b.t(), low=low)
        return out if low else raw_cast(out, torch.promote_types(*ctx.dtypes))

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        low = ctx.low
        g = g.contiguous()
        if low and g.dtype != torch.bfloat16:
            g = raw_cast(g, torch.bfloat16)
        ga = gb = None
        if ctx.needs_input_grad[0]:
            ga = raw_cast(_gemm_nt(g, b, low=low), ctx.dtypes[0])
        if ctx.needs_input_grad[1]:
            gb = raw_cast(_gemm_nt(a.t(), g.t(), low=low, out_dtype=torch.float32), ctx.dtypes[1])
        return ga, gb, None


class _BmmFn(Function):
    """Batched fp32 matmul on the SIMT kernel (grid.z = batch)."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return _gemm.gemm_f32(a, b.transpose(1, 2))

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        g = g.contiguous()
        ga = _gemm.gemm_f32(g, b) if ctx.needs_input_grad[0] else None
        gb = _gemm.gemm_f32(a.transpose(1, 2), g.transpose(1, 2)) if ctx.needs_input_grad[1] else None
        return ga, gb


def _bmm_operand(t):
    t = t if t.dtype == torch.bfloat16 else raw_cast(t, torch.bfloat16)
    return t if _gemm.batched_operand_ok(t) else t.contiguous()


class _BmmLowFn(Function):
    """Batched ``alpha * a @ b`` over 4-D operands on the tcgen05 kernel (bf16 in, bf16 out, fp32 accumulate);
    strided views (heads interleaved in the feature dimension, transposes) are consumed without copies."""

    @staticmethod
    def forward(ctx, a, b, alpha, heads_inner=False):
        a, b = _bmm_operand(a), _bmm_operand(b)
        ctx.save_for_backward(a, b)
        ctx.alpha = alpha
        bt = b.transpose(-1, -2)
        out = None
        if heads_inner:  # result stored [Bo, M, Bi, N] so that merging the heads afterwards is a view
            Bo, Bi, M, _ = a.shape
            out = torch.empty((Bo, M, Bi, b.shape[-1]), device=a.device, dtype=torch.bfloat16).permute(0, 2, 1, 3)
        return _gemm.gemm_bf16_batched(a, bt if _gemm.batched_operand_ok(bt) else bt.contiguous(), out=out,
                                       alpha=alpha)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        g = _bmm_operand(g)
        ga = gb = None
        if ctx.needs_input_grad[0]:   # dA = alpha * g @ b^T
            ga = _gemm.gemm_bf16_batched(g, b, alpha=ctx.alpha)
        if ctx.needs_input_grad[1]:   # dB = alpha * a^T @ g
            gb = _gemm.gemm_bf16_batched(a.transpose(-1, -2), g.transpose(-1, -2), alpha=ctx.alpha)
        return ga, gb, None, None


def bmm_scaled(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, heads_inner: bool = False) -> torch.Tensor:
    """``alpha * a @ b`` for 4-D ``[Bo, Bi, M, K] @ [Bo, Bi, K, N]``: tensor cores under autocast for TMA-describable
    operands (feature extents multiples of 8), the fp32 batched kernel otherwise.  ``heads_inner`` stores the
    result as ``[Bo, M, Bi, N]`` (returned as the permuted view)."""
    if (_native(a) and _native(b) and config.low_precision_active() and a.shape[-1] % 8 == 0
            and b.shape[-1] % 8 == 0):
        return _BmmLowFn.apply(a, b, float(alpha), heads_inner)
    out = matmul(a, b)
    return scalar_op(out, "mul", float(alpha)) if alpha != 1.0 else out


def flash_attention_ok(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, need_no_grad: bool = True,
                       head_dims=(64, 128)) -> bool:
    """True when ``flash_attention`` can take these ``[B, H, S, D]`` operands: CUDA, head dimension 64 or 128
    (``head_dims``) contiguous, other strides multiples of 8 elements and (``need_no_grad``) no gradient needed —
    the kernel records no autograd node."""
    if not (q.is_cuda and q.dim() == 4 and k.dim() == 4 and v.dim() == 4 and q.shape[-1] in head_dims):
        return False
    D = q.shape[-1]
    if need_no_grad and torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return False
    if k.shape != v.shape or q.shape[:2] != k.shape[:2] or k.shape[-1] != D:
        return False
    for t in (q, k, v):
        if t.stride(-1) != 1 or any(s % 8 for s in t.stride()[:-1]) or t.stride(2) < D:
            return False
    return True


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                    return_lse: bool = False, causal: bool = False):
    """``softmax(scale * q @ k^T) @ v`` for ``[B, H, S, D]`` operands (D = 64 or 128) without materialising the
    score matrix: one tcgen05 kernel with online softmax (csrc/kernels/attention.cu).  No autograd node is recorded
    here (:func:`attention_blockwise` is the differentiable form).  ``causal``: query ``i`` sees
    keys ``j <= i + (Skv - Sq)`` and key tiles past the diagonal are skipped.  The result is stored as
    ``[B, Sq, H, D]`` and returned as the ``[B, H, Sq, D]`` view (like ``bmm_scaled(..., heads_inner=True)``)."""
    B, H, Sq, D = q.shape
    Skv = k.shape[2]
    qb, kb, vb = (t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16) for t in (q.detach(), k.detach(), v.detach()))
    out = torch.empty((B, Sq, H, D), device=q.device, dtype=torch.bfloat16)
    lse = torch.empty((B, H, Sq), device=q.device, dtype=torch.float32) if return_lse else None
    rc = _lib.cuda().fb_attention_fwd(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), out.data_ptr(),
                                      lse.data_ptr() if lse is not None else None, B, H, Sq, Skv, D,
                                      qb.stride(0), qb.stride(1), qb.stride(2), kb.stride(0), kb.stride(1),
                                      kb.stride(2), vb.stride(0), vb.stride(1), vb.stride(2), float(scale),
                                      1 if causal else 0, _rt.status_ptr(), _stream())
    _lib.check(rc, "fb_attention_fwd")
    res = out.permute(0, 2, 1, 3)
    return (res, lse) if return_lse else res


class _BlockwiseAttentionFn(Function):
    """``softmax(scale q k^T) v`` with the blockwise tcgen05 kernels in BOTH directions: the forward saves q, k, v,
    the output and one log-sum-exp per row; the backward recomputes the probabilities tile by tile
    (csrc/kernels/attention_bwd.cu).  Nothing of size S x S is ever stored."""

    @staticmethod
    def forward(ctx, q, k, v, scale, causal):
        out, lse = flash_attention(q, k, v, scale, return_lse=True, causal=causal)
        qb, kb, vb = (t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16) for t in (q, k, v))
        ctx.save_for_backward(qb, kb, vb, out, lse)
        ctx.scale, ctx.causal = scale, causal
        ctx.in_dtypes = (q.dtype, k.dtype, v.dtype)
        return out

    @staticmethod
    def backward(ctx, g):
        q, k, v, out, lse = ctx.saved_tensors
        B, H, Sq, D = q.shape
        Skv = k.shape[2]
        o = out.permute(0, 2, 1, 3)                      # the kernel's own [B, Sq, H, D] storage
        if not o.is_contiguous():
            o = o.contiguous()
        go = g.permute(0, 2, 1, 3)
        if go.dtype != torch.bfloat16 or not go.is_contiguous():
            go = go.to(torch.bfloat16).contiguous()
        dq = torch.empty((B, Sq, H, D), device=q.device, dtype=torch.bfloat16)
        dk = torch.empty((B, Skv, H, D), device=q.device, dtype=torch.bfloat16)
        dv = torch.empty((B, Skv, H, D), device=q.device, dtype=torch.bfloat16)
        delta = torch.empty((B, H, Sq), device=q.device, dtype=torch.float32)
        rc = _lib.cuda().fb_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), go.data_ptr(),
                                          lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                          dv.data_ptr(), B, H, Sq, Skv, D, q.stride(0), q.stride(1), q.stride(2),
                                          k.stride(0), k.stride(1), k.stride(2), v.stride(0), v.stride(1),
                                          v.stride(2), float(ctx.scale), 1 if ctx.causal else 0, _rt.status_ptr(),
                                          _stream())
        if -5 <= rc <= -2:  # an operand that no TMA map describes: name it
            name, t = {-2: ("q", q), -3: ("k", k), -4: ("v", v), -5: ("grad_output", go)}[rc]
            raise ValueError(f"fb_attention_bwd: {name} of shape {tuple(t.shape)}, strides {t.stride()}, address "
                             f"{t.data_ptr():#x} cannot be a TMA operand (16-byte aligned pointer, strides multiples of 8; "
                             f"reason {_lib.cuda().fb_attention_bwd_map_error()})")
        _lib.check(rc, "fb_attention_bwd")
        grads = [t.permute(0, 2, 1, 3) for t in (dq, dk, dv)]
        grads = [gr if gr.dtype == dt else gr.to(dt) for gr, dt in zip(grads, ctx.in_dtypes)]
        return grads[0], grads[1], grads[2], None, None


def attention_blockwise(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                        causal: bool = False) -> torch.Tensor:
    """Differentiable blockwise attention for ``[B, H, S, D]`` operands, D = 64 or 128 (see ``flash_attention_ok``):
    forward and backward on the tcgen05 kernels, no S x S matrix in memory in either direction."""
    return _BlockwiseAttentionFn.apply(q, k, v, float(scale), bool(causal))


class _CheckpointedAttentionFn(Function):
    """Attention core with the blockwise kernel in the forward pass and NOTHING of size S x S kept for the backward
    pass: the backward recomputes the scores with the differentiable batched-GEMM path (activation checkpointing
    of the attention core).  Trades one extra score computation for S x S x heads of saved activations."""

    @staticmethod
    def forward(ctx, q, k, v, scale):
        ctx.scale = scale
        ctx.save_for_backward(q, k, v)
        return flash_attention(q, k, v, scale)

    @staticmethod
    def backward(ctx, g):
        q, k, v = ctx.saved_tensors
        # the backward pass runs outside the caller's autocast block: re-enter it for the recomputation
        with torch.enable_grad(), config.autocast():
            qd, kd, vd = (t.detach().requires_grad_(True) for t in (q, k, v))
            attn = softmax(bmm_scaled(qd, kd.transpose(-1, -2), ctx.scale), -1)
            out = bmm_scaled(attn, vd, 1.0, heads_inner=True)
            gq, gk, gv = torch.autograd.grad(out, (qd, kd, vd), g.to(out.dtype))
        return gq, gk, gv, None


def attention_checkpointed(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """Differentiable ``softmax(scale q k^T) v`` that saves only q, k, v (see ``_CheckpointedAttentionFn``);
    operands as for :func:`flash_attention`."""
    return _CheckpointedAttentionFn.apply(q, k, v, float(scale))


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """2D@2D, 2D@1D, 1D@2D (tensor.rs:2433-2485) and batched ND@ND / ND@2D."""
    if not (_native(a) and _native(b)):
        return torch.matmul(a, b)
    low = config.low_precision_active()
    if a.dim() == 1 and b.dim() == 1:
        return reduce(binary(a, b, "mul"), "sum")
    if a.dim() == 1:
        return matmul(a.unsqueeze(0), b).squeeze(-2)
    if b.dim() == 1:
        return matmul(a, b.unsqueeze(1)).squeeze(-1)
    if a.dim() == 2 and b.dim() == 2:
        return _MatmulFn.apply(a, b, low)
    if b.dim() == 2:  # [..., M, K] @ [K, N]
        lead = a.shape[:-1]
        return _MatmulFn.apply(a.reshape(-1, a.shape[-1]), b, low).reshape(*lead, b.shape[1])
    # batched: broadcast batch dims; tensor cores under autocast, else the fp32 batched kernel
    bs = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
    if low and a.shape[-1] % 8 == 0 and b.shape[-1] % 8 == 0:
        a4 = a.expand(*bs, *a.shape[-2:]).reshape(1, -1, *a.shape[-2:])
        b4 = b.expand(*bs, *b.shape[-2:]).reshape(1, -1, *b.shape[-2:])
        return _BmmLowFn.apply(a4, b4, 1.0).reshape(*bs, a.shape[-2], b.shape[-1])
    a3 = _f32(a.expand(*bs, *a.shape[-2:]).reshape(-1, *a.shape[-2:]).contiguous())
    b3 = _f32(b.expand(*bs, *b.shape[-2:]).reshape(-1, *b.shape[-2:]).contiguous())
    out = _BmmFn.apply(a3, b3)
    return raw_cast(out.reshape(*bs, a.shape[-2], b.shape[-1]), torch.promote_types(a.dtype, b.dtype))


class GradSink:
    """Where a Linear's weight gradient is written.

    ``acquire(param)`` returns ``(buffer, accumulate)``: an fp32 tensor shaped like
    the parameter and whether the wgrad GEMM must add to its contents; ``ready(param)``
    is called once the gradient is enqueued on the current stream.  The DDP engine
    implements this to have wgrad written straight into its flat gradient arena.
    """

    def acquire(self, param):  # pragma: no cover - interface
        raise NotImplementedError

    def ready(self, param):  # pragma: no cover - interface
        raise NotImplementedError


def _wgrad_to_sink(sink, weight_ref, g_t: torch.Tensor, x_t: torch.Tensor, low: bool) -> None:
    """dW = g_t @ x_t^T written where the sink wants it: pushed to the shard owners from the GEMM epilogue when the
    sink supports that (data-parallel engine in push mode, bf16 operands), else into the sink's buffer."""
    push = getattr(sink, "try_push", None)
    if push is not None and low and g_t.dtype == torch.bfloat16 and x_t.dtype == torch.bfloat16 and push(
            weight_ref, g_t, x_t):
        return
    buf, acc = sink.acquire(weight_ref)
    _gemm_nt(g_t, x_t, low=low, out=buf, out_dtype=torch.float32, accumulate=acc)


class _LinearFn(Function):
    @staticmethod
    def forward(ctx, x, weight, bias, act, low, w_low, sink):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        ctx.low, ctx.act, ctx.sink = low, act, sink
        ctx.x_dtype, ctx.lead = x.dtype, lead
        ctx.has_bias = bias is not None
        ctx.weight_ref = weight
        if low:
            xb = x2 if x2.dtype == torch.bfloat16 else raw_cast(x2.contiguous(), torch.bfloat16)
            wb = w_low if w_low is not None else raw_cast(weight.detach().contiguous(), torch.bfloat16)
            y = _gemm_nt(xb, wb, bias=bias, act=act, low=True)
            saved_x, saved_w = xb, wb
        else:
            xf = _f32(x2)
            y = _gemm_nt(xf, weight.detach(), bias=bias, act=act, low=False)
            saved_x, saved_w = xf, weight.detach()
        if act is None:
            ctx.save_for_backward(saved_x, saved_w)
        else:
            ctx.save_for_backward(saved_x, saved_w, y)
        return y.reshape(*lead, weight.shape[0])

    @staticmethod
    def backward(ctx, g):
        low, act = ctx.low, ctx.act
        saved = ctx.saved_tensors
        x2, w = saved[0], saved[1]
        g2 = g.reshape(-1, g.shape[-1]).contiguous()
        if low and g2.dtype != torch.bfloat16:
            g2 = raw_cast(g2, torch.bfloat16)
        if not low:
            g2 = _f32(g2)
        if act is not None:
            # only activations whose derivative is a function of the output are fused here
            g2 = raw_unary_bwd(g2, saved[2], act)
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:  # dgrad first: the weight may be overwritten once its bucket is reduced
            gx = _gemm_nt(g2, w.t(), low=low)
            gx = raw_cast(gx, ctx.x_dtype).reshape(*ctx.lead, w.shape[1])
        if ctx.needs_input_grad[1]:
            sink = ctx.sink
            if sink is not None:
                _wgrad_to_sink(sink, ctx.weight_ref, g2.t(), x2.t(), low)
            else:
                gw = _gemm_nt(g2.t(), x2.t(), low=low, out_dtype=torch.float32)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = raw_colsum(g2)
        if ctx.needs_input_grad[1] and ctx.sink is not None:
            ctx.sink.ready(ctx.weight_ref)
        return gx, gw, gb, None, None, None, None


_FUSABLE_ACT = {"relu", "tanh", "sigmoid"}  # derivative expressible from the output


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, act: str | None = None,
           w_low: torch.Tensor | None = None, sink: GradSink | None = None) -> torch.Tensor:
    """``act(x @ weight^T + bias)`` with weight ``[out, in]`` (ferrum-nn/src/linear.rs:78-89).

    On CUDA the bias (and relu/tanh/sigmoid) run in the GEMM epilogue.  ``w_low`` is an
    up-to-date bf16 copy of ``weight`` (kept by the optimizer) used under bf16 precision.
    """
    if not _native(x):
        y = torch.nn.functional.linear(x, weight, bias)
        return _unary_cpu(y, act, 0.0, 0.0) if act else y
    low = config.low_precision_active()
    needs_grad = torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad)
    if act is not None and act not in _FUSABLE_ACT and needs_grad:
        y = _LinearFn.apply(x, weight, bias, None, low, w_low, sink)
        return unary(y, act)
    return _LinearFn.apply(x, weight, bias, act, low, w_low, sink)


# =============================================================================== normalisation
class _LayerNormFn(Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, pre_act, want_colsum):
        cols = x.shape[-1]
        x2 = x.reshape(-1, cols).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, device=x.device, dtype=torch.float32)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        g = gamma.detach().contiguous() if gamma is not None else None
        b = beta.detach().contiguous() if beta is not None else None
        _rt.status_ptr()  # the wide-row kernels report bounded-wait failures to the status block
        _lib.check(_lib.cuda().fb_layernorm_fwd(x2.data_ptr(), _ptr(g), _ptr(b), y.data_ptr(), mean.data_ptr(),
                                                rstd.data_ptr(), rows, cols, eps, UNARY[pre_act or "none"],
                                                _dt(x2), _stream()), "fb_layernorm_fwd")
        ctx.save_for_backward(x2, g, mean, rstd)
        ctx.pre_act, ctx.shape, ctx.want_colsum = pre_act, x.shape, want_colsum
        ctx.has_gamma, ctx.has_beta = gamma is not None, beta is not None
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, gy):
        x2, g, mean, rstd = ctx.saved_tensors
        rows, cols = x2.shape
        gy2 = gy.reshape(rows, cols).contiguous()
        if gy2.dtype != x2.dtype:
            gy2 = raw_cast(gy2, x2.dtype)
        lib = _lib.cuda()
        dx = torch.empty_like(x2)
        nblk = lib.fb_layernorm_bwd_blocks(rows, cols)
        partial = torch.empty((max(nblk, 1), 3, cols), device=x2.device, dtype=torch.float32)
        stats = torch.zeros((3, cols), device=x2.device, dtype=torch.float32)
        _lib.check(lib.fb_layernorm_bwd(gy2.data_ptr(), x2.data_ptr(), None, _ptr(g), mean.data_ptr(), rstd.data_ptr(),
                                        dx.data_ptr(), partial.data_ptr(), stats.data_ptr(), rows, cols,
                                        UNARY[ctx.pre_act or "none"], _dt(x2), nblk, 1 if ctx.want_colsum else 0,
                                        _stream()), "fb_layernorm_bwd")
        dgamma = stats[0] if ctx.has_gamma else None
        dbeta = stats[1] if ctx.has_beta else None
        dcol = stats[2] if ctx.want_colsum else None
        ctx.colsum = dcol
        return dx.reshape(ctx.shape), dgamma, dbeta, None, None, None


def layer_norm(x: torch.Tensor, gamma=None, beta=None, eps: float = 1e-5, pre_act: str | None = None,
               n_norm_dims: int = 1) -> torch.Tensor:
    """Normalise over the last ``n_norm_dims`` dimensions; optional fused GELU before the statistics."""
    if n_norm_dims != 1:
        lead = x.shape[:-n_norm_dims]
        flat = x.reshape(*lead, -1)
        g = gamma.reshape(-1) if gamma is not None else None
        b = beta.reshape(-1) if beta is not None else None
        return layer_norm(flat, g, b, eps, pre_act, 1).reshape(x.shape)
    if _native(x):
        return _LayerNormFn.apply(x, gamma, beta, float(eps), pre_act, False)
    a = _unary_cpu(x, pre_act, 0.0, 0.0) if pre_act else x
    mu = a.mean(-1, keepdim=True)
    var = ((a - mu) ** 2).mean(-1, keepdim=True)
    y = (a - mu) / torch.sqrt(var + eps)
    if gamma is not None:
        y = y * gamma
    if beta is not None:
        y = y + beta
    return y


class _LinearActNormFn(Function):
    """One autograd node for the block ``LayerNorm(act(x W^T + b))``.

    Forward (tensor-core path): the GEMM epilogue writes act(z) and act'(z) in bf16, the LayerNorm kernel reads
    act(z) and writes y.  Backward: one streaming kernel turns dy into dz (using the stored derivative) and also
    yields d_gamma, d_beta and the column sum of dz (= the bias gradient), then the dgrad and wgrad GEMMs run on
    dz.  On the fp32 path z itself is stored and the activation is evaluated inside the normalisation kernels.
    """

    @staticmethod
    def forward(ctx, x, weight, bias, gamma, beta, eps, act, low, w_low, sink):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if low:
            xs = x2 if x2.dtype == torch.bfloat16 else raw_cast(x2.contiguous(), torch.bfloat16)
            ws = w_low if w_low is not None else raw_cast(weight.detach().contiguous(), torch.bfloat16)
        else:
            xs, ws = _f32(x2), weight.detach()
        # Tensor-core path: the GEMM epilogue stores act(z) and act'(z), so the normalisation kernels are pure
        # streaming code.  fp32 path: z is stored and the GELU is evaluated inside the normalisation kernels.
        dual = low and act is not None and xs.dtype == torch.bfloat16 and _gemm.bf16_operand_ok(xs) \
            and _gemm.bf16_operand_ok(ws)
        if dual:
            z = torch.empty((xs.shape[0], ws.shape[0]), device=xs.device, dtype=torch.bfloat16)
            dact = torch.empty_like(z)
            _gemm.gemm_bf16(xs, ws, bias=bias, act=act, out=z, act_grad=dact)
            pre = "none"
        else:
            z = _gemm_nt(xs, ws, bias=bias, act=None, low=low)
            dact, pre = None, act or "none"
        rows, cols = z.shape
        y = torch.empty_like(z)
        mean = torch.empty(rows, device=z.device, dtype=torch.float32)
        rstd = torch.empty(rows, device=z.device, dtype=torch.float32)
        g = gamma.detach().contiguous()
        b = beta.detach().contiguous()
        _rt.status_ptr()  # the wide-row kernels report bounded-wait failures to the status block
        _lib.check(_lib.cuda().fb_layernorm_fwd(z.data_ptr(), g.data_ptr(), b.data_ptr(), y.data_ptr(),
                                                mean.data_ptr(), rstd.data_ptr(), rows, cols, eps, UNARY[pre], _dt(z),
                                                _stream()), "fb_layernorm_fwd")
        if dual:
            ctx.save_for_backward(xs, ws, z, g, mean, rstd, dact)
        else:
            ctx.save_for_backward(xs, ws, z, g, mean, rstd)
        ctx.dual = dual
        ctx.low, ctx.act, ctx.sink, ctx.weight_ref = low, pre, sink, weight
        ctx.x_dtype, ctx.lead, ctx.has_bias = x.dtype, lead, bias is not None
        return y.reshape(*lead, cols)

    @staticmethod
    def backward(ctx, gy):
        if ctx.dual:
            xs, ws, z, g, mean, rstd, dact = ctx.saved_tensors
        else:
            xs, ws, z, g, mean, rstd = ctx.saved_tensors
            dact = None
        rows, cols = z.shape
        low = ctx.low
        gy2 = gy.reshape(rows, cols).contiguous()
        if gy2.dtype != z.dtype:
            gy2 = raw_cast(gy2, z.dtype)
        lib = _lib.cuda()
        dz = torch.empty_like(z)
        nblk = lib.fb_layernorm_bwd_blocks(rows, cols)
        partial = torch.empty((max(nblk, 1), 3, cols), device=z.device, dtype=torch.float32)
        stats = torch.zeros((3, cols), device=z.device, dtype=torch.float32)  # d_gamma, d_beta, colsum(dz)
        _lib.check(lib.fb_layernorm_bwd(gy2.data_ptr(), z.data_ptr(), _ptr(dact), g.data_ptr(), mean.data_ptr(),
                                        rstd.data_ptr(), dz.data_ptr(), partial.data_ptr(), stats.data_ptr(), rows,
                                        cols, UNARY[ctx.act], _dt(z), nblk, 1, _stream()), "fb_layernorm_bwd")
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = raw_cast(_gemm_nt(dz, ws.t(), low=low), ctx.x_dtype).reshape(*ctx.lead, ws.shape[1])
        if ctx.needs_input_grad[1]:
            if ctx.sink is not None:
                _wgrad_to_sink(ctx.sink, ctx.weight_ref, dz.t(), xs.t(), low)
                ctx.sink.ready(ctx.weight_ref)
            else:
                gw = _gemm_nt(dz.t(), xs.t(), low=low, out_dtype=torch.float32)
        gb = stats[2] if ctx.has_bias else None
        return gx, gw, gb, stats[0], stats[1], None, None, None, None, None


def linear_act_layernorm(x, weight, bias, gamma, beta, eps: float = 1e-5, act: str = "gelu", w_low=None,
                         sink: GradSink | None = None):
    """``LayerNorm(act(x @ weight^T + bias)) * gamma + beta`` as one fused block (CUDA); composed ops on CPU."""
    if _native(x) and gamma is not None and beta is not None:
        return _LinearActNormFn.apply(x, weight, bias, gamma, beta, float(eps), act, config.low_precision_active(),
                                      w_low, sink)
    return layer_norm(linear(x, weight, bias, None, w_low, sink), gamma, beta, eps, act)


class _BatchNormFn(Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, running_mean, running_var, eps, momentum, training):
        x2 = _f32(x).contiguous()
        rows, cols = x2.shape
        y = torch.empty_like(x2)
        sm = torch.empty(cols, device=x.device, dtype=torch.float32)
        sr = torch.empty(cols, device=x.device, dtype=torch.float32)
        g = gamma.detach().contiguous() if gamma is not None else None
        b = beta.detach().contiguous() if beta is not None else None
        _lib.check(_lib.cuda().fb_batchnorm_fwd(x2.data_ptr(), _ptr(g), _ptr(b), y.data_ptr(), sm.data_ptr(),
                                                sr.data_ptr(), _ptr(running_mean), _ptr(running_var), rows, cols,
                                                eps, momentum, 1 if training else 0, _stream()),
                   "fb_batchnorm_fwd")
        if not training:
            sm = running_mean.detach().clone()
            sr = torch.rsqrt(running_var.detach() + eps)
        ctx.save_for_backward(x2, g, sm, sr)
        ctx.training = training
        ctx.flags = (gamma is not None, beta is not None)
        ctx.src_dtype = x.dtype
        return raw_cast(y, x.dtype)

    @staticmethod
    def backward(ctx, gy):
        x2, g, sm, sr = ctx.saved_tensors
        rows, cols = x2.shape
        gy2 = _f32(gy).contiguous()
        if ctx.training:
            dx = torch.empty_like(x2)
            dgamma = torch.empty(cols, device=x2.device, dtype=torch.float32)
            dbeta = torch.empty(cols, device=x2.device, dtype=torch.float32)
            _lib.check(_lib.cuda().fb_batchnorm_bwd(gy2.data_ptr(), x2.data_ptr(), _ptr(g), sm.data_ptr(),
                                                    sr.data_ptr(), dx.data_ptr(), dgamma.data_ptr(),
                                                    dbeta.data_ptr(), rows, cols, _stream()), "fb_batchnorm_bwd")
        else:  # statistics are constants in eval mode
            scale = sr if g is None else raw_binary(sr, g, "mul")
            dx = raw_binary(gy2, scale, "mul")
            xhat = raw_binary(raw_binary(x2, sm, "sub"), sr, "mul")
            dgamma = raw_reduce(raw_binary(gy2, xhat, "mul"), "sum", 0)
            dbeta = raw_reduce(gy2, "sum", 0)
        return (raw_cast(dx, ctx.src_dtype), dgamma if ctx.flags[0] else None, dbeta if ctx.flags[1] else None,
                None, None, None, None, None)


def batch_norm(x: torch.Tensor, gamma, beta, running_mean, running_var, training: bool, momentum: float = 0.1,
               eps: float = 1e-5) -> torch.Tensor:
    """Per-feature batch normalisation of ``[B, F]`` input with running-stat update."""
    if x.dim() != 2:
        raise ValueError("batch_norm expects [batch, features]")
    if _native(x):
        return _BatchNormFn.apply(x, gamma, beta, running_mean, running_var, float(eps), float(momentum),
                                  bool(training))
    if training:
        mu = x.mean(0)
        var = ((x - mu) ** 2).mean(0)
        if running_mean is not None:
            with torch.no_grad():
                n = x.shape[0]
                running_mean.mul_(1 - momentum).add_(momentum * mu.detach())
                running_var.mul_(1 - momentum).add_(momentum * var.detach() * (n / (n - 1) if n > 1 else 1.0))
    else:
        mu, var = running_mean, running_var
    y = (x - mu) / torch.sqrt(var + eps)
    if gamma is not None:
        y = y * gamma
    if beta is not None:
        y = y + beta
    return y


# =============================================================================== softmax / losses
class _SoftmaxFn(Function):
    @staticmethod
    def forward(ctx, x, log_mode):
        cols = x.shape[-1]
        x2 = x.reshape(-1, cols).contiguous()
        y = torch.empty_like(x2)
        _lib.check(_lib.cuda().fb_softmax_fwd(x2.data_ptr(), y.data_ptr(), x2.shape[0], cols, 1 if log_mode else 0,
                                              _dt(x2), _stream()), "fb_softmax_fwd")
        ctx.save_for_backward(y)
        ctx.log_mode, ctx.shape = log_mode, x.shape
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        rows, cols = y.shape
        g2 = g.reshape(rows, cols).contiguous()
        if g2.dtype != y.dtype:
            g2 = raw_cast(g2, y.dtype)
        dx = torch.empty_like(y)
        _lib.check(_lib.cuda().fb_softmax_bwd(g2.data_ptr(), y.data_ptr(), dx.data_ptr(), rows, cols,
                                              1 if ctx.log_mode else 0, _dt(y), _stream()), "fb_softmax_bwd")
        return dx.reshape(ctx.shape), None


def _softmax_any_dim(x, dim, log_mode):
    nd = x.dim()
    if nd == 0:
        x = x.reshape(1)
        nd, dim = 1, 0
    d = dim + nd if dim < 0 else dim
    if _native(x):
        if d != nd - 1:
            return _SoftmaxFn.apply(x.transpose(d, -1), log_mode).transpose(d, -1)
        return _SoftmaxFn.apply(x, log_mode)
    return torch.log_softmax(x, d) if log_mode else torch.softmax(x, d)


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Numerically stable softmax along ``dim`` (per-row spec of ferrum-cuda/src/kernels.rs:501-560)."""
    return _softmax_any_dim(x, dim, False)


def log_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return _softmax_any_dim(x, dim, True)


class _CEFn(Function):
    """Fused log-softmax + NLL over integer labels: one kernel yields loss rows and the logit gradient."""

    @staticmethod
    def forward(ctx, logits, labels, scale):
        rows, cols = logits.shape
        lg = logits.contiguous()
        row_loss = torch.empty(rows, device=lg.device, dtype=torch.float32)
        need_grad = ctx.needs_input_grad[0]
        dl = torch.empty_like(lg) if need_grad else None
        _lib.check(_lib.cuda().fb_ce_fwd_bwd(lg.data_ptr(), labels.data_ptr(), row_loss.data_ptr(), _ptr(dl), rows,
                                             cols, scale, _dt(lg), _dt(lg), _stream()), "fb_ce_fwd_bwd")
        if need_grad:
            ctx.save_for_backward(dl)
        loss = raw_reduce(row_loss, "sum", None)
        return raw_unary(loss, "mul_scalar", scale)

    @staticmethod
    def backward(ctx, g):
        (dl,) = ctx.saved_tensors
        # dl already carries the 1/rows factor; scale by the incoming scalar gradient
        gf = _f32(g).reshape(1).contiguous()
        out = torch.empty_like(dl)
        _lib.check(_lib.cuda().fb_scale_by_device_scalar(dl.data_ptr(), gf.data_ptr(), out.data_ptr(), dl.numel(),
                                                         _dt(dl), _stream()), "fb_scale_by_device_scalar")
        return out, None, None


def cross_entropy_logits(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Mean over the batch of ``-log softmax(logits)[label]`` for integer ``labels`` (fused kernel on CUDA)."""
    if logits.dim() != 2:
        logits = logits.reshape(-1, logits.shape[-1])
        labels = labels.reshape(-1)
    labels = labels.to(torch.int64)
    if _native(logits):
        x = logits
        if not torch.is_grad_enabled():
            x = logits.detach()
        return _CEFn.apply(x, labels.contiguous(), 1.0 / logits.shape[0])
    lp = torch.log_softmax(logits.float(), -1)
    return -lp.gather(1, labels.unsqueeze(1)).mean()


class _ElemLossFn(Function):
    @staticmethod
    def forward(ctx, pred, target, kind):
        p, t = _f32(pred).contiguous(), _f32(target).contiguous()
        out = torch.zeros((), device=p.device, dtype=torch.float32)
        n = p.numel()
        _lib.check(_lib.cuda().fb_loss_fwd(p.data_ptr(), t.data_ptr(), out.data_ptr(), n, LOSS[kind], 1.0 / n,
                                           _stream()), "fb_loss_fwd")
        ctx.save_for_backward(p, t)
        ctx.kind, ctx.shape, ctx.dtype = kind, pred.shape, pred.dtype
        return out

    @staticmethod
    def backward(ctx, g):
        p, t = ctx.saved_tensors
        gf = _f32(g).contiguous()
        dp = torch.empty_like(p)
        n = p.numel()
        _lib.check(_lib.cuda().fb_loss_bwd(p.data_ptr(), t.data_ptr(), gf.data_ptr(), dp.data_ptr(), n,
                                           LOSS[ctx.kind], 1.0 / n, _stream()), "fb_loss_bwd")
        return raw_cast(dp.reshape(ctx.shape), ctx.dtype), None, None


def elementwise_loss(pred: torch.Tensor, target: torch.Tensor, kind: str) -> torch.Tensor:
    """mse / bce / l1 / smooth_l1, mean over all elements (ferrum-nn/src/loss.rs:24-105)."""
    if tuple(pred.shape) != tuple(target.shape):
        target = target.expand_as(pred)
    if _native(pred) and pred.numel() > 0:
        return _ElemLossFn.apply(pred, target.detach(), kind)
    d = pred - target
    if kind == "mse":
        return (d * d).mean()
    if kind == "bce":
        eps = 1e-7
        pc = pred + eps
        q = (1.0 + eps) - pc
        return -(target * torch.log(pc) + (1.0 - target) * torch.log(q)).mean()
    if kind == "l1":
        return d.abs().mean()
    a = d.abs()
    return torch.where(a < 1.0, 0.5 * d * d, a - 0.5).mean()


# =============================================================================== dropout / embedding / gather
_dropout_offset = 0


_capturable_rng = {}  # device index -> uint64 counter tensor; non-empty while steps are recorded in CUDA graphs


def set_capturable_rng(flag: bool) -> None:
    """Draw dropout offsets from a device-side counter that advances on the stream, so a step recorded in a CUDA
    graph draws a new mask at every replay (a host-side counter would be frozen into the graph)."""
    if not flag:
        _capturable_rng.clear()
    elif torch.cuda.is_available() and torch.cuda.current_device() not in _capturable_rng:
        _capturable_rng[torch.cuda.current_device()] = torch.zeros(1, dtype=torch.int64, device="cuda")


class _DropoutFn(Function):
    @staticmethod
    def forward(ctx, x, p, seed, offset):
        x2 = x.contiguous()
        y = torch.empty_like(x2)
        mask = torch.empty(x2.shape, device=x.device, dtype=torch.uint8)
        ctr = _capturable_rng.get(x.device.index)
        if ctr is not None:
            _lib.check(_lib.cuda().fb_dropout_fwd_dyn(x2.data_ptr(), y.data_ptr(), mask.data_ptr(), x2.numel(), p,
                                                      seed, offset << 20, ctr.data_ptr(), _dt(x2), _stream()),
                       "fb_dropout_fwd_dyn")
        else:
            _lib.check(_lib.cuda().fb_dropout_fwd(x2.data_ptr(), y.data_ptr(), mask.data_ptr(), x2.numel(), p, seed,
                                                  offset, _dt(x2), _stream()), "fb_dropout_fwd")
        ctx.save_for_backward(mask)
        ctx.p = p
        return y

    @staticmethod
    def backward(ctx, g):
        (mask,) = ctx.saved_tensors
        g2 = g.contiguous()
        dx = torch.empty_like(g2)
        _lib.check(_lib.cuda().fb_dropout_bwd(g2.data_ptr(), mask.data_ptr(), dx.data_ptr(), g2.numel(), ctx.p,
                                              _dt(g2), _stream()), "fb_dropout_bwd")
        return dx, None, None, None


def dropout(x: torch.Tensor, p: float, training: bool, seed: int | None = None) -> torch.Tensor:
    """Inverted dropout: keep with probability 1-p and scale by 1/(1-p) while training; identity otherwise."""
    global _dropout_offset
    if not training or p <= 0.0:
        return x
    if p >= 1.0:
        return x * 0.0
    if _native(x):
        if seed is None:
            seed = torch.initial_seed()
        _dropout_offset += 1
        return _DropoutFn.apply(x, float(p), int(seed) & 0xFFFFFFFFFFFFFFFF, _dropout_offset)
    return torch.nn.functional.dropout(x, p, True)


def _sorted_indices(idx_flat: torch.Tensor):
    """(sorted indices, original positions): a radix sort of the looked-up ids."""
    return torch.sort(idx_flat, stable=True)


class _EmbeddingFn(Function):
    @staticmethod
    def forward(ctx, weight, idx, padding_idx, out_dtype, pool, sink=None):
        ctx.sink, ctx.weight_ref = sink, weight
        w = weight.detach().contiguous()
        V, D = w.shape
        idx_c = idx.contiguous()
        lib = _lib.cuda()
        if pool:
            B, S = idx_c.shape
            out = torch.empty((B, D), device=w.device, dtype=out_dtype)
            _lib.check(lib.fb_embedding_meanpool_fwd(w.data_ptr(), idx_c.data_ptr(), out.data_ptr(), B, S, D, V,
                                                     F32 if out_dtype == torch.float32 else BF16, _stream()),
                       "fb_embedding_meanpool_fwd")
            ctx.group = S
        else:
            out = torch.empty((*idx_c.shape, D), device=w.device, dtype=out_dtype)
            _lib.check(lib.fb_embedding_fwd(w.data_ptr(), idx_c.data_ptr(), out.data_ptr(), idx_c.numel(), D, V,
                                            -1 if padding_idx is None else padding_idx,
                                            F32 if out_dtype == torch.float32 else BF16, _rt.status_ptr(),
                                            _stream()), "fb_embedding_fwd")
            ctx.group = 1
        ctx.save_for_backward(idx_c)
        ctx.wshape, ctx.padding_idx, ctx.pool = (V, D), padding_idx, pool
        return out

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        V, D = ctx.wshape
        g2 = g.reshape(-1, D).contiguous()
        flat = idx.reshape(-1)
        sidx, perm = _sorted_indices(flat)
        if ctx.sink is not None:  # accumulate straight into the data-parallel gradient arena
            dw, acc = ctx.sink.acquire(ctx.weight_ref)
            if not acc:
                dw.zero_()
        else:
            dw = torch.zeros((V, D), device=g.device, dtype=torch.float32)
        scale = 1.0 / ctx.group if ctx.pool else 1.0
        _lib.check(_lib.cuda().fb_embedding_bwd_sorted(g2.data_ptr(), sidx.data_ptr(), perm.data_ptr(),
                                                       dw.data_ptr(), flat.numel(), D, ctx.group, scale,
                                                       -1 if ctx.padding_idx is None else ctx.padding_idx, V,
                                                       _dt(g2), _stream()), "fb_embedding_bwd_sorted")
        if ctx.sink is not None:
            ctx.sink.ready(ctx.weight_ref)
            return None, None, None, None, None, None
        return dw, None, None, None, None, None


def embedding(weight: torch.Tensor, idx: torch.Tensor, padding_idx: int | None = None,
              out_dtype: torch.dtype | None = None, sink: GradSink | None = None) -> torch.Tensor:
    """Row gather ``weight[idx]`` -> ``[*idx.shape, D]``; rows at ``padding_idx`` are zero (embedding.rs:122-208)."""
    idx = idx.to(torch.int64)
    if weight.is_cuda and weight.dtype == torch.float32:
        return _EmbeddingFn.apply(weight, idx, padding_idx, out_dtype or torch.float32, False, sink)
    out = torch.nn.functional.embedding(idx, weight)
    if padding_idx is not None:
        out = out * (idx != padding_idx).unsqueeze(-1).to(out.dtype)
    return out


def embedding_mean_pool(weight: torch.Tensor, idx: torch.Tensor, out_dtype: torch.dtype | None = None,
                        sink: GradSink | None = None):
    """``mean_s weight[idx[b, s]]`` for ``idx [B, S]`` without materialising ``[B, S, D]``."""
    idx = idx.to(torch.int64)
    if weight.is_cuda and weight.dtype == torch.float32 and idx.dim() == 2 and idx.shape[1] * 8 <= 48 * 1024:
        return _EmbeddingFn.apply(weight, idx, None, out_dtype or torch.float32, True, sink)
    return torch.nn.functional.embedding(idx, weight).mean(1)


def gather_rows(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """``src[idx]`` along dim 0 for a contiguous device-resident tensor (DataLoader collate)."""
    if not src.is_cuda:
        return src.index_select(0, idx.to(torch.int64))
    src = src.contiguous()
    idx = idx.to(device=src.device, dtype=torch.int64).contiguous()
    out = torch.empty((idx.numel(), *src.shape[1:]), device=src.device, dtype=src.dtype)
    row_bytes = src[0].numel() * src.element_size() if src.shape[0] else 0
    if idx.numel() == 0 or row_bytes == 0:
        return out
    # an index outside the source is reported through the status block and its row comes back as zeros
    _lib.check(_lib.cuda().fb_gather_rows(src.data_ptr(), idx.data_ptr(), out.data_ptr(), idx.numel(), row_bytes,
                                          src.shape[0], _rt.status_ptr(), _stream()), "fb_gather_rows")
    return out


def transpose_2d(x: torch.Tensor) -> torch.Tensor:
    """Materialised transpose of a 2-D tensor (ferrum-cuda/src/kernels.rs:442-494)."""
    if not (x.is_cuda and x.element_size() in (2, 4)):
        return x.t().contiguous()
    x = x.contiguous()
    out = torch.empty((x.shape[1], x.shape[0]), device=x.device, dtype=x.dtype)
    _lib.check(_lib.cuda().fb_transpose_2d(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], x.element_size(),
                                           _stream()), "fb_transpose_2d")
    return out


# ============================================================ secondary layers: recurrent gates, conv lowering, pooling
class _LstmGatesFn(Function):
    """(h', c') from the gate pre-activations ``xi + hh`` ([B, 4H]: input, forget, cell, output) in one kernel."""

    @staticmethod
    def forward(ctx, xi, hh, c_prev):
        xi, hh, c_prev = _f32(xi).contiguous(), _f32(hh).contiguous(), _f32(c_prev).contiguous()
        B, H = c_prev.shape
        h, c = torch.empty_like(c_prev), torch.empty_like(c_prev)
        gates = torch.empty_like(xi)
        _lib.check(_lib.cuda().fb_lstm_gates_fwd(xi.data_ptr(), hh.data_ptr(), c_prev.data_ptr(), h.data_ptr(),
                                                 c.data_ptr(), gates.data_ptr(), B, H, _stream()), "fb_lstm_gates_fwd")
        ctx.save_for_backward(gates, c_prev, c)
        return h, c

    @staticmethod
    def backward(ctx, dh, dc):
        gates, c_prev, c = ctx.saved_tensors
        B, H = c_prev.shape
        dh = _f32(dh).contiguous() if dh is not None else None
        dc = _f32(dc).contiguous() if dc is not None else None
        dpre, dc_prev = torch.empty_like(gates), torch.empty_like(c_prev)
        _lib.check(_lib.cuda().fb_lstm_gates_bwd(dh.data_ptr() if dh is not None else None,
                                                 dc.data_ptr() if dc is not None else None, gates.data_ptr(),
                                                 c_prev.data_ptr(), c.data_ptr(), dpre.data_ptr(), dc_prev.data_ptr(),
                                                 B, H, _stream()), "fb_lstm_gates_bwd")
        return dpre, dpre, dc_prev


def lstm_gates(xi, hh, c_prev):
    """LSTM cell update from the two projections (ferrum-nn/src/rnn.rs:188-227)."""
    if _native(xi) and xi.dim() == 2:
        return _LstmGatesFn.apply(xi, hh, c_prev)
    i, f, g, o = (xi + hh).chunk(4, -1)
    c = torch.sigmoid(f) * c_prev + torch.sigmoid(i) * torch.tanh(g)
    return torch.sigmoid(o) * torch.tanh(c), c


class _GruGatesFn(Function):
    """h' = (1 - z) n + z h with r, z = sigmoid, n = tanh(xn + r * hn), from xi, hh [B, 3H] in one kernel."""

    @staticmethod
    def forward(ctx, xi, hh, h_prev):
        xi, hh, h_prev = _f32(xi).contiguous(), _f32(hh).contiguous(), _f32(h_prev).contiguous()
        B, H = h_prev.shape
        h = torch.empty_like(h_prev)
        saved = torch.empty((B, 4 * H), device=h.device, dtype=torch.float32)
        _lib.check(_lib.cuda().fb_gru_gates_fwd(xi.data_ptr(), hh.data_ptr(), h_prev.data_ptr(), h.data_ptr(),
                                                saved.data_ptr(), B, H, _stream()), "fb_gru_gates_fwd")
        ctx.save_for_backward(saved, h_prev)
        return h

    @staticmethod
    def backward(ctx, dh):
        saved, h_prev = ctx.saved_tensors
        B, H = h_prev.shape
        dh = _f32(dh).contiguous()
        dxi = torch.empty((B, 3 * H), device=dh.device, dtype=torch.float32)
        dhh, dhp = torch.empty_like(dxi), torch.empty_like(h_prev)
        _lib.check(_lib.cuda().fb_gru_gates_bwd(dh.data_ptr(), saved.data_ptr(), h_prev.data_ptr(), dxi.data_ptr(),
                                                dhh.data_ptr(), dhp.data_ptr(), B, H, _stream()), "fb_gru_gates_bwd")
        return dxi, dhh, dhp


def gru_gates(xi, hh, h_prev):
    """GRU cell update from the two projections (ferrum-nn/src/rnn.rs:318-372)."""
    if _native(xi) and xi.dim() == 2:
        return _GruGatesFn.apply(xi, hh, h_prev)
    xr, xz, xn = xi.chunk(3, -1)
    hr, hz, hn = hh.chunk(3, -1)
    r, z = torch.sigmoid(xr + hr), torch.sigmoid(xz + hz)
    n = torch.tanh(xn + r * hn)
    return (1 - z) * n + z * h_prev


def conv_out_size(size, k, stride, pad, dil):
    return (size + 2 * pad - dil * (k - 1) - 1) // stride + 1


class _Im2colFn(Function):
    """[B, C, H, W] -> window matrix [B*Ho*Wo, C*kh*kw], K contiguous: the A operand of the convolution GEMM."""

    @staticmethod
    def forward(ctx, x, kernel, stride, padding, dilation):
        x = _f32(x).contiguous()
        B, C, H, W = x.shape
        (kh, kw), (sh, sw), (ph, pw), (dh, dw) = kernel, stride, padding, dilation
        Ho, Wo = conv_out_size(H, kh, sh, ph, dh), conv_out_size(W, kw, sw, pw, dw)
        K = C * kh * kw
        cols = torch.empty((B * Ho * Wo, K), device=x.device, dtype=torch.float32)
        ctx.geom = (B, C, H, W, kh, kw, Ho, Wo, sh, sw, ph, pw, dh, dw)
        _lib.check(_lib.cuda().fb_im2col(x.data_ptr(), cols.data_ptr(), *ctx.geom, K, _dt(cols), _stream()),
                   "fb_im2col")
        return cols

    @staticmethod
    def backward(ctx, g):
        g = _f32(g).contiguous()
        B, C, H, W = ctx.geom[:4]
        dx = torch.empty((B, C, H, W), device=g.device, dtype=torch.float32)
        _lib.check(_lib.cuda().fb_col2im(g.data_ptr(), dx.data_ptr(), *ctx.geom, g.shape[1], _stream()), "fb_col2im")
        return dx, None, None, None, None


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def _to_nhwc_bf16(x: torch.Tensor) -> torch.Tensor:
    """[B, C, H, W] fp32 -> [B, H, W, Cp] bf16 with the channels padded by zeros to a multiple of 8."""
    x = _f32(x).contiguous()
    B, C, H, W = x.shape
    y = torch.empty((B, H, W, _pad8(C)), device=x.device, dtype=torch.bfloat16)
    _lib.check(_lib.cuda().fb_nchw_to_nhwc_bf16(x.data_ptr(), y.data_ptr(), B, C, H * W, y.shape[3], _stream()),
               "fb_nchw_to_nhwc_bf16")
    return y


def _to_nchw_f32(y: torch.Tensor, C: int) -> torch.Tensor:
    """[B, H, W, ld] fp32 (first C channels) -> [B, C, H, W] fp32."""
    B, H, W, ld = y.shape
    out = torch.empty((B, C, H, W), device=y.device, dtype=torch.float32)
    _lib.check(_lib.cuda().fb_nhwc_to_nchw_f32(y.data_ptr(), out.data_ptr(), B, C, H * W, ld, _stream()),
               "fb_nhwc_to_nchw_f32")
    return out


def _conv_igemm(xh: torch.Tensor, wk: torch.Tensor, bias, O: int, kernel, padding, dilation) -> torch.Tensor:
    """NHWC bf16 ``xh`` [B, H, W, Cp] * ``wk`` [O, kh * kw * Cp] -> NHWC fp32 [B, Ho, Wo, O] on the tensor cores."""
    B, H, W, Cp = xh.shape
    (kh, kw), (ph, pw), (dh, dw) = kernel, padding, dilation
    Ho, Wo = H + 2 * ph - dh * (kh - 1), W + 2 * pw - dw * (kw - 1)
    y = torch.empty((B, Ho, Wo, O), device=xh.device, dtype=torch.float32)
    _lib.check(_lib.cuda().fb_conv_igemm(xh.data_ptr(), wk.data_ptr(), y.data_ptr(), _ptr(bias), B, H, W, Cp, O, kh,
                                         kw, ph, pw, dh, dw, O, 0, _rt.status_ptr(), _stream()), "fb_conv_igemm")
    return y


class _ConvIgemmFn(Function):
    """Stride-1, ungrouped 2-D convolution without a window matrix (csrc/gemm/tcgen05_gemm.cu, conv forms): all three
    products — forward, data gradient, weight gradient — read NHWC bf16 activations through 4-D TMA boxes shifted by
    the filter tap (zero fill = padding) and run on tcgen05.  Counterpart of the reference's direct loops
    (ferrum-nn/src/conv.rs:209-330)."""

    @staticmethod
    def forward(ctx, x, weight, bias, padding, dilation):
        B, C, H, W = x.shape
        O, _, kh, kw = weight.shape
        xh = _to_nhwc_bf16(x)                                              # [B, H, W, Cp]
        wk = _to_nhwc_bf16(weight.detach()).reshape(O, -1)                 # [O, kh * kw * Cp]
        b = _f32(bias.detach()).contiguous() if bias is not None else None
        y = _conv_igemm(xh, wk, b, O, (kh, kw), padding, dilation)
        ctx.save_for_backward(xh, weight)
        ctx.geom = (C, tuple(padding), tuple(dilation), bias is not None)
        return _to_nchw_f32(y, O)

    @staticmethod
    def backward(ctx, g):
        xh, weight = ctx.saved_tensors
        C, (ph, pw), (dh, dw), has_bias = ctx.geom
        B, H, W, Cp = xh.shape
        O, _, kh, kw = weight.shape
        gh = _to_nhwc_bf16(g)                                              # [B, Ho, Wo, Op]
        Op = gh.shape[3]
        dx = dwt = db = None
        if ctx.needs_input_grad[0]:
            # dx = dy convolved with the filters flipped in both directions and input / output channels exchanged
            wt = _to_nhwc_bf16(weight.detach().transpose(0, 1).flip(2, 3)).reshape(C, -1)   # [C, kh * kw * Op]
            dxh = _conv_igemm(gh, wt, None, C, (kh, kw), (dh * (kh - 1) - ph, dw * (kw - 1) - pw), (dh, dw))
            dx = _to_nchw_f32(dxh, C)
        if ctx.needs_input_grad[1]:
            lib = _lib.cuda()
            Ho, Wo = gh.shape[1], gh.shape[2]
            splits = lib.fb_conv_wgrad_splits(B, Ho, Wo, O, Cp, kh * kw)
            part = torch.empty((splits, O, kh * kw * Cp), device=g.device, dtype=torch.float32)
            _lib.check(lib.fb_conv_wgrad(gh.data_ptr(), xh.data_ptr(), part.data_ptr(), B, H, W, Cp, O, Op, kh, kw, ph,
                                         pw, dh, dw, _rt.status_ptr(), _stream()), "fb_conv_wgrad")
            full = raw_reduce(part, "sum", 0) if splits > 1 else part[0]
            dwt = full.reshape(O, kh, kw, Cp)[..., :C].permute(0, 3, 1, 2).contiguous()
        if has_bias and ctx.needs_input_grad[2]:
            db = raw_colsum(gh.reshape(-1, Op))[:O]
        return dx, dwt, db, None, None


class _ConvS2dFn(Function):
    """Strided, undilated, ungrouped 2-D convolution on the implicit-GEMM kernels: the input goes through a
    space-to-depth layout change (``z[b, I, J, (rh, rw, c)] = x[b, c, I * sh + rh - ph, J * sw + rw - pw]``), after
    which the stride-(sh, sw) convolution with a kh x kw filter IS a stride-1 convolution with a
    ceil(kh / sh) x ceil(kw / sw) filter over sh * sw * C channels (filter taps that do not exist are zero).  A
    patch embedding (kernel = stride) becomes one plain GEMM."""

    @staticmethod
    def _geometry(x_shape, w_shape, stride, padding):
        B, C, H, W = x_shape
        O, _, kh, kw = w_shape
        (sh, sw), (ph, pw) = stride, padding
        Ho, Wo = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        k2h, k2w = -(-kh // sh), -(-kw // sw)
        return Ho, Wo, k2h, k2w, Ho + k2h - 1, Wo + k2w - 1, _pad8(sh * sw * C)

    @staticmethod
    def _filters(weight, stride, k2h, k2w, Cz):
        """[O, C, kh, kw] -> [O, k2h, k2w, Cz] fp32 in the channel order (rh, rw, c) of the space-to-depth input."""
        O, C, kh, kw = weight.shape
        sh, sw = stride
        w = torch.zeros((O, C, k2h * sh, k2w * sw), device=weight.device, dtype=torch.float32)
        w[:, :, :kh, :kw] = weight.detach().float()
        w = w.view(O, C, k2h, sh, k2w, sw).permute(0, 2, 4, 3, 5, 1).reshape(O, k2h, k2w, sh * sw * C)
        out = torch.zeros((O, k2h, k2w, Cz), device=weight.device, dtype=torch.float32)
        out[..., :sh * sw * C] = w
        return out

    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding):
        x = _f32(x).contiguous()
        B, C, H, W = x.shape
        O = weight.shape[0]
        (sh, sw), (ph, pw) = stride, padding
        Ho, Wo, k2h, k2w, Hz, Wz, Cz = _ConvS2dFn._geometry(x.shape, weight.shape, stride, padding)
        z = torch.empty((B, Hz, Wz, Cz), device=x.device, dtype=torch.bfloat16)
        _lib.check(_lib.cuda().fb_nchw_to_s2d_nhwc_bf16(x.data_ptr(), z.data_ptr(), B, C, H, W, sh, sw, ph, pw, Hz, Wz,
                                                        Cz, _stream()), "fb_nchw_to_s2d_nhwc_bf16")
        w2 = _ConvS2dFn._filters(weight, stride, k2h, k2w, Cz)
        b = _f32(bias.detach()).contiguous() if bias is not None else None
        y = _conv_igemm(z, w2.reshape(O, -1).to(torch.bfloat16), b, O, (k2h, k2w), (0, 0), (1, 1))
        ctx.save_for_backward(z, weight)
        ctx.geom = (x.shape, tuple(stride), tuple(padding), bias is not None)
        return _to_nchw_f32(y, O)

    @staticmethod
    def backward(ctx, g):
        z, weight = ctx.saved_tensors
        x_shape, (sh, sw), (ph, pw), has_bias = ctx.geom
        B, C, H, W = x_shape
        O, _, kh, kw = weight.shape
        Ho, Wo, k2h, k2w, Hz, Wz, Cz = _ConvS2dFn._geometry(x_shape, weight.shape, (sh, sw), (ph, pw))
        gh = _to_nhwc_bf16(g)                                              # [B, Ho, Wo, Op]
        Op = gh.shape[3]
        lib = _lib.cuda()
        dx = dwt = db = None
        if ctx.needs_input_grad[0]:
            w2 = _ConvS2dFn._filters(weight, (sh, sw), k2h, k2w, Cz)       # [O, k2h, k2w, Cz]
            wt = torch.zeros((Cz, k2h, k2w, Op), device=g.device, dtype=torch.float32)
            wt[..., :O] = w2.permute(3, 1, 2, 0).flip(1, 2)
            dz = _conv_igemm(gh, wt.reshape(Cz, -1).to(torch.bfloat16), None, Cz, (k2h, k2w), (k2h - 1, k2w - 1), (1, 1))
            dx = torch.empty(x_shape, device=g.device, dtype=torch.float32)
            _lib.check(lib.fb_s2d_nhwc_to_nchw_f32(dz.data_ptr(), dx.data_ptr(), B, C, H, W, sh, sw, ph, pw, Hz, Wz, Cz,
                                                   _stream()), "fb_s2d_nhwc_to_nchw_f32")
        if ctx.needs_input_grad[1]:
            splits = lib.fb_conv_wgrad_splits(B, Ho, Wo, O, Cz, k2h * k2w)
            part = torch.empty((splits, O, k2h * k2w * Cz), device=g.device, dtype=torch.float32)
            _lib.check(lib.fb_conv_wgrad(gh.data_ptr(), z.data_ptr(), part.data_ptr(), B, Hz, Wz, Cz, O, Op, k2h, k2w, 0, 0,
                                         1, 1, _rt.status_ptr(), _stream()), "fb_conv_wgrad")
            full = raw_reduce(part, "sum", 0) if splits > 1 else part[0]
            d2 = full.reshape(O, k2h, k2w, Cz)[..., :sh * sw * C].reshape(O, k2h, k2w, sh, sw, C)
            dwt = d2.permute(0, 5, 1, 3, 2, 4).reshape(O, C, k2h * sh, k2w * sw)[:, :, :kh, :kw].contiguous()
        if has_bias and ctx.needs_input_grad[2]:
            db = raw_colsum(gh.reshape(-1, Op))[:O]
        return dx, dwt, db, None, None


def conv_igemm_ok(x: torch.Tensor, stride, dilation, padding, kernel, groups: int) -> bool:
    """True when ``conv2d`` can take the implicit-GEMM path: CUDA, bf16 autocast on, one group, and either stride 1
    with a data gradient whose padding ``dilation * (kernel - 1) - padding`` is not negative, or any stride without
    dilation (space-to-depth form)."""
    if not (_native(x) and x.dim() == 4 and config.low_precision_active() and groups == 1):
        return False
    if tuple(stride) == (1, 1):
        return (dilation[0] * (kernel[0] - 1) - padding[0] >= 0 and dilation[1] * (kernel[1] - 1) - padding[1] >= 0)
    return tuple(dilation) == (1, 1) and padding[0] >= 0 and padding[1] >= 0


def conv2d_igemm(x, weight, bias, padding=(0, 0), dilation=(1, 1), stride=(1, 1)):
    if tuple(stride) != (1, 1):
        return _ConvS2dFn.apply(x, weight, bias, tuple(stride), tuple(padding))
    return _ConvIgemmFn.apply(x, weight, bias, tuple(padding), tuple(dilation))


def im2col(x, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """Window matrix of a convolution with rows ordered (b, oh, ow) and columns (c, ki, kj)."""
    if _native(x):
        return _Im2colFn.apply(x, tuple(kernel), tuple(stride), tuple(padding), tuple(dilation))
    cols = torch.nn.functional.unfold(x, kernel, dilation=dilation, padding=padding, stride=stride)
    return cols.transpose(1, 2).reshape(-1, cols.shape[1])


class _Pool2dFn(Function):
    @staticmethod
    def forward(ctx, x, kernel, stride, op):
        x = _f32(x).contiguous()
        B, C, H, W = x.shape
        (kh, kw), (sh, sw) = kernel, stride
        Ho, Wo = (H - kh) // sh + 1, (W - kw) // sw + 1
        y = torch.empty((B, C, Ho, Wo), device=x.device, dtype=torch.float32)
        arg = torch.empty((B, C, Ho, Wo), device=x.device, dtype=torch.int32) if op == 0 else None
        ctx.geom, ctx.op = (B, C, H, W, kh, kw, Ho, Wo, sh, sw), op
        _lib.check(_lib.cuda().fb_pool2d_fwd(x.data_ptr(), y.data_ptr(), arg.data_ptr() if arg is not None else None,
                                             *ctx.geom, op, _stream()), "fb_pool2d_fwd")
        ctx.save_for_backward(arg) if arg is not None else None
        return y

    @staticmethod
    def backward(ctx, g):
        g = _f32(g).contiguous()
        arg = ctx.saved_tensors[0] if ctx.op == 0 else None
        B, C, H, W = ctx.geom[:4]
        dx = torch.empty((B, C, H, W), device=g.device, dtype=torch.float32)
        _lib.check(_lib.cuda().fb_pool2d_bwd(g.data_ptr(), arg.data_ptr() if arg is not None else None, dx.data_ptr(),
                                             *ctx.geom, ctx.op, _stream()), "fb_pool2d_bwd")
        return dx, None, None, None


def pool2d(x, kernel, stride, op: str):
    """Max / average pooling over unpadded windows (ferrum-nn/src/conv.rs:340-441)."""
    if _native(x) and x.dim() == 4:
        return _Pool2dFn.apply(x, tuple(kernel), tuple(stride), 0 if op == "max" else 1)
    fn = torch.nn.functional.max_pool2d if op == "max" else torch.nn.functional.avg_pool2d
    return fn(x, kernel, stride)
