"""Raw (non-autograd) GEMM launchers.

``gemm_bf16``  — the tcgen05/TMEM kernel (``csrc/gemm/tcgen05_gemm.cu``).
``gemm_f32``   — the fp32 SIMT kernel with arbitrary strides (``csrc/gemm/simt_gemm.cu``).

Both compute ``out = act(A @ B^T + bias)`` in the "NT" convention used by
``Linear`` (reference forward: ferrum-nn/src/linear.rs:78-89), where operand
layouts are described by flags instead of transposed copies.
"""
from __future__ import annotations

import os

import torch

from .. import _lib
from ..utils import runtime as _rt

ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2, "silu": 3, "tanh": 4, "sigmoid": 5}

_max_ctas = 0  # 0 = all SMs; the DDP engine lowers this to leave SMs for the comm kernel
# CTA-pair kernel (tcgen05 cta_group::2, 256x256 tile per two SMs) for large problems (default);
# FERRUM_GEMM_2CTA=0 selects the single-CTA kernel everywhere.
_use_2cta = os.environ.get("FERRUM_GEMM_2CTA", "1") == "1"


def set_gemm_2cta(flag: bool) -> None:
    """Choose between the CTA-pair kernel (large shapes) and the single-CTA kernel."""
    global _use_2cta
    _use_2cta = bool(flag)


def set_gemm_cta_limit(n: int) -> None:
    """Cap the persistent GEMM grid (0 = one CTA per SM)."""
    global _max_ctas
    _max_ctas = int(n)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def bf16_operand_ok(t: torch.Tensor) -> bool:
    """True when a 2-D bf16 tensor can be described by a TMA map (either major)."""
    if t.dtype != torch.bfloat16 or t.dim() != 2:
        return False
    if t.data_ptr() % 16:
        return False
    s0, s1 = t.stride()
    if s1 == 1:
        return (s0 * 2) % 16 == 0 and s0 >= t.shape[1]
    if s0 == 1:
        return (s1 * 2) % 16 == 0 and s1 >= t.shape[0]
    return False


def _major(t: torch.Tensor):
    """(mn_major flag, row pitch in elements) of an operand given as an [MN, K] view."""
    s0, s1 = t.stride()
    if s1 == 1:
        return 0, s0  # stored [MN][K]: K-major
    if s0 == 1:
        return 1, s1  # stored [K][MN]: MN-major
    raise ValueError("GEMM operand needs one unit stride")


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None, act: str | None = None,
              out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
              accumulate: bool = False, act_grad: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M,N] = act(a[M,K] @ b[N,K]^T + bias)`` on the tcgen05 tensor cores.

    ``a`` and ``b`` are bf16 2-D tensors with one unit stride (any of the two);
    a transposed view (``x.t()``) is consumed as an MN-major operand without a copy.
    ``act_grad`` (bf16, shaped and strided like a bf16 ``out``) additionally receives ``act'(a @ b^T + bias)``.
    """
    assert a.is_cuda and b.is_cuda and a.dim() == 2 and b.dim() == 2
    M, K = a.shape
    N, Kb = b.shape
    assert K == Kb, f"inner dimensions differ: {a.shape} x {b.shape}^T"
    a_mn, lda = _major(a)
    b_mn, ldb = _major(b)
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype)
    assert out.stride(1) == 1 and out.shape == (M, N)
    if accumulate:
        assert out.dtype == torch.float32, "accumulate needs an fp32 output"
    if act_grad is not None:
        assert out.dtype == torch.bfloat16 and act_grad.dtype == torch.bfloat16 and act_grad.shape == out.shape
        assert act_grad.stride() == out.stride()
    aux = act_grad.data_ptr() if act_grad is not None else None
    lib = _lib.cuda()
    pair = _use_2cta and M >= 512 and N >= 128
    fn = lib.fb_gemm_bf16_2cta if pair else lib.fb_gemm_bf16
    rc = fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), aux, bias.data_ptr() if bias is not None else None,
            M, N, K, lda, ldb, out.stride(0), a_mn, b_mn, 1 if out.dtype == torch.bfloat16 else 0,
            ACT[act], 1 if accumulate else 0, _max_ctas, _rt.status_ptr(), _stream())
    if rc == -3:  # CTA pairs cannot be scheduled on this device
        rc = lib.fb_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), aux,
                              bias.data_ptr() if bias is not None else None, M, N, K, lda, ldb, out.stride(0), a_mn, b_mn, 1 if out.dtype == torch.bfloat16 else 0,
                              ACT[act], 1 if accumulate else 0, _max_ctas, _rt.status_ptr(), _stream())
    _lib.check(rc, "fb_gemm_bf16")
    return out


def push_operands_ok(a: torch.Tensor, b: torch.Tensor) -> bool:
    """True when ``a @ b^T`` can run on the CTA-pair kernel with the pushing epilogue."""
    return (_use_2cta and bf16_operand_ok(a) and bf16_operand_ok(b) and a.shape[0] >= 512 and b.shape[0] >= 128
            and b.shape[0] % 4 == 0)


def gemm_bf16_push(a: torch.Tensor, b: torch.Tensor, ctx, bucket_off: int, out_rel: int, per: int,
                   bucket_len: int) -> bool:
    """``a[M,K] @ b[N,K]^T`` in fp32 with the gradient reduce-scatter fused into the epilogue: every 16-byte piece
    of the result is stored over NVLink into the bucket region of the rank that owns it (element ``e`` of the
    bucket belongs to shard ``e // per``; this rank's value lands in its slot of that shard).  ``ctx`` is the
    arena context (``SymmetricArena.ctx``), ``bucket_off`` the byte offset of the bucket's gradient region,
    ``out_rel`` the bucket-relative element index of the result's first element (row pitch = N).  Returns False
    where CTA pairs cannot be launched (the caller then takes the ordinary path)."""
    M, K = a.shape
    N = b.shape[0]
    a_mn, lda = _major(a)
    b_mn, ldb = _major(b)
    rc = _lib.cuda().fb_gemm_bf16_2cta_push(a.data_ptr(), b.data_ptr(), M, N, K, lda, ldb, N, a_mn, b_mn, ctx,
                                            bucket_off, out_rel, per, bucket_len, _max_ctas, _rt.status_ptr(),
                                            _stream())
    if rc == -3:
        return False
    _lib.check(rc, "fb_gemm_bf16_2cta_push")
    return True


def tf32_operand_ok(t: torch.Tensor) -> bool:
    """True when a 2-D fp32 tensor can be described by a TMA map (either major): 16-byte aligned base and pitch."""
    if t.dtype != torch.float32 or t.dim() != 2 or t.data_ptr() % 16:
        return False
    s0, s1 = t.stride()
    if s1 == 1:
        return s0 % 4 == 0 and s0 >= t.shape[1]
    if s0 == 1:
        return s1 % 4 == 0 and s1 >= t.shape[0]
    return False


def gemm_tf32(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None, act: str | None = None,
              out: torch.Tensor | None = None, accumulate: bool = False, kernel: str | None = None) -> torch.Tensor:
    """``out[M,N] = act(a[M,K] @ b[N,K]^T + bias)`` with fp32 tensors on the tensor cores (TF32 operands, fp32
    accumulation and output).  Same layout rules as :func:`gemm_bf16`.  ``kernel`` forces "1cta" or "2cta";
    by default outputs of at least 512 x 256 run on CTA pairs."""
    assert a.is_cuda and a.dim() == 2 and b.dim() == 2 and a.dtype == torch.float32 and b.dtype == torch.float32
    M, K = a.shape
    N, Kb = b.shape
    assert K == Kb, f"inner dimensions differ: {a.shape} x {b.shape}^T"
    a_mn, lda = _major(a)
    b_mn, ldb = _major(b)
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=torch.float32)
    assert out.dtype == torch.float32 and out.stride(1) == 1 and out.shape == (M, N)
    pair = (M >= 512 and N >= 256) if kernel is None else kernel == "2cta"
    lib = _lib.cuda()
    args = (a.data_ptr(), b.data_ptr(), out.data_ptr(), bias.data_ptr() if bias is not None else None, M, N, K,
            lda, ldb, out.stride(0), a_mn, b_mn, ACT[act], 1 if accumulate else 0, _max_ctas, _rt.status_ptr(),
            _stream())
    rc = -3
    if pair:
        rc = lib.fb_gemm_tf32_2cta(*args)
    if rc == -3:  # CTA pairs not used or not launchable on this device
        rc = lib.fb_gemm_tf32(*args)
    _lib.check(rc, "fb_gemm_tf32")
    return out


def batched_operand_ok(t: torch.Tensor) -> bool:
    """True when a 4-D bf16 tensor ``[Bo, Bi, rows, cols]`` can be described by a 4-D TMA map."""
    if t.dtype != torch.bfloat16 or t.dim() != 4 or t.data_ptr() % 16:
        return False
    so, si, s0, s1 = t.stride()
    if s1 == 1:
        ld, ok = s0, s0 >= t.shape[3]
    elif s0 == 1:
        ld, ok = s1, s1 >= t.shape[2]
    else:
        return False
    if not ok or ld % 8:
        return False
    return (t.shape[0] == 1 or (so > 0 and so % 8 == 0)) and (t.shape[1] == 1 or (si > 0 and si % 8 == 0))


def gemm_bf16_batched(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None,
                      out_dtype: torch.dtype = torch.bfloat16, alpha: float = 1.0,
                      accumulate: bool = False) -> torch.Tensor:
    """``out[o,i] = alpha * a[o,i] @ b[o,i]^T`` for 4-D operands ``a [Bo,Bi,M,K]``, ``b [Bo,Bi,N,K]``.

    Any strides over the two batch dimensions (multiples of 8 elements) and either unit-stride major in the
    last two, so ``x.view(B, S, H, D).permute(0, 2, 1, 3)`` and ``.transpose(-1, -2)`` views are used in place.
    """
    assert a.dim() == 4 and b.dim() == 4 and a.shape[:2] == b.shape[:2] and a.shape[3] == b.shape[3]
    Bo, Bi, M, K = a.shape
    N = b.shape[2]
    a_mn, lda = _major(a[0, 0])
    b_mn, ldb = _major(b[0, 0])
    if out is None:
        out = torch.empty((Bo, Bi, M, N), device=a.device, dtype=out_dtype)
    assert out.shape == (Bo, Bi, M, N) and out.stride(3) == 1
    if accumulate:
        assert out.dtype == torch.float32
    rc = _lib.cuda().fb_gemm_bf16_batched(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, lda, ldb, out.stride(2), Bo, Bi,
        a.stride(0), a.stride(1), b.stride(0), b.stride(1), out.stride(0), out.stride(1), a_mn, b_mn,
        1 if out.dtype == torch.bfloat16 else 0, 1 if accumulate else 0, float(alpha), _rt.status_ptr(), _stream())
    _lib.check(rc, "fb_gemm_bf16_batched")
    return out


def gemm_f32(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None, act: str | None = None,
             out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """fp32 ``out = act(a @ b^T + bias)`` with arbitrary strides; ``a``/``b`` may be 2-D or batched 3-D."""
    assert a.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32
    batched = a.dim() == 3
    if batched:
        Bt, M, K = a.shape
        _, N, _ = b.shape
        sam, sak = a.stride(1), a.stride(2)
        sbn, sbk = b.stride(1), b.stride(2)
        bsa, bsb = a.stride(0), b.stride(0)
    else:
        Bt = 1
        M, K = a.shape
        N, _ = b.shape
        sam, sak = a.stride()
        sbn, sbk = b.stride()
        bsa = bsb = 0
    if out is None:
        out = torch.empty((Bt, M, N) if batched else (M, N), device=a.device, dtype=torch.float32)
    ldc = out.stride(-2)
    bsc = out.stride(0) if batched else 0
    lib = _lib.cuda()
    rc = lib.fb_gemm_f32_simt(a.data_ptr(), b.data_ptr(), out.data_ptr(),
                              bias.data_ptr() if bias is not None else None, M, N, K, sam, sak, sbk, sbn, ldc,
                              ACT[act], 1 if accumulate else 0, Bt, bsa, bsb, bsc, _stream())
    _lib.check(rc, "fb_gemm_f32_simt")
    return out
