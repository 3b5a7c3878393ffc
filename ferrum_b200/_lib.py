"""ctypes access to the two native libraries built by :mod:`ferrum_b200._build`.

``cuda()`` returns the sm_100a kernel library, ``host()`` the CUDA-free host
library.  Neither is built on import: if a library is missing it is built once
(nvcc cross-compiles without a GPU); set ``FERRUM_B200_NO_AUTOBUILD=1`` to get an
error instead.  On a machine with a GPU the CUDA library is mandatory — ops
raise rather than falling back to another implementation.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int32, c_longlong, c_ulonglong, c_void_p, POINTER

from . import _build

_lock = threading.Lock()
_cuda = None
_host = None


class NativeLibraryError(RuntimeError):
    pass


def bounds_build_active() -> bool:
    """True when this process uses the debug kernel library with device-side index checks."""
    return os.environ.get("FERRUM_BOUNDS") == "1"


def _ensure(path) -> None:
    if path.exists():
        return
    if os.environ.get("FERRUM_B200_NO_AUTOBUILD") == "1":
        raise NativeLibraryError(f"{path} is missing; run `python -m ferrum_b200._build`")
    if path == _build.CUDA_LIB_BOUNDS:
        _build.build_bounds(verbose=False)
    else:
        _build.build(verbose=False)
    if not path.exists():
        raise NativeLibraryError(f"building {path} failed")


class AdamH(ctypes.Structure):
    _fields_ = [(n, c_float) for n in
                ("lr", "beta1", "beta2", "eps", "weight_decay", "bias_corr1", "bias_corr2", "grad_scale")]


class SgdH(ctypes.Structure):
    _fields_ = [("lr", c_float), ("momentum", c_float), ("weight_decay", c_float), ("grad_scale", c_float),
                ("nesterov", c_int), ("first_step", c_int)]


class DeviceProps(ctypes.Structure):
    _fields_ = [
        ("name", ctypes.c_char * 256), ("total_memory", c_ulonglong), ("multiprocessor_count", c_int),
        ("major", c_int), ("minor", c_int), ("max_threads_per_block", c_int), ("max_block_dim", c_int * 3),
        ("max_grid_dim", c_int * 3), ("warp_size", c_int), ("shared_mem_per_block", c_ulonglong),
        ("shared_mem_per_block_optin", c_ulonglong), ("unified_addressing", c_int), ("l2_cache_bytes", c_int),
        ("clock_khz", c_int), ("memory_clock_khz", c_int), ("memory_bus_width", c_int), ("cluster_launch", c_int),
        ("can_map_host", c_int),
    ]


P = c_void_p
LL = c_longlong
I = c_int
F = c_float
U64 = c_ulonglong

_CUDA_SIGS = {
    # runtime
    "fb_rt_device_count": (I, []),
    "fb_rt_set_device": (I, [I]),
    "fb_rt_get_device": (I, []),
    "fb_rt_synchronize": (I, []),
    "fb_rt_device_props": (I, [I, POINTER(DeviceProps)]),
    "fb_rt_mem_info": (I, [POINTER(U64), POINTER(U64)]),
    "fb_rt_can_access_peer": (I, [I, I]),
    "fb_rt_status_ptr": (P, []),
    "fb_rt_status_read": (I, [POINTER(c_int32), I]),
    "fb_rt_pool_alloc": (P, [U64]),
    "fb_rt_pool_free": (I, [P, U64]),
    "fb_rt_pool_clear": (I, []),
    "fb_rt_pool_allocated": (LL, []),
    "fb_rt_pool_cached": (LL, []),
    "fb_rt_pool_round": (U64, [U64]),
    "fb_rt_memcpy_h2d": (I, [P, P, U64, P]),
    "fb_rt_memcpy_d2h": (I, [P, P, U64, P]),
    "fb_rt_memcpy_d2d": (I, [P, P, U64, P]),
    "fb_rt_memset": (I, [P, I, U64, P]),
    "fb_rt_stream_create": (P, [I]),
    "fb_rt_stream_destroy": (I, [P]),
    "fb_rt_stream_synchronize": (I, [P]),
    "fb_rt_stream_query": (I, [P]),
    "fb_rt_event_create": (P, [I]),
    "fb_rt_event_destroy": (I, [P]),
    "fb_rt_event_record": (I, [P, P]),
    "fb_rt_stream_wait_event": (I, [P, P]),
    "fb_rt_event_synchronize": (I, [P]),
    "fb_rt_event_query": (I, [P]),
    "fb_rt_event_elapsed_ms": (F, [P, P]),
    "fb_rt_error_string": (c_char_p, [I]),
    # gemm
    "fb_gemm_bf16_supported": (I, [P, P, LL, LL]),
    "fb_gemm_bf16": (I, [P, P, P, P, P, I, I, I, LL, LL, LL, I, I, I, I, I, I, P, P]),
    "fb_gemm_bf16_2cta": (I, [P, P, P, P, P, I, I, I, LL, LL, LL, I, I, I, I, I, I, P, P]),
    "fb_gemm_bf16_2cta_pairs": (I, []),
    "fb_gemm_tf32": (I, [P, P, P, P, I, I, I, LL, LL, LL, I, I, I, I, I, P, P]),
    "fb_gemm_tf32_2cta": (I, [P, P, P, P, I, I, I, LL, LL, LL, I, I, I, I, I, P, P]),
    "fb_gemm_bf16_2cta_set_profile": (None, [P]),
    "fb_gemm_bf16_2cta_set_group_m": (I, [I]),
    "fb_gemm_bf16_batched": (I, [P, P, P, I, I, I, LL, LL, LL, I, I, LL, LL, LL, LL, LL, LL, I, I, I, I, F, P, P]),
    "fb_gemm_f32_simt": (I, [P, P, P, P, I, I, I, LL, LL, LL, LL, LL, I, I, I, LL, LL, LL, P]),
    # secondary layers
    "fb_lstm_gates_fwd": (I, [P, P, P, P, P, P, LL, I, P]),
    "fb_lstm_gates_bwd": (I, [P, P, P, P, P, P, P, LL, I, P]),
    "fb_gru_gates_fwd": (I, [P, P, P, P, P, LL, I, P]),
    "fb_gru_gates_bwd": (I, [P, P, P, P, P, P, LL, I, P]),
    "fb_im2col": (I, [P, P] + [I] * 14 + [LL, I, P]),
    "fb_conv_igemm": (I, [P, P, P, P] + [I] * 11 + [LL, I, P, P]),
    "fb_conv_wgrad_splits": (I, [I] * 6),
    "fb_conv_wgrad": (I, [P, P, P] + [I] * 12 + [P, P]),
    "fb_nchw_to_nhwc_bf16": (I, [P, P, I, I, LL, I, P]),
    "fb_nhwc_to_nchw_f32": (I, [P, P, I, I, LL, LL, P]),
    "fb_nchw_to_s2d_nhwc_bf16": (I, [P, P] + [I] * 10 + [LL, P]),
    "fb_s2d_nhwc_to_nchw_f32": (I, [P, P] + [I] * 10 + [LL, P]),
    "fb_attention_bwd_map_error": (I, []),
    "fb_col2im": (I, [P, P] + [I] * 14 + [LL, P]),
    "fb_pool2d_fwd": (I, [P, P, P] + [I] * 10 + [I, P]),
    "fb_pool2d_bwd": (I, [P, P, P] + [I] * 10 + [I, P]),
    # elementwise
    "fb_unary_fwd": (I, [P, P, LL, I, F, F, I, P]),
    "fb_scale_by_device_scalar": (I, [P, P, P, LL, I, P]),
    "fb_unary_bwd": (I, [P, P, P, LL, I, F, F, I, P]),
    "fb_binary_fwd": (I, [P, P, P, I, I, POINTER(LL), POINTER(LL), POINTER(LL), P]),
    "fb_cast": (I, [P, P, LL, I, I, P]),
    "fb_transpose_2d": (I, [P, P, I, I, I, P]),
    # reductions
    "fb_reduce_scratch_elems": (LL, [LL, LL, LL]),
    "fb_reduce": (I, [P, P, LL, LL, LL, I, P, LL, P]),
    "fb_arg_reduce": (I, [P, P, P, LL, LL, LL, I, P]),
    "fb_colsum": (I, [P, P, LL, LL, I, I, P]),
    # norms
    "fb_layernorm_fwd": (I, [P, P, P, P, P, P, LL, I, F, I, I, P]),
    "fb_layernorm_set_status": (None, [P]),
    "fb_layernorm_bwd": (I, [P, P, P, P, P, P, P, P, P, LL, I, I, I, I, I, P]),
    "fb_layernorm_bwd_blocks": (I, [LL, I]),
    "fb_batchnorm_fwd": (I, [P, P, P, P, P, P, P, P, LL, I, F, F, I, P]),
    "fb_batchnorm_bwd": (I, [P, P, P, P, P, P, P, P, LL, I, P]),
    # softmax / losses
    "fb_softmax_fwd": (I, [P, P, LL, I, I, I, P]),
    "fb_softmax_bwd": (I, [P, P, P, LL, I, I, I, P]),
    "fb_ce_fwd_bwd": (I, [P, P, P, P, LL, I, F, I, I, P]),
    "fb_loss_fwd": (I, [P, P, P, LL, I, F, P]),
    "fb_loss_bwd": (I, [P, P, P, P, LL, I, F, P]),
    # dropout / embedding / gather
    "fb_dropout_fwd": (I, [P, P, P, LL, F, U64, U64, I, P]),
    "fb_dropout_fwd_dyn": (I, [P, P, P, LL, F, U64, U64, P, I, P]),
    "fb_dropout_bwd": (I, [P, P, P, LL, F, I, P]),
    "fb_embedding_fwd": (I, [P, P, P, LL, I, LL, LL, I, P, P]),
    "fb_embedding_meanpool_fwd": (I, [P, P, P, LL, I, I, LL, I, P]),
    "fb_embedding_bwd_sorted": (I, [P, P, P, P, LL, I, I, F, LL, LL, I, P]),
    "fb_gather_rows": (I, [P, P, P, LL, LL, LL, P, P]),
    "fb_attention_fwd": (I, [P, P, P, P, P, I, I, I, I, I, LL, LL, LL, LL, LL, LL, LL, LL, LL, F, I, P, P]),
    "fb_attention_bwd": (I, [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, LL, LL, LL, LL, LL, LL, LL, LL, LL, F, I, P, P]),
    # optimizers
    "fb_adam_flat": (I, [P, P, P, P, P, LL, AdamH, P]),
    "fb_sgd_flat": (I, [P, P, P, P, LL, SgdH, P]),
    "fb_adam_multi": (I, [P, P, P, P, P, P, I, AdamH, P]),
    "fb_sgd_multi": (I, [P, P, P, P, P, I, SgdH, P]),
    "fb_adam_multi_dyn": (I, [P, P, P, P, P, P, I, AdamH, P, P]),
    "fb_sgd_multi_dyn": (I, [P, P, P, P, P, I, SgdH, P, P]),
    "fb_optim_advance": (I, [P, F, F, P]),
    # amp
    "fb_unscale_check": (I, [P, P, I, F, P, P]),
    "fb_sumsq_multi": (I, [P, P, I, P, P]),
    "fb_scale_multi": (I, [P, P, I, P, F, F, I, P]),
}


def _bind(lib, sigs, strict: bool = False):
    for name, (res, args) in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if strict:
                raise
            continue
        fn.restype = res
        fn.argtypes = args
    return lib


_launches = 0


class _CountingLib:
    """Forwards attribute access to the CDLL and counts calls of kernel launchers.

    Every entry point that is not part of the runtime layer (``fb_rt_*``) or a pure
    query enqueues at least one of this package's kernels, so the count is a lower
    bound on kernel launches; ``launch_count()`` reads it.
    """

    _NO_COUNT = ("fb_rt_", "fb_reduce_scratch_elems", "fb_layernorm_bwd_blocks", "fb_gemm_bf16_supported", "fb_gemm_bf16_2cta_pairs",
                 "fb_dist_query_")

    def __init__(self, lib):
        self._lib = lib

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if name.startswith(self._NO_COUNT):
            setattr(self, name, fn)
            return fn

        def counted(*args, _fn=fn):
            global _launches
            _launches += 1
            return _fn(*args)

        setattr(self, name, counted)
        return counted


def launch_count() -> int:
    """Number of kernel-launcher calls made through this module so far."""
    return _launches


def cuda():
    """The sm_100a kernel library (``lib/libferrum_b200_cuda.so``)."""
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                path = _build.CUDA_LIB_BOUNDS if bounds_build_active() else _build.CUDA_LIB
                _ensure(path)
                lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
                _bind(lib, _CUDA_SIGS)
                from . import _lib_dist  # signatures of the inter-GPU entry points
                _bind(lib, _lib_dist.SIGS)
                _cuda = _CountingLib(lib)
    return _cuda


def host():
    """The CUDA-free host library (``lib/libferrum_b200_host.so``)."""
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                _ensure(_build.HOST_LIB)
                lib = ctypes.CDLL(str(_build.HOST_LIB))
                from . import _lib_host
                _bind(lib, _lib_host.SIGS)
                _host = lib
    return _host


def check(code: int, what: str = "") -> None:
    """Raise for a non-zero return code of a native launcher."""
    if code == 0:
        return
    if code > 0:
        msg = cuda().fb_rt_error_string(code).decode()
        raise RuntimeError(f"{what}: CUDA error {code}: {msg}")
    raise ValueError(f"{what}: invalid argument (code {code})")
