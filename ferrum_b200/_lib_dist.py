"""ctypes signatures of the inter-GPU entry points (csrc/dist)."""
import ctypes
from ctypes import POINTER, c_float, c_int, c_int32, c_longlong, c_uint, c_ulonglong, c_void_p

MAX_RANKS = 8


class DistCtx(ctypes.Structure):
    """Mirror of ``fb_dist_ctx`` (csrc/dist/dist_ctx.h)."""

    _fields_ = [("rank", c_int), ("world", c_int), ("arena", c_void_p * MAX_RANKS), ("mc_arena", c_void_p),
                ("status", c_void_p), ("timeout_ns", c_ulonglong)]


def _sigs():
    from ._lib import AdamH, SgdH

    P, LL, I, F, U = c_void_p, c_longlong, c_int, c_float, c_uint
    return {
        "fb_symm_alloc": (P, [c_ulonglong]),
        "fb_symm_free": (I, [P]),
        "fb_symm_handle_bytes": (I, []),
        "fb_symm_export": (I, [P, P]),
        "fb_symm_import": (P, [P, POINTER(c_int)]),
        "fb_symm_close": (I, [P]),
        "fb_symm_enable_peer": (I, [I]),
        "fb_dist_query_flag_bytes": (I, []),
        "fb_dist_query_max_blocks": (I, []),
        "fb_dist_query_channels": (I, []),
        "fb_dist_allreduce": (I, [POINTER(DistCtx), I, I, I, U, LL, LL, LL, LL, I, F, POINTER(AdamH), POINTER(SgdH),
                                  P, P, I, I, I, P]),
        "fb_dist_allreduce_dyn": (I, [POINTER(DistCtx), I, I, I, P, LL, LL, LL, LL, I, F, POINTER(AdamH), POINTER(SgdH),
                                      P, P, I, I, I, P, P]),
        "fb_dist_allreduce_staged": (I, [POINTER(DistCtx), I, I, U, LL, LL, I, F, P, P, LL, I, I, P]),
        "fb_dist_allreduce_staged_emulated": (I, [POINTER(DistCtx), I, I, U, LL, LL, I, F, POINTER(c_void_p),
                                                  POINTER(c_void_p), LL, I, I, P]),
        "fb_dist_allreduce_emulated": (I, [POINTER(DistCtx), I, I, I, U, LL, LL, LL, LL, I, F, POINTER(AdamH),
                                           POINTER(SgdH), POINTER(c_void_p), POINTER(c_void_p), I, I, I, P]),
        "fb_dist_collective": (I, [POINTER(DistCtx), I, I, U, I, LL, LL, LL, I, F, I, P]),
        "fb_dist_collective_emulated": (I, [POINTER(DistCtx), I, I, I, U, I, LL, LL, LL, I, F, I, P]),
        "fb_dist_collective_staged": (I, [POINTER(DistCtx), I, I, U, I, LL, LL, I, F, P, P, I, P]),
        "fb_dist_collective_staged_emulated": (I, [POINTER(DistCtx), I, I, I, U, I, LL, LL, I, F, POINTER(c_void_p),
                                                   POINTER(c_void_p), I, P]),
        "fb_gemm_bf16_2cta_push": (I, [P, P, I, I, I, LL, LL, LL, I, I, POINTER(DistCtx), LL, LL, LL, LL, I, P, P]),
        "fb_dist_set_pushed_ranges": (I, [I, POINTER(ctypes.c_longlong), POINTER(ctypes.c_longlong)]),
        "fb_dist_barrier": (I, [POINTER(DistCtx), I, U, P]),
        "fb_dist_allreduce_oneshot": (I, [POINTER(DistCtx), I, U, LL, LL, I, F, P, P, I, I, P]),
        "fb_dist_allreduce_oneshot_emulated": (I, [POINTER(DistCtx), I, I, U, LL, LL, I, F, POINTER(c_void_p),
                                                   POINTER(c_void_p), I, I, P]),
        "fb_dist_reduce_scatter_shard": (I, [POINTER(DistCtx), I, I, U, P, LL, LL, F, I, I, P]),
        "fb_dist_shard_update": (I, [POINTER(DistCtx), I, I, I, U, P, LL, LL, LL, P, I, POINTER(AdamH), POINTER(SgdH),
                                     P, P, I, I, P, P]),
        "fb_dist_reduce_scatter_shard_emulated": (I, [POINTER(DistCtx), I, I, U, LL, LL, F, I, I, P]),
        "fb_dist_shard_update_emulated": (I, [POINTER(DistCtx), I, I, I, U, LL, LL, LL, P, I, POINTER(AdamH),
                                              POINTER(SgdH), POINTER(c_void_p), POINTER(c_void_p), I, I, P]),
    }


class _Lazy(dict):
    def items(self):
        if not self:
            self.update(_sigs())
        return super().items()


SIGS = _Lazy()
