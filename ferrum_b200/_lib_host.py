"""ctypes signatures of the host library (csrc/host)."""
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

P, LL, I, F, D, U64 = c_void_p, c_longlong, c_int, c_float, c_double, c_ulonglong
PLL, PI = POINTER(c_longlong), POINTER(c_int)

SIGS = {
    # checkpoint container
    "fb_ser_save": (I, [c_char_p, I, POINTER(c_char_p), PI, PLL, PI, POINTER(c_void_p), POINTER(U64), c_char_p, I]),
    "fb_ser_open": (P, [c_char_p, c_char_p, I]),
    "fb_ser_count": (I, [P]),
    "fb_ser_version": (c_uint, [P]),
    "fb_ser_meta": (I, [P, I, c_char_p, I, PI, PLL, I, PI, POINTER(U64), POINTER(U64)]),
    "fb_ser_name_len": (I, [P, I]),
    "fb_ser_read": (I, [P, I, P]),
    "fb_ser_close": (None, [P]),
    # samplers
    "fb_sampler_permutation": (None, [LL, U64, P]),
    "fb_sampler_shuffle": (None, [P, LL, U64]),
    "fb_sampler_weighted": (I, [P, LL, LL, U64, P]),
    "fb_sampler_distributed": (LL, [LL, I, I, I, U64, P, LL]),
    "fb_sampler_num_batches": (LL, [LL, LL, I]),
    "fb_sampler_subset": (None, [P, LL, U64, P]),
    "fb_sampler_zipf": (I, [LL, D, LL, U64, P]),
    # batch assembler of the DataLoader
    "fb_loader_create": (P, [I, POINTER(c_void_p), PLL, LL, I, POINTER(c_void_p), I]),
    "fb_loader_submit": (I, [P, I, P, LL]),
    "fb_loader_wait": (I, [P, I]),
    "fb_loader_destroy": (None, [P]),
    # bucket planner
    "fb_plan_buckets": (LL, [I, PLL, LL, LL, LL, PLL, PI, PLL, PLL, PI]),
    "fb_plan_buckets_kinds": (LL, [I, PLL, PI, LL, LL, LL, PLL, PI, PLL, PLL, PI]),
    "fb_plan_shard": (None, [LL, I, I, PLL, PLL]),
    # CPU reference loops
    "fb_ref_matmul": (None, [P, P, P, I, I, I]),
    "fb_ref_linear": (None, [P, P, P, P, I, I, I]),
    "fb_ref_softmax_rows": (None, [P, P, I, I, I]),
    "fb_ref_layernorm_rows": (None, [P, P, P, P, I, I, F]),
    "fb_ref_adam_step": (None, [P, P, P, P, LL, F, F, F, F, F, I]),
    "fb_ref_sgd_step": (None, [P, P, P, LL, F, F, F, I, I]),
    "fb_ref_train_xor": (None, [P, P, P, P, I, F, I, I, P]),
}
