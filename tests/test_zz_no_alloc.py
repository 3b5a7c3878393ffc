"""fb_reduce_noalloc: the reduction entry point for callers that are not allowed to allocate.

A host that embeds the library inside a fixed device-memory budget (a plugin, a C application that only owns the
buffers it was given) can neither grow an allocator nor call cudaMalloc at run time, so it cannot hand fb_reduce
the workspace that tall reductions need.  This variant carries a small built-in workspace instead.  The test
reaches it the way such a caller would — through the exported C symbol of the shared library, not through the
Python wrappers — and compares it with the ordinary entry point on two consecutive calls (the workspace is
shared between calls and keeps stale contents, so the second call must not be disturbed by the first).
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

P, LL, I = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
TOO_LARGE = -5


def _symbols():
    from ferrum_b200 import _build

    lib = ctypes.CDLL(str(_build.CUDA_LIB))
    lib.fb_reduce_noalloc.restype = I
    lib.fb_reduce_noalloc.argtypes = [P, P, LL, LL, LL, I, P, ctypes.c_char_p, I]
    lib.fb_reduce.restype = I
    lib.fb_reduce.argtypes = [P, P, LL, LL, LL, I, P, LL, P]
    lib.fb_reduce_scratch_elems.restype = LL
    lib.fb_reduce_scratch_elems.argtypes = [LL, LL, LL]
    return lib


def _existing(lib, x, outer, R, inner, op):
    out = torch.empty(outer * inner, device="cuda")
    want = lib.fb_reduce_scratch_elems(outer, R, inner)
    scratch = torch.empty(max(want, 1), device="cuda")
    rc = lib.fb_reduce(x.data_ptr(), out.data_ptr(), outer, R, inner, op, scratch.data_ptr() if want else None, want,
                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return out


def _noalloc(lib, x, outer, R, inner, op):
    out = torch.empty(outer * inner, device="cuda")
    err = ctypes.create_string_buffer(256)
    rc = lib.fb_reduce_noalloc(x.data_ptr(), out.data_ptr(), outer, R, inner, op,
                               torch.cuda.current_stream().cuda_stream, err, 256)
    return rc, out, err.value.decode()


@pytest.mark.parametrize("outer,R,inner,op", [(1, 1 << 22, 1, 0), (1, 3_000_001, 1, 1), (3, 100_000, 1, 2),
                                               (1, 20_000, 7, 0), (2, 9000, 33, 3), (64, 50, 1, 0)])
def test_noalloc_matches_existing_entry_point_twice_in_a_row(outer, R, inner, op):
    lib = _symbols()
    torch.manual_seed(outer + R + inner)
    for call in range(2):  # the second call starts from whatever the first left in the workspace
        x = torch.randn(outer * R * inner, device="cuda") * (call + 1)
        ref = _existing(lib, x, outer, R, inner, op)
        rc, got, msg = _noalloc(lib, x, outer, R, inner, op)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.allclose(got, ref, atol=1e-3 if op == 0 else 1e-5, rtol=1e-5), (call, outer, R, inner, op)
        exact = x.double().reshape(outer, R, inner)
        exact = {0: exact.sum(1), 1: exact.mean(1), 2: exact.max(1).values, 3: exact.min(1).values}[op].reshape(-1)
        assert torch.allclose(got.double(), exact, atol=1e-2 if op == 0 else 1e-4, rtol=1e-4)


def test_noalloc_rejects_shapes_beyond_the_builtin_workspace():
    lib = _symbols()
    outer, R, inner = 1, 8192, 550  # the split needs 2 x 550 partial sums; the workspace holds 1024
    assert lib.fb_reduce_scratch_elems(outer, R, inner) > 1024
    x = torch.zeros(outer * R * inner, device="cuda")
    sentinel = torch.full((inner,), -7.0, device="cuda")
    err = ctypes.create_string_buffer(256)
    rc = lib.fb_reduce_noalloc(x.data_ptr(), sentinel.data_ptr(), outer, R, inner, 0,
                               torch.cuda.current_stream().cuda_stream, err, 256)
    torch.cuda.synchronize()
    assert rc == TOO_LARGE
    assert "workspace" in err.value.decode()
    assert torch.all(sentinel == -7.0)  # nothing was launched
