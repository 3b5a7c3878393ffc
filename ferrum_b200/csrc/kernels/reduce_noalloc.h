// fb_reduce_noalloc — reduction entry point for callers that must not allocate.
//
// This entry point has no counterpart in the reference; it exists for hosts that
// embed this library under a fixed device-memory budget.  Think of a plugin inside
// somebody else's process, or a C host that was handed its input and output buffers
// and nothing else: such a caller owns no allocator it may grow at run time, and it
// may not call cudaMalloc / cudaFree itself, because those calls can fail late, they
// stall every stream of the device while they run, and they change a footprint that
// the embedding application sized once at start-up.  fb_reduce() needs a workspace
// from its caller for tall reductions; this variant brings its own.
//
// Same computation as fb_reduce (input viewed as [outer, R, inner], op = FB_RED_*),
// same kernels.  The workspace is a file-scope device array of
// FB_REDUCE_NOALLOC_MAX_FLOATS floats (4 KiB) that every GPU loading the library
// holds until the process exits.  Problems whose split needs more partial sums than
// that are rejected: the call returns FB_REDUCE_NOALLOC_TOO_LARGE and writes a
// message into `err` (when err != NULL); nothing is launched then.
//
// The function itself performs no allocation of any kind: no cudaMalloc / cudaFree,
// no allocating library routine.  The caller passes `x` and `out` as usual.
//
// First call on a device: the address of the array is looked up once per device
// (with that device current) and cached.  Make that first call ahead of any stream
// capture you intend to do on that device.
//
// Sharing: all calls on a device use the one array, and it keeps whatever the last
// call left in it.  Nothing in it has to start at zero — each call overwrites every
// slot it later reads — but two calls whose kernels overlap on the GPU (different
// streams, no ordering between them) race on it.  Order such calls yourself.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FB_REDUCE_NOALLOC_MAX_FLOATS 1024
#define FB_REDUCE_NOALLOC_TOO_LARGE (-5)

int fb_reduce_noalloc(const float* x, float* out, long long outer, long long R, long long inner, int op,
                      cudaStream_t stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
