// Reductions over a tensor viewed as [outer, R, inner]: sum / mean / max / min /
// prod, argmax / argmin, and the column-sum used for bias gradients.
//
// Reference: ferrum-cuda/src/kernels.rs:264-369 (reduce_op, outer x reduce x inner
// loops) and ferrum-core/src/tensor.rs:1611-2243 (sum, mean, sum_dim, mean_dim,
// argmax, argmin, max_dim, min_dim).
//
// inner == 1  : one block per row (vector loads, warp-shuffle + smem tree).
// inner  > 1  : one thread per output column, coalesced across `inner`.
// When there are too few outputs to fill the GPU, R is split across blockIdx.y
// and the partials go through a caller-provided scratch buffer (two launches,
// deterministic order).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>

#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

__device__ __forceinline__ float red_identity(int op) {
  switch (op) {
    case FB_RED_MAX: return -FLT_MAX;
    case FB_RED_MIN: return FLT_MAX;
    case FB_RED_PROD: return 1.f;
    default: return 0.f;
  }
}
__device__ __forceinline__ float red_combine(float a, float b, int op) {
  switch (op) {
    case FB_RED_MAX: return fmaxf(a, b);
    case FB_RED_MIN: return fminf(a, b);
    case FB_RED_PROD: return a * b;
    default: return a + b;
  }
}

__device__ __forceinline__ float block_reduce(float v, int op, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = red_combine(v, __shfl_xor_sync(0xffffffffu, v, o), op);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  v = (threadIdx.x < nw) ? smem[threadIdx.x] : red_identity(op);
  if (warp == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = red_combine(v, __shfl_xor_sync(0xffffffffu, v, o), op);
  }
  return v;  // valid in thread 0
}

// x: [outer, R]; block (row = blockIdx.x, split = blockIdx.y) reduces its segment.  The combining op is a template
// parameter (a per-element switch made the kernel issue-bound) and four 16-byte loads are in flight per thread.
template <int OP>
__device__ __forceinline__ float combine_t(float a, float b) {
  if (OP == FB_RED_MAX) return fmaxf(a, b);
  if (OP == FB_RED_MIN) return fminf(a, b);
  if (OP == FB_RED_PROD) return a * b;
  return a + b;
}
template <int OP>
__device__ __forceinline__ float fold4(float acc, const float4 v) {
  return combine_t<OP>(acc, combine_t<OP>(combine_t<OP>(v.x, v.y), combine_t<OP>(v.z, v.w)));
}

template <int OP>
__global__ void __launch_bounds__(256)
reduce_rows_kernel_t(const float* __restrict__ x, float* __restrict__ out, long long R, float scale, int splits) {
  __shared__ float smem[32];
  const long long row = blockIdx.x;
  const long long seg = (R + splits - 1) / splits;
  const long long lo = blockIdx.y * seg;
  const long long hi = min(R, lo + seg);
  const float* p = x + row * R;
  float acc = red_identity(OP);
  // vector body when the segment start is 16-byte aligned
  long long i = lo + threadIdx.x;
  if (((reinterpret_cast<uintptr_t>(p + lo) & 15) == 0) && hi - lo >= 4) {
    const long long n4 = (hi - lo) >> 2;
    const float4* p4 = reinterpret_cast<const float4*>(p + lo);
    long long k = threadIdx.x;
    float a1 = red_identity(OP), a2 = red_identity(OP), a3 = red_identity(OP);
    for (; k + 3 * blockDim.x < n4; k += 4 * blockDim.x) {
      const float4 v0 = p4[k], v1 = p4[k + blockDim.x], v2 = p4[k + 2 * blockDim.x], v3 = p4[k + 3 * blockDim.x];
      acc = fold4<OP>(acc, v0);
      a1 = fold4<OP>(a1, v1);
      a2 = fold4<OP>(a2, v2);
      a3 = fold4<OP>(a3, v3);
    }
    for (; k < n4; k += blockDim.x) acc = fold4<OP>(acc, p4[k]);
    acc = combine_t<OP>(combine_t<OP>(acc, a1), combine_t<OP>(a2, a3));
    i = lo + (n4 << 2) + threadIdx.x;
  }
  for (; i < hi; i += blockDim.x) acc = combine_t<OP>(acc, p[i]);
  acc = block_reduce(acc, OP, smem);
  if (threadIdx.x == 0) out[row * splits + blockIdx.y] = acc * scale;
}

void launch_reduce_rows(dim3 grid, cudaStream_t stream, const float* x, float* out, long long R, int op, float scale,
                        int splits) {
  const int cop = (op == FB_RED_MEAN) ? FB_RED_SUM : op;
  switch (cop) {
    case FB_RED_MAX: reduce_rows_kernel_t<FB_RED_MAX><<<grid, 256, 0, stream>>>(x, out, R, scale, splits); break;
    case FB_RED_MIN: reduce_rows_kernel_t<FB_RED_MIN><<<grid, 256, 0, stream>>>(x, out, R, scale, splits); break;
    case FB_RED_PROD: reduce_rows_kernel_t<FB_RED_PROD><<<grid, 256, 0, stream>>>(x, out, R, scale, splits); break;
    default: reduce_rows_kernel_t<FB_RED_SUM><<<grid, 256, 0, stream>>>(x, out, R, scale, splits); break;
  }
}

// x: [outer, R, inner]; thread per (outer, inner), optional split of R over blockIdx.y.
__global__ void reduce_cols_kernel(const float* __restrict__ x, float* __restrict__ out, long long outer,
                                   long long R, long long inner, int op, float scale, int splits) {
  const long long col = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (col >= outer * inner) return;
  const long long o = col / inner, in = col % inner;
  const long long seg = (R + splits - 1) / splits;
  const long long lo = blockIdx.y * seg;
  const long long hi = min(R, lo + seg);
  const int cop = (op == FB_RED_MEAN) ? FB_RED_SUM : op;
  float acc = red_identity(cop);
  const float* p = x + o * R * inner + in;
  for (long long r = lo; r < hi; ++r) acc = red_combine(acc, p[r * inner], cop);
  // partial layout: [splits, outer*inner]
  out[static_cast<long long>(blockIdx.y) * outer * inner + col] = acc * scale;
}

// x: [outer, R, inner] with inner % 4 == 0: block = 128 adjacent columns x a chunk of R (blockIdx.y) of one
// outer slice (blockIdx.z); lanes own 4 columns (16-byte loads), the 8 warps walk the rows four at a time and
// meet in shared memory.  Output layout [row_blocks, outer * inner]; a second launch folds the row blocks.
__global__ void __launch_bounds__(256)
reduce_cols_vec_kernel(const float* __restrict__ x, float* __restrict__ out, long long R, long long inner, int op,
                       float scale, long long rows_per_block, long long outs) {
  __shared__ float sm[8][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long c0 = static_cast<long long>(blockIdx.x) * 128 + lane * 4;
  const long long r_lo = static_cast<long long>(blockIdx.y) * rows_per_block;
  const long long r_hi = min(R, r_lo + rows_per_block);
  const int cop = (op == FB_RED_MEAN) ? FB_RED_SUM : op;
  const float id = red_identity(cop);
  float a0 = id, a1 = id, a2 = id, a3 = id;
  const float* base = x + static_cast<long long>(blockIdx.z) * R * inner;
  if (c0 < inner) {
    for (long long r = r_lo + warp; r < r_hi; r += 32) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long rr = r + 8 * u;
        v[u] = rr < r_hi ? *reinterpret_cast<const float4*>(base + rr * inner + c0) : make_float4(id, id, id, id);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a0 = red_combine(a0, v[u].x, cop);
        a1 = red_combine(a1, v[u].y, cop);
        a2 = red_combine(a2, v[u].z, cop);
        a3 = red_combine(a3, v[u].w, cop);
      }
    }
  }
  sm[warp][lane * 4 + 0] = a0;
  sm[warp][lane * 4 + 1] = a1;
  sm[warp][lane * 4 + 2] = a2;
  sm[warp][lane * 4 + 3] = a3;
  __syncthreads();
  if (threadIdx.x < 128) {
    float s = sm[0][threadIdx.x];
#pragma unroll
    for (int w = 1; w < 8; ++w) s = red_combine(s, sm[w][threadIdx.x], cop);
    const long long c = static_cast<long long>(blockIdx.x) * 128 + threadIdx.x;
    if (c < inner)
      out[static_cast<long long>(blockIdx.y) * outs + static_cast<long long>(blockIdx.z) * inner + c] = s * scale;
  }
}

// One 128-thread block per row: 16-byte loads (two in flight per thread), then a warp-shuffle tournament on
// (value, index) with ties going to the lower index, then four warp winners through shared memory.
__global__ void __launch_bounds__(128)
arg_rows_kernel(const float* __restrict__ x, long long* __restrict__ idx, float* __restrict__ val, long long R,
                int is_max) {
  __shared__ float sv[4];
  __shared__ long long si[4];
  const long long row = blockIdx.x;
  const float* p = x + row * R;
  float best = is_max ? -FLT_MAX : FLT_MAX;
  long long bi = 0x7fffffffffffffffLL;
  auto consider = [&](float v, long long i) {
    if (is_max ? (v > best) : (v < best)) {  // strict: the first occurrence wins inside a thread (i increases)
      best = v;
      bi = i;
    }
  };
  const long long head = min(R, static_cast<long long>((16 - (reinterpret_cast<uintptr_t>(p) & 15)) & 15) / 4);
  for (long long i = threadIdx.x; i < head; i += blockDim.x) consider(p[i], i);
  const float4* q = reinterpret_cast<const float4*>(p + head);
  const long long nv = (R - head) >> 2;
  for (long long i = threadIdx.x; i < nv; i += 2 * blockDim.x) {
    const long long j = i + blockDim.x;
    const float4 a = q[i];
    float4 b = a;
    if (j < nv) b = q[j];
    const long long ia = head + 4 * i, ib = head + 4 * j;
    consider(a.x, ia); consider(a.y, ia + 1); consider(a.z, ia + 2); consider(a.w, ia + 3);
    if (j < nv) {
      consider(b.x, ib); consider(b.y, ib + 1); consider(b.z, ib + 2); consider(b.w, ib + 3);
    }
  }
  for (long long i = head + (nv << 2) + threadIdx.x; i < R; i += blockDim.x) consider(p[i], i);
  auto merge = [&](float ov, long long oi) {
    const bool better = is_max ? (ov > best) : (ov < best);
    if (better || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
    merge(ov, oi);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    for (int w = 1; w < nw; ++w) merge(sv[w], si[w]);
    idx[row] = bi == 0x7fffffffffffffffLL ? 0 : bi;
    if (val) val[row] = best;
  }
}

__global__ void arg_cols_kernel(const float* __restrict__ x, long long* __restrict__ idx, float* __restrict__ val,
                                long long outer, long long R, long long inner, int is_max) {
  const long long col = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (col >= outer * inner) return;
  const long long o = col / inner, in = col % inner;
  const float* p = x + o * R * inner + in;
  float best = p[0];
  long long bi = 0;
  for (long long r = 1; r < R; ++r) {
    const float v = p[r * inner];
    if (is_max ? (v > best) : (v < best)) {
      best = v;
      bi = r;
    }
  }
  idx[col] = bi;
  if (val) val[col] = best;
}

// Column sums of [rows, cols]: a block covers 32 x V adjacent columns (V = elements per 16 bytes: 4 fp32, 8 bf16)
// and a chunk of rows; its 8 warps walk the rows, a lane owns V adjacent columns and keeps eight independent
// 16-byte loads in flight; the partials meet in shared memory and leave with one atomicAdd per column per block.
template <typename T>
struct ColVec {
  static constexpr int kV = 16 / sizeof(T);
};

template <typename T>
__global__ void __launch_bounds__(256)
colsum_kernel(const T* __restrict__ x, float* __restrict__ out, long long rows, long long cols,
              long long rows_per_block) {
  constexpr int kV = ColVec<T>::kV, kCols = 32 * kV, kU = 8;
  __shared__ float sm[8][kCols];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long c0 = static_cast<long long>(blockIdx.x) * kCols + lane * kV;
  const long long r_lo = static_cast<long long>(blockIdx.y) * rows_per_block;
  const long long r_hi = min(rows, r_lo + rows_per_block);
  float acc[kV];
#pragma unroll
  for (int i = 0; i < kV; ++i) acc[i] = 0.f;
  const bool vec = (cols % kV == 0) && (c0 + kV - 1 < cols) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  if (vec) {
    for (long long r = r_lo + warp; r < r_hi; r += 8 * kU) {
      uint4 v[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const long long rr = r + 8 * u;
        v[u] = rr < r_hi ? *reinterpret_cast<const uint4*>(x + rr * cols + c0) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
        if constexpr (sizeof(T) == 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i] += __uint_as_float(w[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {  // bf16 -> fp32 is a 16-bit shift
            acc[2 * i] += __uint_as_float(w[i] << 16);
            acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
          }
        }
      }
    }
  } else {
    for (long long r = r_lo + warp; r < r_hi; r += 8) {
      const T* p = x + r * cols + c0;
#pragma unroll
      for (int i = 0; i < kV; ++i)
        if (c0 + i < cols) acc[i] += static_cast<float>(p[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < kV; ++i) sm[warp][lane * kV + i] = acc[i];
  __syncthreads();
  for (int t = threadIdx.x; t < kCols; t += 256) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += sm[w][t];
    const long long c = static_cast<long long>(blockIdx.x) * kCols + t;
    if (c < cols) atomicAdd(out + c, s);
  }
}

int sm_count() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace
}  // namespace fb

using namespace fb;

// Number of scratch floats fb_reduce wants for this problem (0 = single pass).
// Row blocks the vectorised column reduction uses for [outer, R, inner] (0 = not applicable).
static long long vec_row_blocks(long long outer, long long R, long long inner) {
  if (inner % 4 != 0 || inner < 4 || outer > 65535) return 0;
  const long long col_blocks = ((inner + 127) / 128) * outer;
  long long rb = (static_cast<long long>(sm_count()) * 4 + col_blocks - 1) / col_blocks;
  const long long max_rb = (R + 31) / 32;
  if (rb > max_rb) rb = max_rb;
  if (rb > 65535) rb = 65535;
  return rb < 1 ? 1 : rb;
}

// Number of scratch floats fb_reduce wants for this problem (0 = single pass).
extern "C" long long fb_reduce_scratch_elems(long long outer, long long R, long long inner) {
  const long long outs = outer * inner;
  if (outs <= 0) return 0;
  if (inner > 1) {
    const long long rb = vec_row_blocks(outer, R, inner);
    if (rb > 1) return rb * outs;
  }
  if (R < 4096) return 0;
  // blocks a single pass would launch: one per row (inner == 1) or one per 256 columns
  const long long blocks = inner == 1 ? outs : (outs + 255) / 256;
  const long long target = static_cast<long long>(sm_count()) * 4;
  if (blocks >= target / 2) return 0;
  long long splits = (target + blocks - 1) / blocks;
  const long long max_splits = (R + 1023) / 1024;
  if (splits > max_splits) splits = max_splits;
  if (splits <= 1) return 0;
  return splits * outs;
}

extern "C" int fb_reduce(const float* x, float* out, long long outer, long long R, long long inner, int op,
                         float* scratch, long long scratch_elems, cudaStream_t stream) {
  if (outer <= 0 || inner <= 0) return 0;
  if (R <= 0) return -1;
  const long long outs = outer * inner;
  const float final_scale = (op == FB_RED_MEAN) ? 1.f / static_cast<float>(R) : 1.f;
  int splits = 1;
  if (scratch != nullptr && scratch_elems >= 2 * outs) {
    const long long want = fb_reduce_scratch_elems(outer, R, inner);
    if (want > 0 && want <= scratch_elems) splits = static_cast<int>(want / outs);
  }
  const int stage_op = (op == FB_RED_MEAN) ? FB_RED_SUM : op;
  if (inner == 1) {
    if (outer > 2147483647LL) return -1;
    if (splits == 1) {
      launch_reduce_rows(dim3(static_cast<unsigned>(outer), 1), stream, x, out, R, op, final_scale, 1);
    } else {
      launch_reduce_rows(dim3(static_cast<unsigned>(outer), splits), stream, x, scratch, R, stage_op, 1.f, splits);
      launch_reduce_rows(dim3(static_cast<unsigned>(outer), 1), stream, scratch, out, splits, stage_op, final_scale,
                         1);
    }
  } else if (vec_row_blocks(outer, R, inner) > 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
             (vec_row_blocks(outer, R, inner) == 1 ||
              (scratch != nullptr && scratch_elems >= vec_row_blocks(outer, R, inner) * outs))) {
    const long long rb = vec_row_blocks(outer, R, inner);
    const long long rpb = (R + rb - 1) / rb;
    const dim3 grid(static_cast<unsigned>((inner + 127) / 128), static_cast<unsigned>(rb),
                    static_cast<unsigned>(outer));
    if (rb == 1) {
      reduce_cols_vec_kernel<<<grid, 256, 0, stream>>>(x, out, R, inner, op, final_scale, rpb, outs);
    } else {
      reduce_cols_vec_kernel<<<grid, 256, 0, stream>>>(x, scratch, R, inner, stage_op, 1.f, rpb, outs);
      const unsigned gx = static_cast<unsigned>((outs + 255) / 256);
      reduce_cols_kernel<<<dim3(gx, 1), 256, 0, stream>>>(scratch, out, 1, rb, outs, stage_op, final_scale, 1);
    }
  } else {
    const unsigned gx = static_cast<unsigned>((outs + 255) / 256);
    if (splits == 1) {
      reduce_cols_kernel<<<dim3(gx, 1), 256, 0, stream>>>(x, out, outer, R, inner, op, final_scale, 1);
    } else {
      reduce_cols_kernel<<<dim3(gx, splits), 256, 0, stream>>>(x, scratch, outer, R, inner, stage_op, 1.f, splits);
      reduce_cols_kernel<<<dim3(gx, 1), 256, 0, stream>>>(scratch, out, 1, splits, outs, stage_op, final_scale, 1);
    }
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_arg_reduce(const float* x, long long* idx, float* val, long long outer, long long R,
                             long long inner, int is_max, cudaStream_t stream) {
  if (outer <= 0 || inner <= 0) return 0;
  if (R <= 0) return -1;
  if (inner == 1) {
    arg_rows_kernel<<<static_cast<unsigned>(outer), 128, 0, stream>>>(x, idx, val, R, is_max);
  } else {
    const long long outs = outer * inner;
    arg_cols_kernel<<<static_cast<unsigned>((outs + 255) / 256), 256, 0, stream>>>(x, idx, val, outer, R, inner,
                                                                                  is_max);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_colsum(const void* x, float* out, long long rows, long long cols, int dtype, int accumulate,
                         cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (!accumulate) {
    cudaError_t e = cudaMemsetAsync(out, 0, cols * sizeof(float), stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const long long per_block = dtype == FB_DT_BF16 ? 256 : 128;  // 32 lanes x 16 bytes
  const long long col_blocks = (cols + per_block - 1) / per_block;
  long long row_blocks = (static_cast<long long>(sm_count()) * 4 + col_blocks - 1) / col_blocks;
  const long long max_rb = (rows + 63) / 64;
  if (row_blocks > max_rb) row_blocks = max_rb;
  if (row_blocks < 1) row_blocks = 1;
  if (row_blocks > 65535) row_blocks = 65535;
  const long long rpb = (rows + row_blocks - 1) / row_blocks;
  dim3 grid(static_cast<unsigned>(col_blocks), static_cast<unsigned>(row_blocks));
  if (dtype == FB_DT_F32) {
    colsum_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), out, rows, cols, rpb);
  } else if (dtype == FB_DT_BF16) {
    colsum_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), out, rows, cols,
                                                           rpb);
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

// ----------------------------------------------------------------------------
// Allocation-free variant (declared in reduce_noalloc.h).
#include <cstdio>
#include <mutex>

#include "reduce_noalloc.h"

namespace {

// Workspace of fb_reduce_noalloc.  In host code this name is only a handle for
// cudaGetSymbolAddress; the device address it yields is what kernels receive.
static __device__ __align__(256) float g_reduce_noalloc_scratch[FB_REDUCE_NOALLOC_MAX_FLOATS];

constexpr int kNoAllocMaxDevices = 64;
float* g_noalloc_ptr[kNoAllocMaxDevices] = {};
std::mutex g_noalloc_mu;

void noalloc_err(char* err, int err_len, const char* msg) {
  if (err != nullptr && err_len > 0) std::snprintf(err, static_cast<size_t>(err_len), "%s", msg);
}

}  // namespace

extern "C" int fb_reduce_noalloc(const float* x, float* out, long long outer, long long R, long long inner,
                                 int op, cudaStream_t stream, char* err, int err_len) {
  if (err != nullptr && err_len > 0) err[0] = '\0';
  if (outer <= 0 || inner <= 0) return 0;
  if (R <= 0) {
    noalloc_err(err, err_len, "fb_reduce_noalloc: reduced extent R must be positive");
    return -1;
  }
  const long long want = fb_reduce_scratch_elems(outer, R, inner);
  if (want > FB_REDUCE_NOALLOC_MAX_FLOATS) {
    char msg[200];
    std::snprintf(msg, sizeof(msg),
                  "fb_reduce_noalloc: this shape needs %lld partial sums, the built-in workspace holds %d; "
                  "use fb_reduce with a caller-provided workspace",
                  want, FB_REDUCE_NOALLOC_MAX_FLOATS);
    noalloc_err(err, err_len, msg);
    return FB_REDUCE_NOALLOC_TOO_LARGE;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kNoAllocMaxDevices) {
    noalloc_err(err, err_len, "fb_reduce_noalloc: device ordinal out of range");
    return -1;
  }
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
      // once per device, with that device current
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_reduce_noalloc_scratch);
      if (e != cudaSuccess) {
        noalloc_err(err, err_len, "fb_reduce_noalloc: cudaGetSymbolAddress failed");
        return static_cast<int>(e);
      }
      g_noalloc_ptr[dev] = static_cast<float*>(p);
    }
    scratch = g_noalloc_ptr[dev];
  }
  return fb_reduce(x, out, outer, R, inner, op, want > 0 ? scratch : nullptr,
                   want > 0 ? FB_REDUCE_NOALLOC_MAX_FLOATS : 0, stream);
}
