// Dropout (Philox mask), Embedding gather / mean-pool / scatter-add, generic
// row gather for device-resident DataLoader batches, and BatchNorm1d.
//
// Reference behaviour these replace:
//   ferrum-nn/src/norm.rs:171-219      Dropout (reference multiplies by (1-p) without a
//                                      mask; this is real inverted dropout)
//   ferrum-nn/src/embedding.rs:122-208 Embedding.forward (host gather, padding_idx rows
//                                      zero, out-of-range index is an error, no backward)
//   ferrum-nn/src/norm.rs:75-165,242-283 BatchNorm1d (reference uses one global mean /
//                                      variance and never updates running stats; this is
//                                      per feature with running-stat update, full-grid passes)
//   ferrum-data/src/dataloader.rs:144-165 per-index dataset.get (here: one row-gather launch)
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../common/status.h"
#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

// ------------------------------------------------------------------ Philox
struct Philox {
  uint32_t c[4];
  uint32_t k[2];
};
__device__ __forceinline__ void philox_round(Philox& s) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, s.c[0]), lo0 = 0xD2511F53u * s.c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, s.c[2]), lo1 = 0xCD9E8D57u * s.c[2];
  const uint32_t n0 = hi1 ^ s.c[1] ^ s.k[0];
  const uint32_t n2 = hi0 ^ s.c[3] ^ s.k[1];
  s.c[0] = n0;
  s.c[1] = lo1;
  s.c[2] = n2;
  s.c[3] = lo0;
  s.k[0] += 0x9E3779B9u;
  s.k[1] += 0xBB67AE85u;
}
__device__ __forceinline__ void philox4x32_10(unsigned long long seed, unsigned long long ctr,
                                              unsigned long long offset, uint32_t (&out)[4]) {
  Philox s;
  s.c[0] = static_cast<uint32_t>(ctr);
  s.c[1] = static_cast<uint32_t>(ctr >> 32);
  s.c[2] = static_cast<uint32_t>(offset);
  s.c[3] = static_cast<uint32_t>(offset >> 32);
  s.k[0] = static_cast<uint32_t>(seed);
  s.k[1] = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) philox_round(s);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = s.c[i];
}

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void stf(T* p, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// One Philox call covers 4 consecutive elements.
// One Philox call yields 128 random bits = eight 16-bit draws: a thread handles eight consecutive elements per
// call (one 16-byte load / store of bf16, two of fp32, one 8-byte mask store).  Keep-probability resolution 2^-16.
template <typename T>
__global__ void __launch_bounds__(256)
dropout_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ mask, long long n, float p,
                   unsigned long long seed, unsigned long long offset,
                   const unsigned long long* __restrict__ dev_offset) {
  if (dev_offset != nullptr) offset += *dev_offset;  // advanced on the stream between calls: graph replays differ
  const float scale = 1.f / (1.f - p);
  const uint32_t thresh = static_cast<uint32_t>(fminf(fmaxf(p, 0.f), 1.f) * 65536.0f);  // keep when draw >= thresh
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long n8 = (n + 7) >> 3;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(mask) & 7) == 0;
  for (long long q = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; q < n8; q += stride) {
    uint32_t r[4];
    philox4x32_10(seed, static_cast<unsigned long long>(q), offset, r);
    bool keep[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) keep[j] = ((r[j >> 1] >> ((j & 1) * 16)) & 0xffffu) >= thresh;
    const long long i0 = q * 8;
    if (aligned && i0 + 8 <= n) {
      float v[8];
      if constexpr (sizeof(T) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + i0);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          v[2 * e] = f.x;
          v[2 * e + 1] = f.y;
        }
      } else {
        const float4 a = *reinterpret_cast<const float4*>(x + i0);
        const float4 b = *reinterpret_cast<const float4*>(x + i0 + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
      }
      uint32_t m0 = 0, m1 = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[j] = keep[j] ? v[j] * scale : 0.f;
        if (keep[j]) (j < 4 ? m0 : m1) |= 1u << ((j & 3) * 8);
      }
      *reinterpret_cast<uint2*>(mask + i0) = make_uint2(m0, m1);
      if constexpr (sizeof(T) == 2) {
        uint4 out;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
        *reinterpret_cast<uint4*>(y + i0) = out;
      } else {
        *reinterpret_cast<float4*>(y + i0) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(y + i0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const long long i = i0 + j;
        if (i < n) {
          mask[i] = keep[j] ? 1 : 0;
          stf(y + i, keep[j] ? ldf(x + i) * scale : 0.f);
        }
      }
    }
  }
}
template <typename T>
__global__ void __launch_bounds__(256)
dropout_bwd_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ mask, T* __restrict__ dx, long long n,
                   float p) {
  const float scale = 1.f / (1.f - p);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(mask) & 7) == 0;
  const long long n8 = aligned ? (n >> 3) : 0;
  for (long long q = tid; q < n8; q += stride) {
    const long long i0 = q * 8;
    const uint2 m = *reinterpret_cast<const uint2*>(mask + i0);
    float v[8];
    if constexpr (sizeof(T) == 2) {
      const uint4 raw = *reinterpret_cast<const uint4*>(dy + i0);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        v[2 * e] = f.x;
        v[2 * e + 1] = f.y;
      }
    } else {
      const float4 a = *reinterpret_cast<const float4*>(dy + i0);
      const float4 b = *reinterpret_cast<const float4*>(dy + i0 + 4);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t bits = (j < 4 ? m.x : m.y) >> ((j & 3) * 8);
      v[j] = (bits & 0xffu) ? v[j] * scale : 0.f;
    }
    if constexpr (sizeof(T) == 2) {
      uint4 out;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
      *reinterpret_cast<uint4*>(dx + i0) = out;
    } else {
      *reinterpret_cast<float4*>(dx + i0) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(dx + i0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
  for (long long i = (n8 << 3) + tid; i < n; i += stride) stf(dx + i, mask[i] ? ldf(dy + i) * scale : 0.f);
}

__global__ void counter_add_kernel(unsigned long long* ctr, unsigned long long inc) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *ctr += inc;
}

// --------------------------------------------------------------- Embedding
// One warp per looked-up row.
template <typename O>
__global__ void embedding_fwd_kernel(const float* __restrict__ w, const long long* __restrict__ idx,
                                     O* __restrict__ out, long long n_idx, int dim, long long vocab,
                                     long long padding_idx, int32_t* status) {
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long i = warp; i < n_idx; i += nwarps) {
    const long long id = idx[i];
    const bool oob = id < 0 || id >= vocab;
    if (oob && lane == 0) report_status(status, kStatusBoundsViolation, 10, static_cast<int32_t>(i),
                                        static_cast<int32_t>(id));
    const bool zero = oob || id == padding_idx;
    const float* src = w + (zero ? 0 : id) * dim;
    O* dst = out + i * dim;
    for (int c = lane; c < dim; c += 32) stf(dst + c, zero ? 0.f : src[c]);
  }
}

// out[b, :] = (1/seq) * sum_s W[idx[b, s], :]; one block per batch row, threads over dim.
template <typename O>
__global__ void embedding_meanpool_kernel(const float* __restrict__ w, const long long* __restrict__ idx,
                                          O* __restrict__ out, long long batch, int seq, int dim,
                                          long long vocab) {
  extern __shared__ long long sidx[];
  for (long long b = blockIdx.x; b < batch; b += gridDim.x) {
    __syncthreads();
    for (int s = threadIdx.x; s < seq; s += blockDim.x) {
      const long long id = idx[b * seq + s];
      sidx[s] = (id < 0 || id >= vocab) ? -1 : id;
    }
    __syncthreads();
    const float inv = 1.f / static_cast<float>(seq);
    if ((dim & 3) == 0) {
      for (int c4 = threadIdx.x; c4 < (dim >> 2); c4 += blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < seq; ++s) {
          const long long id = sidx[s];
          if (id >= 0) {
            const float4 v = reinterpret_cast<const float4*>(w + id * dim)[c4];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
        }
        O* dst = out + b * dim + c4 * 4;
        stf(dst, acc.x * inv); stf(dst + 1, acc.y * inv); stf(dst + 2, acc.z * inv); stf(dst + 3, acc.w * inv);
      }
    } else {
      for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < seq; ++s) {
          const long long id = sidx[s];
          if (id >= 0) acc += w[id * dim + c];
        }
        stf(out + b * dim + c, acc * inv);
      }
    }
  }
}

// Scatter-add over a SORTED index list: a block walks a chunk of 32 consecutive positions, sums runs of equal
// indices in registers and flushes each run once, so heavily repeated tokens cost one flush per chunk instead of
// one per occurrence.  perm[i] is the original position.  The chunk's ids and source rows are staged in shared
// memory once (one 64-bit division per position instead of one per thread and position); with dim % 4 == 0 a
// thread owns four adjacent columns: 8- or 16-byte loads of dout and one vector atomic (red.global.add.v4.f32)
// per run.
template <typename G>
__global__ void embedding_bwd_sorted_kernel(const G* __restrict__ dout, const long long* __restrict__ sorted_idx,
                                            const long long* __restrict__ perm, float* __restrict__ dw,
                                            long long n_idx, int dim, int group, float scale,
                                            long long padding_idx, long long vocab, int32_t* bstatus) {
  constexpr int kChunk = 32;
  __shared__ long long s_id[kChunk];
  __shared__ long long s_row[kChunk];
  const long long lo = static_cast<long long>(blockIdx.x) * kChunk;
  const int cnt = static_cast<int>(min(n_idx, lo + kChunk) - lo);
  if (threadIdx.x < cnt) {
    long long id = sorted_idx[lo + threadIdx.x];
    const long long row = perm[lo + threadIdx.x] / group;
    // ids outside the table were reported by the forward pass; their gradient rows are dropped, never written.
    if (id >= vocab) id = -1;
    if (!FB_INDEX_OK(bstatus, 40, row, (n_idx + group - 1) / group)) id = -1;
    s_id[threadIdx.x] = id;
    s_row[threadIdx.x] = id < 0 ? 0 : row;
  }
  __syncthreads();
  const bool vec = dim % 4 == 0 && (reinterpret_cast<uintptr_t>(dw) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(dout) & (4 * sizeof(G) - 1)) == 0;
  if (vec) {
    for (int c = threadIdx.x * 4; c < dim; c += blockDim.x * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      long long cur = -1;
      auto flush = [&]() {
        if (cur >= 0 && cur != padding_idx)
          atomicAdd(reinterpret_cast<float4*>(dw + cur * dim + c),
                    make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale));
      };
#pragma unroll 4
      for (int k = 0; k < cnt; ++k) {
        const long long id = s_id[k];
        if (id != cur) {
          flush();
          cur = id;
          acc = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const G* src = dout + s_row[k] * dim + c;
        if constexpr (sizeof(G) == 2) {
          const uint2 u = *reinterpret_cast<const uint2*>(src);
          const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
          const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
          acc.x += f0.x; acc.y += f0.y; acc.z += f1.x; acc.w += f1.y;
        } else {
          const float4 f = *reinterpret_cast<const float4*>(src);
          acc.x += f.x; acc.y += f.y; acc.z += f.z; acc.w += f.w;
        }
      }
      flush();
    }
  } else {
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      float acc = 0.f;
      long long cur = -1;
      for (int k = 0; k < cnt; ++k) {
        const long long id = s_id[k];
        if (id != cur) {
          if (cur >= 0 && cur != padding_idx) atomicAdd(dw + cur * dim + c, acc * scale);
          cur = id;
          acc = 0.f;
        }
        acc += ldf(dout + s_row[k] * dim + c);
      }
      if (cur >= 0 && cur != padding_idx) atomicAdd(dw + cur * dim + c, acc * scale);
    }
  }
}

// An index outside [0, n_rows) is reported (site 11) and its output row is zero-filled; the source is not read.
__global__ void gather_rows_kernel(const uint8_t* __restrict__ src, const long long* __restrict__ idx,
                                   uint8_t* __restrict__ dst, long long n_idx, long long row_bytes,
                                   long long n_rows, int32_t* status) {
  const bool vec = (row_bytes % 16 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
  for (long long i = blockIdx.x; i < n_idx; i += gridDim.x) {
    const long long id = idx[i];
    const bool oob = id < 0 || id >= n_rows;
    if (oob && threadIdx.x == 0)
      report_status(status, kStatusBoundsViolation, 11, static_cast<int32_t>(i), static_cast<int32_t>(id));
    uint8_t* d = dst + i * row_bytes;
    if (oob) {  // block-uniform: the whole row is zero-filled, the source is not read
      for (long long k = threadIdx.x; k < row_bytes; k += blockDim.x) d[k] = 0;
      continue;
    }
    const uint8_t* s = src + id * row_bytes;
    if (vec) {
      const long long nv = row_bytes >> 4;
      for (long long k = threadIdx.x; k < nv; k += blockDim.x)
        reinterpret_cast<uint4*>(d)[k] = reinterpret_cast<const uint4*>(s)[k];
    } else {
      for (long long k = threadIdx.x; k < row_bytes; k += blockDim.x) d[k] = s[k];
    }
  }
}

// --------------------------------------------------------------- BatchNorm
// BatchNorm1d over [rows, cols] fp32.  Column statistics come from full-grid passes (a block = 128 columns x a
// chunk of rows, lanes own 4 adjacent columns with 16-byte loads, warps walk the rows four at a time, partials
// meet in shared memory and leave with one atomicAdd per column per block), so a 1024-feature layer uses the
// whole GPU instead of 32 blocks.  Training forward = ONE statistics pass (sums of x - k and (x - k)^2 with k = the
// column's first row: shifted data, so the variance is not a difference of two large numbers), finalize, apply;
// backward = one two-statistic pass (d_beta, d_gamma) and one elementwise pass.
//   MODE 2: a += dy, b += dy * (x - mean) * rstd
//   MODE 3: a += x - k, b += (x - k)^2      k = x[0, column] (read by the kernel; `mean` unused)
template <int MODE>
__global__ void __launch_bounds__(256)
bn_colstats_kernel(const float* __restrict__ x, const float* __restrict__ dy, const float* __restrict__ mean,
                   const float* __restrict__ rstd, float* __restrict__ out_a, float* __restrict__ out_b,
                   long long rows, int cols, long long rows_per_block) {
  __shared__ float sm_a[8][128];
  __shared__ float sm_b[MODE >= 2 ? 8 : 1][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = blockIdx.x * 128 + lane * 4;
  const long long r_lo = static_cast<long long>(blockIdx.y) * rows_per_block;
  const long long r_hi = min(rows, r_lo + rows_per_block);
  const bool vec = (cols % 4 == 0) && (c0 + 3 < cols);
  float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
  float mu[4] = {0.f, 0.f, 0.f, 0.f}, rs[4] = {0.f, 0.f, 0.f, 0.f};
  {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (c0 + j < cols) {
        mu[j] = MODE == 3 ? x[c0 + j] : mean[c0 + j];
        if (MODE == 2) rs[j] = rstd[c0 + j];
      }
  }
  auto accum = [&](const float (&xv)[4], const float (&gv)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (MODE == 2) {
        a[j] += gv[j];
        b[j] = fmaf(gv[j], (xv[j] - mu[j]) * rs[j], b[j]);
      }
      if (MODE == 3) {
        const float d = xv[j] - mu[j];
        a[j] += d;
        b[j] = fmaf(d, d, b[j]);
      }
    }
  };
  if (vec) {
    for (long long r = r_lo + warp; r < r_hi; r += 32) {
      float4 xv[4], gv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {  // four independent rows in flight per thread
        const long long rr = r + 8 * u;
        const bool ok = rr < r_hi;
        xv[u] = ok ? *reinterpret_cast<const float4*>(x + rr * cols + c0) : make_float4(mu[0], mu[1], mu[2], mu[3]);
        if (MODE == 2) gv[u] = ok ? *reinterpret_cast<const float4*>(dy + rr * cols + c0) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        // padded rows equal the shift / the mean: no effect
        const float xa[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
        const float ga[4] = {gv[u].x, gv[u].y, gv[u].z, gv[u].w};
        accum(xa, ga);
      }
    }
  } else {
    for (long long r = r_lo + warp; r < r_hi; r += 8) {
      float xa[4] = {mu[0], mu[1], mu[2], mu[3]}, ga[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c0 + j < cols) {
          xa[j] = x[r * cols + c0 + j];
          if (MODE == 2) ga[j] = dy[r * cols + c0 + j];
        }
      accum(xa, ga);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    sm_a[warp][lane * 4 + j] = a[j];
    if (MODE >= 2) sm_b[warp][lane * 4 + j] = b[j];
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    const int c = blockIdx.x * 128 + threadIdx.x;
    float ta = 0.f, tb = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      ta += sm_a[w][threadIdx.x];
      if (MODE >= 2) tb += sm_b[w][threadIdx.x];
    }
    if (c < cols) {
      atomicAdd(out_a + c, ta);
      if (MODE >= 2) atomicAdd(out_b + c, tb);
    }
  }
}

// mean holds sum(x - k), rstd holds sum((x - k)^2), k = x0[column] (the first row): both statistics and the
// running buffers are finished here.
__global__ void bn_finalize_kernel(float* __restrict__ mean, float* __restrict__ rstd, float* __restrict__ running_mean,
                                   float* __restrict__ running_var, long long rows, int cols, float eps,
                                   float momentum, const float* __restrict__ x0) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const float m = mean[c] / static_cast<float>(rows);  // mean of the shifted data
  const float var = fmaxf(rstd[c] / static_cast<float>(rows) - m * m, 0.f);
  mean[c] = x0[c] + m;
  rstd[c] = rsqrtf(var + eps);
  if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mean[c];
  if (running_var) {
    const float unbiased = rows > 1 ? var * static_cast<float>(rows) / static_cast<float>(rows - 1) : var;
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * unbiased;
  }
}

// y = (x - mean) * rstd * gamma + beta  (eval: statistics from the running buffers).  A thread owns four fixed
// columns (when cols % 4 == 0 and the grid stride is a multiple of cols / 4), so scale and shift sit in registers.
__global__ void __launch_bounds__(256)
bn_apply_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                const float* __restrict__ mean, const float* __restrict__ rstd_or_var, float* __restrict__ y,
                long long rows, int cols, float eps, int stats_are_running) {
  const long long n = rows * cols;
  auto scale_shift = [&](int c, float& sc, float& sh) {
    const float rs = stats_are_running ? rsqrtf(rstd_or_var[c] + eps) : rstd_or_var[c];
    sc = rs * (gamma ? gamma[c] : 1.f);
    sh = (beta ? beta[c] : 0.f) - mean[c] * sc;
  };
  if (cols % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
    const int vpr = cols / 4;  // vectors per row
    const long long nv = n / 4;
    // stride chosen by the launcher as a multiple of vpr: the thread's columns never change
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (first >= nv) return;
    const bool fixed = stride % vpr == 0;
    float sc[4], sh[4];
    const int c0 = static_cast<int>(first % vpr) * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) scale_shift(c0 + j, sc[j], sh[j]);
    for (long long i = first; i < nv; i += stride) {
      if (!fixed) {
        const int c = static_cast<int>(i % vpr) * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) scale_shift(c + j, sc[j], sh[j]);
      }
      float4 v = reinterpret_cast<const float4*>(x)[i];
      v.x = fmaf(v.x, sc[0], sh[0]);
      v.y = fmaf(v.y, sc[1], sh[1]);
      v.z = fmaf(v.z, sc[2], sh[2]);
      v.w = fmaf(v.w, sc[3], sh[3]);
      reinterpret_cast<float4*>(y)[i] = v;
    }
  } else {
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float sc, sh;
      scale_shift(static_cast<int>(i % cols), sc, sh);
      y[i] = fmaf(x[i], sc, sh);
    }
  }
}

// dx = gamma * rstd / rows * (rows * dy - d_beta - xhat * d_gamma), rewritten per column as
// dx = A * dy + B * x + C with A = gamma rstd, B = -gamma rstd^2 d_gamma / rows,
// C = -(gamma rstd / rows) d_beta - B mean.  Thread-fixed columns as in bn_apply_kernel.
__global__ void __launch_bounds__(256)
bn_dx_kernel(const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
             const float* __restrict__ mean, const float* __restrict__ rstd, const float* __restrict__ dgamma,
             const float* __restrict__ dbeta, float* __restrict__ dx, long long rows, int cols) {
  const long long n = rows * cols;
  const float inv_rows = 1.f / static_cast<float>(rows);
  auto coeffs = [&](int c, float& A, float& B, float& C) {
    const float rs = rstd[c], g = gamma ? gamma[c] : 1.f;
    A = g * rs;
    B = -g * rs * rs * dgamma[c] * inv_rows;
    C = -A * inv_rows * dbeta[c] - B * mean[c];
  };
  const bool vec = cols % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) |
                                      reinterpret_cast<uintptr_t>(dx)) & 15) == 0;
  if (vec) {
    const int vpr = cols / 4;
    const long long nv = n / 4;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (first >= nv) return;
    const bool fixed = stride % vpr == 0;
    float A[4], B[4], C[4];
    const int c0 = static_cast<int>(first % vpr) * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) coeffs(c0 + j, A[j], B[j], C[j]);
    for (long long i = first; i < nv; i += stride) {
      if (!fixed) {
        const int c = static_cast<int>(i % vpr) * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) coeffs(c + j, A[j], B[j], C[j]);
      }
      const float4 g = reinterpret_cast<const float4*>(dy)[i];
      const float4 v = reinterpret_cast<const float4*>(x)[i];
      float4 o;
      o.x = fmaf(A[0], g.x, fmaf(B[0], v.x, C[0]));
      o.y = fmaf(A[1], g.y, fmaf(B[1], v.y, C[1]));
      o.z = fmaf(A[2], g.z, fmaf(B[2], v.z, C[2]));
      o.w = fmaf(A[3], g.w, fmaf(B[3], v.w, C[3]));
      reinterpret_cast<float4*>(dx)[i] = o;
    }
  } else {
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float A, B, C;
      coeffs(static_cast<int>(i % cols), A, B, C);
      dx[i] = fmaf(A, dy[i], fmaf(B, x[i], C));
    }
  }
}

int sm_count() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}
int grid1d(long long items, int block) {
  long long nb = (items + block - 1) / block;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (nb > cap) nb = cap;
  if (nb < 1) nb = 1;
  return static_cast<int>(nb);
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" int fb_dropout_fwd(const void* x, void* y, uint8_t* mask, long long n, float p, unsigned long long seed,
                              unsigned long long offset, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (p < 0.f || p >= 1.f) return -1;
  const int g = grid1d((n + 7) / 8, 256);
  if (dtype == FB_DT_F32)
    dropout_fwd_kernel<float><<<g, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<float*>(y), mask, n,
                                                    p, seed, offset, nullptr);
  else if (dtype == FB_DT_BF16)
    dropout_fwd_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), mask, n, p, seed, offset, nullptr);
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}

// Graph-capturable form: the Philox offset is `offset + *dev_counter`, and the counter is advanced by one on the
// stream after the launch, so every replay of a captured step draws a new mask.
extern "C" int fb_dropout_fwd_dyn(const void* x, void* y, uint8_t* mask, long long n, float p,
                                  unsigned long long seed, unsigned long long offset,
                                  unsigned long long* dev_counter, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (p < 0.f || p >= 1.f || dev_counter == nullptr) return -1;
  const int g = grid1d((n + 7) / 8, 256);
  if (dtype == FB_DT_F32)
    dropout_fwd_kernel<float><<<g, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<float*>(y), mask, n,
                                                    p, seed, offset, dev_counter);
  else if (dtype == FB_DT_BF16)
    dropout_fwd_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), mask, n, p, seed, offset, dev_counter);
  else
    return -1;
  counter_add_kernel<<<1, 32, 0, stream>>>(dev_counter, 1ull);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int fb_dropout_bwd(const void* dy, const uint8_t* mask, void* dx, long long n, float p, int dtype,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  const int g = grid1d((n + 7) / 8, 256);
  if (dtype == FB_DT_F32)
    dropout_bwd_kernel<float><<<g, 256, 0, stream>>>(static_cast<const float*>(dy), mask, static_cast<float*>(dx),
                                                    n, p);
  else if (dtype == FB_DT_BF16)
    dropout_bwd_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(dy), mask,
                                                            static_cast<__nv_bfloat16*>(dx), n, p);
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_embedding_fwd(const float* weight, const long long* idx, void* out, long long n_idx, int dim,
                                long long vocab, long long padding_idx, int out_dtype, int32_t* status,
                                cudaStream_t stream) {
  if (n_idx <= 0 || dim <= 0) return 0;
  const int g = grid1d(n_idx * 32, 256);
  if (out_dtype == FB_DT_F32)
    embedding_fwd_kernel<float><<<g, 256, 0, stream>>>(weight, idx, static_cast<float*>(out), n_idx, dim, vocab,
                                                      padding_idx, status);
  else if (out_dtype == FB_DT_BF16)
    embedding_fwd_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(weight, idx, static_cast<__nv_bfloat16*>(out), n_idx,
                                                              dim, vocab, padding_idx, status);
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_embedding_meanpool_fwd(const float* weight, const long long* idx, void* out, long long batch,
                                         int seq, int dim, long long vocab, int out_dtype, cudaStream_t stream) {
  if (batch <= 0 || seq <= 0 || dim <= 0) return 0;
  const int g = static_cast<int>(batch < sm_count() * 8LL ? batch : sm_count() * 8LL);
  const size_t smem = static_cast<size_t>(seq) * sizeof(long long);
  if (smem > 48 * 1024) return -1;
  if (out_dtype == FB_DT_F32)
    embedding_meanpool_kernel<float><<<g, 256, smem, stream>>>(weight, idx, static_cast<float*>(out), batch, seq,
                                                              dim, vocab);
  else if (out_dtype == FB_DT_BF16)
    embedding_meanpool_kernel<__nv_bfloat16><<<g, 256, smem, stream>>>(
        weight, idx, static_cast<__nv_bfloat16*>(out), batch, seq, dim, vocab);
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_embedding_bwd_sorted(const void* dout, const long long* sorted_idx, const long long* perm,
                                       float* dweight, long long n_idx, int dim, int group, float scale,
                                       long long padding_idx, long long vocab, int dtype, cudaStream_t stream) {
  if (n_idx <= 0 || dim <= 0) return 0;
  if (group < 1) return -1;
  const long long nb = (n_idx + 31) / 32;
  if (nb > 2147483647LL) return -1;
  const int threads = dim >= 256 ? 256 : (dim >= 128 ? 128 : 64);
  if (dtype == FB_DT_F32)
    embedding_bwd_sorted_kernel<float><<<static_cast<unsigned>(nb), threads, 0, stream>>>(
        static_cast<const float*>(dout), sorted_idx, perm, dweight, n_idx, dim, group, scale, padding_idx, vocab,
        bounds_status_ref());
  else if (dtype == FB_DT_BF16)
    embedding_bwd_sorted_kernel<__nv_bfloat16><<<static_cast<unsigned>(nb), threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(dout), sorted_idx, perm, dweight, n_idx, dim, group, scale, padding_idx,
        vocab, bounds_status_ref());
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_gather_rows(const void* src, const long long* idx, void* dst, long long n_idx,
                              long long row_bytes, long long n_rows, int32_t* status, cudaStream_t stream) {
  if (n_idx <= 0 || row_bytes <= 0) return 0;
  if (n_rows <= 0) return -1;
  const int g = static_cast<int>(n_idx < sm_count() * 16LL ? n_idx : sm_count() * 16LL);
  const int threads = row_bytes >= 4096 ? 256 : 64;
  gather_rows_kernel<<<g, threads, 0, stream>>>(static_cast<const uint8_t*>(src), idx, static_cast<uint8_t*>(dst),
                                                n_idx, row_bytes, n_rows, status);
  return static_cast<int>(cudaGetLastError());
}

namespace {
// 2-D grid of the column-statistics passes: 128-column blocks x enough row blocks to fill the GPU.
dim3 bn_stats_grid(long long rows, int cols, long long* rows_per_block) {
  const long long col_blocks = (cols + 127) / 128;
  long long rb = (static_cast<long long>(fb::sm_count()) * 4 + col_blocks - 1) / col_blocks;
  const long long max_rb = (rows + 31) / 32;
  if (rb > max_rb) rb = max_rb;
  if (rb < 1) rb = 1;
  if (rb > 65535) rb = 65535;
  *rows_per_block = (rows + rb - 1) / rb;
  return dim3(static_cast<unsigned>(col_blocks), static_cast<unsigned>(rb));
}
// Grid of the elementwise passes (256 threads): the grid stride is a multiple of the vectors per row where
// possible, so a thread keeps its columns and their per-column coefficients stay in registers.
int bn_elementwise_grid(long long rows, int cols) {
  long long blocks = static_cast<long long>(fb::sm_count()) * 6;
  const long long nv = (rows * cols + 3) / 4;
  if (cols % 4 == 0) {
    const long long vpr = cols / 4;            // vectors per row
    long long threads = blocks * 256;
    if (threads > vpr && (threads / vpr * vpr) % 256 == 0) blocks = threads / vpr * vpr / 256;
  }
  const long long need = (nv + 255) / 256;
  if (blocks > need) blocks = need;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}
}  // namespace

// Training: save_mean / save_rstd are required (they double as the accumulators of the statistics passes).
extern "C" int fb_batchnorm_fwd(const float* x, const float* gamma, const float* beta, float* y, float* save_mean,
                                float* save_rstd, float* running_mean, float* running_var, long long rows, int cols,
                                float eps, float momentum, int training, cudaStream_t stream) {
  using namespace fb;
  if (rows <= 0 || cols <= 0) return 0;
  if (!training && (running_mean == nullptr || running_var == nullptr)) return -1;
  const int apply_grid = bn_elementwise_grid(rows, cols);
  if (training) {
    if (save_mean == nullptr || save_rstd == nullptr) return -1;
    cudaError_t e = cudaMemsetAsync(save_mean, 0, cols * sizeof(float), stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(save_rstd, 0, cols * sizeof(float), stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    long long rpb = 0;
    const dim3 grid = bn_stats_grid(rows, cols, &rpb);
    const int fgrid = (cols + 255) / 256;
    bn_colstats_kernel<3><<<grid, 256, 0, stream>>>(x, nullptr, nullptr, nullptr, save_mean, save_rstd, rows, cols, rpb);
    bn_finalize_kernel<<<fgrid, 256, 0, stream>>>(save_mean, save_rstd, running_mean, running_var, rows, cols, eps,
                                                  momentum, x);
    bn_apply_kernel<<<apply_grid, 256, 0, stream>>>(x, gamma, beta, save_mean, save_rstd, y, rows, cols, eps, 0);
  } else {
    bn_apply_kernel<<<apply_grid, 256, 0, stream>>>(x, gamma, beta, running_mean, running_var, y, rows, cols, eps, 1);
  }
  return static_cast<int>(cudaGetLastError());
}
// dgamma / dbeta are required (they are the accumulators of the statistics pass).
extern "C" int fb_batchnorm_bwd(const float* dy, const float* x, const float* gamma, const float* save_mean,
                                const float* save_rstd, float* dx, float* dgamma, float* dbeta, long long rows,
                                int cols, cudaStream_t stream) {
  using namespace fb;
  if (rows <= 0 || cols <= 0) return 0;
  if (dgamma == nullptr || dbeta == nullptr) return -1;
  cudaError_t e = cudaMemsetAsync(dgamma, 0, cols * sizeof(float), stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(dbeta, 0, cols * sizeof(float), stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  long long rpb = 0;
  const dim3 grid = bn_stats_grid(rows, cols, &rpb);
  bn_colstats_kernel<2><<<grid, 256, 0, stream>>>(x, dy, save_mean, save_rstd, dbeta, dgamma, rows, cols, rpb);
  bn_dx_kernel<<<bn_elementwise_grid(rows, cols), 256, 0, stream>>>(dy, x, gamma, save_mean, save_rstd, dgamma, dbeta,
                                                                    dx, rows, cols);
  return static_cast<int>(cudaGetLastError());
}
