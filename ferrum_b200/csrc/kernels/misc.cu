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
//                                      per feature with running-stat update)
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
template <typename T>
__global__ void dropout_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ mask,
                                   long long n, float p, unsigned long long seed, unsigned long long offset) {
  const float scale = 1.f / (1.f - p);
  const uint32_t thresh = static_cast<uint32_t>(fminf(p, 1.f) * 4294967295.0f);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long n4 = (n + 3) >> 2;
  for (long long q = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; q < n4; q += stride) {
    uint32_t r[4];
    philox4x32_10(seed, static_cast<unsigned long long>(q), offset, r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = q * 4 + j;
      if (i < n) {
        const bool keep = r[j] >= thresh;
        mask[i] = keep ? 1 : 0;
        stf(y + i, keep ? ldf(x + i) * scale : 0.f);
      }
    }
  }
}
template <typename T>
__global__ void dropout_bwd_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ mask, T* __restrict__ dx,
                                   long long n, float p) {
  const float scale = 1.f / (1.f - p);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    stf(dx + i, mask[i] ? ldf(dy + i) * scale : 0.f);
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

// Scatter-add over a SORTED index list: a block walks a chunk of 32 consecutive
// positions, sums runs of equal indices in registers and flushes each run with
// one atomicAdd per element, so heavily repeated tokens cost one flush per
// chunk instead of one per occurrence.  perm[i] is the original position.
template <typename G>
__global__ void embedding_bwd_sorted_kernel(const G* __restrict__ dout, const long long* __restrict__ sorted_idx,
                                            const long long* __restrict__ perm, float* __restrict__ dw,
                                            long long n_idx, int dim, int group, float scale,
                                            long long padding_idx) {
  constexpr int kChunk = 32;
  const long long lo = static_cast<long long>(blockIdx.x) * kChunk;
  const long long hi = min(n_idx, lo + kChunk);
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float acc = 0.f;
    long long cur = -1;
    for (long long i = lo; i < hi; ++i) {
      const long long id = sorted_idx[i];
      if (id != cur) {
        if (cur >= 0 && cur != padding_idx) atomicAdd(dw + cur * dim + c, acc * scale);
        cur = id;
        acc = 0.f;
      }
      acc += ldf(dout + (perm[i] / group) * dim + c);
    }
    if (cur >= 0 && cur != padding_idx) atomicAdd(dw + cur * dim + c, acc * scale);
  }
}

__global__ void gather_rows_kernel(const uint8_t* __restrict__ src, const long long* __restrict__ idx,
                                   uint8_t* __restrict__ dst, long long n_idx, long long row_bytes) {
  const bool vec = (row_bytes % 16 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
  for (long long i = blockIdx.x; i < n_idx; i += gridDim.x) {
    const uint8_t* s = src + idx[i] * row_bytes;
    uint8_t* d = dst + i * row_bytes;
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
// Block = 32 columns x 8 row groups.  Column statistics by two passes.
__device__ __forceinline__ float col_sum_8(float v, float (*sm)[33]) {
  __syncthreads();
  sm[threadIdx.y][threadIdx.x] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) s += sm[j][threadIdx.x];
  return s;
}

__global__ void batchnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, float* __restrict__ y,
                                     float* __restrict__ save_mean, float* __restrict__ save_rstd,
                                     float* __restrict__ running_mean, float* __restrict__ running_var,
                                     long long rows, int cols, float eps, float momentum, int training) {
  __shared__ float sm[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const bool live = c < cols;
  float mu, rs;
  if (training) {
    float s = 0.f;
    if (live)
      for (long long r = threadIdx.y; r < rows; r += 8) s += x[r * cols + c];
    mu = col_sum_8(s, sm) / static_cast<float>(rows);
    float q = 0.f;
    if (live)
      for (long long r = threadIdx.y; r < rows; r += 8) {
        const float d = x[r * cols + c] - mu;
        q += d * d;
      }
    const float var = col_sum_8(q, sm) / static_cast<float>(rows);
    rs = rsqrtf(var + eps);
    if (live && threadIdx.y == 0) {
      if (save_mean) save_mean[c] = mu;
      if (save_rstd) save_rstd[c] = rs;
      if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mu;
      if (running_var) {
        const float unbiased = rows > 1 ? var * static_cast<float>(rows) / static_cast<float>(rows - 1) : var;
        running_var[c] = (1.f - momentum) * running_var[c] + momentum * unbiased;
      }
    }
  } else {
    mu = live ? running_mean[c] : 0.f;
    rs = live ? rsqrtf(running_var[c] + eps) : 0.f;
  }
  if (live) {
    const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
    for (long long r = threadIdx.y; r < rows; r += 8) y[r * cols + c] = (x[r * cols + c] - mu) * rs * g + b;
  }
}

__global__ void batchnorm_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                     const float* __restrict__ gamma, const float* __restrict__ save_mean,
                                     const float* __restrict__ save_rstd, float* __restrict__ dx,
                                     float* __restrict__ dgamma, float* __restrict__ dbeta, long long rows,
                                     int cols) {
  __shared__ float sm[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const bool live = c < cols;
  const float mu = live ? save_mean[c] : 0.f, rs = live ? save_rstd[c] : 0.f;
  float sg = 0.f, sb = 0.f;
  if (live)
    for (long long r = threadIdx.y; r < rows; r += 8) {
      const float g = dy[r * cols + c];
      sg += g * (x[r * cols + c] - mu) * rs;
      sb += g;
    }
  const float dg = col_sum_8(sg, sm);
  const float db = col_sum_8(sb, sm);
  if (live) {
    if (threadIdx.y == 0) {
      if (dgamma) dgamma[c] = dg;
      if (dbeta) dbeta[c] = db;
    }
    const float w = (gamma ? gamma[c] : 1.f) * rs / static_cast<float>(rows);
    for (long long r = threadIdx.y; r < rows; r += 8) {
      const float h = (x[r * cols + c] - mu) * rs;
      dx[r * cols + c] = w * (static_cast<float>(rows) * dy[r * cols + c] - db - h * dg);
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
  const int g = grid1d((n + 3) / 4, 256);
  if (dtype == FB_DT_F32)
    dropout_fwd_kernel<float><<<g, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<float*>(y), mask, n,
                                                    p, seed, offset);
  else if (dtype == FB_DT_BF16)
    dropout_fwd_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                            static_cast<__nv_bfloat16*>(y), mask, n, p, seed, offset);
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}
extern "C" int fb_dropout_bwd(const void* dy, const uint8_t* mask, void* dx, long long n, float p, int dtype,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  const int g = grid1d(n, 256);
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
                                       long long padding_idx, int dtype, cudaStream_t stream) {
  if (n_idx <= 0 || dim <= 0) return 0;
  if (group < 1) return -1;
  const long long nb = (n_idx + 31) / 32;
  if (nb > 2147483647LL) return -1;
  const int threads = dim >= 256 ? 256 : (dim >= 128 ? 128 : 64);
  if (dtype == FB_DT_F32)
    embedding_bwd_sorted_kernel<float><<<static_cast<unsigned>(nb), threads, 0, stream>>>(
        static_cast<const float*>(dout), sorted_idx, perm, dweight, n_idx, dim, group, scale, padding_idx);
  else if (dtype == FB_DT_BF16)
    embedding_bwd_sorted_kernel<__nv_bfloat16><<<static_cast<unsigned>(nb), threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(dout), sorted_idx, perm, dweight, n_idx, dim, group, scale, padding_idx);
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_gather_rows(const void* src, const long long* idx, void* dst, long long n_idx,
                              long long row_bytes, cudaStream_t stream) {
  if (n_idx <= 0 || row_bytes <= 0) return 0;
  const int g = static_cast<int>(n_idx < sm_count() * 16LL ? n_idx : sm_count() * 16LL);
  const int threads = row_bytes >= 4096 ? 256 : 64;
  gather_rows_kernel<<<g, threads, 0, stream>>>(static_cast<const uint8_t*>(src), idx, static_cast<uint8_t*>(dst),
                                                n_idx, row_bytes);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_batchnorm_fwd(const float* x, const float* gamma, const float* beta, float* y, float* save_mean,
                                float* save_rstd, float* running_mean, float* running_var, long long rows, int cols,
                                float eps, float momentum, int training, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (!training && (running_mean == nullptr || running_var == nullptr)) return -1;
  dim3 block(32, 8), grid((cols + 31) / 32);
  batchnorm_fwd_kernel<<<grid, block, 0, stream>>>(x, gamma, beta, y, save_mean, save_rstd, running_mean,
                                                   running_var, rows, cols, eps, momentum, training);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int fb_batchnorm_bwd(const float* dy, const float* x, const float* gamma, const float* save_mean,
                                const float* save_rstd, float* dx, float* dgamma, float* dbeta, long long rows,
                                int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  dim3 block(32, 8), grid((cols + 31) / 32);
  batchnorm_bwd_kernel<<<grid, block, 0, stream>>>(dy, x, gamma, save_mean, save_rstd, dx, dgamma, dbeta, rows,
                                                   cols);
  return static_cast<int>(cudaGetLastError());
}
