// Row softmax / log-softmax (forward, backward), the fused log-softmax + NLL /
// cross-entropy kernel that also emits the logit gradient, and the fused
// elementwise losses (mse, bce, l1, smooth-l1) with their backward.
//
// Reference:
//   ferrum-cuda/src/kernels.rs:501-621  softmax / log_softmax: per row over the last
//                                       dimension, max-subtracted (the nn versions at
//                                       ferrum-nn/src/activation.rs:235-251 are global
//                                       and unstabilised; the per-row form is built)
//   ferrum-nn/src/loss.rs:24-151        mse / bce (eps 1e-7) / l1 / smooth_l1 /
//                                       cross_entropy / nll
// Rows of any width: each row is owned by one warp (cols <= 1024) or one block;
// the row is read from DRAM once and re-read from L1 for the later passes.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>

#include "../common/status.h"
#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

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

template <int TPR, bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, u) : v + u;
  }
  if (TPR == 32) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = IS_MAX ? -FLT_MAX : 0.f;
#pragma unroll
  for (int w = 0; w < TPR / 32; ++w) t = IS_MAX ? fmaxf(t, smem[w]) : t + smem[w];
  return t;
}


// Rows of 8-element-multiple width up to 4096 (16-byte aligned): a warp owns a row and keeps it in registers
// (K vectors of 8 per lane), so the row is read once, exp is evaluated once per element and the reductions are
// warp shuffles.  Used for both dtypes; the scalar kernels below remain for ragged widths and very wide rows.
template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 t = __bfloat1622float2(h[e]);
      f[2 * e] = t.x;
      f[2 * e + 1] = t.y;
    }
  } else {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 out;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
    *reinterpret_cast<uint4*>(p) = out;
  } else {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
}

template <typename T, int K>
__global__ void __launch_bounds__(256)
softmax_fwd_warp_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int cols, int log_mode) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  const long long warp_id = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = warp_id; row < rows; row += nwarps) {
    const T* xr = x + row * cols;
    float v[K][8];
    float m = -FLT_MAX;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        ld8(xr + vi * 8, v[k]);
#pragma unroll
        for (int e = 0; e < 8; ++e) m = fmaxf(m, v[k][e]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[k][e] = -FLT_MAX;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
    float ex[K][8];
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        ex[k][e] = expf(v[k][e] - m);
        s += ex[k][e];
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float inv = 1.f / s, lse = m + logf(s);
    T* yr = y + row * cols;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = log_mode ? v[k][e] - lse : ex[k][e] * inv;
        st8(yr + vi * 8, o);
      }
    }
  }
}

template <typename T, int K>
__global__ void __launch_bounds__(256)
softmax_bwd_warp_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, long long rows,
                        int cols, int log_mode) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  const long long warp_id = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = warp_id; row < rows; row += nwarps) {
    const long long base = row * cols;
    float g[K][8], v[K][8];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        ld8(dy + base + vi * 8, g[k]);
        ld8(y + base + vi * 8, v[k]);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += log_mode ? g[k][e] : g[k][e] * v[k][e];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = log_mode ? g[k][e] - expf(v[k][e]) * s : v[k][e] * (g[k][e] - s);
        st8(dx + base + vi * 8, o);
      }
    }
  }
}

// One group of TPR threads per row; 256 threads per block.
template <typename T, int TPR>
__global__ void __launch_bounds__(256)
softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int cols, int log_mode) {
  __shared__ float smem[8];
  constexpr int kRPB = 256 / TPR;
  const int sub = threadIdx.x / TPR, t = threadIdx.x % TPR;
  for (long long row0 = static_cast<long long>(blockIdx.x) * kRPB; row0 < rows;
       row0 += static_cast<long long>(gridDim.x) * kRPB) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const T* xr = x + (live ? row : 0) * cols;
    float m = -FLT_MAX;
    if (live)
      for (int c = t; c < cols; c += TPR) m = fmaxf(m, ldf(xr + c));
    m = group_reduce<TPR, true>(m, smem);
    float s = 0.f;
    if (live)
      for (int c = t; c < cols; c += TPR) s += expf(ldf(xr + c) - m);
    s = group_reduce<TPR, false>(s, smem);
    if (live) {
      T* yr = y + row * cols;
      if (log_mode) {
        const float lse = m + logf(s);
        for (int c = t; c < cols; c += TPR) stf(yr + c, ldf(xr + c) - lse);
      } else {
        const float inv = 1.f / s;
        for (int c = t; c < cols; c += TPR) stf(yr + c, expf(ldf(xr + c) - m) * inv);
      }
    }
  }
}

// softmax:     dx = y * (dy - sum(dy * y))
// log_softmax: dx = dy - exp(y) * sum(dy)
template <typename T, int TPR>
__global__ void __launch_bounds__(256)
softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, long long rows, int cols,
                   int log_mode) {
  __shared__ float smem[8];
  constexpr int kRPB = 256 / TPR;
  const int sub = threadIdx.x / TPR, t = threadIdx.x % TPR;
  for (long long row0 = static_cast<long long>(blockIdx.x) * kRPB; row0 < rows;
       row0 += static_cast<long long>(gridDim.x) * kRPB) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const long long base = (live ? row : 0) * cols;
    float s = 0.f;
    if (live)
      for (int c = t; c < cols; c += TPR) {
        const float g = ldf(dy + base + c);
        s += log_mode ? g : g * ldf(y + base + c);
      }
    s = group_reduce<TPR, false>(s, smem);
    if (live)
      for (int c = t; c < cols; c += TPR) {
        const float g = ldf(dy + base + c), v = ldf(y + base + c);
        stf(dx + base + c, log_mode ? g - expf(v) * s : v * (g - s));
      }
  }
}

template <typename T, typename G, int TPR>
__global__ void __launch_bounds__(256)
ce_kernel(const T* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ row_loss,
          G* __restrict__ dlogits, long long rows, int cols, float grad_scale, int32_t* bstatus) {
  __shared__ float smem[8];
  constexpr int kRPB = 256 / TPR;
  const int sub = threadIdx.x / TPR, t = threadIdx.x % TPR;
  for (long long row0 = static_cast<long long>(blockIdx.x) * kRPB; row0 < rows;
       row0 += static_cast<long long>(gridDim.x) * kRPB) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const T* xr = logits + (live ? row : 0) * cols;
    float m = -FLT_MAX;
    if (live)
      for (int c = t; c < cols; c += TPR) m = fmaxf(m, ldf(xr + c));
    m = group_reduce<TPR, true>(m, smem);
    float s = 0.f;
    if (live)
      for (int c = t; c < cols; c += TPR) s += expf(ldf(xr + c) - m);
    s = group_reduce<TPR, false>(s, smem);
    if (live) {
      long long lab = labels[row];
      const bool valid = lab >= 0 && lab < cols;  // out-of-range labels contribute nothing
      if (!valid && t == 0) (void)FB_INDEX_OK(bstatus, 41, lab, cols);  // the debug build also reports them
      if (t == 0 && row_loss) row_loss[row] = valid ? (m + logf(s) - ldf(xr + lab)) : 0.f;
      if (dlogits) {
        const float inv = 1.f / s;
        G* gr = dlogits + row * cols;
        for (int c = t; c < cols; c += TPR) {
          float p = expf(ldf(xr + c) - m) * inv;
          if (c == lab) p -= 1.f;
          stf(gr + c, valid ? p * grad_scale : 0.f);
        }
      }
    }
  }
}


// bf16 rows of 264..4096 columns (multiples of 8, 16-byte aligned): a warp owns a row, every lane keeps its
// elements in registers (K vectors of 8), so the row is read once, exp is evaluated once per element and the
// three reductions are warp shuffles without a block barrier.
template <int K>
__global__ void __launch_bounds__(256, K <= 4 ? 4 : (K <= 8 ? 2 : 1))
ce_warp_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
               float* __restrict__ row_loss, __nv_bfloat16* __restrict__ dlogits, long long rows, int cols,
               float grad_scale, int32_t* bstatus) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  const long long warp_id = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = warp_id; row < rows; row += nwarps) {
    const __nv_bfloat16* xr = logits + row * cols;
    float v[K][8];
    float m = -FLT_MAX;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr + vi * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          v[k][2 * e] = f.x;
          v[k][2 * e + 1] = f.y;
          m = fmaxf(m, fmaxf(f.x, f.y));
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[k][e] = -FLT_MAX;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[k][e] = __expf(v[k][e] - m);  // padded lanes: exp(-huge) = 0
        s += v[k][e];
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const long long lab = labels[row];
    const bool valid = lab >= 0 && lab < cols;
    if (!valid && lane == 0) (void)FB_INDEX_OK(bstatus, 41, lab, cols);
    if (lane == 0 && row_loss) row_loss[row] = valid ? (m + logf(s) - __bfloat162float(xr[lab])) : 0.f;
    if (dlogits) {
      const float inv = valid ? grad_scale / s : 0.f;
      __nv_bfloat16* gr = dlogits + row * cols;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int vi = lane + 32 * k;
        if (vi < nvec) {
          uint4 out;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float a = v[k][2 * e] * inv, b = v[k][2 * e + 1] * inv;
            if (valid && vi * 8 + 2 * e == lab) a -= grad_scale;
            if (valid && vi * 8 + 2 * e + 1 == lab) b -= grad_scale;
            h[e] = __floats2bfloat162_rn(a, b);
          }
          *reinterpret_cast<uint4*>(gr + vi * 8) = out;
        }
      }
    }
  }
}

// ------------------------------------------------------- elementwise losses
__device__ __forceinline__ float loss_elem(float p, float t, int kind) {
  const float d = p - t;
  switch (kind) {
    case FB_LOSS_MSE: return d * d;
    case FB_LOSS_BCE: {
      const float eps = 1e-7f;
      const float pc = p + eps;
      const float q = (1.f + eps) - pc;
      return -(t * logf(pc) + (1.f - t) * logf(q));
    }
    case FB_LOSS_L1: return fabsf(d);
    default: {
      const float a = fabsf(d);
      return a < 1.f ? 0.5f * d * d : a - 0.5f;
    }
  }
}
__device__ __forceinline__ float loss_grad(float p, float t, int kind) {
  const float d = p - t;
  switch (kind) {
    case FB_LOSS_MSE: return 2.f * d;
    case FB_LOSS_BCE: {
      const float eps = 1e-7f;
      const float pc = p + eps;
      const float q = (1.f + eps) - pc;
      return -(t / pc - (1.f - t) / q);
    }
    case FB_LOSS_L1: return d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
    default: {
      const float a = fabsf(d);
      return a < 1.f ? d : (d > 0.f ? 1.f : -1.f);
    }
  }
}

__global__ void loss_fwd_kernel(const float* __restrict__ p, const float* __restrict__ t, float* __restrict__ out,
                                long long n, int kind, float scale) {
  __shared__ float smem[8];
  float acc = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    acc += loss_elem(p[i], t[i], kind);
  acc = group_reduce<256, false>(acc, smem);
  if (threadIdx.x == 0) atomicAdd(out, acc * scale);
}

__global__ void loss_bwd_kernel(const float* __restrict__ p, const float* __restrict__ t,
                                const float* __restrict__ gout, float* __restrict__ dp, long long n, int kind,
                                float scale) {
  const float g = (gout ? gout[0] : 1.f) * scale;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    dp[i] = g * loss_grad(p[i], t[i], kind);
}

int sm_count() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}
int row_grid(long long rows, int rpb) {
  const long long nb = (rows + rpb - 1) / rpb;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  return static_cast<int>(nb < cap ? nb : cap);
}

bool warp_rows_ok(const void* a, const void* b, const void* c, int cols) {
  return cols % 8 == 0 && cols >= 64 && cols <= 2048 &&
         ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0;
}

template <typename T>
int softmax_fwd_t(const void* x, void* y, long long rows, int cols, int log_mode, cudaStream_t st) {
  if (warp_rows_ok(x, y, nullptr, cols)) {
    const int k = (cols / 8 + 31) / 32, grid = row_grid(rows, 8);
    const T* xp = static_cast<const T*>(x);
    T* yp = static_cast<T*>(y);
    if (k <= 2) softmax_fwd_warp_kernel<T, 2><<<grid, 256, 0, st>>>(xp, yp, rows, cols, log_mode);
    else if (k <= 4) softmax_fwd_warp_kernel<T, 4><<<grid, 256, 0, st>>>(xp, yp, rows, cols, log_mode);
    else softmax_fwd_warp_kernel<T, 8><<<grid, 256, 0, st>>>(xp, yp, rows, cols, log_mode);
    return static_cast<int>(cudaGetLastError());
  }
  if (cols <= 1024)
    softmax_fwd_kernel<T, 32><<<row_grid(rows, 8), 256, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), rows,
                                                                cols, log_mode);
  else
    softmax_fwd_kernel<T, 256><<<row_grid(rows, 1), 256, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y),
                                                                 rows, cols, log_mode);
  return static_cast<int>(cudaGetLastError());
}
template <typename T>
int softmax_bwd_t(const void* dy, const void* y, void* dx, long long rows, int cols, int log_mode,
                  cudaStream_t st) {
  if (warp_rows_ok(dy, y, dx, cols)) {
    const int kk = (cols / 8 + 31) / 32, grid = row_grid(rows, 8);
    const T* gp = static_cast<const T*>(dy);
    const T* yp = static_cast<const T*>(y);
    T* dp = static_cast<T*>(dx);
    if (kk <= 2) softmax_bwd_warp_kernel<T, 2><<<grid, 256, 0, st>>>(gp, yp, dp, rows, cols, log_mode);
    else if (kk <= 4) softmax_bwd_warp_kernel<T, 4><<<grid, 256, 0, st>>>(gp, yp, dp, rows, cols, log_mode);
    else softmax_bwd_warp_kernel<T, 8><<<grid, 256, 0, st>>>(gp, yp, dp, rows, cols, log_mode);
    return static_cast<int>(cudaGetLastError());
  }
  if (cols <= 1024)
    softmax_bwd_kernel<T, 32><<<row_grid(rows, 8), 256, 0, st>>>(static_cast<const T*>(dy), static_cast<const T*>(y),
                                                                static_cast<T*>(dx), rows, cols, log_mode);
  else
    softmax_bwd_kernel<T, 256><<<row_grid(rows, 1), 256, 0, st>>>(
        static_cast<const T*>(dy), static_cast<const T*>(y), static_cast<T*>(dx), rows, cols, log_mode);
  return static_cast<int>(cudaGetLastError());
}
// bf16 logits with bf16 gradient, vectorisable rows: the warp-per-row kernel.
bool ce_warp_launch(const void* logits, const long long* labels, float* row_loss, void* dlogits, long long rows,
                    int cols, float gs, cudaStream_t st) {
  if (cols % 8 != 0 || cols < 264 || cols > 4096) return false;
  if (((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits)) & 15) != 0) return false;
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(logits);
  __nv_bfloat16* g = static_cast<__nv_bfloat16*>(dlogits);
  const int grid = row_grid(rows, 8);
  const int k = (cols / 8 + 31) / 32;
  if (k <= 4)
    ce_warp_kernel<4><<<grid, 256, 0, st>>>(x, labels, row_loss, g, rows, cols, gs, bounds_status_ref());
  else if (k <= 8)
    ce_warp_kernel<8><<<grid, 256, 0, st>>>(x, labels, row_loss, g, rows, cols, gs, bounds_status_ref());
  else
    ce_warp_kernel<16><<<grid, 256, 0, st>>>(x, labels, row_loss, g, rows, cols, gs, bounds_status_ref());
  return true;
}

template <typename T, typename G>
int ce_t(const void* logits, const long long* labels, float* row_loss, void* dlogits, long long rows, int cols,
         float gs, cudaStream_t st) {
  if (sizeof(T) == 2 && sizeof(G) == 2 && ce_warp_launch(logits, labels, row_loss, dlogits, rows, cols, gs, st))
    return static_cast<int>(cudaGetLastError());
  if (cols <= 512)
    ce_kernel<T, G, 32><<<row_grid(rows, 8), 256, 0, st>>>(static_cast<const T*>(logits), labels, row_loss,
                                                          static_cast<G*>(dlogits), rows, cols, gs,
                                                          bounds_status_ref());
  else
    ce_kernel<T, G, 256><<<row_grid(rows, 1), 256, 0, st>>>(static_cast<const T*>(logits), labels, row_loss,
                                                           static_cast<G*>(dlogits), rows, cols, gs,
                                                          bounds_status_ref());
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" int fb_softmax_fwd(const void* x, void* y, long long rows, int cols, int log_mode, int dtype,
                              cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (dtype == FB_DT_F32) return softmax_fwd_t<float>(x, y, rows, cols, log_mode, stream);
  if (dtype == FB_DT_BF16) return softmax_fwd_t<__nv_bfloat16>(x, y, rows, cols, log_mode, stream);
  return -1;
}
extern "C" int fb_softmax_bwd(const void* dy, const void* y, void* dx, long long rows, int cols, int log_mode,
                              int dtype, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (dtype == FB_DT_F32) return softmax_bwd_t<float>(dy, y, dx, rows, cols, log_mode, stream);
  if (dtype == FB_DT_BF16) return softmax_bwd_t<__nv_bfloat16>(dy, y, dx, rows, cols, log_mode, stream);
  return -1;
}
extern "C" int fb_ce_fwd_bwd(const void* logits, const long long* labels, float* row_loss, void* dlogits,
                             long long rows, int cols, float grad_scale, int dtype, int dlogits_dtype,
                             cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (dtype == FB_DT_F32 && dlogits_dtype == FB_DT_F32)
    return ce_t<float, float>(logits, labels, row_loss, dlogits, rows, cols, grad_scale, stream);
  if (dtype == FB_DT_F32 && dlogits_dtype == FB_DT_BF16)
    return ce_t<float, __nv_bfloat16>(logits, labels, row_loss, dlogits, rows, cols, grad_scale, stream);
  if (dtype == FB_DT_BF16 && dlogits_dtype == FB_DT_BF16)
    return ce_t<__nv_bfloat16, __nv_bfloat16>(logits, labels, row_loss, dlogits, rows, cols, grad_scale, stream);
  if (dtype == FB_DT_BF16 && dlogits_dtype == FB_DT_F32)
    return ce_t<__nv_bfloat16, float>(logits, labels, row_loss, dlogits, rows, cols, grad_scale, stream);
  return -1;
}
extern "C" int fb_loss_fwd(const float* pred, const float* target, float* out, long long n, int kind, float scale,
                           cudaStream_t stream) {
  if (n <= 0) return 0;
  long long nb = (n + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 4;
  if (nb > cap) nb = cap;
  loss_fwd_kernel<<<static_cast<int>(nb), 256, 0, stream>>>(pred, target, out, n, kind, scale);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int fb_loss_bwd(const float* pred, const float* target, const float* gout, float* dpred, long long n,
                           int kind, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long nb = (n + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (nb > cap) nb = cap;
  loss_bwd_kernel<<<static_cast<int>(nb), 256, 0, stream>>>(pred, target, gout, dpred, n, kind, scale);
  return static_cast<int>(cudaGetLastError());
}
