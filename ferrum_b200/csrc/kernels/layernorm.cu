// Per-row LayerNorm forward / backward, optionally fused with a preceding GELU
// (the Linear -> GELU -> LayerNorm block reads the pre-activation once and
// writes the normalised output once; the backward produces the gradient of the
// pre-activation plus the three column reductions d_gamma, d_beta and the
// column sum of dx, which is the bias gradient of the preceding Linear).
//
// Reference: ferrum-nn/src/norm.rs:13-68,226-239 (module + functional; the
// reference normalises with the statistics of the whole tensor — this kernel
// normalises each row of `normalized_shape`, like the row-wise variant at
// ferrum-nn/src/transformer.rs:316-342) and ferrum-nn/src/activation.rs:254-262 (GELU).
//
// Fast path: a row lives in registers (TPR threads x 4-element vectors x KMAX),
// two-pass mean / variance on registers, column partials accumulate in
// registers across the rows a block owns and are written once to
// partial[nblk][3][cols]; a second kernel folds the partials.
// Generic path (odd widths, very wide rows): scalar accesses, re-reads the row,
// column sums by atomicAdd.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

constexpr float kGeluC = 0.7978845608028654f;
constexpr float kGeluA = 0.044715f;
constexpr int kKMax = 8;

__device__ __forceinline__ float gelu_f(float x) {
  return 0.5f * x * (1.f + tanhf(kGeluC * (x + kGeluA * x * x * x)));
}
__device__ __forceinline__ float gelu_grad(float x) {
  const float t = tanhf(kGeluC * (x + kGeluA * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * kGeluC * (1.f + 3.f * kGeluA * x * x);
}

template <typename T>
struct V4;
template <>
struct V4<float> {
  static __device__ __forceinline__ float4 ld(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void st(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
  static __device__ __forceinline__ float ld1(const float* p) { return *p; }
  static __device__ __forceinline__ void st1(float* p, float v) { *p = v; }
};
template <>
struct V4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 ld(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float4 v) {
    uint2 u;
    *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = u;
  }
  static __device__ __forceinline__ float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// Sum across the TPR threads that share a row (TPR = 32: one warp; 256: the block).
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (TPR == 32) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // protect smem reuse across calls
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < TPR / 32; ++w) t += smem[w];
  return t;
}

template <typename T, int TPR>
__global__ void __launch_bounds__(256)
ln_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
              T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, long long rows,
              int cols, float eps, int pre_act) {
  __shared__ float smem[8];
  constexpr int kRowsPerBlock = 256 / TPR;
  const int sub = threadIdx.x / TPR;  // row slot inside the block
  const int t = threadIdx.x % TPR;
  const int nvec = cols >> 2;
  const float inv_n = 1.f / static_cast<float>(cols);
  for (long long row0 = static_cast<long long>(blockIdx.x) * kRowsPerBlock; row0 < rows;
       row0 += static_cast<long long>(gridDim.x) * kRowsPerBlock) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    float4 v[kKMax];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kKMax; ++k) {
      const int vi = t + k * TPR;
      if (live && vi < nvec) {
        float4 a = V4<T>::ld(x + row * cols + vi * 4);
        if (pre_act == FB_ACT_GELU) {
          a.x = gelu_f(a.x); a.y = gelu_f(a.y); a.z = gelu_f(a.z); a.w = gelu_f(a.w);
        }
        v[k] = a;
        s += a.x + a.y + a.z + a.w;
      } else {
        v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    const float mu = row_sum<TPR>(s, smem) * inv_n;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < kKMax; ++k) {
      const int vi = t + k * TPR;
      if (live && vi < nvec) {
        const float dx0 = v[k].x - mu, dx1 = v[k].y - mu, dx2 = v[k].z - mu, dx3 = v[k].w - mu;
        q += dx0 * dx0 + dx1 * dx1 + dx2 * dx2 + dx3 * dx3;
      }
    }
    const float var = row_sum<TPR>(q, smem) * inv_n;
    const float rs = rsqrtf(var + eps);
    if (live && t == 0) {
      if (mean_out) mean_out[row] = mu;
      if (rstd_out) rstd_out[row] = rs;
    }
#pragma unroll
    for (int k = 0; k < kKMax; ++k) {
      const int vi = t + k * TPR;
      if (live && vi < nvec) {
        const float4 g = gamma ? *reinterpret_cast<const float4*>(gamma + vi * 4) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 b = beta ? *reinterpret_cast<const float4*>(beta + vi * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 o;
        o.x = (v[k].x - mu) * rs * g.x + b.x;
        o.y = (v[k].y - mu) * rs * g.y + b.y;
        o.z = (v[k].z - mu) * rs * g.z + b.z;
        o.w = (v[k].w - mu) * rs * g.w + b.w;
        V4<T>::st(y + row * cols + vi * 4, o);
      }
    }
  }
}

template <typename T, int TPR>
__global__ void __launch_bounds__(256)
ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
              const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
              float* __restrict__ partial, long long rows, int cols, int pre_act, int want_colsum) {
  __shared__ float smem[8];
  __shared__ float fold[3][kKMax * 4 * 32];  // used only when several rows share a block (TPR == 32)
  constexpr int kRowsPerBlock = 256 / TPR;
  const int sub = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const int nvec = cols >> 2;
  const float inv_n = 1.f / static_cast<float>(cols);
  float4 acc_g[kKMax], acc_b[kKMax], acc_c[kKMax];
#pragma unroll
  for (int k = 0; k < kKMax; ++k) {
    acc_g[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    acc_b[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    acc_c[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (long long row0 = static_cast<long long>(blockIdx.x) * kRowsPerBlock; row0 < rows;
       row0 += static_cast<long long>(gridDim.x) * kRowsPerBlock) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const float mu = live ? mean[row] : 0.f;
    const float rs = live ? rstd[row] : 0.f;
    float4 xh[kKMax], dh[kKMax];  // x-hat and dy*gamma
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < kKMax; ++k) {
      const int vi = t + k * TPR;
      if (live && vi < nvec) {
        float4 a = V4<T>::ld(x + row * cols + vi * 4);
        if (pre_act == FB_ACT_GELU) {
          a.x = gelu_f(a.x); a.y = gelu_f(a.y); a.z = gelu_f(a.z); a.w = gelu_f(a.w);
        }
        const float4 g = V4<T>::ld(dy + row * cols + vi * 4);
        const float4 w = gamma ? *reinterpret_cast<const float4*>(gamma + vi * 4) : make_float4(1.f, 1.f, 1.f, 1.f);
        float4 h;
        h.x = (a.x - mu) * rs; h.y = (a.y - mu) * rs; h.z = (a.z - mu) * rs; h.w = (a.w - mu) * rs;
        acc_g[k].x += g.x * h.x; acc_g[k].y += g.y * h.y; acc_g[k].z += g.z * h.z; acc_g[k].w += g.w * h.w;
        acc_b[k].x += g.x; acc_b[k].y += g.y; acc_b[k].z += g.z; acc_b[k].w += g.w;
        float4 d;
        d.x = g.x * w.x; d.y = g.y * w.y; d.z = g.z * w.z; d.w = g.w * w.w;
        xh[k] = h;
        dh[k] = d;
        s1 += d.x + d.y + d.z + d.w;
        s2 += d.x * h.x + d.y * h.y + d.z * h.z + d.w * h.w;
      } else {
        xh[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        dh[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    const float m1 = row_sum<TPR>(s1, smem) * inv_n;
    const float m2 = row_sum<TPR>(s2, smem) * inv_n;
#pragma unroll
    for (int k = 0; k < kKMax; ++k) {
      const int vi = t + k * TPR;
      if (live && vi < nvec) {
        float4 o;
        o.x = rs * (dh[k].x - m1 - xh[k].x * m2);
        o.y = rs * (dh[k].y - m1 - xh[k].y * m2);
        o.z = rs * (dh[k].z - m1 - xh[k].z * m2);
        o.w = rs * (dh[k].w - m1 - xh[k].w * m2);
        if (pre_act == FB_ACT_GELU) {
          const float4 raw = V4<T>::ld(x + row * cols + vi * 4);
          o.x *= gelu_grad(raw.x); o.y *= gelu_grad(raw.y); o.z *= gelu_grad(raw.z); o.w *= gelu_grad(raw.w);
        }
        if (want_colsum) {
          acc_c[k].x += o.x; acc_c[k].y += o.y; acc_c[k].z += o.z; acc_c[k].w += o.w;
        }
        V4<T>::st(dx + row * cols + vi * 4, o);
      }
    }
  }
  // ---- write this block's column partials: partial[blockIdx][3][cols]
  float* pg = partial + static_cast<long long>(blockIdx.x) * 3 * cols;
  float* pb = pg + cols;
  float* pc = pb + cols;
  if (TPR == 256) {
#pragma unroll
    for (int k = 0; k < kKMax; ++k) {
      const int vi = t + k * TPR;
      if (vi < nvec) {
        *reinterpret_cast<float4*>(pg + vi * 4) = acc_g[k];
        *reinterpret_cast<float4*>(pb + vi * 4) = acc_b[k];
        *reinterpret_cast<float4*>(pc + vi * 4) = acc_c[k];
      }
    }
  } else {
    // 8 row slots share the columns: fold them through shared memory, slot by slot.
    for (int pass = 0; pass < 3; ++pass) {
      for (int sidx = 0; sidx < kRowsPerBlock; ++sidx) {
        __syncthreads();
        if (sub == sidx) {
#pragma unroll
          for (int k = 0; k < kKMax; ++k) {
            const int vi = t + k * TPR;
            if (vi < nvec) {
              const float4 a = pass == 0 ? acc_g[k] : (pass == 1 ? acc_b[k] : acc_c[k]);
              float* f = &fold[pass][vi * 4];
              if (sidx == 0) {
                f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
              } else {
                f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
              }
            }
          }
        }
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      pg[c] = fold[0][c];
      pb[c] = fold[1][c];
      pc[c] = fold[2][c];
    }
  }
}

// Fold partial[nblk][3][cols] into the three outputs (each may be NULL); outputs are accumulated into.
__global__ void ln_fold_kernel(const float* __restrict__ partial, float* __restrict__ dgamma,
                               float* __restrict__ dbeta, float* __restrict__ dcolsum, int nblk, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int which = blockIdx.y;
  float* out = which == 0 ? dgamma : (which == 1 ? dbeta : dcolsum);
  if (c >= cols || out == nullptr) return;
  float s = 0.f;
  for (int b = 0; b < nblk; ++b) s += partial[(static_cast<long long>(b) * 3 + which) * cols + c];
  out[c] += s;
}

// ---------------------------------------------------------------- generic path
template <typename T>
__global__ void ln_fwd_generic(const T* __restrict__ x, const float* __restrict__ gamma,
                               const float* __restrict__ beta, T* __restrict__ y, float* __restrict__ mean_out,
                               float* __restrict__ rstd_out, long long rows, int cols, float eps, int pre_act) {
  __shared__ float smem[8];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) {
      float a = V4<T>::ld1(xr + c);
      if (pre_act == FB_ACT_GELU) a = gelu_f(a);
      s += a;
    }
    const float mu = row_sum<256>(s, smem) / cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) {
      float a = V4<T>::ld1(xr + c);
      if (pre_act == FB_ACT_GELU) a = gelu_f(a);
      q += (a - mu) * (a - mu);
    }
    const float rs = rsqrtf(row_sum<256>(q, smem) / cols + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mu;
      if (rstd_out) rstd_out[row] = rs;
    }
    for (int c = threadIdx.x; c < cols; c += 256) {
      float a = V4<T>::ld1(xr + c);
      if (pre_act == FB_ACT_GELU) a = gelu_f(a);
      const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
      V4<T>::st1(y + row * cols + c, (a - mu) * rs * g + b);
    }
  }
}

template <typename T>
__global__ void ln_bwd_generic(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                               const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                               float* __restrict__ dgamma, float* __restrict__ dbeta, float* __restrict__ dcolsum,
                               long long rows, int cols, int pre_act) {
  __shared__ float smem[8];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) {
      float a = V4<T>::ld1(x + row * cols + c);
      if (pre_act == FB_ACT_GELU) a = gelu_f(a);
      const float h = (a - mu) * rs;
      const float g = V4<T>::ld1(dy + row * cols + c);
      const float d = g * (gamma ? gamma[c] : 1.f);
      s1 += d;
      s2 += d * h;
      if (dgamma) atomicAdd(dgamma + c, g * h);
      if (dbeta) atomicAdd(dbeta + c, g);
    }
    const float m1 = row_sum<256>(s1, smem) / cols;
    const float m2 = row_sum<256>(s2, smem) / cols;
    for (int c = threadIdx.x; c < cols; c += 256) {
      const float raw = V4<T>::ld1(x + row * cols + c);
      const float a = pre_act == FB_ACT_GELU ? gelu_f(raw) : raw;
      const float h = (a - mu) * rs;
      const float d = V4<T>::ld1(dy + row * cols + c) * (gamma ? gamma[c] : 1.f);
      float o = rs * (d - m1 - h * m2);
      if (pre_act == FB_ACT_GELU) o *= gelu_grad(raw);
      if (dcolsum) atomicAdd(dcolsum + c, o);
      V4<T>::st1(dx + row * cols + c, o);
    }
  }
}

int sm_count() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

bool fast_ok(int cols, const void* a, const void* b, const void* c) {
  const uintptr_t m =
      reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c);
  return cols % 4 == 0 && cols <= 256 * 4 * kKMax && (m & 15) == 0;
}

template <typename T>
int fwd_t(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, long long rows,
          int cols, float eps, int pre_act, cudaStream_t st) {
  const T* xp = static_cast<const T*>(x);
  T* yp = static_cast<T*>(y);
  if (fast_ok(cols, x, y, gamma) && ((reinterpret_cast<uintptr_t>(beta) & 15) == 0)) {
    if (cols <= 32 * 4 * kKMax) {
      const long long nb = (rows + 7) / 8;
      const int grid = static_cast<int>(nb < sm_count() * 8LL ? nb : sm_count() * 8LL);
      ln_fwd_kernel<T, 32><<<grid, 256, 0, st>>>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps, pre_act);
    } else {
      const int grid = static_cast<int>(rows < sm_count() * 8LL ? rows : sm_count() * 8LL);
      ln_fwd_kernel<T, 256><<<grid, 256, 0, st>>>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps, pre_act);
    }
  } else {
    const int grid = static_cast<int>(rows < sm_count() * 8LL ? rows : sm_count() * 8LL);
    ln_fwd_generic<T><<<grid, 256, 0, st>>>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps, pre_act);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
}  // namespace fb

using namespace fb;

// Number of blocks (= rows of `partial`) the fast backward uses; 0 means the
// generic path runs and no partial buffer is needed.
extern "C" int fb_layernorm_bwd_blocks(long long rows, int cols) {
  if (cols % 4 != 0 || cols > 256 * 4 * kKMax) return 0;
  const long long sms = sm_count();
  if (cols <= 32 * 4 * kKMax) {
    const long long nb = (rows + 7) / 8;
    return static_cast<int>(nb < sms * 2 ? nb : sms * 2);
  }
  return static_cast<int>(rows < sms * 2 ? rows : sms * 2);
}

extern "C" int fb_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean,
                                float* rstd, long long rows, int cols, float eps, int pre_act, int dtype,
                                cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (dtype == FB_DT_F32) return fwd_t<float>(x, gamma, beta, y, mean, rstd, rows, cols, eps, pre_act, stream);
  if (dtype == FB_DT_BF16)
    return fwd_t<__nv_bfloat16>(x, gamma, beta, y, mean, rstd, rows, cols, eps, pre_act, stream);
  return -1;
}

template <typename T>
static int bwd_t(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, void* dx,
                 float* partial, float* dgamma, float* dbeta, float* dcolsum, long long rows, int cols, int pre_act,
                 int nblk, cudaStream_t st) {
  const T* dyp = static_cast<const T*>(dy);
  const T* xp = static_cast<const T*>(x);
  T* dxp = static_cast<T*>(dx);
  const bool fast = nblk > 0 && partial != nullptr && fast_ok(cols, dy, x, dx) &&
                    ((reinterpret_cast<uintptr_t>(gamma) & 15) == 0) &&
                    ((reinterpret_cast<uintptr_t>(partial) & 15) == 0);
  if (fast) {
    if (cols <= 32 * 4 * kKMax)
      ln_bwd_kernel<T, 32><<<nblk, 256, 0, st>>>(dyp, xp, gamma, mean, rstd, dxp, partial, rows, cols, pre_act,
                                                 dcolsum != nullptr);
    else
      ln_bwd_kernel<T, 256><<<nblk, 256, 0, st>>>(dyp, xp, gamma, mean, rstd, dxp, partial, rows, cols, pre_act,
                                                  dcolsum != nullptr);
    dim3 grid((cols + 255) / 256, 3);
    ln_fold_kernel<<<grid, 256, 0, st>>>(partial, dgamma, dbeta, dcolsum, nblk, cols);
  } else {
    const int grid = static_cast<int>(rows < sm_count() * 4LL ? rows : sm_count() * 4LL);
    ln_bwd_generic<T><<<grid, 256, 0, st>>>(dyp, xp, gamma, mean, rstd, dxp, dgamma, dbeta, dcolsum, rows, cols,
                                            pre_act);
  }
  return static_cast<int>(cudaGetLastError());
}

// dgamma / dbeta / dcolsum (each optional) are ACCUMULATED into: zero them for a fresh gradient.
extern "C" int fb_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean,
                                const float* rstd, void* dx, float* partial, float* dgamma, float* dbeta,
                                float* dcolsum, long long rows, int cols, int pre_act, int dtype, int nblk,
                                cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (dtype == FB_DT_F32)
    return bwd_t<float>(dy, x, gamma, mean, rstd, dx, partial, dgamma, dbeta, dcolsum, rows, cols, pre_act, nblk,
                        stream);
  if (dtype == FB_DT_BF16)
    return bwd_t<__nv_bfloat16>(dy, x, gamma, mean, rstd, dx, partial, dgamma, dbeta, dcolsum, rows, cols, pre_act,
                                nblk, stream);
  return -1;
}
