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
// Fast path: a row lives in registers (TPR threads x K vectors of 8 elements, 16-byte
// accesses), two-pass mean / variance on registers, column partials accumulate in
// registers across the rows a block owns and are written once to
// partial[nblk][3][cols]; a second kernel folds the partials.  Register budgets are
// kept small enough for two to four 256-thread blocks per SM: these kernels are
// bandwidth-bound and need the bytes in flight.
// Generic path (odd widths, very wide rows): scalar accesses, re-reads the row,
// column sums by atomicAdd.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

constexpr float kGeluC = 0.7978845608028654f;
constexpr float kGeluA = 0.044715f;

// FAST = hardware tanh.approx (bf16 data: its 2^-11 error is below the storage rounding);
// otherwise the accurate tanhf (fp32 parity path).
template <bool FAST>
__device__ __forceinline__ float tanh_sel(float u) {
  if (FAST) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    return t;
  }
  return tanhf(u);
}
template <bool FAST>
__device__ __forceinline__ float gelu_f(float x) {
  return 0.5f * x * (1.f + tanh_sel<FAST>(kGeluC * (x + kGeluA * x * x * x)));
}
// value and derivative from one tanh
template <bool FAST>
__device__ __forceinline__ void gelu_both(float x, float& val, float& der) {
  const float t = tanh_sel<FAST>(kGeluC * (x + kGeluA * x * x * x));
  val = 0.5f * x * (1.f + t);
  der = 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * kGeluC * (1.f + 3.f * kGeluA * x * x);
}

// Eight consecutive elements: one 16-byte access for bf16, two for fp32.
template <typename T>
struct V8;
template <>
struct V8<float> {
  static constexpr bool kFastMath = false;
  struct Raw { float4 a, b; };
  static __device__ __forceinline__ Raw ld(const float* p) {
    Raw r;
    r.a = *reinterpret_cast<const float4*>(p);
    r.b = *reinterpret_cast<const float4*>(p + 4);
    return r;
  }
  static __device__ __forceinline__ void unpack(const Raw& r, float (&f)[8]) {
    f[0] = r.a.x; f[1] = r.a.y; f[2] = r.a.z; f[3] = r.a.w; f[4] = r.b.x; f[5] = r.b.y; f[6] = r.b.z; f[7] = r.b.w;
  }
  static __device__ __forceinline__ void st(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
  static __device__ __forceinline__ float ld1(const float* p) { return *p; }
  static __device__ __forceinline__ void st1(float* p, float v) { *p = v; }
};
template <>
struct V8<__nv_bfloat16> {
  static constexpr bool kFastMath = true;
  using Raw = uint4;
  static __device__ __forceinline__ Raw ld(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ void unpack(const Raw& r, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  static __device__ __forceinline__ float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

__device__ __forceinline__ void ld8f(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// Sum over the TPR threads that share a row.  256-thread blocks hold 256 / TPR rows; every thread of the
// block calls this the same number of times (rows are processed in lockstep).
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float (*smem)[8]) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (TPR == 32) return v;
  constexpr int kWarps = TPR / 32;
  const int sub = threadIdx.x / TPR;
  const int w = (threadIdx.x % TPR) >> 5;
  __syncthreads();  // previous use of smem is over
  if ((threadIdx.x & 31) == 0) smem[sub][w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kWarps; ++i) t += smem[sub][i];
  return t;
}

// Forward.  A row lives in registers: TPR threads x K vectors of 8 elements.
template <typename T, int TPR, int K>
__global__ void __launch_bounds__(256, (K * sizeof(T) <= 2) ? 4 : ((K * sizeof(T) <= 4) ? 3 : ((K * sizeof(T) <= 8) ? 2 : 1)))
ln_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
              T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, long long rows,
              int cols, float eps, int pre_act) {
  __shared__ float smem[8][8];
  constexpr int kRowsPerBlock = 256 / TPR;
  constexpr bool kFast = V8<T>::kFastMath;
  const int sub = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const int nvec = cols >> 3;
  const float inv_n = 1.f / static_cast<float>(cols);
  const long long row_stride = static_cast<long long>(gridDim.x) * kRowsPerBlock;
  using Raw = typename V8<T>::Raw;
  auto load = [&](long long r, Raw (&buf)[K]) {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = t + k * TPR;
      if (r < rows && vi < nvec) buf[k] = V8<T>::ld(x + r * cols + vi * 8);
    }
  };
  auto process = [&](long long row, const Raw (&raw)[K]) {
    const bool live = row < rows;
    float v[K][8];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = t + k * TPR;
      if (live && vi < nvec) {
        V8<T>::unpack(raw[k], v[k]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (pre_act == FB_ACT_GELU) v[k][i] = gelu_f<kFast>(v[k][i]);
          s += v[k][i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[k][i] = 0.f;
      }
    }
    const float mu = row_sum<TPR>(s, smem) * inv_n;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = t + k * TPR;
      if (live && vi < nvec) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = v[k][i] - mu;
          q += d * d;
        }
      }
    }
    const float var = row_sum<TPR>(q, smem) * inv_n;
    const float rs = rsqrtf(var + eps);
    if (live && t == 0) {
      if (mean_out) mean_out[row] = mu;
      if (rstd_out) rstd_out[row] = rs;
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = t + k * TPR;
      if (live && vi < nvec) {
        float g[8], b[8], o[8];
        if (gamma) ld8f(gamma + vi * 8, g);
        if (beta) ld8f(beta + vi * 8, b);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          o[i] = (v[k][i] - mu) * rs * (gamma ? g[i] : 1.f) + (beta ? b[i] : 0.f);
        V8<T>::st(y + row * cols + vi * 8, o);
      }
    }
  };
  // Three register sets rotating by name (loop unrolled by three): the loads of the next two rows stay in
  // flight while a row is reduced and written, and no register-to-register rotation waits on the newest load.
  // Row slots of a block advance in lockstep (row0 is uniform), so the barriers inside row_sum stay uniform.
  Raw b0[K], b1[K], b2[K];
  long long row0 = static_cast<long long>(blockIdx.x) * kRowsPerBlock;
  load(row0 + sub, b0);
  load(row0 + row_stride + sub, b1);
  while (row0 < rows) {
    load(row0 + 2 * row_stride + sub, b2);
    process(row0 + sub, b0);
    row0 += row_stride;
    if (row0 >= rows) break;
    load(row0 + 2 * row_stride + sub, b0);
    process(row0 + sub, b1);
    row0 += row_stride;
    if (row0 >= rows) break;
    load(row0 + 2 * row_stride + sub, b1);
    process(row0 + sub, b2);
    row0 += row_stride;
  }
}

// Backward.  x and dy stay packed in registers between the statistics pass and the output pass; the
// three column partials (dy*xhat, dy, dx) accumulate in registers over all rows the block visits and are
// written once to partial[blockIdx][3][cols].
template <typename T, int TPR, int K>
__global__ void __launch_bounds__(256, 2)
ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ act_grad,
              const float* __restrict__ gamma, const float* __restrict__ mean, const float* __restrict__ rstd,
              T* __restrict__ dx, float* __restrict__ partial, long long rows, int cols, int pre_act,
              int want_colsum) {
  __shared__ float smem[8][8];
  constexpr int kRowsPerBlock = 256 / TPR;
  constexpr bool kFast = V8<T>::kFastMath;
  const int sub = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const int nvec = cols >> 3;
  const float inv_n = 1.f / static_cast<float>(cols);
  float acc_g[K][8], acc_b[K][8], acc_c[K][8];
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc_g[k][i] = acc_b[k][i] = acc_c[k][i] = 0.f;

  const long long row_stride = static_cast<long long>(gridDim.x) * kRowsPerBlock;
  typename V8<T>::Raw xr[K], gr[K], xn[K], gn[K];
  {
    const long long r0 = static_cast<long long>(blockIdx.x) * kRowsPerBlock + sub;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = t + k * TPR;
      if (r0 < rows && vi < nvec) {
        xr[k] = V8<T>::ld(x + r0 * cols + vi * 8);
        gr[k] = V8<T>::ld(dy + r0 * cols + vi * 8);
      }
    }
  }
  for (long long row0 = static_cast<long long>(blockIdx.x) * kRowsPerBlock; row0 < rows; row0 += row_stride) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    {  // prefetch the next row while this one is processed
      const long long rn = row + row_stride;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int vi = t + k * TPR;
        if (rn < rows && vi < nvec) {
          xn[k] = V8<T>::ld(x + rn * cols + vi * 8);
          gn[k] = V8<T>::ld(dy + rn * cols + vi * 8);
        }
      }
    }
    const float mu = live ? mean[row] : 0.f;
    const float rs = live ? rstd[row] : 0.f;
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = t + k * TPR;
      if (live && vi < nvec) {
        float xv[8], gv[8], w[8];
        V8<T>::unpack(xr[k], xv);
        V8<T>::unpack(gr[k], gv);
        if (gamma) ld8f(gamma + vi * 8, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float a = pre_act == FB_ACT_GELU ? gelu_f<kFast>(xv[i]) : xv[i];
          const float h = (a - mu) * rs;
          const float d = gv[i] * (gamma ? w[i] : 1.f);
          acc_g[k][i] += gv[i] * h;
          acc_b[k][i] += gv[i];
          s1 += d;
          s2 += d * h;
        }
      }
    }
    const float m1 = row_sum<TPR>(s1, smem) * inv_n;
    const float m2 = row_sum<TPR>(s2, smem) * inv_n;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = t + k * TPR;
      if (live && vi < nvec) {
        float xv[8], gv[8], w[8], o[8];
        V8<T>::unpack(xr[k], xv);
        V8<T>::unpack(gr[k], gv);
        if (gamma) ld8f(gamma + vi * 8, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float a = xv[i], da = 1.f;
          if (pre_act == FB_ACT_GELU) gelu_both<kFast>(xv[i], a, da);
          const float h = (a - mu) * rs;
          const float d = gv[i] * (gamma ? w[i] : 1.f);
          o[i] = rs * (d - m1 - h * m2) * da;
        }
        if (act_grad != nullptr) {  // x holds act(z); its derivative was stored by the producer
          float ag[8];
          V8<T>::unpack(V8<T>::ld(act_grad + row * cols + vi * 8), ag);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] *= ag[i];
        }
        if (want_colsum) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc_c[k][i] += o[i];
        }
        V8<T>::st(dx + row * cols + vi * 8, o);
      }
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      xr[k] = xn[k];
      gr[k] = gn[k];
    }
  }

  // ---- column partials of this block: partial[blockIdx][3][cols]
  float* pg = partial + static_cast<long long>(blockIdx.x) * 3 * cols;
  float* pb = pg + cols;
  float* pc = pb + cols;
  if (kRowsPerBlock == 1) {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = t + k * TPR;
      if (vi < nvec) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          pg[vi * 8 + i] = acc_g[k][i];
          pb[vi * 8 + i] = acc_b[k][i];
          pc[vi * 8 + i] = acc_c[k][i];
        }
      }
    }
  } else {
    // several row slots own the same columns: slot 0 stores, the others add, one slot at a time
    for (int sidx = 0; sidx < kRowsPerBlock; ++sidx) {
      __syncthreads();
      if (sub == sidx) {
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const int vi = t + k * TPR;
          if (vi < nvec) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int c = vi * 8 + i;
              if (sidx == 0) {
                pg[c] = acc_g[k][i]; pb[c] = acc_b[k][i]; pc[c] = acc_c[k][i];
              } else {
                pg[c] += acc_g[k][i]; pb[c] += acc_b[k][i]; pc[c] += acc_c[k][i];
              }
            }
          }
        }
      }
      __threadfence_block();
    }
  }
}

// Backward for rows of 2056..4096 bf16 elements whose activation derivative (if any) is given as a tensor:
// pure streaming arithmetic, so the kernel is organised around bytes in flight.  One 512-thread block per
// SM walks its rows one at a time; a thread owns ONE 16-byte vector of each operand and keeps the loads of
// the next two rows outstanding while it works on the current one.  The three register sets rotate by NAME
// (the row loop is unrolled by three): a register-to-register rotation would make every trip wait for the
// newest load.  A row costs a single __syncthreads (the two row sums travel together through a
// double-buffered shared-memory slot).  gamma and the three column accumulators stay in registers.
struct WideRow {
  uint4 g, x, a;
  float mu, rs;
};

__global__ void __launch_bounds__(512, 1)
ln_bwd_wide_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ act_grad, const float* __restrict__ gamma,
                   const float* __restrict__ mean, const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ partial, long long rows, int cols, int want_colsum) {
  using V = V8<__nv_bfloat16>;
  __shared__ float2 red[2][16];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int nvec = cols >> 3;
  const bool has = t < nvec;
  const float inv_n = 1.f / static_cast<float>(cols);
  const long long stride = gridDim.x;
  const bool use_ag = act_grad != nullptr;

  float w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = 1.f;
  if (has && gamma != nullptr) ld8f(gamma + t * 8, w);
  float acc_g[8], acc_b[8], acc_c[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc_g[i] = acc_b[i] = acc_c[i] = 0.f;
  int par = 0;

  auto load = [&](long long r, WideRow& b) {
    if (r < rows) {
      b.mu = mean[r];
      b.rs = rstd[r];
      if (has) {
        const long long o = r * cols + t * 8;
        b.g = V::ld(dy + o);
        b.x = V::ld(x + o);
        if (use_ag) b.a = V::ld(act_grad + o);
      }
    }
  };
  auto process = [&](long long row, const WideRow& b) {
    float gv[8], h[8];
    V::unpack(b.g, gv);
    V::unpack(b.x, h);
    const float shift = -b.mu * b.rs;
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      h[i] = fmaf(h[i], b.rs, shift);
      acc_b[i] += gv[i];
      acc_g[i] = fmaf(gv[i], h[i], acc_g[i]);
      gv[i] *= w[i];  // d = dy * gamma
      s1 += gv[i];
      s2 = fmaf(gv[i], h[i], s2);
    }
    if (!has) s1 = s2 = 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (lane == 0) red[par][warp] = make_float2(s1, s2);
    __syncthreads();
    float m1 = 0.f, m2 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 v = red[par][i];
      m1 += v.x;
      m2 += v.y;
    }
    par ^= 1;
    m1 *= inv_n;
    m2 *= inv_n;
    if (has) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = b.rs * (gv[i] - m1 - h[i] * m2);
      if (use_ag) {
        float ag[8];
        V::unpack(b.a, ag);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] *= ag[i];
      }
      if (want_colsum) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc_c[i] += o[i];
      }
      V::st(dx + row * cols + t * 8, o);
    }
  };

  WideRow b0, b1, b2;
  b0.g = b0.x = b0.a = b1.g = b1.x = b1.a = b2.g = b2.x = b2.a = make_uint4(0u, 0u, 0u, 0u);
  b0.mu = b0.rs = b1.mu = b1.rs = b2.mu = b2.rs = 0.f;
  long long row = blockIdx.x;
  load(row, b0);
  load(row + stride, b1);
  while (row < rows) {  // every condition below is uniform over the block
    load(row + 2 * stride, b2);
    process(row, b0);
    row += stride;
    if (row >= rows) break;
    load(row + 2 * stride, b0);
    process(row, b1);
    row += stride;
    if (row >= rows) break;
    load(row + 2 * stride, b1);
    process(row, b2);
    row += stride;
  }
  if (has) {
    float* pg = partial + static_cast<long long>(blockIdx.x) * 3 * cols + t * 8;
    float* pb = pg + cols;
    float* pc = pb + cols;
    *reinterpret_cast<float4*>(pg) = make_float4(acc_g[0], acc_g[1], acc_g[2], acc_g[3]);
    *reinterpret_cast<float4*>(pg + 4) = make_float4(acc_g[4], acc_g[5], acc_g[6], acc_g[7]);
    *reinterpret_cast<float4*>(pb) = make_float4(acc_b[0], acc_b[1], acc_b[2], acc_b[3]);
    *reinterpret_cast<float4*>(pb + 4) = make_float4(acc_b[4], acc_b[5], acc_b[6], acc_b[7]);
    *reinterpret_cast<float4*>(pc) = make_float4(acc_c[0], acc_c[1], acc_c[2], acc_c[3]);
    *reinterpret_cast<float4*>(pc + 4) = make_float4(acc_c[4], acc_c[5], acc_c[6], acc_c[7]);
  }
}

// Fold partial[nblk][3*cols] into stats[3*cols] (accumulated into): block = 128 columns x a chunk of the
// nblk rows, lanes own 4 adjacent columns, partials leave with one atomicAdd per column per block.
__global__ void __launch_bounds__(256)
ln_fold_kernel(const float* __restrict__ partial, float* __restrict__ stats, int nblk, int ncols,
               int rows_per_block) {
  __shared__ float sm[8][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = blockIdx.x * 128 + lane * 4;
  const int r_lo = blockIdx.y * rows_per_block;
  const int r_hi = min(nblk, r_lo + rows_per_block);
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c0 < ncols) {
    for (int r = r_lo + warp; r < r_hi; r += 8) {
      const float4 v = *reinterpret_cast<const float4*>(partial + static_cast<long long>(r) * ncols + c0);
      a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
  }
  sm[warp][lane * 4 + 0] = a.x;
  sm[warp][lane * 4 + 1] = a.y;
  sm[warp][lane * 4 + 2] = a.z;
  sm[warp][lane * 4 + 3] = a.w;
  __syncthreads();
  if (threadIdx.x < 128) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += sm[w][threadIdx.x];
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c < ncols) atomicAdd(stats + c, s);
  }
}

// ---------------------------------------------------------------- generic path
template <typename T>
__global__ void ln_fwd_generic(const T* __restrict__ x, const float* __restrict__ gamma,
                               const float* __restrict__ beta, T* __restrict__ y, float* __restrict__ mean_out,
                               float* __restrict__ rstd_out, long long rows, int cols, float eps, int pre_act) {
  __shared__ float smem[8][8];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) {
      float a = V8<T>::ld1(xr + c);
      if (pre_act == FB_ACT_GELU) a = gelu_f<false>(a);
      s += a;
    }
    const float mu = row_sum<256>(s, smem) / cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) {
      float a = V8<T>::ld1(xr + c);
      if (pre_act == FB_ACT_GELU) a = gelu_f<false>(a);
      q += (a - mu) * (a - mu);
    }
    const float rs = rsqrtf(row_sum<256>(q, smem) / cols + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mu;
      if (rstd_out) rstd_out[row] = rs;
    }
    for (int c = threadIdx.x; c < cols; c += 256) {
      float a = V8<T>::ld1(xr + c);
      if (pre_act == FB_ACT_GELU) a = gelu_f<false>(a);
      const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
      V8<T>::st1(y + row * cols + c, (a - mu) * rs * g + b);
    }
  }
}

// stats = [3][cols] (d_gamma, d_beta, column sum of dx), accumulated into with atomics.
template <typename T>
__global__ void ln_bwd_generic(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ act_grad,
                               const float* __restrict__ gamma, const float* __restrict__ mean,
                               const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ stats,
                               long long rows, int cols, int pre_act, int want_colsum) {
  __shared__ float smem[8][8];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) {
      float a = V8<T>::ld1(x + row * cols + c);
      if (pre_act == FB_ACT_GELU) a = gelu_f<false>(a);
      const float h = (a - mu) * rs;
      const float g = V8<T>::ld1(dy + row * cols + c);
      const float d = g * (gamma ? gamma[c] : 1.f);
      s1 += d;
      s2 += d * h;
      atomicAdd(stats + c, g * h);
      atomicAdd(stats + cols + c, g);
    }
    const float m1 = row_sum<256>(s1, smem) / cols;
    const float m2 = row_sum<256>(s2, smem) / cols;
    for (int c = threadIdx.x; c < cols; c += 256) {
      const float raw = V8<T>::ld1(x + row * cols + c);
      float a = raw, da = 1.f;
      if (pre_act == FB_ACT_GELU) gelu_both<false>(raw, a, da);
      const float h = (a - mu) * rs;
      const float d = V8<T>::ld1(dy + row * cols + c) * (gamma ? gamma[c] : 1.f);
      float o = rs * (d - m1 - h * m2) * da;
      if (act_grad != nullptr) o *= V8<T>::ld1(act_grad + row * cols + c);
      if (want_colsum) atomicAdd(stats + 2 * cols + c, o);
      V8<T>::st1(dx + row * cols + c, o);
    }
  }
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

// Fast-path geometry for a row of `cols` elements: threads per row and 8-element vectors per thread.
struct Geo {
  int tpr, k;
};
bool geometry(int cols, Geo* g) {
  if (cols % 8 != 0 || cols > 8192 || cols <= 0) return false;
  const int nvec = cols / 8;
  if (nvec <= 32) *g = {32, 1};
  else if (nvec <= 64) *g = {32, 2};
  else if (nvec <= 128) *g = {128, 1};
  else if (nvec <= 256) *g = {128, 2};
  else if (nvec <= 512) *g = {256, 2};
  else *g = {256, 4};
  return true;
}
bool aligned16(const void* a, const void* b, const void* c, const void* d) {
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
           reinterpret_cast<uintptr_t>(d)) & 15) == 0;
}

// Persistent grid: exactly the blocks that are resident at once, so every block walks the same number of rows.
template <typename T, int TPR, int K>
void launch_fwd(const T* xp, const float* gamma, const float* beta, T* yp, float* mean, float* rstd, long long rows,
                int cols, float eps, int pre_act, long long nb, cudaStream_t st) {
  static int occ = 0;
  if (occ == 0 &&
      (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, ln_fwd_kernel<T, TPR, K>, 256, 0) != cudaSuccess || occ < 1))
    occ = 1;
  const long long cap = static_cast<long long>(sm_count()) * occ;
  const int grid = static_cast<int>(nb < cap ? nb : cap);
  ln_fwd_kernel<T, TPR, K><<<grid, 256, 0, st>>>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps, pre_act);
}

template <typename T>
int fwd_t(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, long long rows,
          int cols, float eps, int pre_act, cudaStream_t st) {
  const T* xp = static_cast<const T*>(x);
  T* yp = static_cast<T*>(y);
  Geo g;
  if (geometry(cols, &g) && aligned16(x, y, gamma, beta)) {
    const long long rpb = 256 / g.tpr;
    const long long nb = (rows + rpb - 1) / rpb;
#define FB_LN_FWD(TPR, K) \
  launch_fwd<T, TPR, K>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps, pre_act, nb, st)
    if (g.tpr == 32 && g.k == 1) FB_LN_FWD(32, 1);
    else if (g.tpr == 32) FB_LN_FWD(32, 2);
    else if (g.tpr == 128 && g.k == 1) FB_LN_FWD(128, 1);
    else if (g.tpr == 128) FB_LN_FWD(128, 2);
    else if (g.k == 2) FB_LN_FWD(256, 2);
    else FB_LN_FWD(256, 4);
#undef FB_LN_FWD
  } else {
    const int grid = static_cast<int>(rows < sm_count() * 8LL ? rows : sm_count() * 8LL);
    ln_fwd_generic<T><<<grid, 256, 0, st>>>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps, pre_act);
  }
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
bool launch_wide(const T*, const T*, const T*, const float*, const float*, const float*, T*, float*, long long, int,
                 int, int, cudaStream_t) {
  return false;
}
// bf16 rows of 257..512 vectors with no activation to re-evaluate: the streaming kernel, one block per SM.
template <>
bool launch_wide<__nv_bfloat16>(const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* ag,
                                const float* gamma, const float* mean, const float* rstd, __nv_bfloat16* dx,
                                float* partial, long long rows, int cols, int blocks, int want_colsum,
                                cudaStream_t st) {
  ln_bwd_wide_kernel<<<blocks, 512, 0, st>>>(dy, x, ag, gamma, mean, rstd, dx, partial, rows, cols, want_colsum);
  return true;
}

template <typename T>
int bwd_t(const void* dy, const void* x, const void* act_grad, const float* gamma, const float* mean,
          const float* rstd, void* dx, float* partial, float* stats, long long rows, int cols, int pre_act, int nblk,
          int want_colsum, cudaStream_t st) {
  const T* dyp = static_cast<const T*>(dy);
  const T* xp = static_cast<const T*>(x);
  const T* agp = static_cast<const T*>(act_grad);
  T* dxp = static_cast<T*>(dx);
  Geo g;
  const bool fast = nblk > 0 && partial != nullptr && geometry(cols, &g) && aligned16(dy, x, dx, gamma) &&
                    aligned16(partial, stats, act_grad, nullptr);
  if (fast) {
    int used = nblk;
    const int nvec = cols / 8;
    const int wide_blocks = nblk < sm_count() ? nblk : sm_count();
    if (pre_act == FB_ACT_NONE && nvec > 256 && nvec <= 512 &&
        launch_wide<T>(dyp, xp, agp, gamma, mean, rstd, dxp, partial, rows, cols, wide_blocks, want_colsum, st)) {
      used = wide_blocks;
    } else {
#define FB_LN_BWD(TPR, K) \
  ln_bwd_kernel<T, TPR, K><<<nblk, 256, 0, st>>>(dyp, xp, agp, gamma, mean, rstd, dxp, partial, rows, cols, pre_act, \
                                                 want_colsum)
    if (g.tpr == 32 && g.k == 1) FB_LN_BWD(32, 1);
    else if (g.tpr == 32) FB_LN_BWD(32, 2);
    else if (g.tpr == 128 && g.k == 1) FB_LN_BWD(128, 1);
    else if (g.tpr == 128) FB_LN_BWD(128, 2);
    else if (g.k == 2) FB_LN_BWD(256, 2);
    else FB_LN_BWD(256, 4);
#undef FB_LN_BWD
    }
    const int ncols = 3 * cols;
    const int col_blocks = (ncols + 127) / 128;
    int row_blocks = (sm_count() * 2 + col_blocks - 1) / col_blocks;
    const int max_rb = (used + 15) / 16;
    if (row_blocks > max_rb) row_blocks = max_rb;
    if (row_blocks < 1) row_blocks = 1;
    const int rpb = (used + row_blocks - 1) / row_blocks;
    ln_fold_kernel<<<dim3(col_blocks, row_blocks), 256, 0, st>>>(partial, stats, used, ncols, rpb);
  } else {
    const int grid = static_cast<int>(rows < sm_count() * 4LL ? rows : sm_count() * 4LL);
    ln_bwd_generic<T><<<grid, 256, 0, st>>>(dyp, xp, agp, gamma, mean, rstd, dxp, stats, rows, cols, pre_act,
                                            want_colsum);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
}  // namespace fb

using namespace fb;

// Number of blocks (= rows of `partial`, each 3 * cols floats) the fast backward uses; 0 means the
// generic path runs and no partial buffer is needed.
extern "C" int fb_layernorm_bwd_blocks(long long rows, int cols) {
  Geo g;
  if (!geometry(cols, &g)) return 0;
  const long long rpb = 256 / g.tpr;
  const long long nb = (rows + rpb - 1) / rpb;
  const long long cap = static_cast<long long>(sm_count()) * 2;
  return static_cast<int>(nb < cap ? nb : cap);
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

// stats = [3][cols] fp32: d_gamma, d_beta and the column sum of dx.  All three are ACCUMULATED into
// (zero the buffer for a fresh gradient); the column sum is produced only when want_colsum != 0.
// act_grad (optional, dtype of x): x then holds act(z) of an activation applied before the normalisation and
// act_grad its derivative act'(z); dx is the gradient of z.  (pre_act instead re-evaluates a GELU from z.)
extern "C" int fb_layernorm_bwd(const void* dy, const void* x, const void* act_grad, const float* gamma,
                                const float* mean, const float* rstd, void* dx, float* partial, float* stats,
                                long long rows, int cols, int pre_act, int dtype, int nblk, int want_colsum,
                                cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (stats == nullptr) return -1;
  if (act_grad != nullptr && pre_act != FB_ACT_NONE) return -1;
  if (dtype == FB_DT_F32)
    return bwd_t<float>(dy, x, act_grad, gamma, mean, rstd, dx, partial, stats, rows, cols, pre_act, nblk,
                        want_colsum, stream);
  if (dtype == FB_DT_BF16)
    return bwd_t<__nv_bfloat16>(dy, x, act_grad, gamma, mean, rstd, dx, partial, stats, rows, cols, pre_act, nblk,
                                want_colsum, stream);
  return -1;
}
