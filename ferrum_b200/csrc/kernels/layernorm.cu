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

#include <cstdlib>

#include "../common/ptx.cuh"
#include "../common/status.h"
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
__global__ void __launch_bounds__(256)
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
  typename V8<T>::Raw raw[K], nxt[K];
  {
    const long long r0 = static_cast<long long>(blockIdx.x) * kRowsPerBlock + sub;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = t + k * TPR;
      if (r0 < rows && vi < nvec) raw[k] = V8<T>::ld(x + r0 * cols + vi * 8);
    }
  }
  for (long long row0 = static_cast<long long>(blockIdx.x) * kRowsPerBlock; row0 < rows; row0 += row_stride) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    {  // the next row's loads are in flight while this row is reduced and written
      const long long rn = row + row_stride;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int vi = t + k * TPR;
        if (rn < rows && vi < nvec) nxt[k] = V8<T>::ld(x + rn * cols + vi * 8);
      }
    }
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
#pragma unroll
    for (int k = 0; k < K; ++k) raw[k] = nxt[k];
  }
}

__device__ __forceinline__ void ld_pairs_f32(const float* p, float2 (&o)[4]);

// Forward, one WARP per row (bf16, 1024..4096 columns): a lane keeps its K 16-byte vectors packed in registers,
// all K loads are issued back to back (up to 8 KB in flight per warp), the statistics are one pass of shifted sums
// (x - c with c = the row's first element) reduced by warp shuffles, and there is no block barrier at all: warps
// stream rows independently.  Packed fp32x2 arithmetic; gamma / beta come through L1.
template <int K>
__global__ void __launch_bounds__(256, 2)
ln_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                   long long rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  const float inv_n = 1.f / static_cast<float>(cols);
  const long long warp_id = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = warp_id; row < rows; row += nwarps) {
    const __nv_bfloat16* xr = x + row * cols;
    uint4 raw[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = lane + 32 * k;
      raw[k] = vi < nvec ? *reinterpret_cast<const uint4*>(xr + vi * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
    // c = element 0 of the row = low half of lane 0's first word
    const float c = __uint_as_float(__shfl_sync(0xffffffffu, raw[0].x, 0) << 16);
    const float2 nc = make_float2(-c, -c);
    float2 s2 = make_float2(0.f, 0.f), q2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (lane + 32 * k < nvec) {
        const uint32_t w[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 v = make_float2(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xffff0000u));
          const float2 d = __fadd2_rn(v, nc);
          s2 = __fadd2_rn(s2, d);
          q2 = __ffma2_rn(d, d, q2);
        }
      }
    }
    float s = s2.x + s2.y, q = q2.x + q2.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      q += __shfl_xor_sync(0xffffffffu, q, o);
    }
    const float ms = s * inv_n;
    const float var = fmaxf(q * inv_n - ms * ms, 0.f);
    const float mu = c + ms;
    const float rs = rsqrtf(var + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mu;
      if (rstd_out) rstd_out[row] = rs;
    }
    const float2 rs2 = make_float2(rs, rs), sh2 = make_float2(-mu * rs, -mu * rs);
    __nv_bfloat16* yr = y + row * cols;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        const uint32_t w[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
        float2 g[4], b[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          g[e] = make_float2(1.f, 1.f);
          b[e] = make_float2(0.f, 0.f);
        }
        if (gamma) ld_pairs_f32(gamma + vi * 8, g);
        if (beta) ld_pairs_f32(beta + vi * 8, b);
        uint4 out;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 v = make_float2(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xffff0000u));
          const float2 o = __ffma2_rn(__ffma2_rn(v, rs2, sh2), g[e], b[e]);
          const __nv_bfloat162 pk = __float22bfloat162_rn(o);
          ow[e] = *reinterpret_cast<const uint32_t*>(&pk);
        }
        *reinterpret_cast<uint4*>(yr + vi * 8) = out;
      }
    }
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

// ----------------------------------------------------------------------------------------------------
// Wide rows (2 KB .. 8 KB of bf16 / 16 KB of fp32, i.e. up to 4096 columns): shared-memory ring fed by bulk
// async copies, organised for few instructions per element.
//
// Measured on the register-tiled kernels above and on a first ring version: with ~30-40 instructions per
// element these kernels are bound by instruction issue (issue slots 55-60 % busy, the rest barrier / dependency
// stalls), not by HBM.  So:
//   * a thread owns 16 elements of a row (two 16-byte vectors of bf16), which halves the per-row fixed cost
//     (shuffles, shared-memory exchange, barrier) per element;
//   * the forward needs ONE reduction per row: sums of (x - c) and (x - c)^2 with c = the row's first element
//     (shifted sums: no cancellation unless the row's spread is tiny against |x0 - mean|);
//   * a 512-thread block is two independent groups of 256 threads, each with its own ring, mbarriers and named
//     barrier, so one group's barrier wait overlaps the other group's arithmetic;
//   * rows arrive by cp.async.bulk into the ring, up to three rows ahead per group: no registers or scoreboards
//     are tied up by prefetched data;
//   * the arithmetic is packed fp32x2 (FFMA2 / FADD2 / FMUL2).
// Measured at 8192 x 4096 bf16: backward 64-66 us against 128 us for the register-tiled kernel; the forward
// (42-45 us) does not beat the register-tiled forward (39-40 us), so the forward ring is opt-in
// (FERRUM_LN_RING_FWD=1) and the default forward stays on the register-tiled kernel.  A slot is refilled at the top of the iteration after the one that read it (every
//     thread of the group has passed that iteration's barrier by then).
// Packed fp32x2 arithmetic (Blackwell FFMA2 / FADD2 / FMUL2): one issue slot does two fp32 operations, which
// matters here because these kernels are bound by instruction issue, not by HBM.
__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ float2 f2s(float a) { return make_float2(a, a); }
template <typename T>
__device__ __forceinline__ void unpack_pairs(const typename V8<T>::Raw& r, float2 (&p)[4]) {
  float f[8];
  V8<T>::unpack(r, f);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = make_float2(f[2 * i], f[2 * i + 1]);
}
template <typename T>
__device__ __forceinline__ void store_pairs(T* dst, const float2 (&p)[4]) {
  float f[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = p[i].x;
    f[2 * i + 1] = p[i].y;
  }
  V8<T>::st(dst, f);
}
__device__ __forceinline__ void ld_pairs_f32(const float* p, float2 (&o)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = make_float2(a.x, a.y);
  o[1] = make_float2(a.z, a.w);
  o[2] = make_float2(b.x, b.y);
  o[3] = make_float2(b.z, b.w);
}
// Sum of (a, b) over the eight warps of a 256-thread group: lane 0 of every warp has written its partial to
// slot[warp]; after the group barrier every thread folds the eight partials with three shuffles.
__device__ __forceinline__ float2 fold8(const float2* slot, int lane) {
  float2 v = slot[lane & 7];
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
  }
  return v;
}

constexpr int kRingThreads = 512;
constexpr int kGroupThreads = 256;
constexpr int kMaxRingStages = 4;  // per group (measured: 2 .. 6 stages perform alike; the kernels are issue-bound)
constexpr int kStatRows = 128;   // per-group cache of mean / rstd (backward)

struct RingCtl {
  uint64_t full[2][kMaxRingStages];
  int abort_flag;
};

__device__ __forceinline__ void group_sync(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(kGroupThreads) : "memory");
}
__device__ __forceinline__ bool ring_wait(RingCtl* ctl, int group, int i, int stages) {
  return ptx::mbar_wait(&ctl->full[group][i % stages], static_cast<uint32_t>((i / stages) & 1), &ctl->abort_flag,
                        2000000000ull);
}
// Before a group with copies in flight may exit, let them land (bounded).
__device__ __forceinline__ void ring_drain(RingCtl* ctl, int group, int issued, int consumed, int stages) {
  for (int i = consumed; i < issued; ++i) {
    const uint64_t t0 = ptx::globaltimer();
    while (!ptx::mbar_try_wait(&ctl->full[group][i % stages], static_cast<uint32_t>((i / stages) & 1))) {
      if (ptx::globaltimer() - t0 > 2000000000ull) break;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kRingThreads, sizeof(T) == 2 ? 2 : 1)
ln_fwd_ring_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                   T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, long long rows,
                   int cols, float eps, int pre_act, int stages, int32_t* status) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ RingCtl ctl;
  __shared__ float2 red[2][2][8];
  constexpr bool kFast = V8<T>::kFastMath;
  const int group = threadIdx.x >> 8, t = threadIdx.x & 255, lane = t & 31, warp = t >> 5;
  const int nvec = cols >> 3;
  const uint32_t row_bytes = static_cast<uint32_t>(cols) * sizeof(T);
  uint8_t* my_ring = ring + group * stages * row_bytes;
  const float inv_n = 1.f / static_cast<float>(cols);
  // the block's rows are first + j * stride; group g takes j = 2 i + g
  const long long first = blockIdx.x, stride = gridDim.x;
  const long long n_block = first < rows ? (rows - first + stride - 1) / stride : 0;
  const int n_mine = static_cast<int>((n_block - group + 1) / 2);
  auto row_of = [&](int i) { return first + (2LL * i + group) * stride; };
  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    for (int g = 0; g < 2; ++g)
      for (int s = 0; s < stages; ++s) ptx::mbar_init(&ctl.full[g][s], 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  auto issue = [&](int idx) {
    const int sl = idx % stages;
    ptx::mbar_arrive_expect_tx(&ctl.full[group][sl], row_bytes);
    ptx::bulk_load_1d(my_ring + sl * row_bytes, x + row_of(idx) * cols, row_bytes, &ctl.full[group][sl]);
  };
  int issued = 0;
  if (t == 0)
    for (; issued < stages - 1 && issued < n_mine; ++issued) issue(issued);

  const bool has[2] = {t < nvec, t + kGroupThreads < nvec};
  int i = 0, par = 0;
  for (; i < n_mine; ++i) {
    const long long row = row_of(i);
    if (t == 0 && issued < n_mine) issue(issued++);  // refills the slot that iteration i - 1 read
    if (!ring_wait(&ctl, group, i, stages)) break;
    const T* src = reinterpret_cast<const T*>(my_ring + (i % stages) * row_bytes);
    float2 v[2][4];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (has[k]) {
        unpack_pairs<T>(V8<T>::ld(src + (t + k * kGroupThreads) * 8), v[k]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[k][e] = f2s(0.f);
      }
    }
    float c = V8<T>::ld1(src);
    if (pre_act == FB_ACT_GELU) {
      c = gelu_f<kFast>(c);
#pragma unroll
      for (int k = 0; k < 2; ++k)
#pragma unroll
        for (int e = 0; e < 4; ++e) v[k][e] = f2(gelu_f<kFast>(v[k][e].x), gelu_f<kFast>(v[k][e].y));
    }
    const float2 nc = f2s(-c);
    float2 s2 = f2s(0.f), q2 = f2s(0.f);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (has[k]) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 d = __fadd2_rn(v[k][e], nc);
          s2 = __fadd2_rn(s2, d);
          q2 = __ffma2_rn(d, d, q2);
        }
      }
    }
    float s = s2.x + s2.y, q = q2.x + q2.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      q += __shfl_xor_sync(0xffffffffu, q, o);
    }
    if (lane == 0) red[group][par][warp] = make_float2(s, q);
    group_sync(group);
    const float2 tot = fold8(red[group][par], lane);
    par ^= 1;
    const float ms = tot.x * inv_n;                       // mean of (x - c)
    const float var = fmaxf(tot.y * inv_n - ms * ms, 0.f);
    const float mu = c + ms;
    const float rs = rsqrtf(var + eps);
    if (t == 0) {
      if (mean_out) mean_out[row] = mu;
      if (rstd_out) rstd_out[row] = rs;
    }
    const float2 rs2 = f2s(rs), shift2 = f2s(-mu * rs);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int vi = t + k * kGroupThreads;
      if (has[k]) {
        float2 g[4], b[4], o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          g[e] = f2s(1.f);
          b[e] = f2s(0.f);
        }
        if (gamma) ld_pairs_f32(gamma + vi * 8, g);
        if (beta) ld_pairs_f32(beta + vi * 8, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = __ffma2_rn(__ffma2_rn(v[k][e], rs2, shift2), g[e], b[e]);
        store_pairs<T>(y + row * cols + vi * 8, o);
      }
    }
  }
  if (i < n_mine && t == 0) {  // a wait gave up
    report_status(status, kStatusGemmTimeout, 31, blockIdx.x, i);
    ring_drain(&ctl, group, issued, i, stages);
  }
}

// Backward with the activation derivative (if any) given as a tensor: bf16, up to 4096 columns.  A slot
// holds the dy, x and act_grad rows; gamma and the three column accumulators stay in registers; mean / rstd
// of a group's rows are cached in shared memory up front; a row costs one group barrier.  Column partials:
// one row of partial[] per GROUP (2 * gridDim.x rows in all).
__global__ void __launch_bounds__(kRingThreads, 1)
ln_bwd_ring_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ act_grad, const float* __restrict__ gamma,
                   const float* __restrict__ mean, const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ partial, long long rows, int cols, int want_colsum, int stages,
                   int32_t* status) {
  using V = V8<__nv_bfloat16>;
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ RingCtl ctl;
  __shared__ float2 red[2][2][8];
  __shared__ float2 stat[2][kStatRows];
  const int group = threadIdx.x >> 8, t = threadIdx.x & 255, lane = t & 31, warp = t >> 5;
  const int nvec = cols >> 3;
  const bool use_ag = act_grad != nullptr;
  const uint32_t row_bytes = static_cast<uint32_t>(cols) * 2u;
  const uint32_t slot_bytes = row_bytes * (use_ag ? 3u : 2u);
  uint8_t* my_ring = ring + group * stages * slot_bytes;
  const float inv_n = 1.f / static_cast<float>(cols);
  const long long first = blockIdx.x, stride = gridDim.x;
  const long long n_block = first < rows ? (rows - first + stride - 1) / stride : 0;
  const int n_mine = static_cast<int>((n_block - group + 1) / 2);
  auto row_of = [&](int i) { return first + (2LL * i + group) * stride; };

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    for (int g = 0; g < 2; ++g)
      for (int s = 0; s < stages; ++s) ptx::mbar_init(&ctl.full[g][s], 1);
    ptx::fence_mbar_init();
  }
  for (int r = t; r < n_mine && r < kStatRows; r += kGroupThreads)
    stat[group][r] = make_float2(mean[row_of(r)], rstd[row_of(r)]);
  __syncthreads();
  auto issue = [&](int idx) {
    const int sl = idx % stages;
    uint8_t* dst = my_ring + sl * slot_bytes;
    const long long off = row_of(idx) * cols;
    ptx::mbar_arrive_expect_tx(&ctl.full[group][sl], slot_bytes);
    ptx::bulk_load_1d(dst, dy + off, row_bytes, &ctl.full[group][sl]);
    ptx::bulk_load_1d(dst + row_bytes, x + off, row_bytes, &ctl.full[group][sl]);
    if (use_ag) ptx::bulk_load_1d(dst + 2 * row_bytes, act_grad + off, row_bytes, &ctl.full[group][sl]);
  };
  int issued = 0;
  if (t == 0)
    for (; issued < stages - 1 && issued < n_mine; ++issued) issue(issued);

  const bool has[2] = {t < nvec, t + kGroupThreads < nvec};
  float2 w[2][4], acc_g[2][4], acc_b[2][4], acc_c[2][4];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      w[k][e] = f2s(1.f);
      acc_g[k][e] = acc_b[k][e] = acc_c[k][e] = f2s(0.f);
    }
    if (has[k] && gamma != nullptr) ld_pairs_f32(gamma + (t + k * kGroupThreads) * 8, w[k]);
  }

  int i = 0, par = 0;
  for (; i < n_mine; ++i) {
    const long long row = row_of(i);
    if (t == 0 && issued < n_mine) issue(issued++);  // refills the slot that iteration i - 1 read
    if (!ring_wait(&ctl, group, i, stages)) break;
    const float2 st = i < kStatRows ? stat[group][i] : make_float2(mean[row], rstd[row]);
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(my_ring + (i % stages) * slot_bytes);
    float2 d[2][4], h[2][4];
    const float2 rs2 = f2s(st.y), shift2 = f2s(-st.x * st.y);
    float2 s1 = f2s(0.f), s2 = f2s(0.f);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (has[k]) {
        const int vi = t + k * kGroupThreads;
        unpack_pairs<__nv_bfloat16>(V::ld(src + vi * 8), d[k]);
        unpack_pairs<__nv_bfloat16>(V::ld(src + cols + vi * 8), h[k]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          h[k][e] = __ffma2_rn(h[k][e], rs2, shift2);
          acc_b[k][e] = __fadd2_rn(acc_b[k][e], d[k][e]);
          acc_g[k][e] = __ffma2_rn(d[k][e], h[k][e], acc_g[k][e]);
          d[k][e] = __fmul2_rn(d[k][e], w[k][e]);  // d = dy * gamma
          s1 = __fadd2_rn(s1, d[k][e]);
          s2 = __ffma2_rn(d[k][e], h[k][e], s2);
        }
      }
    }
    float a1 = s1.x + s1.y, a2 = s2.x + s2.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a1 += __shfl_xor_sync(0xffffffffu, a1, o);
      a2 += __shfl_xor_sync(0xffffffffu, a2, o);
    }
    if (lane == 0) red[group][par][warp] = make_float2(a1, a2);
    group_sync(group);
    const float2 tot = fold8(red[group][par], lane);
    par ^= 1;
    // o = rstd * (d - m1 - h m2) with rstd folded into the two means
    const float2 nm1 = f2s(-tot.x * inv_n * st.y), nm2 = f2s(-tot.y * inv_n * st.y);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (has[k]) {
        const int vi = t + k * kGroupThreads;
        float2 o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = __ffma2_rn(h[k][e], nm2, __ffma2_rn(d[k][e], rs2, nm1));
        if (use_ag) {
          float2 ag[4];
          unpack_pairs<__nv_bfloat16>(V::ld(src + 2 * cols + vi * 8), ag);
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] = __fmul2_rn(o[e], ag[e]);
        }
        if (want_colsum) {
#pragma unroll
          for (int e = 0; e < 4; ++e) acc_c[k][e] = __fadd2_rn(acc_c[k][e], o[e]);
        }
        store_pairs<__nv_bfloat16>(dx + row * cols + vi * 8, o);
      }
    }
  }
  if (i < n_mine && t == 0) {
    report_status(status, kStatusGemmTimeout, 32, blockIdx.x, i);
    ring_drain(&ctl, group, issued, i, stages);
  }
  float* base = partial + (2LL * blockIdx.x + group) * 3 * cols;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    if (has[k]) {
      float* pg = base + (t + k * kGroupThreads) * 8;
      float* pb = pg + cols;
      float* pc = pb + cols;
      *reinterpret_cast<float4*>(pg) = make_float4(acc_g[k][0].x, acc_g[k][0].y, acc_g[k][1].x, acc_g[k][1].y);
      *reinterpret_cast<float4*>(pg + 4) = make_float4(acc_g[k][2].x, acc_g[k][2].y, acc_g[k][3].x, acc_g[k][3].y);
      *reinterpret_cast<float4*>(pb) = make_float4(acc_b[k][0].x, acc_b[k][0].y, acc_b[k][1].x, acc_b[k][1].y);
      *reinterpret_cast<float4*>(pb + 4) = make_float4(acc_b[k][2].x, acc_b[k][2].y, acc_b[k][3].x, acc_b[k][3].y);
      *reinterpret_cast<float4*>(pc) = make_float4(acc_c[k][0].x, acc_c[k][0].y, acc_c[k][1].x, acc_c[k][1].y);
      *reinterpret_cast<float4*>(pc + 4) = make_float4(acc_c[k][2].x, acc_c[k][2].y, acc_c[k][3].x, acc_c[k][3].y);
    }
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

int32_t* g_ln_status = nullptr;  // host-mapped status block for the bounded waits of the ring kernels

// FERRUM_LN_RING=0 keeps wide rows on the register-tiled kernels (for A/B measurements).
bool ring_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("FERRUM_LN_RING");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <typename T, int TPR, int K>
void launch_fwd(const T* xp, const float* gamma, const float* beta, T* yp, float* mean, float* rstd, long long rows,
                int cols, float eps, int pre_act, long long nb, cudaStream_t st) {
  const int grid = static_cast<int>(nb < sm_count() * 8LL ? nb : sm_count() * 8LL);
  ln_fwd_kernel<T, TPR, K><<<grid, 256, 0, st>>>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps, pre_act);
}

int env_int(const char* name, int dflt) {
  const char* e = getenv(name);
  return e != nullptr ? atoi(e) : dflt;
}

// Stages per group for slots of `slot_bytes`: as many as fit in `budget` bytes for the two groups of a block,
// at most kMaxRingStages.
int ring_stages(size_t slot_bytes, size_t budget) {
  size_t fit = budget / (2 * slot_bytes);
  static const int forced = env_int("FERRUM_LN_STAGES", 0);  // measurement knob
  if (forced >= 2 && static_cast<size_t>(forced) < fit) fit = forced;
  return static_cast<int>(fit > kMaxRingStages ? kMaxRingStages : fit);
}

// Warp-per-row forward: bf16 rows of 1024 .. 4096 columns without a fused activation (FERRUM_LN_WARP_FWD=0 = off).
template <typename T>
bool launch_fwd_warp(const T*, const float*, const float*, T*, float*, float*, long long, int, float, int,
                     cudaStream_t) {
  return false;
}
template <>
bool launch_fwd_warp<__nv_bfloat16>(const __nv_bfloat16* xp, const float* gamma, const float* beta,
                                    __nv_bfloat16* yp, float* mean, float* rstd, long long rows, int cols, float eps,
                                    int pre_act, cudaStream_t st) {
  static const int enabled = env_int("FERRUM_LN_WARP_FWD", 1);
  if (!enabled || pre_act != FB_ACT_NONE || cols < 1024 || cols > 4096) return false;
  const int k = (cols / 8 + 31) / 32;
  const long long want = (rows + 7) / 8;  // eight warps per block
  const long long cap = static_cast<long long>(sm_count()) * 2;
  const int grid = static_cast<int>(want < cap ? want : cap);
  if (k <= 4)
    ln_fwd_warp_kernel<4><<<grid, 256, 0, st>>>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps);
  else if (k <= 8)
    ln_fwd_warp_kernel<8><<<grid, 256, 0, st>>>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps);
  else
    ln_fwd_warp_kernel<16><<<grid, 256, 0, st>>>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps);
  return true;
}

// Ring kernel for rows of at least 2 KB and at most 4096 columns; false if it cannot be launched.
template <typename T>
bool launch_fwd_ring(const T* xp, const float* gamma, const float* beta, T* yp, float* mean, float* rstd,
                     long long rows, int cols, float eps, int pre_act, cudaStream_t st) {
  // 2-byte rows run two blocks per SM (register budget of the kernel), so each gets half of the shared memory
  constexpr int kBlocksPerSm = sizeof(T) == 2 ? 2 : 1;
  const int stages = ring_stages(static_cast<size_t>(cols) * sizeof(T), (200u * 1024u) / kBlocksPerSm);
  if (stages < 2) return false;
  const size_t smem = static_cast<size_t>(2 * stages) * cols * sizeof(T);
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(ln_fwd_ring_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    configured = smem;
  }
  const long long want = (rows + 1) / 2;  // a block needs two rows to keep both groups busy
  const long long cap = static_cast<long long>(sm_count()) * kBlocksPerSm;
  const int grid = static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
  ln_fwd_ring_kernel<T><<<grid, kRingThreads, smem, st>>>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps, pre_act,
                                                         stages, g_ln_status);
  return true;
}

template <typename T>
int fwd_t(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, long long rows,
          int cols, float eps, int pre_act, cudaStream_t st) {
  const T* xp = static_cast<const T*>(x);
  T* yp = static_cast<T*>(y);
  Geo g;
  if (geometry(cols, &g) && aligned16(x, y, gamma, beta)) {
    const int nvec = cols / 8;
    if (launch_fwd_warp<T>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps, pre_act, st))
      return static_cast<int>(cudaGetLastError());
    static const int ring_fwd = env_int("FERRUM_LN_RING_FWD", 0);
    if (ring_fwd && ring_enabled() && static_cast<size_t>(cols) * sizeof(T) >= 2048 && nvec <= 2 * kGroupThreads &&
        launch_fwd_ring<T>(xp, gamma, beta, yp, mean, rstd, rows, cols, eps, pre_act, st))
      return static_cast<int>(cudaGetLastError());
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
// bf16 rows of 2 KB .. 8 KB with no activation to re-evaluate: the ring kernel, one block per SM.
template <>
bool launch_wide<__nv_bfloat16>(const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* ag,
                                const float* gamma, const float* mean, const float* rstd, __nv_bfloat16* dx,
                                float* partial, long long rows, int cols, int blocks, int want_colsum,
                                cudaStream_t st) {
  const int stages = ring_stages(static_cast<size_t>(cols) * 2 * (ag != nullptr ? 3 : 2), 200u * 1024u);
  if (stages < 2) return false;
  const size_t smem = static_cast<size_t>(2 * stages) * (ag != nullptr ? 3 : 2) * cols * 2;
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(ln_bwd_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    configured = smem;
  }
  ln_bwd_ring_kernel<<<blocks, kRingThreads, smem, st>>>(dy, x, ag, gamma, mean, rstd, dx, partial, rows, cols,
                                                         want_colsum, stages, g_ln_status);
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
    const int wide_blocks = nblk / 2 < sm_count() ? nblk / 2 : sm_count();  // two rows of partial[] per block
    if (ring_enabled() && pre_act == FB_ACT_NONE && cols * 2 >= 2048 && nvec <= 2 * kGroupThreads &&
        wide_blocks >= 1 &&
        launch_wide<T>(dyp, xp, agp, gamma, mean, rstd, dxp, partial, rows, cols, wide_blocks, want_colsum, st)) {
      used = 2 * wide_blocks;
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

// Status block (host-mapped, see common/status.h) that the bounded waits of the wide-row kernels report to.
extern "C" void fb_layernorm_set_status(int32_t* status) { g_ln_status = status; }

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
