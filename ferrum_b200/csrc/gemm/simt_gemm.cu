// fp32 SIMT GEMM with arbitrary element strides, optional batch, bias,
// activation and accumulate.  It is the exact-fp32 path for parity runs and
// for shapes the TMA-fed tensor-core kernel cannot take (row pitch not a
// multiple of 16 bytes, 1-D operands), and the on-device oracle for it.
// Same contract as the reference's matmul_2d (ferrum-core/src/tensor.rs:2487-2558)
// and bmm (ferrum-ops/src/matmul.rs:176-178).
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>

#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

constexpr int kTile = 64;
constexpr int kTk = 16;

__device__ __forceinline__ float act_f32(float x, int act) {
  switch (act) {
    case FB_ACT_RELU:
      return fmaxf(x, 0.f);
    case FB_ACT_GELU: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    case FB_ACT_SILU:
      return x / (1.f + expf(-x));
    case FB_ACT_TANH:
      return tanhf(x);
    case FB_ACT_SIGMOID:
      return 1.f / (1.f + expf(-x));
    default:
      return x;
  }
}

// 256 threads, each computes a 4x4 micro-tile of a 64x64 output tile.
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                const float* __restrict__ bias, int M, int N, int K, long long sam, long long sak, long long sbk,
                long long sbn, long long ldc, int act, int beta, long long bsa, long long bsb, long long bsc) {
  __shared__ float As[kTk][kTile + 1];
  __shared__ float Bs[kTk][kTile + 1];
  a += blockIdx.z * bsa;
  b += blockIdx.z * bsb;
  out += blockIdx.z * bsc;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += kTk) {
    for (int i = threadIdx.x; i < kTile * kTk; i += 256) {
      // Pick the loop order that follows the contiguous dimension of each operand.
      int mm, kk;
      if (sak == 1) {
        kk = i % kTk;
        mm = i / kTk;
      } else {
        mm = i % kTile;
        kk = i / kTile;
      }
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? a[gm * sam + gk * sak] : 0.f;
      int nn, kb;
      if (sbk == 1) {
        kb = i % kTk;
        nn = i / kTk;
      } else {
        nn = i % kTile;
        kb = i / kTile;
      }
      const int gn = n0 + nn, gkb = k0 + kb;
      Bs[kb][nn] = (gn < N && gkb < K) ? b[gkb * sbk + gn * sbn] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTk; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += bias[gn];
      v = act_f32(v, act);
      float* o = out + static_cast<long long>(gm) * ldc + gn;
      *o = beta ? (*o + v) : v;
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Fast path for regular operands (each operand has a unit stride in one of its two dimensions, 16-byte aligned
// base and pitch): 128 x 128 x 16 tiles, 256 threads, an 8 x 8 register tile per thread held as four 4 x 4 blocks
// (rows ty*4 and 64 + ty*4, columns tx*4 and 64 + tx*4, so a warp's shared-memory reads are conflict-free
// 16-byte broadcasts), shared memory double-buffered, the next k-slice fetched from global memory into registers
// while the current one is multiplied.  Shared memory holds both operands K-outer ([k][m], [k][n]) whatever
// their layout in global memory: an MN-contiguous operand is copied with 16-byte loads and stores, a
// K-contiguous one is loaded 16 bytes along K and scattered.
constexpr int kFT = 128;   // tile edge
constexpr int kFK = 16;    // k-slice

template <bool kAContigK, bool kBContigK>
__global__ void __launch_bounds__(256)
gemm_f32_fast_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                     const float* __restrict__ bias, int M, int N, int K, long long lda, long long ldb,
                     long long ldc, int act, int beta, long long bsa, long long bsb, long long bsc) {
  __shared__ __align__(16) float As[2][kFK][kFT];
  __shared__ __align__(16) float Bs[2][kFK][kFT];
  a += blockIdx.z * bsa;
  b += blockIdx.z * bsb;
  out += blockIdx.z * bsc;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * kFT, n0 = blockIdx.x * kFT;

  // Each thread moves two 16-byte pieces of each operand per k-slice.
  //   K-contiguous operand [rows][K]: piece = 4 consecutive k of one row      -> row = id / 4, k = (id % 4) * 4
  //   MN-contiguous operand [K][rows]: piece = 4 consecutive rows of one k    -> k = id / 32, row = (id % 32) * 4
  float4 ra[2], rb[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int id = tid + h * 256;
      if (kAContigK) {
        const int r = id >> 2, kk = (id & 3) << 2;
        const int gm = m0 + r, gk = k0 + kk;
        const float* p = a + static_cast<long long>(gm) * lda + gk;
        if (gm < M && gk + 3 < K) ra[h] = *reinterpret_cast<const float4*>(p);
        else {
          ra[h] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gm < M) {
            if (gk < K) ra[h].x = p[0];
            if (gk + 1 < K) ra[h].y = p[1];
            if (gk + 2 < K) ra[h].z = p[2];
          }
        }
      } else {
        const int kk = id >> 5, r = (id & 31) << 2;
        const int gm = m0 + r, gk = k0 + kk;
        const float* p = a + static_cast<long long>(gk) * lda + gm;
        if (gk < K && gm + 3 < M) ra[h] = *reinterpret_cast<const float4*>(p);
        else {
          ra[h] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gk < K) {
            if (gm < M) ra[h].x = p[0];
            if (gm + 1 < M) ra[h].y = p[1];
            if (gm + 2 < M) ra[h].z = p[2];
          }
        }
      }
      if (kBContigK) {
        const int r = id >> 2, kk = (id & 3) << 2;
        const int gn = n0 + r, gk = k0 + kk;
        const float* p = b + static_cast<long long>(gn) * ldb + gk;
        if (gn < N && gk + 3 < K) rb[h] = *reinterpret_cast<const float4*>(p);
        else {
          rb[h] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gn < N) {
            if (gk < K) rb[h].x = p[0];
            if (gk + 1 < K) rb[h].y = p[1];
            if (gk + 2 < K) rb[h].z = p[2];
          }
        }
      } else {
        const int kk = id >> 5, r = (id & 31) << 2;
        const int gn = n0 + r, gk = k0 + kk;
        const float* p = b + static_cast<long long>(gk) * ldb + gn;
        if (gk < K && gn + 3 < N) rb[h] = *reinterpret_cast<const float4*>(p);
        else {
          rb[h] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gk < K) {
            if (gn < N) rb[h].x = p[0];
            if (gn + 1 < N) rb[h].y = p[1];
            if (gn + 2 < N) rb[h].z = p[2];
          }
        }
      }
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int id = tid + h * 256;
      if (kAContigK) {
        const int r = id >> 2, kk = (id & 3) << 2;
        As[buf][kk][r] = ra[h].x; As[buf][kk + 1][r] = ra[h].y; As[buf][kk + 2][r] = ra[h].z; As[buf][kk + 3][r] = ra[h].w;
      } else {
        const int kk = id >> 5, r = (id & 31) << 2;
        *reinterpret_cast<float4*>(&As[buf][kk][r]) = ra[h];
      }
      if (kBContigK) {
        const int r = id >> 2, kk = (id & 3) << 2;
        Bs[buf][kk][r] = rb[h].x; Bs[buf][kk + 1][r] = rb[h].y; Bs[buf][kk + 2][r] = rb[h].z; Bs[buf][kk + 3][r] = rb[h].w;
      } else {
        const int kk = id >> 5, r = (id & 31) << 2;
        *reinterpret_cast<float4*>(&Bs[buf][kk][r]) = rb[h];
      }
    }
  };

  float acc[8][8] = {};
  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += kFK) {
    const bool more = k0 + kFK < K;
    if (more) fetch(k0 + kFK);  // in flight while this slice is multiplied
#pragma unroll
    for (int kk = 0; kk < kFK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (more) {
      stash(buf ^ 1);  // the other buffer was last read before the previous barrier
      __syncthreads();
      buf ^= 1;
    }
  }

  const bool vec_out = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (gm >= M) continue;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int gn = n0 + jh * 64 + tx * 4;
      if (gn >= N) continue;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[j] = acc[i][jh * 4 + j];
        if (bias != nullptr && gn + j < N) v[j] += bias[gn + j];
        v[j] = act_f32(v[j], act);
      }
      float* o = out + static_cast<long long>(gm) * ldc + gn;
      if (vec_out && gn + 3 < N) {
        float4 x = make_float4(v[0], v[1], v[2], v[3]);
        if (beta) {
          const float4 old = *reinterpret_cast<const float4*>(o);
          x.x += old.x; x.y += old.y; x.z += old.z; x.w += old.w;
        }
        *reinterpret_cast<float4*>(o) = x;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (gn + j < N) o[j] = beta ? o[j] + v[j] : v[j];
      }
    }
  }
}

}  // namespace
}  // namespace fb

extern "C" int fb_gemm_f32_simt(const float* a, const float* b, float* out, const float* bias, int M, int N, int K,
                                long long sam, long long sak, long long sbk, long long sbn, long long ldc, int act,
                                int beta, int batch, long long bsa, long long bsb, long long bsc,
                                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return -1;
  {
    // fast path: every operand contiguous along K or along its M / N dimension, 16-byte aligned base, pitch and
    // batch stride; worth it from one full tile up
    const bool a_k = sak == 1, a_m = sam == 1 && !a_k;
    const bool b_k = sbk == 1, b_n = sbn == 1 && !b_k;
    const long long lda = a_k ? sam : sak, ldb = b_k ? sbn : sbk;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    static int fast_off = -1;
    if (fast_off < 0) {
      const char* e = getenv("FERRUM_SIMT_FAST");
      fast_off = (e != nullptr && e[0] == '0') ? 1 : 0;
    }
    if (!fast_off && (a_k || a_m) && (b_k || b_n) && lda % 4 == 0 && ldb % 4 == 0 && al(a) && al(b) &&
        bsa % 4 == 0 && bsb % 4 == 0 && M >= 64 && N >= 64 && K >= 16 && lda > 0 && ldb > 0) {
      dim3 grid((N + fb::kFT - 1) / fb::kFT, (M + fb::kFT - 1) / fb::kFT, batch);
      if (a_k && b_k)
        fb::gemm_f32_fast_kernel<true, true><<<grid, 256, 0, stream>>>(a, b, out, bias, M, N, K, lda, ldb, ldc, act,
                                                                       beta, bsa, bsb, bsc);
      else if (a_k)
        fb::gemm_f32_fast_kernel<true, false><<<grid, 256, 0, stream>>>(a, b, out, bias, M, N, K, lda, ldb, ldc,
                                                                        act, beta, bsa, bsb, bsc);
      else if (b_k)
        fb::gemm_f32_fast_kernel<false, true><<<grid, 256, 0, stream>>>(a, b, out, bias, M, N, K, lda, ldb, ldc,
                                                                        act, beta, bsa, bsb, bsc);
      else
        fb::gemm_f32_fast_kernel<false, false><<<grid, 256, 0, stream>>>(a, b, out, bias, M, N, K, lda, ldb, ldc,
                                                                         act, beta, bsa, bsb, bsc);
      return static_cast<int>(cudaGetLastError());
    }
  }
  dim3 grid((N + fb::kTile - 1) / fb::kTile, (M + fb::kTile - 1) / fb::kTile, batch);
  fb::gemm_f32_kernel<<<grid, 256, 0, stream>>>(a, b, out, bias, M, N, K, sam, sak, sbk, sbn, ldc, act, beta, bsa,
                                                bsb, bsc);
  return static_cast<int>(cudaGetLastError());
}
