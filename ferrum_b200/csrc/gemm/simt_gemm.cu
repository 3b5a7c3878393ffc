// fp32 SIMT GEMM with arbitrary element strides, optional batch, bias,
// activation and accumulate.  It is the exact-fp32 path for parity runs and
// for shapes the TMA-fed tensor-core kernel cannot take (row pitch not a
// multiple of 16 bytes, 1-D operands), and the on-device oracle for it.
// Same contract as the reference's matmul_2d (ferrum-core/src/tensor.rs:2487-2558)
// and bmm (ferrum-ops/src/matmul.rs:176-178).
#include <cuda_runtime.h>

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

}  // namespace
}  // namespace fb

extern "C" int fb_gemm_f32_simt(const float* a, const float* b, float* out, const float* bias, int M, int N, int K,
                                long long sam, long long sak, long long sbk, long long sbn, long long ldc, int act,
                                int beta, int batch, long long bsa, long long bsb, long long bsc,
                                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return -1;
  dim3 grid((N + fb::kTile - 1) / fb::kTile, (M + fb::kTile - 1) / fb::kTile, batch);
  fb::gemm_f32_kernel<<<grid, 256, 0, stream>>>(a, b, out, bias, M, N, K, sam, sak, sbk, sbn, ldc, act, beta, bsa,
                                                bsb, bsc);
  return static_cast<int>(cudaGetLastError());
}
