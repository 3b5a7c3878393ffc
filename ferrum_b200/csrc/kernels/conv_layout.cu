// Layout changes around the implicit-GEMM convolution (csrc/gemm/tcgen05_gemm.cu, fb_conv_igemm): the reference
// keeps activations as NCHW fp32 (ferrum-nn/src/conv.rs:209-330); the tensor-core kernels read NHWC bf16 through
// 4-D TMA boxes, with the channel count padded to a multiple of 8 so that every pixel starts on a 16-byte boundary.
//
//   fb_nchw_to_nhwc_bf16   [B, C, P] fp32 -> [B, P, Cp] bf16   (P = H * W; channels C .. Cp - 1 are written as zero)
//   fb_nhwc_to_nchw_f32    [B, P, ld] fp32 (first C of ld channels) -> [B, C, P] fp32
//
// Both are 32 x 32 tile transposes through shared memory: coalesced reads along P (NCHW) or C (NHWC), coalesced
// writes along the other.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

__global__ void __launch_bounds__(256)
nchw_to_nhwc_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, int C, long long P, int Cp) {
  __shared__ float tile[32][33];
  const long long b = blockIdx.z;
  const long long p0 = static_cast<long long>(blockIdx.x) * 32;
  const int c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const float* xb = x + b * C * P;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + 8 * i;
    const long long p = p0 + tx;
    tile[ty + 8 * i][tx] = (c < C && p < P) ? xb[c * P + p] : 0.f;
  }
  __syncthreads();
  __nv_bfloat16* yb = y + b * P * Cp;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long p = p0 + ty + 8 * i;
    const int c = c0 + tx;
    if (p < P && c < Cp) yb[p * Cp + c] = __float2bfloat16_rn(tile[tx][ty + 8 * i]);
  }
}

__global__ void __launch_bounds__(256)
nhwc_to_nchw_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int C, long long P, long long ld) {
  __shared__ float tile[32][33];
  const long long b = blockIdx.z;
  const long long p0 = static_cast<long long>(blockIdx.x) * 32;
  const int c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const float* xb = x + b * P * ld;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long p = p0 + ty + 8 * i;
    const int c = c0 + tx;
    tile[ty + 8 * i][tx] = (p < P && c < C) ? xb[p * ld + c] : 0.f;
  }
  __syncthreads();
  float* yb = y + b * C * P;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + 8 * i;
    const long long p = p0 + tx;
    if (c < C && p < P) yb[c * P + p] = tile[tx][ty + 8 * i];
  }
}

}  // namespace
}  // namespace fb

extern "C" int fb_nchw_to_nhwc_bf16(const float* x, void* y, int B, int C, long long P, int Cp, cudaStream_t stream) {
  if (B <= 0 || C <= 0 || P <= 0 || Cp < C || B > 65535 || (Cp + 31) / 32 > 65535) return -1;
  dim3 grid(static_cast<unsigned>((P + 31) / 32), static_cast<unsigned>((Cp + 31) / 32), static_cast<unsigned>(B));
  fb::nchw_to_nhwc_bf16_kernel<<<grid, 256, 0, stream>>>(x, static_cast<__nv_bfloat16*>(y), C, P, Cp);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_nhwc_to_nchw_f32(const float* x, float* y, int B, int C, long long P, long long ld,
                                   cudaStream_t stream) {
  if (B <= 0 || C <= 0 || P <= 0 || ld < C || B > 65535 || (C + 31) / 32 > 65535) return -1;
  dim3 grid(static_cast<unsigned>((P + 31) / 32), static_cast<unsigned>((C + 31) / 32), static_cast<unsigned>(B));
  fb::nhwc_to_nchw_f32_kernel<<<grid, 256, 0, stream>>>(x, y, C, P, ld);
  return static_cast<int>(cudaGetLastError());
}
