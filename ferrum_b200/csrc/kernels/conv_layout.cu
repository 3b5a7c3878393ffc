// Layout changes around the implicit-GEMM convolution (csrc/gemm/tcgen05_gemm.cu, fb_conv_igemm): the reference
// keeps activations as NCHW fp32 (ferrum-nn/src/conv.rs:209-330); the tensor-core kernels read NHWC bf16 through
// 4-D TMA boxes, with the channel count padded to a multiple of 8 so that every pixel starts on a 16-byte boundary.
//
//   fb_nchw_to_nhwc_bf16   [B, C, P] fp32 -> [B, P, Cp] bf16   (P = H * W; channels C .. Cp - 1 are written as zero)
//   fb_nhwc_to_nchw_f32    [B, P, ld] fp32 (first C of ld channels) -> [B, C, P] fp32
//
//   fb_nchw_to_s2d_nhwc_bf16  strided convolutions: [B, C, H, W] fp32 -> space-to-depth NHWC bf16
//                             z[b, I, J, (rh * sw + rw) * C + c] = x[b, c, I * sh + rh - ph, J * sw + rw - pw]
//                             (zero outside the image), which turns a stride-(sh, sw) convolution with a kh x kw
//                             filter into a stride-1 one with a ceil(kh / sh) x ceil(kw / sw) filter over sh * sw * C
//                             channels, i.e. into the implicit-GEMM kernel's case
//   fb_s2d_nhwc_to_nchw_f32   the inverse, for the data gradient: [B, Hz, Wz, ld] fp32 -> [B, C, H, W] fp32
//
// All are 32 x 32 tile transposes through shared memory: coalesced reads along P (NCHW) or C (NHWC), coalesced
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

// Space-to-depth geometry shared by the two strided-convolution layout kernels.
struct S2d {
  int C, H, W, sh, sw, ph, pw, Hz, Wz;
  long long ld;  // channels per pixel of the NHWC side (>= sh * sw * C)
};

// Block = image row (b, i) x 32 columns x 32 channels of the NCHW side.
__global__ void __launch_bounds__(256)
nchw_to_s2d_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ z, const S2d g) {
  __shared__ float tile[32][33];
  const long long bi = blockIdx.x;
  const long long b = bi / g.H;
  const int i = static_cast<int>(bi - b * g.H);
  const int I = (i + g.ph) / g.sh, rh = (i + g.ph) % g.sh;
  if (I >= g.Hz) return;  // a row no window reaches (uniform over the block)
  const int j0 = blockIdx.y * 32, c0 = blockIdx.z * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const float* xr = x + (b * g.C * g.H + i) * static_cast<long long>(g.W);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = c0 + ty + 8 * k, j = j0 + tx;
    tile[ty + 8 * k][tx] = (c < g.C && j < g.W) ? xr[static_cast<long long>(c) * g.H * g.W + j] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int j = j0 + ty + 8 * k, c = c0 + tx;
    if (j >= g.W || c >= g.C) continue;
    const int J = (j + g.pw) / g.sw, rw = (j + g.pw) % g.sw;
    if (J >= g.Wz) continue;
    z[((b * g.Hz + I) * g.Wz + J) * g.ld + static_cast<long long>(rh * g.sw + rw) * g.C + c] =
        __float2bfloat16_rn(tile[tx][ty + 8 * k]);
  }
}

__global__ void __launch_bounds__(256)
s2d_to_nchw_kernel(const float* __restrict__ z, float* __restrict__ x, const S2d g) {
  __shared__ float tile[32][33];
  const long long bi = blockIdx.x;
  const long long b = bi / g.H;
  const int i = static_cast<int>(bi - b * g.H);
  const int I = (i + g.ph) / g.sh, rh = (i + g.ph) % g.sh;
  const int j0 = blockIdx.y * 32, c0 = blockIdx.z * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int j = j0 + ty + 8 * k, c = c0 + tx;
    float v = 0.f;
    if (I < g.Hz && j < g.W && c < g.C) {
      const int J = (j + g.pw) / g.sw, rw = (j + g.pw) % g.sw;
      if (J < g.Wz) v = z[((b * g.Hz + I) * g.Wz + J) * g.ld + static_cast<long long>(rh * g.sw + rw) * g.C + c];
    }
    tile[ty + 8 * k][tx] = v;
  }
  __syncthreads();
  float* xr = x + (b * g.C * g.H + i) * static_cast<long long>(g.W);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = c0 + ty + 8 * k, j = j0 + tx;
    if (c < g.C && j < g.W) xr[static_cast<long long>(c) * g.H * g.W + j] = tile[tx][ty + 8 * k];
  }
}

bool s2d_ok(int B, const S2d& g) {
  return B > 0 && g.C > 0 && g.H > 0 && g.W > 0 && g.sh > 0 && g.sw > 0 && g.ph >= 0 && g.pw >= 0 && g.Hz > 0 &&
         g.Wz > 0 && g.ld >= static_cast<long long>(g.sh) * g.sw * g.C && static_cast<long long>(B) * g.H < 0x7fffffffll &&
         (g.W + 31) / 32 <= 65535 && (g.C + 31) / 32 <= 65535;
}

}  // namespace
}  // namespace fb

// z (bf16, [B, Hz, Wz, ld]) is zeroed first: pixels outside the image and channels sh * sw * C .. ld - 1 stay zero.
extern "C" int fb_nchw_to_s2d_nhwc_bf16(const float* x, void* z, int B, int C, int H, int W, int sh, int sw, int ph,
                                        int pw, int Hz, int Wz, long long ld, cudaStream_t stream) {
  const fb::S2d g{C, H, W, sh, sw, ph, pw, Hz, Wz, ld};
  if (!fb::s2d_ok(B, g)) return -1;
  cudaError_t e = cudaMemsetAsync(z, 0, static_cast<size_t>(B) * Hz * Wz * ld * 2, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(static_cast<unsigned>(B) * H, static_cast<unsigned>((W + 31) / 32), static_cast<unsigned>((C + 31) / 32));
  fb::nchw_to_s2d_kernel<<<grid, 256, 0, stream>>>(x, static_cast<__nv_bfloat16*>(z), g);
  return static_cast<int>(cudaGetLastError());
}

// x[b, c, i, j] = z[b, (i + ph) / sh, (j + pw) / sw, (((i + ph) % sh) * sw + (j + pw) % sw) * C + c], zero where no
// window reaches.
extern "C" int fb_s2d_nhwc_to_nchw_f32(const float* z, float* x, int B, int C, int H, int W, int sh, int sw, int ph,
                                       int pw, int Hz, int Wz, long long ld, cudaStream_t stream) {
  const fb::S2d g{C, H, W, sh, sw, ph, pw, Hz, Wz, ld};
  if (!fb::s2d_ok(B, g)) return -1;
  dim3 grid(static_cast<unsigned>(B) * H, static_cast<unsigned>((W + 31) / 32), static_cast<unsigned>((C + 31) / 32));
  fb::s2d_to_nchw_kernel<<<grid, 256, 0, stream>>>(z, x, g);
  return static_cast<int>(cudaGetLastError());
}

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
