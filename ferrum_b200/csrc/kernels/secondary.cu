// Kernels of the secondary layers: recurrent gate arithmetic, the im2col / col2im
// data movement that lowers convolution to GEMM, and 2-D pooling.
//
// Reference behaviour these replace (all forward-only host loops there):
//   ferrum-nn/src/rnn.rs:112-227   LSTM / GRU gate arithmetic on host vectors
//   ferrum-nn/src/conv.rs:209-330  direct 7-deep convolution loops
//   ferrum-nn/src/conv.rs:340-497  max / average / adaptive pooling loops
//
// The matrix products (input and hidden projections, the convolution itself) run
// on the GEMM kernels; what is left is bandwidth-bound elementwise work, fused here
// so that one recurrent step is two GEMMs plus ONE kernel each way instead of a
// dozen elementwise launches, and so that the convolution's window matrix is
// written directly in the K-major layout that the GEMM's TMA loads expect.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

inline int grid_for(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  return static_cast<int>(b > 148LL * 16 ? 148LL * 16 : (b < 1 ? 1 : b));
}

// ------------------------------------------------------------------ LSTM
// pre = xi + hh, laid out [B, 4H] as (input, forget, cell, output) blocks of H.
// Saves the ACTIVATED gates (i, f, g, o) for the backward pass.
__global__ void lstm_gates_fwd_kernel(const float* __restrict__ xi, const float* __restrict__ hh,
                                      const float* __restrict__ c_prev, float* __restrict__ h_out,
                                      float* __restrict__ c_out, float* __restrict__ gates, long long B, int H) {
  const long long n = B * H;
  for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < n;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = e / H;
    const int j = static_cast<int>(e - b * H);
    const long long base = b * 4 * H + j;
    const float i = sigmoidf_(xi[base] + hh[base]);
    const float f = sigmoidf_(xi[base + H] + hh[base + H]);
    const float g = tanhf(xi[base + 2 * H] + hh[base + 2 * H]);
    const float o = sigmoidf_(xi[base + 3 * H] + hh[base + 3 * H]);
    const float c = f * c_prev[e] + i * g;
    c_out[e] = c;
    h_out[e] = o * tanhf(c);
    gates[base] = i;
    gates[base + H] = f;
    gates[base + 2 * H] = g;
    gates[base + 3 * H] = o;
  }
}

// d_pre [B, 4H] (gradient of xi and of hh alike) and d_c_prev from d_h, d_c.
__global__ void lstm_gates_bwd_kernel(const float* __restrict__ dh, const float* __restrict__ dc,
                                      const float* __restrict__ gates, const float* __restrict__ c_prev,
                                      const float* __restrict__ c_out, float* __restrict__ dpre,
                                      float* __restrict__ dc_prev, long long B, int H) {
  const long long n = B * H;
  for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < n;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = e / H;
    const int j = static_cast<int>(e - b * H);
    const long long base = b * 4 * H + j;
    const float i = gates[base], f = gates[base + H], g = gates[base + 2 * H], o = gates[base + 3 * H];
    const float tc = tanhf(c_out[e]);
    const float gh = dh != nullptr ? dh[e] : 0.f;
    const float gc = (dc != nullptr ? dc[e] : 0.f) + gh * o * (1.f - tc * tc);
    dpre[base] = gc * g * i * (1.f - i);
    dpre[base + H] = gc * c_prev[e] * f * (1.f - f);
    dpre[base + 2 * H] = gc * i * (1.f - g * g);
    dpre[base + 3 * H] = gh * tc * o * (1.f - o);
    dc_prev[e] = gc * f;
  }
}

// ------------------------------------------------------------------- GRU
// xi, hh: [B, 3H] as (reset, update, new).  h' = (1 - z) n + z h,  n = tanh(xn + r * hn).
// Saves r, z, n and hn ([B, 4H]) for the backward pass.
__global__ void gru_gates_fwd_kernel(const float* __restrict__ xi, const float* __restrict__ hh,
                                     const float* __restrict__ h_prev, float* __restrict__ h_out,
                                     float* __restrict__ saved, long long B, int H) {
  const long long n = B * H;
  for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < n;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = e / H;
    const int j = static_cast<int>(e - b * H);
    const long long b3 = b * 3 * H + j, b4 = b * 4 * H + j;
    const float r = sigmoidf_(xi[b3] + hh[b3]);
    const float z = sigmoidf_(xi[b3 + H] + hh[b3 + H]);
    const float hn = hh[b3 + 2 * H];
    const float nn = tanhf(xi[b3 + 2 * H] + r * hn);
    h_out[e] = (1.f - z) * nn + z * h_prev[e];
    saved[b4] = r;
    saved[b4 + H] = z;
    saved[b4 + 2 * H] = nn;
    saved[b4 + 3 * H] = hn;
  }
}

__global__ void gru_gates_bwd_kernel(const float* __restrict__ dh, const float* __restrict__ saved,
                                     const float* __restrict__ h_prev, float* __restrict__ dxi,
                                     float* __restrict__ dhh, float* __restrict__ dh_prev, long long B, int H) {
  const long long n = B * H;
  for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < n;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = e / H;
    const int j = static_cast<int>(e - b * H);
    const long long b3 = b * 3 * H + j, b4 = b * 4 * H + j;
    const float r = saved[b4], z = saved[b4 + H], nn = saved[b4 + 2 * H], hn = saved[b4 + 3 * H];
    const float g = dh[e];
    const float dn = g * (1.f - z) * (1.f - nn * nn);  // through tanh
    const float dz = g * (h_prev[e] - nn) * z * (1.f - z);
    const float dr = dn * hn * r * (1.f - r);
    dxi[b3] = dr;
    dxi[b3 + H] = dz;
    dxi[b3 + 2 * H] = dn;
    dhh[b3] = dr;
    dhh[b3 + H] = dz;
    dhh[b3 + 2 * H] = dn * r;
    dh_prev[e] = g * z;
  }
}

// ---------------------------------------------------------------- im2col
struct ConvGeom {
  int B, C, H, W, kh, kw, Ho, Wo, sh, sw, ph, pw, dh, dw;
};

// cols[(b * Ho*Wo + l), (c * kh*kw + ki * kw + kj)] = x[b, c, oh*sh - ph + ki*dh, ow*sw - pw + kj*dw] (0 outside):
// one row per output position, K = C*kh*kw contiguous — the A operand of the convolution GEMM, no transpose.
template <typename T>
__global__ void im2col_kernel(const float* __restrict__ x, T* __restrict__ cols, ConvGeom g, long long ldk) {
  const int Kc = g.C * g.kh * g.kw;
  const long long total = static_cast<long long>(g.B) * g.Ho * g.Wo * Kc;
  for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = e / Kc;
    const int k = static_cast<int>(e - row * Kc);
    const int kj = k % g.kw, ki = (k / g.kw) % g.kh, c = k / (g.kw * g.kh);
    const int ow = static_cast<int>(row % g.Wo), oh = static_cast<int>((row / g.Wo) % g.Ho);
    const int b = static_cast<int>(row / (static_cast<long long>(g.Wo) * g.Ho));
    const int ih = oh * g.sh - g.ph + ki * g.dh, iw = ow * g.sw - g.pw + kj * g.dw;
    float v = 0.f;
    if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) v = x[((static_cast<long long>(b) * g.C + c) * g.H + ih) * g.W + iw];
    if constexpr (sizeof(T) == 2)
      cols[row * ldk + k] = __float2bfloat16_rn(v);
    else
      cols[row * ldk + k] = v;
  }
}

// Same result, organised so that index arithmetic is paid once per row and once per four columns: a warp owns one
// output position (row of the window matrix), decomposes it into (b, oh, ow) once, and its lanes walk the K columns
// in groups of four — (c, ki, kj) of the group's first column by two 32-bit divisions, the next three by
// increment-with-carry — and store 16 bytes (fp32) or 8 bytes (bf16) at a time.  The element-per-thread kernel above
// spends seven 64-bit divisions per element and reached 8 % of the memory rate; it remains for pitches or pointers
// that rule out vector stores.
template <typename T>
__global__ void __launch_bounds__(256)
im2col_rows_kernel(const float* __restrict__ x, T* __restrict__ cols, ConvGeom g, long long ldk, long long rows) {
  const int Kc = g.C * g.kh * g.kw;
  const int khw = g.kh * g.kw;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long plane = static_cast<long long>(g.H) * g.W;
  for (long long row = warp0; row < rows; row += nwarps) {
    const unsigned hw = static_cast<unsigned>(g.Ho) * g.Wo;
    const unsigned b = static_cast<unsigned>(row / hw);
    const unsigned l = static_cast<unsigned>(row - static_cast<long long>(b) * hw);
    const int oh = static_cast<int>(l / static_cast<unsigned>(g.Wo));
    const int ow = static_cast<int>(l - static_cast<unsigned>(oh) * g.Wo);
    const int ih0 = oh * g.sh - g.ph, iw0 = ow * g.sw - g.pw;
    const float* xb = x + static_cast<long long>(b) * g.C * plane;
    T* out = cols + row * ldk;
    for (int k = lane * 4; k < Kc; k += 128) {
      int c = static_cast<unsigned>(k) / static_cast<unsigned>(khw);
      const int rem = k - c * khw;
      int ki = static_cast<unsigned>(rem) / static_cast<unsigned>(g.kw);
      int kj = rem - ki * g.kw;
      float v[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int ih = ih0 + ki * g.dh, iw = iw0 + kj * g.dw;
        v[q] = 0.f;
        if (k + q < Kc && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) v[q] = __ldg(xb + c * plane + ih * g.W + iw);
        if (++kj == g.kw) {
          kj = 0;
          if (++ki == g.kh) {
            ki = 0;
            ++c;
          }
        }
      }
      if (k + 3 < Kc) {
        if constexpr (sizeof(T) == 2) {
          const __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
          uint2 w;
          w.x = *reinterpret_cast<const uint32_t*>(&p0);
          w.y = *reinterpret_cast<const uint32_t*>(&p1);
          *reinterpret_cast<uint2*>(out + k) = w;
        } else {
          *reinterpret_cast<float4*>(out + k) = make_float4(v[0], v[1], v[2], v[3]);
        }
      } else {
        for (int q = 0; q < 4 && k + q < Kc; ++q) {
          if constexpr (sizeof(T) == 2) out[k + q] = __float2bfloat16_rn(v[q]);
          else out[k + q] = v[q];
        }
      }
    }
  }
}

// Gradient of im2col in gather form (no atomics): every input pixel sums the window
// entries that read it.
__global__ void col2im_kernel(const float* __restrict__ dcols, float* __restrict__ dx, ConvGeom g, long long ldk) {
  const long long total = static_cast<long long>(g.B) * g.C * g.H * g.W;
  for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const unsigned hw = static_cast<unsigned>(g.H) * g.W;
    const long long bcq = e / hw;  // b * C + c
    const unsigned l = static_cast<unsigned>(e - bcq * hw);
    const int ih = static_cast<int>(l / static_cast<unsigned>(g.W)), iw = static_cast<int>(l - (l / g.W) * g.W);
    const int b = static_cast<int>(bcq / g.C), c = static_cast<int>(bcq - static_cast<long long>(b) * g.C);
    float acc = 0.f;
    for (int ki = 0; ki < g.kh; ++ki) {
      const int th = ih + g.ph - ki * g.dh;
      if (th < 0 || th % g.sh) continue;
      const int oh = th / g.sh;
      if (oh >= g.Ho) continue;
      for (int kj = 0; kj < g.kw; ++kj) {
        const int tw = iw + g.pw - kj * g.dw;
        if (tw < 0 || tw % g.sw) continue;
        const int ow = tw / g.sw;
        if (ow >= g.Wo) continue;
        const long long row = (static_cast<long long>(b) * g.Ho + oh) * g.Wo + ow;
        acc += dcols[row * ldk + (c * g.kh + ki) * g.kw + kj];
      }
    }
    dx[e] = acc;
  }
}

// --------------------------------------------------------------- pooling
// op 0 = max (records the flat input offset of the winner), 1 = average.
__global__ void pool2d_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int* __restrict__ arg,
                                  ConvGeom g, int op) {
  const long long total = static_cast<long long>(g.B) * g.C * g.Ho * g.Wo;
  for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    // one 64-bit and one 32-bit division per element instead of three 64-bit ones
    const unsigned hw = static_cast<unsigned>(g.Ho) * g.Wo;
    const long long bc = e / hw;
    const unsigned l = static_cast<unsigned>(e - bc * hw);
    const int oh = static_cast<int>(l / static_cast<unsigned>(g.Wo)), ow = static_cast<int>(l - (l / g.Wo) * g.Wo);
    const float* plane = x + bc * g.H * g.W;
    float best = -INFINITY, sum = 0.f;
    int besti = 0;
    for (int ki = 0; ki < g.kh; ++ki)
      for (int kj = 0; kj < g.kw; ++kj) {
        const int ih = oh * g.sh + ki, iw = ow * g.sw + kj;  // windows lie inside the input (no padding)
        const float v = plane[ih * g.W + iw];
        sum += v;
        if (v > best) {
          best = v;
          besti = ih * g.W + iw;
        }
      }
    if (op == 0) {
      y[e] = best;
      if (arg != nullptr) arg[e] = besti;
    } else {
      y[e] = sum / static_cast<float>(g.kh * g.kw);
    }
  }
}

// Gather-form backward: each input pixel collects from the windows that cover it.
__global__ void pool2d_bwd_kernel(const float* __restrict__ dy, const int* __restrict__ arg, float* __restrict__ dx,
                                  ConvGeom g, int op) {
  const long long total = static_cast<long long>(g.B) * g.C * g.H * g.W;
  const float inv = 1.f / static_cast<float>(g.kh * g.kw);
  for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const unsigned hw = static_cast<unsigned>(g.H) * g.W;
    const long long bc = e / hw;
    const unsigned l = static_cast<unsigned>(e - bc * hw);
    const int ih = static_cast<int>(l / static_cast<unsigned>(g.W)), iw = static_cast<int>(l - (l / g.W) * g.W);
    const int me = ih * g.W + iw;
    float acc = 0.f;
    for (int ki = 0; ki < g.kh; ++ki) {
      const int th = ih - ki;
      if (th < 0 || th % g.sh) continue;
      const int oh = th / g.sh;
      if (oh >= g.Ho) continue;
      for (int kj = 0; kj < g.kw; ++kj) {
        const int tw = iw - kj;
        if (tw < 0 || tw % g.sw) continue;
        const int ow = tw / g.sw;
        if (ow >= g.Wo) continue;
        const long long o = (bc * g.Ho + oh) * g.Wo + ow;
        if (op == 0)
          acc += (arg[o] == me) ? dy[o] : 0.f;
        else
          acc += dy[o] * inv;
      }
    }
    dx[e] = acc;
  }
}

ConvGeom geom(int B, int C, int H, int W, int kh, int kw, int Ho, int Wo, int sh, int sw, int ph, int pw, int dh,
              int dw) {
  ConvGeom g{B, C, H, W, kh, kw, Ho, Wo, sh, sw, ph, pw, dh, dw};
  return g;
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" int fb_lstm_gates_fwd(const float* xi, const float* hh, const float* c_prev, float* h_out, float* c_out,
                                 float* gates, long long B, int H, cudaStream_t st) {
  if (B <= 0 || H <= 0) return 0;
  lstm_gates_fwd_kernel<<<grid_for(B * H, 256), 256, 0, st>>>(xi, hh, c_prev, h_out, c_out, gates, B, H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_lstm_gates_bwd(const float* dh, const float* dc, const float* gates, const float* c_prev,
                                 const float* c_out, float* dpre, float* dc_prev, long long B, int H,
                                 cudaStream_t st) {
  if (B <= 0 || H <= 0) return 0;
  lstm_gates_bwd_kernel<<<grid_for(B * H, 256), 256, 0, st>>>(dh, dc, gates, c_prev, c_out, dpre, dc_prev, B, H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_gru_gates_fwd(const float* xi, const float* hh, const float* h_prev, float* h_out, float* saved,
                                long long B, int H, cudaStream_t st) {
  if (B <= 0 || H <= 0) return 0;
  gru_gates_fwd_kernel<<<grid_for(B * H, 256), 256, 0, st>>>(xi, hh, h_prev, h_out, saved, B, H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_gru_gates_bwd(const float* dh, const float* saved, const float* h_prev, float* dxi, float* dhh,
                                float* dh_prev, long long B, int H, cudaStream_t st) {
  if (B <= 0 || H <= 0) return 0;
  gru_gates_bwd_kernel<<<grid_for(B * H, 256), 256, 0, st>>>(dh, saved, h_prev, dxi, dhh, dh_prev, B, H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_im2col(const float* x, void* cols, int B, int C, int H, int W, int kh, int kw, int Ho, int Wo,
                         int sh, int sw, int ph, int pw, int dh, int dw, long long ldk, int out_dtype,
                         cudaStream_t st) {
  const long long total = static_cast<long long>(B) * Ho * Wo * C * kh * kw;
  if (total <= 0) return 0;
  const ConvGeom g = geom(B, C, H, W, kh, kw, Ho, Wo, sh, sw, ph, pw, dh, dw);
  const long long rows = static_cast<long long>(B) * Ho * Wo;
  const int esz = out_dtype == FB_DT_BF16 ? 2 : 4;
  // warp-per-row kernel: needs vector stores to be legal (pitch and base multiples of 4 elements)
  if (ldk % 4 == 0 && (reinterpret_cast<uintptr_t>(cols) % (4 * esz)) == 0 && static_cast<long long>(Ho) * Wo < (1LL << 31) &&
      static_cast<long long>(C) * H * W < (1LL << 31)) {
    const int grid = grid_for(rows * 32, 256);
    if (out_dtype == FB_DT_BF16)
      im2col_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(x, static_cast<__nv_bfloat16*>(cols), g, ldk, rows);
    else
      im2col_rows_kernel<float><<<grid, 256, 0, st>>>(x, static_cast<float*>(cols), g, ldk, rows);
    return static_cast<int>(cudaGetLastError());
  }
  if (out_dtype == FB_DT_BF16)
    im2col_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, st>>>(x, static_cast<__nv_bfloat16*>(cols), g, ldk);
  else
    im2col_kernel<float><<<grid_for(total, 256), 256, 0, st>>>(x, static_cast<float*>(cols), g, ldk);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_col2im(const float* dcols, float* dx, int B, int C, int H, int W, int kh, int kw, int Ho, int Wo,
                         int sh, int sw, int ph, int pw, int dh, int dw, long long ldk, cudaStream_t st) {
  const long long total = static_cast<long long>(B) * C * H * W;
  if (total <= 0) return 0;
  col2im_kernel<<<grid_for(total, 256), 256, 0, st>>>(dcols, dx, geom(B, C, H, W, kh, kw, Ho, Wo, sh, sw, ph, pw, dh, dw),
                                                      ldk);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_pool2d_fwd(const float* x, float* y, int* arg, int B, int C, int H, int W, int kh, int kw, int Ho,
                             int Wo, int sh, int sw, int op, cudaStream_t st) {
  const long long total = static_cast<long long>(B) * C * Ho * Wo;
  if (total <= 0) return 0;
  pool2d_fwd_kernel<<<grid_for(total, 256), 256, 0, st>>>(x, y, arg, geom(B, C, H, W, kh, kw, Ho, Wo, sh, sw, 0, 0, 1, 1),
                                                          op);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_pool2d_bwd(const float* dy, const int* arg, float* dx, int B, int C, int H, int W, int kh, int kw,
                             int Ho, int Wo, int sh, int sw, int op, cudaStream_t st) {
  const long long total = static_cast<long long>(B) * C * H * W;
  if (total <= 0) return 0;
  pool2d_bwd_kernel<<<grid_for(total, 256), 256, 0, st>>>(dy, arg, dx, geom(B, C, H, W, kh, kw, Ho, Wo, sh, sw, 0, 0, 1, 1),
                                                          op);
  return static_cast<int>(cudaGetLastError());
}
