// Elementwise kernels: the unary / scalar family (forward and backward), the
// broadcasting binary family, dtype casts and a tiled 2-D transpose.
//
// Reference entry points these stand in for:
//   ferrum-cuda/src/kernels.rs:64-123   binary_op  {Add,Sub,Mul,Div,Pow,Max,Min}
//   ferrum-cuda/src/kernels.rs:130-194  unary_op   {Neg,Exp,Log,Sqrt,Abs,Sin,Cos,Tanh,Sigmoid,Relu,LeakyRelu,Gelu,Silu}
//   ferrum-cuda/src/kernels.rs:201-257  scalar_op  {Add,Sub,Mul,Div,Pow}
//   ferrum-cuda/src/kernels.rs:442-494  transpose
//   ferrum-core/src/autograd_ops.rs:476-566  which tensor each backward formula saves
// All are memory-bound: 128-bit accesses, one pass, grid sized to the SM count.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

constexpr float kGeluC = 0.7978845608028654f;
constexpr float kGeluA = 0.044715f;

__device__ __forceinline__ float tanh_fast(float u) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return t;
}
// bf16 storage rounds at 2^-9; the hardware tanh (2^-11) and __expf are accurate enough there and keep the
// kernel memory-bound.
__device__ __forceinline__ float unary_f_fast(float x, int op, float alpha, float beta);
__device__ __forceinline__ float unary_grad_fast(float dy, float s, int op, float alpha, float beta);

__device__ __forceinline__ float unary_f(float x, int op, float alpha, float beta) {
  switch (op) {
    case FB_ACT_NONE: return x;
    case FB_ACT_RELU: return fmaxf(x, 0.f);
    case FB_ACT_GELU: return 0.5f * x * (1.f + tanhf(kGeluC * (x + kGeluA * x * x * x)));
    case FB_ACT_SILU: return x / (1.f + expf(-x));
    case FB_ACT_TANH: return tanhf(x);
    case FB_ACT_SIGMOID: return 1.f / (1.f + expf(-x));
    case FB_ACT_LEAKY_RELU: return x > 0.f ? x : alpha * x;
    case FB_ACT_ELU: return x > 0.f ? x : alpha * (expf(x) - 1.f);
    case FB_UNARY_NEG: return -x;
    case FB_UNARY_EXP: return expf(x);
    case FB_UNARY_LOG: return logf(x);
    case FB_UNARY_SQRT: return sqrtf(x);
    case FB_UNARY_ABS: return fabsf(x);
    case FB_UNARY_SIN: return sinf(x);
    case FB_UNARY_COS: return cosf(x);
    case FB_UNARY_POW: return powf(x, alpha);
    case FB_UNARY_ADD_SCALAR: return x + alpha;
    case FB_UNARY_MUL_SCALAR: return x * alpha;
    case FB_UNARY_RSUB_SCALAR: return alpha - x;
    case FB_UNARY_RDIV_SCALAR: return alpha / x;
    case FB_UNARY_AFFINE: return fmaf(x, alpha, beta);
    case FB_UNARY_CLAMP: return fminf(fmaxf(x, alpha), beta);
    default: return x;
  }
}

// s = saved tensor value: the INPUT for relu/gelu/silu/leaky/elu/log/abs/sin/cos/pow/rdiv/clamp,
// the OUTPUT for tanh/sigmoid/exp/sqrt; unused for the linear ops.
__device__ __forceinline__ float unary_grad(float dy, float s, int op, float alpha, float beta) {
  switch (op) {
    case FB_ACT_NONE: return dy;
    case FB_ACT_RELU: return s > 0.f ? dy : 0.f;
    case FB_ACT_GELU: {
      const float u = kGeluC * (s + kGeluA * s * s * s);
      const float t = tanhf(u);
      const float du = kGeluC * (1.f + 3.f * kGeluA * s * s);
      return dy * (0.5f * (1.f + t) + 0.5f * s * (1.f - t * t) * du);
    }
    case FB_ACT_SILU: {
      const float sg = 1.f / (1.f + expf(-s));
      return dy * (sg * (1.f + s * (1.f - sg)));
    }
    case FB_ACT_TANH: return dy * (1.f - s * s);
    case FB_ACT_SIGMOID: return dy * s * (1.f - s);
    case FB_ACT_LEAKY_RELU: return s > 0.f ? dy : alpha * dy;
    case FB_ACT_ELU: return s > 0.f ? dy : dy * alpha * expf(s);
    case FB_UNARY_NEG: return -dy;
    case FB_UNARY_EXP: return dy * s;
    case FB_UNARY_LOG: return dy / s;
    case FB_UNARY_SQRT: return dy / (2.f * s);
    case FB_UNARY_ABS: return s > 0.f ? dy : (s < 0.f ? -dy : 0.f);
    case FB_UNARY_SIN: return dy * cosf(s);
    case FB_UNARY_COS: return -dy * sinf(s);
    case FB_UNARY_POW: return dy * alpha * powf(s, alpha - 1.f);
    case FB_UNARY_ADD_SCALAR: return dy;
    case FB_UNARY_MUL_SCALAR: return dy * alpha;
    case FB_UNARY_RSUB_SCALAR: return -dy;
    case FB_UNARY_RDIV_SCALAR: return -dy * alpha / (s * s);
    case FB_UNARY_AFFINE: return dy * alpha;
    case FB_UNARY_CLAMP: return (s >= alpha && s <= beta) ? dy : 0.f;
    default: return dy;
  }
}

__device__ __forceinline__ float unary_f_fast(float x, int op, float alpha, float beta) {
  switch (op) {
    case FB_ACT_GELU: return 0.5f * x * (1.f + tanh_fast(kGeluC * (x + kGeluA * x * x * x)));
    case FB_ACT_SILU: return x / (1.f + __expf(-x));
    case FB_ACT_TANH: return tanh_fast(x);
    case FB_ACT_SIGMOID: return 1.f / (1.f + __expf(-x));
    default: return unary_f(x, op, alpha, beta);
  }
}
__device__ __forceinline__ float unary_grad_fast(float dy, float s, int op, float alpha, float beta) {
  switch (op) {
    case FB_ACT_GELU: {
      const float t = tanh_fast(kGeluC * (s + kGeluA * s * s * s));
      const float du = kGeluC * (1.f + 3.f * kGeluA * s * s);
      return dy * (0.5f * (1.f + t) + 0.5f * s * (1.f - t * t) * du);
    }
    case FB_ACT_SILU: {
      const float sg = 1.f / (1.f + __expf(-s));
      return dy * (sg * (1.f + s * (1.f - sg)));
    }
    default: return unary_grad(dy, s, op, alpha, beta);
  }
}

__device__ __forceinline__ void bf16x8_to_f32(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

template <int OP>
__global__ void unary_fwd_f32(const float* __restrict__ x, float* __restrict__ y, long long n, int, float a,
                              float b) {
  const long long n4 = n >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (aligned) {
    for (long long i = tid; i < n4; i += stride) {
      float4 v = reinterpret_cast<const float4*>(x)[i];
      v.x = unary_f(v.x, OP, a, b);
      v.y = unary_f(v.y, OP, a, b);
      v.z = unary_f(v.z, OP, a, b);
      v.w = unary_f(v.w, OP, a, b);
      reinterpret_cast<float4*>(y)[i] = v;
    }
    for (long long i = (n4 << 2) + tid; i < n; i += stride) y[i] = unary_f(x[i], OP, a, b);
  } else {
    for (long long i = tid; i < n; i += stride) y[i] = unary_f(x[i], OP, a, b);
  }
}

template <int OP>
__global__ void unary_bwd_f32(const float* __restrict__ dy, const float* __restrict__ s, float* __restrict__ dx,
                              long long n, int, float a, float b) {
  const long long n4 = n >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const float* sp = s ? s : dy;
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(sp) | reinterpret_cast<uintptr_t>(dx)) & 15) ==
      0;
  if (aligned) {
    for (long long i = tid; i < n4; i += stride) {
      const float4 g = reinterpret_cast<const float4*>(dy)[i];
      const float4 v = reinterpret_cast<const float4*>(sp)[i];
      float4 o;
      o.x = unary_grad(g.x, v.x, OP, a, b);
      o.y = unary_grad(g.y, v.y, OP, a, b);
      o.z = unary_grad(g.z, v.z, OP, a, b);
      o.w = unary_grad(g.w, v.w, OP, a, b);
      reinterpret_cast<float4*>(dx)[i] = o;
    }
    for (long long i = (n4 << 2) + tid; i < n; i += stride) dx[i] = unary_grad(dy[i], sp[i], OP, a, b);
  } else {
    for (long long i = tid; i < n; i += stride) dx[i] = unary_grad(dy[i], sp[i], OP, a, b);
  }
}

template <int OP>
__global__ void unary_fwd_bf16(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n,
                               int, float a, float b) {
  const long long n8 = n >> 3;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (aligned) {
    // two independent 16-byte loads per thread per trip: bf16 rows carry half the bytes of fp32 ones, and
    // the bytes in flight per SM are what buys HBM bandwidth
    for (long long i = tid; i < n8; i += 2 * stride) {
      const long long j = i + stride;
      const uint4 r0 = reinterpret_cast<const uint4*>(x)[i];
      uint4 r1 = make_uint4(0u, 0u, 0u, 0u);
      if (j < n8) r1 = reinterpret_cast<const uint4*>(x)[j];
      float f[8];
      bf16x8_to_f32(r0, f);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = unary_f_fast(f[k], OP, a, b);
      reinterpret_cast<uint4*>(y)[i] = f32_to_bf16x8(f);
      if (j < n8) {
        bf16x8_to_f32(r1, f);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = unary_f_fast(f[k], OP, a, b);
        reinterpret_cast<uint4*>(y)[j] = f32_to_bf16x8(f);
      }
    }
    for (long long i = (n8 << 3) + tid; i < n; i += stride)
      y[i] = __float2bfloat16_rn(unary_f_fast(__bfloat162float(x[i]), OP, a, b));
  } else {
    for (long long i = tid; i < n; i += stride) y[i] = __float2bfloat16_rn(unary_f_fast(__bfloat162float(x[i]), OP, a, b));
  }
}

template <int OP>
__global__ void unary_bwd_bf16(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ s,
                               __nv_bfloat16* __restrict__ dx, long long n, int, float a, float b) {
  const long long n8 = n >> 3;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const __nv_bfloat16* sp = s ? s : dy;
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(sp) | reinterpret_cast<uintptr_t>(dx)) & 15) ==
      0;
  if (aligned) {
    for (long long i = tid; i < n8; i += 2 * stride) {
      const long long j = i + stride;
      const uint4 rg0 = reinterpret_cast<const uint4*>(dy)[i], rv0 = reinterpret_cast<const uint4*>(sp)[i];
      uint4 rg1 = make_uint4(0u, 0u, 0u, 0u), rv1 = rg1;
      if (j < n8) {
        rg1 = reinterpret_cast<const uint4*>(dy)[j];
        rv1 = reinterpret_cast<const uint4*>(sp)[j];
      }
      float g[8], v[8];
      bf16x8_to_f32(rg0, g);
      bf16x8_to_f32(rv0, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = unary_grad_fast(g[k], v[k], OP, a, b);
      reinterpret_cast<uint4*>(dx)[i] = f32_to_bf16x8(g);
      if (j < n8) {
        bf16x8_to_f32(rg1, g);
        bf16x8_to_f32(rv1, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] = unary_grad_fast(g[k], v[k], OP, a, b);
        reinterpret_cast<uint4*>(dx)[j] = f32_to_bf16x8(g);
      }
    }
    for (long long i = (n8 << 3) + tid; i < n; i += stride)
      dx[i] = __float2bfloat16_rn(unary_grad_fast(__bfloat162float(dy[i]), __bfloat162float(sp[i]), OP, a, b));
  } else {
    for (long long i = tid; i < n; i += stride)
      dx[i] = __float2bfloat16_rn(unary_grad_fast(__bfloat162float(dy[i]), __bfloat162float(sp[i]), OP, a, b));
  }
}

__device__ __forceinline__ float binary_f(float a, float b, int op) {
  switch (op) {
    case FB_BIN_ADD: return a + b;
    case FB_BIN_SUB: return a - b;
    case FB_BIN_MUL: return a * b;
    case FB_BIN_DIV: return a / b;
    case FB_BIN_POW: return powf(a, b);
    case FB_BIN_MAX: return fmaxf(a, b);
    case FB_BIN_MIN: return fminf(a, b);
    default: return a;
  }
}

struct BcastDesc {
  int ndim;
  long long shape[6];
  long long sa[6];
  long long sb[6];
};

// Same-shape contiguous operands.
__global__ void binary_contig(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o,
                              long long n, int op) {
  const long long n4 = n >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(o)) & 15) == 0;
  if (aligned) {
    for (long long i = tid; i < n4; i += stride) {
      const float4 x = reinterpret_cast<const float4*>(a)[i];
      const float4 y = reinterpret_cast<const float4*>(b)[i];
      float4 r;
      r.x = binary_f(x.x, y.x, op);
      r.y = binary_f(x.y, y.y, op);
      r.z = binary_f(x.z, y.z, op);
      r.w = binary_f(x.w, y.w, op);
      reinterpret_cast<float4*>(o)[i] = r;
    }
    for (long long i = (n4 << 2) + tid; i < n; i += stride) o[i] = binary_f(a[i], b[i], op);
  } else {
    for (long long i = tid; i < n; i += stride) o[i] = binary_f(a[i], b[i], op);
  }
}

// [rows, cols] (op) [cols]: the second operand is broadcast along rows (bias add, per-feature scaling).
// swap = the broadcast operand is the FIRST argument of the op.
__global__ void binary_rowbcast(const float* __restrict__ full, const float* __restrict__ vec, float* __restrict__ o,
                                long long n, long long cols, int op, int swap) {
  const long long n4 = n >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 x = reinterpret_cast<const float4*>(full)[i];
    const float4 y = *reinterpret_cast<const float4*>(vec + (i << 2) % cols);
    float4 r;
    if (swap) {
      r.x = binary_f(y.x, x.x, op); r.y = binary_f(y.y, x.y, op);
      r.z = binary_f(y.z, x.z, op); r.w = binary_f(y.w, x.w, op);
    } else {
      r.x = binary_f(x.x, y.x, op); r.y = binary_f(x.y, y.y, op);
      r.z = binary_f(x.z, y.z, op); r.w = binary_f(x.w, y.w, op);
    }
    reinterpret_cast<float4*>(o)[i] = r;
  }
}

// General strided / stride-0 broadcast: the output index is decomposed once per element.
__global__ void binary_bcast(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o,
                             long long n, int op, const BcastDesc d) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    long long rem = i, oa = 0, ob = 0;
#pragma unroll
    for (int k = 5; k >= 0; --k) {
      if (k < d.ndim) {
        const long long c = rem % d.shape[k];
        rem /= d.shape[k];
        oa += c * d.sa[k];
        ob += c * d.sb[k];
      }
    }
    o[i] = binary_f(a[oa], b[ob], op);
  }
}

template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ s, D* __restrict__ d, long long n);

template <>
__global__ void cast_kernel<float, __nv_bfloat16>(const float* __restrict__ s, __nv_bfloat16* __restrict__ d,
                                                  long long n) {
  const long long n8 = n >> 3;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15) == 0;
  if (aligned) {
    for (long long i = tid; i < n8; i += stride) {
      const float4 a = reinterpret_cast<const float4*>(s)[2 * i];
      const float4 b = reinterpret_cast<const float4*>(s)[2 * i + 1];
      const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      reinterpret_cast<uint4*>(d)[i] = f32_to_bf16x8(f);
    }
    for (long long i = (n8 << 3) + tid; i < n; i += stride) d[i] = __float2bfloat16_rn(s[i]);
  } else {
    for (long long i = tid; i < n; i += stride) d[i] = __float2bfloat16_rn(s[i]);
  }
}

template <>
__global__ void cast_kernel<__nv_bfloat16, float>(const __nv_bfloat16* __restrict__ s, float* __restrict__ d,
                                                  long long n) {
  const long long n8 = n >> 3;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15) == 0;
  if (aligned) {
    for (long long i = tid; i < n8; i += stride) {
      float f[8];
      bf16x8_to_f32(reinterpret_cast<const uint4*>(s)[i], f);
      reinterpret_cast<float4*>(d)[2 * i] = make_float4(f[0], f[1], f[2], f[3]);
      reinterpret_cast<float4*>(d)[2 * i + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    for (long long i = (n8 << 3) + tid; i < n; i += stride) d[i] = __bfloat162float(s[i]);
  } else {
    for (long long i = tid; i < n; i += stride) d[i] = __bfloat162float(s[i]);
  }
}

// 32x32 tiles through padded shared memory; T is a 2- or 4-byte POD.
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ s, T* __restrict__ d, int rows, int cols) {
  __shared__ T tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = s[static_cast<long long>(r) * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) d[static_cast<long long>(c) * rows + r] = tile[threadIdx.x][j];
  }
}

// 2-byte elements, even rows / cols, 4-byte aligned pitches: 64 x 64 tiles moved as 32-bit pairs, so global
// loads and stores are 128 bytes per warp row (the 32 x 32 kernel above moves 64) and a block has 8 KB in flight.
__global__ void __launch_bounds__(256)
transpose16_pairs_kernel(const uint16_t* __restrict__ s, uint16_t* __restrict__ d, int rows, int cols) {
  __shared__ uint16_t tile[64][66];  // pitch 132 B: 4-byte aligned rows, conflict-free pair stores
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  const int x = threadIdx.x, y = threadIdx.y;  // 32 x 8
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int r = r0 + y + 8 * j, c = c0 + 2 * x;
    uint32_t v = 0;
    if (r < rows && c < cols) v = *reinterpret_cast<const uint32_t*>(s + static_cast<long long>(r) * cols + c);
    *reinterpret_cast<uint32_t*>(&tile[y + 8 * j][2 * x]) = v;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = c0 + y + 8 * j, r = r0 + 2 * x;  // output row c holds input rows r, r + 1
    if (c < cols && r < rows) {
      const uint32_t v = static_cast<uint32_t>(tile[2 * x][y + 8 * j]) |
                         (static_cast<uint32_t>(tile[2 * x + 1][y + 8 * j]) << 16);
      *reinterpret_cast<uint32_t*>(d + static_cast<long long>(c) * rows + r) = v;
    }
  }
}

// y = x * (*scalar): the incoming gradient of a scalar loss applied to a stored gradient, without a host read.
template <typename T>
__global__ void scale_by_scalar_kernel(const T* __restrict__ x, const float* __restrict__ scalar, T* __restrict__ y,
                                       long long n) {
  const float sc = *scalar;
  constexpr int kPer = 16 / sizeof(T);
  const long long nv = n / kPer;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (aligned) {
    for (long long i = tid; i < nv; i += stride) {
      if constexpr (sizeof(T) == 2) {
        float f[8];
        bf16x8_to_f32(reinterpret_cast<const uint4*>(x)[i], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] *= sc;
        reinterpret_cast<uint4*>(y)[i] = f32_to_bf16x8(f);
      } else {
        float4 v = reinterpret_cast<const float4*>(x)[i];
        v.x *= sc; v.y *= sc; v.z *= sc; v.w *= sc;
        reinterpret_cast<float4*>(y)[i] = v;
      }
    }
    for (long long i = nv * kPer + tid; i < n; i += stride) y[i] = static_cast<T>(static_cast<float>(x[i]) * sc);
  } else {
    for (long long i = tid; i < n; i += stride) y[i] = static_cast<T>(static_cast<float>(x[i]) * sc);
  }
}

int grid_for(long long work_items, int block) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long need = (work_items + block - 1) / block;
  const long long cap = static_cast<long long>(sms) * 6;  // 6 x 256 threads: what 40-register kernels keep resident
  if (need > cap) need = cap;
  if (need < 1) need = 1;
  return static_cast<int>(need);
}

}  // namespace
}  // namespace fb

using namespace fb;

// The op is a template parameter of the kernels (a switch evaluated per element costs more issue slots than
// the arithmetic of most ops); this turns the runtime op into the instantiation.
#define FB_UNARY_DISPATCH(OPV, CALL) \
  switch (OPV) {                     \
    case 0: { constexpr int OP = 0; CALL; } break;   \
    case 1: { constexpr int OP = 1; CALL; } break;   \
    case 2: { constexpr int OP = 2; CALL; } break;   \
    case 3: { constexpr int OP = 3; CALL; } break;   \
    case 4: { constexpr int OP = 4; CALL; } break;   \
    case 5: { constexpr int OP = 5; CALL; } break;   \
    case 6: { constexpr int OP = 6; CALL; } break;   \
    case 7: { constexpr int OP = 7; CALL; } break;   \
    case 8: { constexpr int OP = 8; CALL; } break;   \
    case 9: { constexpr int OP = 9; CALL; } break;   \
    case 10: { constexpr int OP = 10; CALL; } break; \
    case 11: { constexpr int OP = 11; CALL; } break; \
    case 12: { constexpr int OP = 12; CALL; } break; \
    case 13: { constexpr int OP = 13; CALL; } break; \
    case 14: { constexpr int OP = 14; CALL; } break; \
    case 15: { constexpr int OP = 15; CALL; } break; \
    case 16: { constexpr int OP = 16; CALL; } break; \
    case 17: { constexpr int OP = 17; CALL; } break; \
    case 18: { constexpr int OP = 18; CALL; } break; \
    case 19: { constexpr int OP = 19; CALL; } break; \
    case 20: { constexpr int OP = 20; CALL; } break; \
    case 21: { constexpr int OP = 21; CALL; } break; \
    default: return -1;              \
  }

extern "C" int fb_unary_fwd(const void* x, void* y, long long n, int op, float alpha, float beta, int dtype,
                            cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dtype == FB_DT_F32) {
    FB_UNARY_DISPATCH(op, (unary_fwd_f32<OP><<<grid_for((n + 3) / 4, 256), 256, 0, stream>>>(
                              static_cast<const float*>(x), static_cast<float*>(y), n, op, alpha, beta)))
  } else if (dtype == FB_DT_BF16) {
    FB_UNARY_DISPATCH(op, (unary_fwd_bf16<OP><<<grid_for((n + 7) / 8, 256), 256, 0, stream>>>(
                              static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, op, alpha, beta)))
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_unary_bwd(const void* dy, const void* saved, void* dx, long long n, int op, float alpha,
                            float beta, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dtype == FB_DT_F32) {
    FB_UNARY_DISPATCH(op, (unary_bwd_f32<OP><<<grid_for((n + 3) / 4, 256), 256, 0, stream>>>(
                              static_cast<const float*>(dy), static_cast<const float*>(saved), static_cast<float*>(dx),
                              n, op, alpha, beta)))
  } else if (dtype == FB_DT_BF16) {
    FB_UNARY_DISPATCH(op, (unary_bwd_bf16<OP><<<grid_for((n + 7) / 8, 256), 256, 0, stream>>>(
                              static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(saved),
                              static_cast<__nv_bfloat16*>(dx), n, op, alpha, beta)))
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_binary_fwd(const float* a, const float* b, float* out, int op, int ndim, const long long* shape,
                             const long long* stride_a, const long long* stride_b, cudaStream_t stream) {
  if (ndim < 0 || ndim > 6) return -1;
  long long n = 1;
  for (int i = 0; i < ndim; ++i) n *= shape[i];
  if (n <= 0) return 0;
  // contiguous same-shape fast path
  bool contig = true;
  long long expect = 1;
  for (int i = ndim - 1; i >= 0; --i) {
    if (shape[i] != 1 && (stride_a[i] != expect || stride_b[i] != expect)) contig = false;
    expect *= shape[i];
  }
  // row-broadcast fast path: one operand contiguous over the full shape, the other only along the last dim
  auto is_full = [&](const long long* st) {
    long long e = 1;
    for (int i = ndim - 1; i >= 0; --i) {
      if (shape[i] != 1 && st[i] != e) return false;
      e *= shape[i];
    }
    return true;
  };
  auto is_row = [&](const long long* st) {
    if (ndim < 2 || st[ndim - 1] != 1) return false;
    for (int i = 0; i < ndim - 1; ++i)
      if (shape[i] != 1 && st[i] != 0) return false;
    return true;
  };
  const long long cols = ndim > 0 ? shape[ndim - 1] : 1;
  const bool al = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                    reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (contig) {
    binary_contig<<<grid_for((n + 3) / 4, 256), 256, 0, stream>>>(a, b, out, n, op);
  } else if (al && cols % 4 == 0 && is_full(stride_a) && is_row(stride_b)) {
    binary_rowbcast<<<grid_for(n / 4, 256), 256, 0, stream>>>(a, b, out, n, cols, op, 0);
  } else if (al && cols % 4 == 0 && is_full(stride_b) && is_row(stride_a)) {
    binary_rowbcast<<<grid_for(n / 4, 256), 256, 0, stream>>>(b, a, out, n, cols, op, 1);
  } else {
    BcastDesc d;
    d.ndim = ndim;
    for (int i = 0; i < 6; ++i) {
      d.shape[i] = i < ndim ? shape[i] : 1;
      d.sa[i] = i < ndim ? stride_a[i] : 0;
      d.sb[i] = i < ndim ? stride_b[i] : 0;
    }
    binary_bcast<<<grid_for(n, 256), 256, 0, stream>>>(a, b, out, n, op, d);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_cast(const void* src, void* dst, long long n, int sd, int dd, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int g = grid_for((n + 7) / 8, 256);
  if (sd == FB_DT_F32 && dd == FB_DT_BF16) {
    cast_kernel<float, __nv_bfloat16><<<g, 256, 0, stream>>>(static_cast<const float*>(src),
                                                             static_cast<__nv_bfloat16*>(dst), n);
  } else if (sd == FB_DT_BF16 && dd == FB_DT_F32) {
    cast_kernel<__nv_bfloat16, float><<<g, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src),
                                                             static_cast<float*>(dst), n);
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_transpose_2d(const void* src, void* dst, int rows, int cols, int elem_size,
                               cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  if (elem_size == 4) {
    transpose_kernel<uint32_t><<<grid, block, 0, stream>>>(static_cast<const uint32_t*>(src),
                                                          static_cast<uint32_t*>(dst), rows, cols);
  } else if (elem_size == 2 && rows % 2 == 0 && cols % 2 == 0 &&
             ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 3) == 0) {
    transpose16_pairs_kernel<<<dim3((cols + 63) / 64, (rows + 63) / 64), block, 0, stream>>>(
        static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), rows, cols);
  } else if (elem_size == 2) {
    transpose_kernel<uint16_t><<<grid, block, 0, stream>>>(static_cast<const uint16_t*>(src),
                                                          static_cast<uint16_t*>(dst), rows, cols);
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_scale_by_device_scalar(const void* x, const float* scalar, void* y, long long n, int dtype,
                                         cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dtype == FB_DT_F32)
    scale_by_scalar_kernel<float><<<grid_for((n + 3) / 4, 256), 256, 0, stream>>>(
        static_cast<const float*>(x), scalar, static_cast<float*>(y), n);
  else if (dtype == FB_DT_BF16)
    scale_by_scalar_kernel<__nv_bfloat16><<<grid_for((n + 7) / 8, 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), scalar, static_cast<__nv_bfloat16*>(y), n);
  else
    return -1;
  return static_cast<int>(cudaGetLastError());
}
