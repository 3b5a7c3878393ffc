// Fused optimizer steps and AMP helpers, one launch for the whole model.
//
// Reference update rules (each a chain of 6 - 14 full-size temporaries there):
//   ferrum-optim/src/sgd.rs:81-120   g += wd*p ; v = mu*v + g (first step v = g) ;
//                                    nesterov: g + mu*v ; p -= lr*upd
//   ferrum-optim/src/adam.rs:91-146  decoupled decay p -= lr*wd*p BEFORE the moments ;
//                                    m, v EMA ; bias correction 1 - beta^t ;
//                                    p -= lr * m_hat / (sqrt(v_hat) + eps)
//   ferrum-optim/src/amp.rs:62-91,198-238  unscale + inf/nan check, clip_grad_norm
//                                    (global L2, +1e-6), clip_grad_value
// One pass over memory: reads g, p and the state, writes p and the state, and
// (optionally) the bf16 shadow copy of p that the next forward GEMM consumes.
// The `flat` variants take one contiguous arena; the `multi` variants take
// device tables of pointers and sizes.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const fb_adam_hparams& h) {
  g *= h.grad_scale;
  if (h.weight_decay != 0.f) p -= h.lr * h.weight_decay * p;
  m = h.beta1 * m + (1.f - h.beta1) * g;
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  const float mh = m / h.bias_corr1;
  const float vh = v / h.bias_corr2;
  p -= h.lr * mh / (sqrtf(vh) + h.eps);
}

__device__ __forceinline__ void sgd_one(float& p, float g, float* buf, long long i, const fb_sgd_hparams& h) {
  g *= h.grad_scale;
  if (h.weight_decay != 0.f) g += h.weight_decay * p;
  float upd = g;
  if (h.momentum != 0.f && buf != nullptr) {
    const float v = h.first_step ? g : h.momentum * buf[i] + g;
    buf[i] = v;
    upd = h.nesterov ? g + h.momentum * v : v;
  }
  p -= h.lr * upd;
}

__device__ __forceinline__ void adam_range(float* __restrict__ p, const float* __restrict__ g,
                                           float* __restrict__ m, float* __restrict__ v,
                                           __nv_bfloat16* __restrict__ sh, long long n, const fb_adam_hparams& h,
                                           long long tid, long long stride) {
  const bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                         reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) == 0 &&
                       (sh == nullptr || (reinterpret_cast<uintptr_t>(sh) & 7) == 0);
  long long done = 0;
  if (aligned) {
    const long long n4 = n >> 2;
    for (long long i = tid; i < n4; i += stride) {
      float4 pp = reinterpret_cast<float4*>(p)[i];
      const float4 gg = reinterpret_cast<const float4*>(g)[i];
      float4 mm = reinterpret_cast<float4*>(m)[i];
      float4 vv = reinterpret_cast<float4*>(v)[i];
      adam_one(pp.x, gg.x, mm.x, vv.x, h);
      adam_one(pp.y, gg.y, mm.y, vv.y, h);
      adam_one(pp.z, gg.z, mm.z, vv.z, h);
      adam_one(pp.w, gg.w, mm.w, vv.w, h);
      reinterpret_cast<float4*>(p)[i] = pp;
      reinterpret_cast<float4*>(m)[i] = mm;
      reinterpret_cast<float4*>(v)[i] = vv;
      if (sh != nullptr) {
        uint2 u;
        *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(pp.x, pp.y);
        *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(pp.z, pp.w);
        reinterpret_cast<uint2*>(sh)[i] = u;
      }
    }
    done = n4 << 2;
  }
  for (long long i = done + tid; i < n; i += stride) {
    float pp = p[i], mm = m[i], vv = v[i];
    adam_one(pp, g[i], mm, vv, h);
    p[i] = pp;
    m[i] = mm;
    v[i] = vv;
    if (sh != nullptr) sh[i] = __float2bfloat16_rn(pp);
  }
}

__device__ __forceinline__ void sgd_range(float* __restrict__ p, const float* __restrict__ g,
                                          float* __restrict__ buf, __nv_bfloat16* __restrict__ sh, long long n,
                                          const fb_sgd_hparams& h, long long tid, long long stride) {
  const bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                         reinterpret_cast<uintptr_t>(buf)) & 15) == 0 &&
                       (sh == nullptr || (reinterpret_cast<uintptr_t>(sh) & 7) == 0);
  long long done = 0;
  if (aligned) {
    const long long n4 = n >> 2;
    const bool mom = h.momentum != 0.f && buf != nullptr;
    for (long long i = tid; i < n4; i += stride) {
      float4 pp = reinterpret_cast<float4*>(p)[i];
      const float4 gg = reinterpret_cast<const float4*>(g)[i];
      float4 vv = mom ? reinterpret_cast<float4*>(buf)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      float* pv = reinterpret_cast<float*>(&pp);
      const float* gv = reinterpret_cast<const float*>(&gg);
      float* bv = reinterpret_cast<float*>(&vv);
#pragma unroll
      for (int k = 0; k < 4; ++k) sgd_one(pv[k], gv[k], mom ? bv : nullptr, k, h);
      reinterpret_cast<float4*>(p)[i] = pp;
      if (mom) reinterpret_cast<float4*>(buf)[i] = vv;
      if (sh != nullptr) {
        uint2 u;
        *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(pp.x, pp.y);
        *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(pp.z, pp.w);
        reinterpret_cast<uint2*>(sh)[i] = u;
      }
    }
    done = n4 << 2;
  }
  for (long long i = done + tid; i < n; i += stride) {
    float pp = p[i];
    sgd_one(pp, g[i], buf, i, h);
    p[i] = pp;
    if (sh != nullptr) sh[i] = __float2bfloat16_rn(pp);
  }
}

__global__ void adam_flat_kernel(float* p, const float* g, float* m, float* v, __nv_bfloat16* sh, long long n,
                                 const fb_adam_hparams h) {
  adam_range(p, g, m, v, sh, n, h, static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x,
             static_cast<long long>(gridDim.x) * blockDim.x);
}
__global__ void sgd_flat_kernel(float* p, const float* g, float* buf, __nv_bfloat16* sh, long long n,
                                const fb_sgd_hparams h) {
  sgd_range(p, g, buf, sh, n, h, static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x,
            static_cast<long long>(gridDim.x) * blockDim.x);
}
constexpr int kChunk = 48;  // tensors per launch; the table travels in the kernel parameters
struct AdamTable {
  float* p[kChunk];
  const float* g[kChunk];
  float* m[kChunk];
  float* v[kChunk];
  void* sh[kChunk];
  long long n[kChunk];
  int count;
};
struct SgdTable {
  float* p[kChunk];
  const float* g[kChunk];
  float* buf[kChunk];
  void* sh[kChunk];
  long long n[kChunk];
  int count;
};
struct GradTable {
  float* g[kChunk];
  long long n[kChunk];
  int count;
};

// dyn (optional): device scalars {lr, bias_corr1, bias_corr2, beta1^t, beta2^t, t} kept current by
// optim_advance_kernel, so that a captured CUDA graph replays with the right step-dependent factors.
__global__ void adam_multi_kernel(const AdamTable t, fb_adam_hparams h, const float* __restrict__ dyn) {
  if (dyn != nullptr) {
    h.lr = dyn[0];
    h.bias_corr1 = dyn[1];
    h.bias_corr2 = dyn[2];
  }
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int i = 0; i < t.count; ++i)
    adam_range(t.p[i], t.g[i], t.m[i], t.v[i], static_cast<__nv_bfloat16*>(t.sh[i]), t.n[i], h, tid, stride);
}
__global__ void sgd_multi_kernel(const SgdTable t, fb_sgd_hparams h, const float* __restrict__ dyn) {
  if (dyn != nullptr) h.lr = dyn[0];
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int i = 0; i < t.count; ++i)
    sgd_range(t.p[i], t.g[i], t.buf[i], static_cast<__nv_bfloat16*>(t.sh[i]), t.n[i], h, tid, stride);
}

// One thread: t += 1, beta^t products and the two bias corrections (Adam) for the launches that follow.
__global__ void optim_advance_kernel(float* dyn, float beta1, float beta2) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    dyn[3] *= beta1;
    dyn[4] *= beta2;
    dyn[1] = 1.f - dyn[3];
    dyn[2] = 1.f - dyn[4];
    dyn[5] += 1.f;
  }
}

// ------------------------------------------------------------------- AMP
// All three walk the tensors with 16-byte accesses, two independent vectors per thread per trip (the head
// up to the first 16-byte boundary and the tail are done element-wise).
template <typename F4, typename F1>
__device__ __forceinline__ void walk_rw(float* p, long long n, long long tid, long long stride, F4 f4, F1 f1) {
  const long long head = min(n, static_cast<long long>((16 - (reinterpret_cast<uintptr_t>(p) & 15)) & 15) / 4);
  for (long long i = tid; i < head; i += stride) p[i] = f1(p[i]);
  float4* q = reinterpret_cast<float4*>(p + head);
  const long long nv = (n - head) >> 2;
  for (long long i = tid; i < nv; i += 2 * stride) {
    const long long j = i + stride;
    float4 a = q[i], b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < nv) b = q[j];
    q[i] = f4(a);
    if (j < nv) q[j] = f4(b);
  }
  for (long long i = head + (nv << 2) + tid; i < n; i += stride) p[i] = f1(p[i]);
}

__global__ void unscale_check_kernel(const GradTable tb, float inv_scale, float* found_inf) {
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  bool bad = false;
  auto f1 = [&](float v) {
    v *= inv_scale;
    if (!isfinite(v)) bad = true;
    return v;
  };
  auto f4 = [&](float4 v) {
    v.x *= inv_scale; v.y *= inv_scale; v.z *= inv_scale; v.w *= inv_scale;
    // a non-finite lane makes the sum of (v - v) NaN: one test for four values
    const float z = (v.x - v.x) + (v.y - v.y) + (v.z - v.z) + (v.w - v.w);
    if (z != 0.f) bad = true;
    return v;
  };
  for (int t = 0; t < tb.count; ++t) walk_rw(tb.g[t], tb.n[t], tid, stride, f4, f1);
  if (bad) *found_inf = 1.f;
}

__global__ void sumsq_multi_kernel(const GradTable tb, float* out) {
  __shared__ float smem[8];
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float acc0 = 0.f, acc1 = 0.f;
  for (int t = 0; t < tb.count; ++t) {
    const float* p = tb.g[t];
    const long long n = tb.n[t];
    const long long head = min(n, static_cast<long long>((16 - (reinterpret_cast<uintptr_t>(p) & 15)) & 15) / 4);
    for (long long i = tid; i < head; i += stride) acc0 = fmaf(p[i], p[i], acc0);
    const float4* q = reinterpret_cast<const float4*>(p + head);
    const long long nv = (n - head) >> 2;
    for (long long i = tid; i < nv; i += 2 * stride) {
      const long long j = i + stride;
      const float4 a = q[i];
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < nv) b = q[j];
      acc0 = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, acc0))));
      acc1 = fmaf(b.x, b.x, fmaf(b.y, b.y, fmaf(b.z, b.z, fmaf(b.w, b.w, acc1))));
    }
    for (long long i = head + (nv << 2) + tid; i < n; i += stride) acc0 = fmaf(p[i], p[i], acc0);
  }
  float acc = acc0 + acc1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += smem[w];
    atomicAdd(out, s);
  }
}

// mode 0: scale by min(1, max_norm / (sqrt(total_sumsq) + 1e-6)); mode 1: clamp to +-clip_value.
__global__ void scale_multi_kernel(const GradTable tb, const float* total_sumsq, float max_norm, float clip_value,
                                   int mode) {
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float coef = 1.f;
  if (mode == 0) {
    coef = max_norm / (sqrtf(*total_sumsq) + 1e-6f);
    if (coef >= 1.f) return;
    auto f1 = [&](float v) { return v * coef; };
    auto f4 = [&](float4 v) { return make_float4(v.x * coef, v.y * coef, v.z * coef, v.w * coef); };
    for (int t = 0; t < tb.count; ++t) walk_rw(tb.g[t], tb.n[t], tid, stride, f4, f1);
  } else {
    auto f1 = [&](float v) { return fminf(fmaxf(v, -clip_value), clip_value); };
    auto f4 = [&](float4 v) { return make_float4(f1(v.x), f1(v.y), f1(v.z), f1(v.w)); };
    for (int t = 0; t < tb.count; ++t) walk_rw(tb.g[t], tb.n[t], tid, stride, f4, f1);
  }
}

int big_grid() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms * 4;
}
int grid_for(long long n) {
  long long nb = (n / 4 + 255) / 256;
  const long long cap = big_grid();
  if (nb > cap) nb = cap;
  if (nb < 1) nb = 1;
  return static_cast<int>(nb);
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" int fb_adam_flat(float* p, const float* g, float* m, float* v, void* shadow, long long n,
                            fb_adam_hparams h, cudaStream_t stream) {
  if (n <= 0) return 0;
  adam_flat_kernel<<<grid_for(n), 256, 0, stream>>>(p, g, m, v, static_cast<__nv_bfloat16*>(shadow), n, h);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int fb_sgd_flat(float* p, const float* g, float* buf, void* shadow, long long n, fb_sgd_hparams h,
                           cudaStream_t stream) {
  if (n <= 0) return 0;
  sgd_flat_kernel<<<grid_for(n), 256, 0, stream>>>(p, g, buf, static_cast<__nv_bfloat16*>(shadow), n, h);
  return static_cast<int>(cudaGetLastError());
}
// The `multi` entry points take HOST arrays of device pointers (NULL gradient = skip the tensor).
static int adam_multi_impl(float* const* p, const float* const* g, float* const* m, float* const* v,
                           void* const* shadow, const long long* sizes, int ntensors, fb_adam_hparams h,
                           const float* dyn, cudaStream_t stream);
extern "C" int fb_adam_multi(float* const* p, const float* const* g, float* const* m, float* const* v,
                             void* const* shadow, const long long* sizes, int ntensors, fb_adam_hparams h,
                             cudaStream_t stream) {
  return adam_multi_impl(p, g, m, v, shadow, sizes, ntensors, h, nullptr, stream);
}
// Graph-capturable form: lr and the bias corrections are read from the device scalars `dyn`
// ({lr, bias_corr1, bias_corr2, beta1^t, beta2^t, t}; see fb_optim_advance).
extern "C" int fb_adam_multi_dyn(float* const* p, const float* const* g, float* const* m, float* const* v,
                                 void* const* shadow, const long long* sizes, int ntensors, fb_adam_hparams h,
                                 const float* dyn, cudaStream_t stream) {
  if (dyn == nullptr) return -1;
  return adam_multi_impl(p, g, m, v, shadow, sizes, ntensors, h, dyn, stream);
}
extern "C" int fb_optim_advance(float* dyn, float beta1, float beta2, cudaStream_t stream) {
  if (dyn == nullptr) return -1;
  optim_advance_kernel<<<1, 32, 0, stream>>>(dyn, beta1, beta2);
  return static_cast<int>(cudaGetLastError());
}
static int adam_multi_impl(float* const* p, const float* const* g, float* const* m, float* const* v,
                           void* const* shadow, const long long* sizes, int ntensors, fb_adam_hparams h,
                           const float* dyn, cudaStream_t stream) {
  AdamTable t;
  t.count = 0;
  for (int i = 0; i <= ntensors; ++i) {
    if (i < ntensors && g[i] != nullptr && sizes[i] > 0) {
      const int k = t.count++;
      t.p[k] = p[i]; t.g[k] = g[i]; t.m[k] = m[i]; t.v[k] = v[i];
      t.sh[k] = shadow ? shadow[i] : nullptr;
      t.n[k] = sizes[i];
    }
    if (t.count == kChunk || (i == ntensors && t.count > 0)) {
      adam_multi_kernel<<<big_grid(), 256, 0, stream>>>(t, h, dyn);
      t.count = 0;
    }
  }
  return static_cast<int>(cudaGetLastError());
}
static int sgd_multi_impl(float* const* p, const float* const* g, float* const* buf, void* const* shadow,
                          const long long* sizes, int ntensors, fb_sgd_hparams h, const float* dyn,
                          cudaStream_t stream);
extern "C" int fb_sgd_multi(float* const* p, const float* const* g, float* const* buf, void* const* shadow,
                            const long long* sizes, int ntensors, fb_sgd_hparams h, cudaStream_t stream) {
  return sgd_multi_impl(p, g, buf, shadow, sizes, ntensors, h, nullptr, stream);
}
extern "C" int fb_sgd_multi_dyn(float* const* p, const float* const* g, float* const* buf, void* const* shadow,
                                const long long* sizes, int ntensors, fb_sgd_hparams h, const float* dyn,
                                cudaStream_t stream) {
  if (dyn == nullptr) return -1;
  return sgd_multi_impl(p, g, buf, shadow, sizes, ntensors, h, dyn, stream);
}
static int sgd_multi_impl(float* const* p, const float* const* g, float* const* buf, void* const* shadow,
                          const long long* sizes, int ntensors, fb_sgd_hparams h, const float* dyn,
                          cudaStream_t stream) {
  SgdTable t;
  t.count = 0;
  for (int i = 0; i <= ntensors; ++i) {
    if (i < ntensors && g[i] != nullptr && sizes[i] > 0) {
      const int k = t.count++;
      t.p[k] = p[i]; t.g[k] = g[i];
      t.buf[k] = buf ? buf[i] : nullptr;
      t.sh[k] = shadow ? shadow[i] : nullptr;
      t.n[k] = sizes[i];
    }
    if (t.count == kChunk || (i == ntensors && t.count > 0)) {
      sgd_multi_kernel<<<big_grid(), 256, 0, stream>>>(t, h, dyn);
      t.count = 0;
    }
  }
  return static_cast<int>(cudaGetLastError());
}

template <typename Launch>
static int for_grad_chunks(float* const* g, const long long* sizes, int ntensors, Launch launch) {
  GradTable t;
  t.count = 0;
  for (int i = 0; i <= ntensors; ++i) {
    if (i < ntensors && g[i] != nullptr && sizes[i] > 0) {
      const int k = t.count++;
      t.g[k] = g[i];
      t.n[k] = sizes[i];
    }
    if (t.count == kChunk || (i == ntensors && t.count > 0)) {
      launch(t);
      t.count = 0;
    }
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_unscale_check(float* const* g, const long long* sizes, int ntensors, float inv_scale,
                                float* found_inf, cudaStream_t stream) {
  return for_grad_chunks(g, sizes, ntensors, [&](const GradTable& t) {
    unscale_check_kernel<<<big_grid(), 256, 0, stream>>>(t, inv_scale, found_inf);
  });
}
extern "C" int fb_sumsq_multi(const float* const* g, const long long* sizes, int ntensors, float* out,
                              cudaStream_t stream) {
  return for_grad_chunks(const_cast<float* const*>(g), sizes, ntensors, [&](const GradTable& t) {
    sumsq_multi_kernel<<<big_grid(), 256, 0, stream>>>(t, out);
  });
}
extern "C" int fb_scale_multi(float* const* g, const long long* sizes, int ntensors, const float* total_sumsq,
                              float max_norm, float clip_value, int mode, cudaStream_t stream) {
  return for_grad_chunks(g, sizes, ntensors, [&](const GradTable& t) {
    scale_multi_kernel<<<big_grid(), 256, 0, stream>>>(t, total_sumsq, max_norm, clip_value, mode);
  });
}
