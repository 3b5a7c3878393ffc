// Activation value and derivative for the GEMM epilogues.  A Linear -> activation -> LayerNorm block
// stores act(z) and act'(z) straight from the accumulator, so neither the normalisation kernel nor its
// backward has to evaluate the activation again (for GELU that is a tanh plus a dozen multiply-adds per
// element in kernels that are otherwise pure streaming).
#pragma once
#include "../include/ferrum_kernels.h"

namespace fb {

__device__ __forceinline__ float tanh_approx(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}

__device__ __forceinline__ void act_both(float x, int act, float& val, float& der) {
  switch (act) {
    case FB_ACT_RELU:
      val = fmaxf(x, 0.f);
      der = x > 0.f ? 1.f : 0.f;
      break;
    case FB_ACT_GELU: {
      const float x2 = x * x;
      const float t = tanh_approx(x * fmaf(x2, 0.7978845608028654f * 0.044715f, 0.7978845608028654f));
      const float hx = 0.5f * x;
      val = fmaf(hx, t, hx);
      der = fmaf(hx * fmaf(-t, t, 1.f), fmaf(x2, 3.f * 0.7978845608028654f * 0.044715f, 0.7978845608028654f),
                 fmaf(t, 0.5f, 0.5f));
      break;
    }
    case FB_ACT_SILU: {
      const float s = 1.f / (1.f + __expf(-x));
      val = x * s;
      der = s * fmaf(x, 1.f - s, 1.f);
      break;
    }
    case FB_ACT_TANH: {
      const float t = tanh_approx(x);
      val = t;
      der = fmaf(-t, t, 1.f);
      break;
    }
    case FB_ACT_SIGMOID: {
      const float s = 1.f / (1.f + __expf(-x));
      val = s;
      der = s * (1.f - s);
      break;
    }
    default:
      val = x;
      der = 1.f;
      break;
  }
}


template <int ACT>
__device__ __forceinline__ float act_value(float x) {
  if (ACT == FB_ACT_RELU) return fmaxf(x, 0.f);
  if (ACT == FB_ACT_GELU) {
    const float t = tanh_approx(x * fmaf(x * x, 0.7978845608028654f * 0.044715f, 0.7978845608028654f));
    const float hx = 0.5f * x;
    return fmaf(hx, t, hx);
  }
  if (ACT == FB_ACT_SILU) return x / (1.f + __expf(-x));
  if (ACT == FB_ACT_TANH) return tanh_approx(x);
  if (ACT == FB_ACT_SIGMOID) return 1.f / (1.f + __expf(-x));
  return x;
}

// The activation is chosen ONCE per 32-column chunk; a switch evaluated per element costs more issue slots
// than the activation itself and made the epilogue the bottleneck of the GEMM.
template <int ACT>
__device__ __forceinline__ void act_chunk_t(float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = act_value<ACT>(v[i]);
}
__device__ __forceinline__ void act_chunk(float (&v)[32], int act) {
  switch (act) {
    case FB_ACT_RELU: act_chunk_t<FB_ACT_RELU>(v); break;
    case FB_ACT_GELU: act_chunk_t<FB_ACT_GELU>(v); break;
    case FB_ACT_SILU: act_chunk_t<FB_ACT_SILU>(v); break;
    case FB_ACT_TANH: act_chunk_t<FB_ACT_TANH>(v); break;
    case FB_ACT_SIGMOID: act_chunk_t<FB_ACT_SIGMOID>(v); break;
    default: break;
  }
}

// v <- act(v), d <- act'(v) for a 32-column chunk.
template <int ACT>
__device__ __forceinline__ void act_both_chunk_t(float (&v)[32], float (&d)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float a, g;
    act_both(v[i], ACT, a, g);  // ACT is a constant here: the switch folds away
    v[i] = a;
    d[i] = g;
  }
}
__device__ __forceinline__ void act_both_chunk(float (&v)[32], float (&d)[32], int act) {
  switch (act) {
    case FB_ACT_RELU: act_both_chunk_t<FB_ACT_RELU>(v, d); break;
    case FB_ACT_GELU: act_both_chunk_t<FB_ACT_GELU>(v, d); break;
    case FB_ACT_SILU: act_both_chunk_t<FB_ACT_SILU>(v, d); break;
    case FB_ACT_TANH: act_both_chunk_t<FB_ACT_TANH>(v, d); break;
    case FB_ACT_SIGMOID: act_both_chunk_t<FB_ACT_SIGMOID>(v, d); break;
    default: act_both_chunk_t<FB_ACT_NONE>(v, d); break;
  }
}

}  // namespace fb
