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

}  // namespace fb
