// Device-side pieces shared by the inter-GPU kernels: the flag slots of the handshake, the bounded block
// handshake itself, and the per-element optimizer rules the fused kernels apply.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "../common/ptx.cuh"
#include "../common/status.h"
#include "../include/ferrum_kernels.h"
#include "dist_ctx.h"

namespace fb {

__device__ __forceinline__ uint32_t* flag_slot(unsigned char* arena, int channel, int block, int src) {
  return reinterpret_cast<uint32_t*>(arena) + ((channel * FB_FLAG_BLOCKS + block) * FB_MAX_RANKS + src);
}

// Called by every thread of the block.  Returns false (for the whole block) if a wait gave up.
__device__ inline bool block_handshake(const fb_dist_ctx& c, int channel, int vblock, uint32_t epoch, int* s_fail,
                                int site) {
  __syncthreads();
  if (threadIdx.x < c.world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    ptx::st_release_sys(flag_slot(c.arena[peer], channel, vblock, c.rank), epoch);
    const uint32_t* mine = flag_slot(c.arena[c.rank], channel, vblock, peer);
    const uint64_t t0 = ptx::globaltimer();
    uint32_t it = 0;
    while (static_cast<int32_t>(ptx::ld_acquire_sys(mine) - epoch) < 0) {
      if (((++it) & 31u) == 0u) {
        if (*reinterpret_cast<volatile int*>(s_fail)) break;
        if (ptx::globaltimer() - t0 > c.timeout_ns) {
          report_status(c.status, kStatusPeerTimeout, site, peer, static_cast<int32_t>(epoch));
          *reinterpret_cast<volatile int*>(s_fail) = 1;
          break;
        }
      }
    }
  }
  __syncthreads();
  return *reinterpret_cast<volatile int*>(s_fail) == 0;
}

__device__ __forceinline__ void adam1(float& p, float g, float& m, float& v, const fb_adam_hparams& h) {
  g *= h.grad_scale;
  if (h.weight_decay != 0.f) p -= h.lr * h.weight_decay * p;
  m = h.beta1 * m + (1.f - h.beta1) * g;
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  p -= h.lr * (m / h.bias_corr1) / (sqrtf(v / h.bias_corr2) + h.eps);
}
__device__ __forceinline__ void sgd1(float& p, float g, float& vel, const fb_sgd_hparams& h) {
  g *= h.grad_scale;
  if (h.weight_decay != 0.f) g += h.weight_decay * p;
  float upd = g;
  if (h.momentum != 0.f) {
    vel = h.first_step ? g : h.momentum * vel + g;
    upd = h.nesterov ? g + h.momentum * vel : vel;
  }
  p -= h.lr * upd;
}

inline bool ctx_ok(const fb_dist_ctx* c) {
  return c != nullptr && c->world >= 1 && c->world <= FB_MAX_RANKS && c->rank >= 0 && c->rank < c->world;
}

}  // namespace fb
