// Data-parallel gradient reduction in two kernels, for engines that keep the optimizer out of the backward pass:
//
//   fb_dist_reduce_scatter_shard   (per bucket, launched behind the bucket's last weight gradient, runs beside the
//                                   remaining backward GEMMs)   rank r sums ITS shard of the bucket over all ranks
//                                   with peer loads (or one multimem.ld_reduce through the NVSwitch), applies the
//                                   1 / world scale and leaves the result in its own gradient arena.
//   fb_dist_shard_update           (once per step, after backward)   for every bucket: SGD-momentum / Adam on the
//                                   rank's shard (fp32 master weights and moments stay with the owner) and the new
//                                   bf16 weights (optionally the fp32 ones too) stored into EVERY rank's arena —
//                                   the all-gather half of the all-reduce fused with the optimizer.
//
// Why two: a kernel that streams optimizer state (7 x 4 bytes per element of the shard) while the weight-gradient
// and data-gradient GEMMs run takes L2 and HBM bandwidth from kernels that are bound by exactly that, and with its
// register appetite it does not even fit on an SM beside a persistent GEMM CTA.  The reduce-scatter kernel is
// small (<= 80 registers, a block fits beside a GEMM CTA), reads each gradient once and writes 1 / world of them;
// the update then runs alone at the full HBM rate on 1 / world of the parameters.
//
// Synchronisation.  The reduce-scatter needs ONE handshake, at entry (all ranks' gradients of the bucket are
// complete).  Nobody overwrites gradients before the next backward pass, and the update kernel's entry handshake
// (every rank has finished its backward pass and all of its reduce-scatter kernels) comes before that, so no
// exit handshake is needed there.  The update kernel's entry handshake also guarantees that no peer still reads
// the bf16 weights it is about to overwrite; its exit handshake tells every rank that all shards have landed in
// its arena.  All waits are bounded (ctx.timeout_ns) and report through the status block.
//
// The reference's counterpart is the no-op loop of ferrum-distributed/src/ddp.rs:96-111 followed by the
// optimizer's own pass (ferrum-optim/src/adam.rs:91-146, sgd.rs).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../common/ptx.cuh"
#include "../common/status.h"
#include "../include/ferrum_kernels.h"
#include "dist_ctx.h"
#include "dist_device.cuh"

namespace fb {
namespace {

struct RsArgs {
  int channel;
  uint32_t epoch;
  const uint32_t* dev_epoch;  // NULL = use `epoch` (graph-capturable launches read the counter)
  long long grad_off;         // byte offset of the bucket's gradients inside every arena
  long long n;                // bucket length in elements (multiple of 4)
  float scale;
};

__device__ __forceinline__ void shard_bounds(long long n, int world, int rank, long long& lo, long long& hi) {
  long long per = (n + world - 1) / world;
  per = (per + 3) & ~3LL;
  lo = min(n, per * rank);
  hi = min(n, lo + per);
}

// One 16-byte group of the shard, all ranks summed (used for the ends that the 32-byte main loop leaves over).
template <bool MC, int W>
__device__ __forceinline__ float4 rs_group4(const fb_dist_ctx& c, long long grad_off, long long i4) {
  if (MC) return ptx::multimem_ld_reduce_add_f4(reinterpret_cast<const float4*>(c.mc_arena + grad_off) + i4);
  float4 g = ptx::ld_relaxed_sys_f4(reinterpret_cast<const float4*>(c.arena[0] + grad_off) + i4);
#pragma unroll
  for (int r = 1; r < W; ++r)
    if (r < c.world) {
      const float4 q = ptx::ld_relaxed_sys_f4(reinterpret_cast<const float4*>(c.arena[r] + grad_off) + i4);
      g.x += q.x; g.y += q.y; g.z += q.z; g.w += q.w;
    }
  return g;
}

// Peer-load form: 32 bytes per load instruction, marked evict-first in L2 and not allocated in L1 — the gradients
// stream past once while the GEMMs that run beside this kernel live on operand tiles cached in L2.  Ranks are read
// in groups of at most four so that U x 4 x 32 bytes are in flight per thread within the register budget.
template <bool MC, int U, int W>
__device__ void rs_body(const fb_dist_ctx& c, int vblock, int nvblocks, const RsArgs& a, int* s_fail) {
  const uint32_t epoch = a.dev_epoch != nullptr ? *a.dev_epoch : a.epoch;
  if (!block_handshake(c, a.channel, vblock, epoch, s_fail, 400)) return;
  long long lo, hi;
  shard_bounds(a.n, c.world, c.rank, lo, hi);
  const long long n4 = (hi - lo) >> 2, lo4 = lo >> 2;
  const long long stride = static_cast<long long>(nvblocks) * blockDim.x;
  float4* mine = reinterpret_cast<float4*>(c.arena[c.rank] + a.grad_off) + lo4;
  const long long tid = static_cast<long long>(vblock) * blockDim.x + threadIdx.x;
  if (MC) {
    for (long long base = tid; base < n4; base += stride * U) {
      float4 g[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i4 = base + u * stride;
        if (i4 < n4)
          g[u] = ptx::multimem_ld_reduce_add_f4(reinterpret_cast<const float4*>(c.mc_arena + a.grad_off) + lo4 + i4);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i4 = base + u * stride;
        if (i4 < n4) mine[i4] = make_float4(g[u].x * a.scale, g[u].y * a.scale, g[u].z * a.scale, g[u].w * a.scale);
      }
    }
    return;
  }
  // 16-byte groups before the first 32-byte boundary (0 or 1; the arenas share their alignment) and after the last
  const long long head = min(n4, static_cast<long long>((reinterpret_cast<uintptr_t>(mine) >> 4) & 1));
  const long long n8 = (n4 - head) >> 1;
  if (tid < head || (tid == 1 && head + 2 * n8 < n4)) {
    const long long i4 = tid < head ? 0 : n4 - 1;
    const float4 g = rs_group4<false, W>(c, a.grad_off, lo4 + i4);
    mine[i4] = make_float4(g.x * a.scale, g.y * a.scale, g.z * a.scale, g.w * a.scale);
  }
  constexpr int kG = W < 4 ? W : 4;  // ranks per group of loads
  const long long off8 = (lo4 + head) * 16;  // byte offset of the first 32-byte group inside the gradient region
  for (long long base = tid; base < n8; base += stride * U) {
    ptx::f8 acc[U];
#pragma unroll
    for (int r0 = 0; r0 < W; r0 += kG) {
      if (r0 >= c.world) break;
      ptx::f8 part[U][kG];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i8 = base + u * stride;
        if (i8 < n8) {
#pragma unroll
          for (int r = 0; r < kG; ++r)
            if (r0 + r < c.world)
              part[u][r] = ptx::ld_relaxed_sys_f8_stream(c.arena[r0 + r] + a.grad_off + off8 + i8 * 32);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int r = 0; r < kG; ++r)
          if (r0 + r < c.world) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              if (r0 + r == 0) acc[u].v[e] = part[u][r].v[e];
              else acc[u].v[e] += part[u][r].v[e];
            }
          }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i8 = base + u * stride;
      if (i8 < n8) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[u].v[e] *= a.scale;
        ptx::st_f8_stream(c.arena[c.rank] + a.grad_off + off8 + i8 * 32, acc[u]);
      }
    }
  }
}

template <bool MC, int U, int W>
__global__ void __launch_bounds__(256, 3)  // <= 80 registers: a block fits on an SM beside a persistent GEMM CTA
rs_kernel(const fb_dist_ctx c, const RsArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  rs_body<MC, U, W>(c, blockIdx.x, gridDim.x, a, &s_fail);
}

struct UpArgs {
  int channel;
  uint32_t epoch;
  const uint32_t* dev_epoch;
  long long grad_off, param_off, shadow_off;  // byte offsets of the three REGIONS (element 0 of the arena layout)
  const long long* table;                     // device: per bucket {start element, length, state offset, publish fp32}
  int nbuckets;
  fb_adam_hparams adam;
  fb_sgd_hparams sgd;
  float* m;  // this rank's moments, concatenated shards (table[][2] = first element of the bucket's shard)
  float* v;
  const float* dyn;  // NULL, or {lr, bias_corr1, bias_corr2, ...} in device memory
};

struct EmuUp {
  fb_dist_ctx c[FB_MAX_RANKS];
  float* m[FB_MAX_RANKS];
  float* v[FB_MAX_RANKS];
  int blocks_per_rank;
};

constexpr int kMaxUpBuckets = 256;  // rows of the bucket table one launch can take (kept in shared memory)

// The shards of all buckets form ONE index space of float4 positions (bucket after bucket), walked with a grid
// stride: a bucket whose shard is smaller than the grid (biases, normalisation parameters; every bucket once the
// world is large) then costs no trip of its own, and no trip ends with most of the grid idle.
template <int FUSE, bool MC, int U, bool CS = true>
__device__ void update_body(const fb_dist_ctx& c, int vblock, int nvblocks, const UpArgs& a, float* m_base,
                            float* v_base, int* s_fail) {
  __shared__ long long s_pre[kMaxUpBuckets + 1];  // first position of bucket k in the joint index space
  __shared__ long long s_e4[kMaxUpBuckets];       // first float4 of the rank's shard inside a region
  __shared__ long long s_so4[kMaxUpBuckets];      // first float4 of the shard inside m / v
  __shared__ unsigned char s_pub[kMaxUpBuckets];  // 1: fp32 values go to every rank
  const uint32_t epoch = a.dev_epoch != nullptr ? *a.dev_epoch : a.epoch;
  fb_adam_hparams adam = a.adam;
  fb_sgd_hparams sgd = a.sgd;
  if (a.dyn != nullptr) {
    adam.lr = a.dyn[0];
    adam.bias_corr1 = a.dyn[1];
    adam.bias_corr2 = a.dyn[2];
    sgd.lr = a.dyn[0];
  }
  for (int k = threadIdx.x; k < a.nbuckets; k += blockDim.x) {
    const long long start = a.table[4 * k], len = a.table[4 * k + 1];
    long long lo, hi;
    shard_bounds(len, c.world, c.rank, lo, hi);
    s_pre[k + 1] = (hi - lo) >> 2;  // lengths first, summed below
    s_e4[k] = (start + lo) >> 2;
    s_so4[k] = a.table[4 * k + 2] >> 2;
    s_pub[k] = a.table[4 * k + 3] != 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    s_pre[0] = 0;
    for (int k = 0; k < a.nbuckets; ++k) s_pre[k + 1] += s_pre[k];
  }
  if (!block_handshake(c, a.channel, vblock, epoch, s_fail, 410)) return;  // (its barriers publish the table)
  const long long total4 = s_pre[a.nbuckets];
  const long long stride = static_cast<long long>(nvblocks) * blockDim.x;
  unsigned char* self = c.arena[c.rank];
  const float4* gp = reinterpret_cast<const float4*>(self + a.grad_off);
  float4* pp = reinterpret_cast<float4*>(self + a.param_off);
  float4* mp = reinterpret_cast<float4*>(m_base);
  float4* vp = reinterpret_cast<float4*>(v_base);
  int cur = 0;  // bucket of this thread's first position of the trip; positions only grow
  for (long long base = static_cast<long long>(vblock) * blockDim.x + threadIdx.x; base < total4; base += stride * U) {
    float4 g[U], p[U], m[U], v[U];
    long long ri[U], si[U];  // float4 index inside a region / inside the moments
    bool pub[U];
    int bk = cur;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i4 = base + u * stride;
      if (i4 < total4) {
        while (i4 >= s_pre[bk + 1]) ++bk;
        if (u == 0) cur = bk;
        const long long j = i4 - s_pre[bk];
        ri[u] = s_e4[bk] + j;
        si[u] = s_so4[bk] + j;
        pub[u] = s_pub[bk] != 0;
        g[u] = CS ? __ldcs(gp + ri[u]) : gp[ri[u]];
        p[u] = pp[ri[u]];
        m[u] = (FUSE == FB_FUSE_ADAM || m_base != nullptr) ? (CS ? __ldcs(mp + si[u]) : mp[si[u]]) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (FUSE == FB_FUSE_ADAM) v[u] = CS ? __ldcs(vp + si[u]) : vp[si[u]];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (base + u * stride >= total4) continue;
      if (FUSE == FB_FUSE_ADAM) {
        adam1(p[u].x, g[u].x, m[u].x, v[u].x, adam);
        adam1(p[u].y, g[u].y, m[u].y, v[u].y, adam);
        adam1(p[u].z, g[u].z, m[u].z, v[u].z, adam);
        adam1(p[u].w, g[u].w, m[u].w, v[u].w, adam);
        if (CS) {
          __stcs(mp + si[u], m[u]);
          __stcs(vp + si[u], v[u]);
        } else {
          mp[si[u]] = m[u];
          vp[si[u]] = v[u];
        }
      } else {
        sgd1(p[u].x, g[u].x, m[u].x, sgd);
        sgd1(p[u].y, g[u].y, m[u].y, sgd);
        sgd1(p[u].z, g[u].z, m[u].z, sgd);
        sgd1(p[u].w, g[u].w, m[u].w, sgd);
        if (m_base != nullptr) __stcs(mp + si[u], m[u]);
      }
      uint2 sh;
      *reinterpret_cast<__nv_bfloat162*>(&sh.x) = __floats2bfloat162_rn(p[u].x, p[u].y);
      *reinterpret_cast<__nv_bfloat162*>(&sh.y) = __floats2bfloat162_rn(p[u].z, p[u].w);
      if (!pub[u]) pp[ri[u]] = p[u];  // the owner keeps the fp32 master; peers only need the bf16 copy
      if (MC) {
        if (pub[u]) ptx::multimem_st_f4(reinterpret_cast<float4*>(c.mc_arena + a.param_off) + ri[u], p[u]);
        if (a.shadow_off >= 0)
          ptx::multimem_st_f2(reinterpret_cast<float2*>(c.mc_arena + a.shadow_off) + ri[u],
                              make_float2(__uint_as_float(sh.x), __uint_as_float(sh.y)));
      } else {
        // Plain (weak) stores, to the peers' memory too: the exit handshake orders them.  Its barrier makes every
        // store of the block happen before the flag writers' fence.sys, which is cumulative, and only then is
        // the flag released; a reader that has seen all flags therefore sees all data.  (Measured level with
        // st.relaxed.sys stores on one and two GPUs; the weak form leaves the hardware free to combine them.)
        for (int r = 0; r < c.world; ++r) {
          if (pub[u]) *(reinterpret_cast<float4*>(c.arena[r] + a.param_off) + ri[u]) = p[u];
          if (a.shadow_off >= 0) *(reinterpret_cast<uint2*>(c.arena[r] + a.shadow_off) + ri[u]) = sh;
        }
      }
    }
  }
  block_handshake(c, a.channel, vblock, epoch + 1, s_fail, 411);
}

// One 16-byte group of g, p, m, v per thread and trip with ordinary loads and stores: measured on one GPU (131 M
// parameters, 592 blocks) 635 us against 646 us with two groups per trip and streaming hints.
template <int FUSE, bool MC, int U = 1, bool CS = false>
__global__ void __launch_bounds__(256)
update_kernel(const fb_dist_ctx c, const UpArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  update_body<FUSE, MC, U, CS>(c, blockIdx.x, gridDim.x, a, a.m, a.v, &s_fail);
}

// All ranks in ONE cooperative launch on one GPU (virtual rank = blockIdx.x / blocks_per_rank): the protocol can
// be exercised where a single GPU is available; separate launches that wait on each other never share a GPU.
struct EmuRs {
  fb_dist_ctx c[FB_MAX_RANKS];
  int blocks_per_rank;
};
__global__ void __launch_bounds__(256)
rs_emulated_kernel(const EmuRs pk, const RsArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  rs_body<false, 1, FB_MAX_RANKS>(pk.c[blockIdx.x / pk.blocks_per_rank], blockIdx.x % pk.blocks_per_rank,
                                  pk.blocks_per_rank, a, &s_fail);
}
template <int FUSE>
__global__ void __launch_bounds__(256)
update_emulated_kernel(const EmuUp pk, const UpArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int vr = blockIdx.x / pk.blocks_per_rank;
  update_body<FUSE, false, 1>(pk.c[vr], blockIdx.x % pk.blocks_per_rank, pk.blocks_per_rank, a, pk.m[vr], pk.v[vr],
                              &s_fail);
}

__global__ void counter_advance_kernel(unsigned* ctr, unsigned inc) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *ctr += inc;
}

bool launch_ok(const fb_dist_ctx* ctx, int channel, int nblocks, int nthreads) {
  return ctx_ok(ctx) && nblocks >= 1 && nblocks <= FB_FLAG_BLOCKS && nthreads >= 32 && nthreads <= 256 &&
         channel >= 0 && channel < FB_FLAG_CHANNELS;
}

}  // namespace
}  // namespace fb

using namespace fb;

// Sum of this rank's shard of the bucket at grad_off (n elements, a multiple of 4) over all ranks, times `scale`,
// left in this rank's own arena.  Consumes `epoch` on `channel` (callers advance by 2, like every collective);
// with dev_epoch the epoch is read from that device counter, which is advanced by 2 on the stream afterwards.
extern "C" int fb_dist_reduce_scatter_shard(const fb_dist_ctx* ctx, int use_mc, int channel, unsigned epoch,
                                            unsigned* dev_epoch, long long grad_off, long long n, float scale,
                                            int nblocks, int nthreads, cudaStream_t stream) {
  if (!launch_ok(ctx, channel, nblocks, nthreads) || n <= 0 || (n & 3) || (grad_off & 15)) return -1;
  if (use_mc && ctx->mc_arena == nullptr) return -2;
  RsArgs a{channel, epoch, dev_epoch, grad_off, n, scale};
  // bytes in flight per thread = U x world x 16 (peer loads): deeper unrolling for small worlds
  if (use_mc) rs_kernel<true, 4, 1><<<nblocks, nthreads, 0, stream>>>(*ctx, a);
  else if (ctx->world <= 2) rs_kernel<false, 2, 2><<<nblocks, nthreads, 0, stream>>>(*ctx, a);
  else if (ctx->world <= 4) rs_kernel<false, 1, 4><<<nblocks, nthreads, 0, stream>>>(*ctx, a);
  else rs_kernel<false, 1, FB_MAX_RANKS><<<nblocks, nthreads, 0, stream>>>(*ctx, a);
  int rc = static_cast<int>(cudaGetLastError());
  if (rc == 0 && dev_epoch != nullptr) {
    counter_advance_kernel<<<1, 32, 0, stream>>>(dev_epoch, 2u);
    rc = static_cast<int>(cudaGetLastError());
  }
  return rc;
}

// Optimizer update of this rank's shards of `nbuckets` buckets and publication of the new weights to all ranks.
// table (device memory, 4 x 64-bit per bucket): {first element of the bucket in the arena layout, length, first
// element of the bucket's shard inside m / v, 1 = the new fp32 values go to every rank / 0 = only the bf16 copy
// does and the owner keeps the fp32 master}.  fuse: FB_FUSE_SGD (m = velocity or NULL) or FB_FUSE_ADAM.  Gradients are
// expected reduced and scaled (grad_scale of the hyper-parameters still applies).  Consumes epoch, epoch + 1.
extern "C" int fb_dist_shard_update(const fb_dist_ctx* ctx, int fuse, int use_mc, int channel, unsigned epoch,
                                    unsigned* dev_epoch, long long grad_off, long long param_off,
                                    long long shadow_off, const long long* table, int nbuckets,
                                    const fb_adam_hparams* adam, const fb_sgd_hparams* sgd, float* m, float* v,
                                    int nblocks, int nthreads, const float* dyn, cudaStream_t stream) {
  if (!launch_ok(ctx, channel, nblocks, nthreads) || table == nullptr || nbuckets < 1 || nbuckets > kMaxUpBuckets)
    return -1;
  if ((grad_off & 15) || (param_off & 15) || (shadow_off >= 0 && (shadow_off & 7))) return -1;
  if (use_mc && ctx->mc_arena == nullptr) return -2;
  UpArgs a{};
  a.channel = channel;
  a.epoch = epoch;
  a.dev_epoch = dev_epoch;
  a.grad_off = grad_off;
  a.param_off = param_off;
  a.shadow_off = shadow_off;
  a.table = table;
  a.nbuckets = nbuckets;
  if (adam) a.adam = *adam;
  if (sgd) a.sgd = *sgd;
  a.m = m;
  a.v = v;
  a.dyn = dyn;
  if (fuse == FB_FUSE_ADAM) {
    if (adam == nullptr || m == nullptr || v == nullptr) return -3;
    if (use_mc) update_kernel<FB_FUSE_ADAM, true><<<nblocks, nthreads, 0, stream>>>(*ctx, a);
    else update_kernel<FB_FUSE_ADAM, false><<<nblocks, nthreads, 0, stream>>>(*ctx, a);
  } else if (fuse == FB_FUSE_SGD) {
    if (sgd == nullptr) return -3;
    if (use_mc) update_kernel<FB_FUSE_SGD, true><<<nblocks, nthreads, 0, stream>>>(*ctx, a);
    else update_kernel<FB_FUSE_SGD, false><<<nblocks, nthreads, 0, stream>>>(*ctx, a);
  } else {
    return -1;
  }
  int rc = static_cast<int>(cudaGetLastError());
  if (rc == 0 && dev_epoch != nullptr) {
    counter_advance_kernel<<<1, 32, 0, stream>>>(dev_epoch, 2u);
    rc = static_cast<int>(cudaGetLastError());
  }
  return rc;
}

// The same two kernels with all `world` ranks emulated on the current GPU in one cooperative launch each.
extern "C" int fb_dist_reduce_scatter_shard_emulated(const fb_dist_ctx* ctxs, int world, int channel, unsigned epoch,
                                                     long long grad_off, long long n, float scale, int nblocks,
                                                     int nthreads, cudaStream_t stream) {
  if (world < 1 || world > FB_MAX_RANKS || n <= 0 || (n & 3) || nblocks < 1 || nblocks > FB_FLAG_BLOCKS) return -1;
  EmuRs pk{};
  for (int r = 0; r < world; ++r) {
    if (!ctx_ok(&ctxs[r]) || ctxs[r].world != world || ctxs[r].rank != r) return -1;
    pk.c[r] = ctxs[r];
  }
  pk.blocks_per_rank = nblocks;
  RsArgs a{channel, epoch, nullptr, grad_off, n, scale};
  void* args[] = {&pk, &a};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(rs_emulated_kernel),
                                                      dim3(world * nblocks), dim3(nthreads), args, 0, stream));
}

extern "C" int fb_dist_shard_update_emulated(const fb_dist_ctx* ctxs, int world, int fuse, int channel,
                                             unsigned epoch, long long grad_off, long long param_off,
                                             long long shadow_off, const long long* table, int nbuckets,
                                             const fb_adam_hparams* adam, const fb_sgd_hparams* sgd,
                                             float* const* m, float* const* v, int nblocks, int nthreads,
                                             cudaStream_t stream) {
  if (world < 1 || world > FB_MAX_RANKS || table == nullptr || nbuckets < 1 || nbuckets > kMaxUpBuckets ||
      nblocks < 1 || nblocks > FB_FLAG_BLOCKS)
    return -1;
  EmuUp pk{};
  for (int r = 0; r < world; ++r) {
    if (!ctx_ok(&ctxs[r]) || ctxs[r].world != world || ctxs[r].rank != r) return -1;
    pk.c[r] = ctxs[r];
    pk.m[r] = m ? m[r] : nullptr;
    pk.v[r] = v ? v[r] : nullptr;
  }
  pk.blocks_per_rank = nblocks;
  UpArgs a{};
  a.channel = channel;
  a.epoch = epoch;
  a.grad_off = grad_off;
  a.param_off = param_off;
  a.shadow_off = shadow_off;
  a.table = table;
  a.nbuckets = nbuckets;
  if (adam) a.adam = *adam;
  if (sgd) a.sgd = *sgd;
  void* args[] = {&pk, &a};
  const void* fn = fuse == FB_FUSE_ADAM ? reinterpret_cast<const void*>(update_emulated_kernel<FB_FUSE_ADAM>)
                                        : reinterpret_cast<const void*>(update_emulated_kernel<FB_FUSE_SGD>);
  return static_cast<int>(cudaLaunchCooperativeKernel(fn, dim3(world * nblocks), dim3(nthreads), args, 0, stream));
}
