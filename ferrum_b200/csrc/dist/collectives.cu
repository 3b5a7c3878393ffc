// Inter-GPU kernels over NVLink 5 / NVSwitch.  Every rank owns a "symmetric
// arena" (same layout on every GPU, mapped into every peer's address space) and
// the kernels move data with plain peer loads / stores issued from inside the
// kernel, or with multimem.ld_reduce / multimem.st through the NVSwitch multicast
// alias when one is set up.  No library collective is called and no TMA multicast
// is used anywhere.
//
//   fused all-reduce (+ 1/world scale) (+ SGD-momentum | Adam update + parameter
//   publish)              -> fb_dist_allreduce          (gradient buckets of DDP)
//   broadcast / all-gather / gather / scatter / reduce-scatter / reduce
//                          -> fb_dist_collective
//   barrier                -> fb_dist_barrier
//
// The reference declares these operations and implements them as no-ops
// (ferrum-distributed/src/collectives.rs:74-129; ddp.rs:96-111 loops over them).
//
// Algorithm of the fused all-reduce (two-shot, shard-owner update): rank r owns the
// r-th shard of the bucket.  After an entry handshake it sums that shard over all
// ranks (reads of the peers' gradient arenas), applies the scale and the optimizer
// rule to its fp32 master copy and the moments it alone keeps for the shard, and
// stores the new fp32 parameters and their bf16 copy into EVERY rank's arena.  An
// exit handshake tells each rank that all shards have arrived and that nobody still
// reads its gradients.  Per element the link carries one gradient read and one
// parameter write per peer — the cost of an all-reduce — and the separate optimizer
// pass over memory disappears.
//
// Handshakes are per (channel, block): block b of every rank writes an epoch into
// slot [channel][b][its rank] of every peer's flag region and waits until its own
// region shows that epoch from every peer.  Waits are bounded by ctx.timeout_ns;
// on expiry the block records {peer, epoch} in the status block, the kernel skips
// the rest of its work and returns.
#include <cuda_bf16.h>

#include <cstdlib>
#include <cuda_runtime.h>

#include "../common/ptx.cuh"
#include "../common/status.h"
#include "../include/ferrum_kernels.h"
#include "dist_ctx.h"
#include "dist_device.cuh"

namespace fb {
namespace {

struct ArArgs {
  int channel;
  uint32_t epoch;
  long long grad_off;    // byte offsets into the arena
  long long param_off;   // fp32 master parameters (fused modes)
  long long shadow_off;  // bf16 copy of the parameters (fused modes; <0 = none)
  long long n;           // bucket length in elements (multiple of 4)
  int op;
  float scale;
  fb_adam_hparams adam;
  fb_sgd_hparams sgd;
  float* m;  // this rank's moment / velocity storage for ITS shard (index 0 = first element of the shard)
  float* v;
  int publish_master;  // 1: new fp32 parameters go to every rank; 0: only the bf16 copy does (owner keeps fp32)
  // Graph-capturable launches: the handshake epoch and the step-dependent optimizer factors come from device
  // memory (advanced by tiny kernels on the same stream), not from the by-value arguments a graph would freeze.
  const uint32_t* dev_epoch;  // NULL = use `epoch`
  const float* dyn;           // NULL = use adam / sgd as given; else {lr, bias_corr1, bias_corr2, ...}
  // Plain all-reduce of a tensor that lives OUTSIDE the arena: each block copies the positions it will handshake
  // for from stage_in into the region at grad_off before the entry handshake and copies the reduced values back to
  // stage_out after the exit handshake, so no separate staging launches are needed.  n_valid <= n elements are
  // real; the rest of the region is zero-filled and never copied back.
  const float* stage_in;
  float* stage_out;
  long long n_valid;
  // Ranges [lo, hi) of the bucket (elements, multiples of 4) whose gradients were PUSHED by the producing GEMMs:
  // source rank s stored its values for shard o at element s * per + j of rank o's bucket region, so the owner
  // finds all contributions in its own memory and reads no peer for them.
  int n_pushed;
  long long pushed_lo[4], pushed_hi[4];
  int streaming;       // local optimizer state moves with evict-first hints (ld/st.global.cs): it is touched once per
                       // step and should not displace the operand tiles of the GEMMs this kernel runs beside
};

__device__ __forceinline__ float4 combine4(float4 a, float4 b, int op) {
  switch (op) {
    case FB_OP_PROD: return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w);
    case FB_OP_MIN: return make_float4(fminf(a.x, b.x), fminf(a.y, b.y), fminf(a.z, b.z), fminf(a.w, b.w));
    case FB_OP_MAX: return make_float4(fmaxf(a.x, b.x), fmaxf(a.y, b.y), fmaxf(a.z, b.z), fmaxf(a.w, b.w));
    default: return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
  }
}

// Copies between a local tensor and this rank's arena region for the positions block `vblock` owns in EVERY
// shard (the same relative positions that the peers' blocks of this index read and write).
template <bool IN>
__device__ void stage_block(const fb_dist_ctx& c, int vblock, int nvblocks, const ArArgs& a) {
  long long per = (a.n + c.world - 1) / c.world;
  per = (per + 3) & ~3LL;
  const long long stride = static_cast<long long>(nvblocks) * blockDim.x;
  float4* region = reinterpret_cast<float4*>(c.arena[c.rank] + a.grad_off);
  const bool vec = ((reinterpret_cast<uintptr_t>(IN ? static_cast<const void*>(a.stage_in)
                                                    : static_cast<const void*>(a.stage_out)) & 15) == 0);
  for (int r = 0; r < c.world; ++r) {
    const long long lo = min(a.n, per * r);
    const long long hi = min(a.n, lo + per);
    const long long n4 = (hi - lo) >> 2, lo4 = lo >> 2;
    long long i4 = static_cast<long long>(vblock) * blockDim.x + threadIdx.x;
    if (vec && hi <= a.n_valid) {
      // whole shard is real data and 16-byte aligned on both sides: eight independent vectors in flight per thread
      constexpr int kU = 8;
      for (; i4 + (kU - 1) * stride < n4; i4 += stride * kU) {
        float4 x[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const long long k = lo4 + i4 + u * stride;
          x[u] = IN ? reinterpret_cast<const float4*>(a.stage_in)[k] : ptx::ld_relaxed_sys_f4(region + k);
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const long long k = lo4 + i4 + u * stride;
          if (IN) region[k] = x[u];
          else reinterpret_cast<float4*>(a.stage_out)[k] = x[u];
        }
      }
    }
    for (; i4 < n4; i4 += stride) {
      const long long e = (lo4 + i4) << 2;  // first element of this float4
      if (IN) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (vec && e + 4 <= a.n_valid) {
          x = *reinterpret_cast<const float4*>(a.stage_in + e);
        } else {
          if (e < a.n_valid) x.x = a.stage_in[e];
          if (e + 1 < a.n_valid) x.y = a.stage_in[e + 1];
          if (e + 2 < a.n_valid) x.z = a.stage_in[e + 2];
          if (e + 3 < a.n_valid) x.w = a.stage_in[e + 3];
        }
        region[lo4 + i4] = x;
      } else {
        if (e >= a.n_valid) continue;
        // read at the L2 (the peers' stores arrive there; this SM's L1 may still hold what stage-in wrote)
        const float4 x = ptx::ld_relaxed_sys_f4(region + lo4 + i4);
        if (vec && e + 4 <= a.n_valid) {
          *reinterpret_cast<float4*>(a.stage_out + e) = x;
        } else {
          a.stage_out[e] = x.x;
          if (e + 1 < a.n_valid) a.stage_out[e + 1] = x.y;
          if (e + 2 < a.n_valid) a.stage_out[e + 2] = x.z;
          if (e + 3 < a.n_valid) a.stage_out[e + 3] = x.w;
        }
      }
    }
  }
}

// Reduce the shard of rank c.rank over all ranks, (optionally) update, publish to all ranks.
// Each thread keeps U independent float4 positions in flight: a peer load costs a round trip over
// NVLink (microseconds), so throughput is set by the bytes outstanding per SM, not by the thread count.
template <int FUSE, bool MC, int U, int W>
__device__ void allreduce_body(const fb_dist_ctx& c, int vblock, int nvblocks, const ArArgs& a, int* s_fail) {
  const uint32_t epoch = a.dev_epoch != nullptr ? *a.dev_epoch : a.epoch;
  fb_adam_hparams adam = a.adam;
  fb_sgd_hparams sgd = a.sgd;
  if (a.dyn != nullptr) {
    adam.lr = a.dyn[0];
    adam.bias_corr1 = a.dyn[1];
    adam.bias_corr2 = a.dyn[2];
    sgd.lr = a.dyn[0];
  }
  if (FUSE == FB_FUSE_NONE && a.stage_in != nullptr) stage_block<true>(c, vblock, nvblocks, a);
  if (!block_handshake(c, a.channel, vblock, epoch, s_fail, 100)) return;

  long long per = (a.n + c.world - 1) / c.world;
  per = (per + 3) & ~3LL;
  const long long lo = min(a.n, per * c.rank);
  const long long hi = min(a.n, lo + per);
  const long long n4 = (hi - lo) >> 2;
  const long long stride = static_cast<long long>(nvblocks) * blockDim.x;
  const long long lo4 = lo >> 2;

  for (long long base = static_cast<long long>(vblock) * blockDim.x + threadIdx.x; base < n4; base += stride * U) {
    float4 g[U];
    if (MC) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i4 = base + u * stride;
        if (i4 < n4)
          g[u] = ptx::multimem_ld_reduce_add_f4(reinterpret_cast<const float4*>(c.mc_arena + a.grad_off) + lo4 + i4);
      }
    } else {
      float4 part[U][W];  // W = compile-time bound on the world size, so the table stays in registers
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i4 = base + u * stride;
        if (i4 < n4) {
          bool pushed = false;
          if (a.n_pushed > 0) {
            const long long e = lo + (i4 << 2);
#pragma unroll
            for (int q = 0; q < 4; ++q) pushed |= (q < a.n_pushed && e >= a.pushed_lo[q] && e < a.pushed_hi[q]);
          }
          if (pushed) {
            // contributions of all ranks already sit in this rank's memory, one slot of `per` elements per source
            const float4* mine = reinterpret_cast<const float4*>(c.arena[c.rank] + a.grad_off);
#pragma unroll
            for (int r = 0; r < W; ++r)
              if (r < c.world) part[u][r] = ptx::ld_relaxed_sys_f4(mine + r * (per >> 2) + i4);
          } else {
#pragma unroll
            for (int r = 0; r < W; ++r)
              if (r < c.world)
                part[u][r] =
                    ptx::ld_relaxed_sys_f4(reinterpret_cast<const float4*>(c.arena[r] + a.grad_off) + lo4 + i4);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (base + u * stride < n4) {
          g[u] = part[u][0];
#pragma unroll
          for (int r = 1; r < W; ++r)
            if (r < c.world) g[u] = combine4(g[u], part[u][r], a.op);
        }
      }
    }
    if (FUSE == FB_FUSE_NONE) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i4 = base + u * stride;
        if (i4 >= n4) continue;
        float4 x = g[u];
        x.x *= a.scale; x.y *= a.scale; x.z *= a.scale; x.w *= a.scale;
        if (MC) {
          ptx::multimem_st_f4(reinterpret_cast<float4*>(c.mc_arena + a.grad_off) + lo4 + i4, x);
        } else {
#pragma unroll
          for (int r = 0; r < W; ++r)
            if (r < c.world) ptx::st_relaxed_sys_f4(reinterpret_cast<float4*>(c.arena[r] + a.grad_off) + lo4 + i4, x);
        }
      }
    } else {
      float4 p[U], m[U], v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i4 = base + u * stride;
        if (i4 < n4) {
          p[u] = *(reinterpret_cast<const float4*>(c.arena[c.rank] + a.param_off) + lo4 + i4);
          if (FUSE == FB_FUSE_ADAM) {
            if (a.streaming) {
              m[u] = __ldcs(reinterpret_cast<const float4*>(a.m) + i4);
              v[u] = __ldcs(reinterpret_cast<const float4*>(a.v) + i4);
            } else {
              m[u] = reinterpret_cast<const float4*>(a.m)[i4];
              v[u] = reinterpret_cast<const float4*>(a.v)[i4];
            }
          } else {
            m[u] = a.m != nullptr ? reinterpret_cast<const float4*>(a.m)[i4] : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i4 = base + u * stride;
        if (i4 >= n4) continue;
        if (FUSE == FB_FUSE_ADAM) {
          adam1(p[u].x, g[u].x, m[u].x, v[u].x, adam);
          adam1(p[u].y, g[u].y, m[u].y, v[u].y, adam);
          adam1(p[u].z, g[u].z, m[u].z, v[u].z, adam);
          adam1(p[u].w, g[u].w, m[u].w, v[u].w, adam);
          if (a.streaming) {
            __stcs(reinterpret_cast<float4*>(a.m) + i4, m[u]);
            __stcs(reinterpret_cast<float4*>(a.v) + i4, v[u]);
          } else {
            reinterpret_cast<float4*>(a.m)[i4] = m[u];
            reinterpret_cast<float4*>(a.v)[i4] = v[u];
          }
        } else {
          sgd1(p[u].x, g[u].x, m[u].x, sgd);
          sgd1(p[u].y, g[u].y, m[u].y, sgd);
          sgd1(p[u].z, g[u].z, m[u].z, sgd);
          sgd1(p[u].w, g[u].w, m[u].w, sgd);
          if (a.m != nullptr) reinterpret_cast<float4*>(a.m)[i4] = m[u];
        }
        uint2 sh;
        *reinterpret_cast<__nv_bfloat162*>(&sh.x) = __floats2bfloat162_rn(p[u].x, p[u].y);
        *reinterpret_cast<__nv_bfloat162*>(&sh.y) = __floats2bfloat162_rn(p[u].z, p[u].w);
        if (!a.publish_master)
          *(reinterpret_cast<float4*>(c.arena[c.rank] + a.param_off) + lo4 + i4) = p[u];
        if (MC) {
          if (a.publish_master)
            ptx::multimem_st_f4(reinterpret_cast<float4*>(c.mc_arena + a.param_off) + lo4 + i4, p[u]);
          if (a.shadow_off >= 0)
            ptx::multimem_st_f2(reinterpret_cast<float2*>(c.mc_arena + a.shadow_off) + lo4 + i4,
                                make_float2(__uint_as_float(sh.x), __uint_as_float(sh.y)));
        } else {
#pragma unroll
          for (int r = 0; r < W; ++r)
            if (r < c.world) {
              if (a.publish_master)
                ptx::st_relaxed_sys_f4(reinterpret_cast<float4*>(c.arena[r] + a.param_off) + lo4 + i4, p[u]);
              if (a.shadow_off >= 0)
                ptx::st_relaxed_sys_u2(reinterpret_cast<uint2*>(c.arena[r] + a.shadow_off) + lo4 + i4, sh);
            }
        }
      }
    }
  }
  const bool done = block_handshake(c, a.channel, vblock, epoch + 1, s_fail, 101);
  if (FUSE == FB_FUSE_NONE && a.stage_out != nullptr && done) stage_block<false>(c, vblock, nvblocks, a);
}

template <int FUSE, bool MC, int U, int W>
__global__ void __launch_bounds__(256)
allreduce_kernel(const fb_dist_ctx c, const ArArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  allreduce_body<FUSE, MC, U, W>(c, blockIdx.x, gridDim.x, a, &s_fail);
}

// All ranks of a job emulated by ONE cooperative launch on one GPU: virtual rank =
// blockIdx.x / blocks_per_rank.  Used to exercise the multi-rank protocol where only a
// single GPU is available (separate launches that wait on each other must never share a GPU).
struct EmuPack {
  fb_dist_ctx c[FB_MAX_RANKS];
  float* m[FB_MAX_RANKS];
  float* v[FB_MAX_RANKS];
  const float* stage_in[FB_MAX_RANKS];  // per virtual rank: tensor outside the arena (NULL = none)
  float* stage_out[FB_MAX_RANKS];
  int blocks_per_rank;
};

template <int FUSE>
__global__ void __launch_bounds__(256)
allreduce_emulated_kernel(const EmuPack pk, ArArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int vr = blockIdx.x / pk.blocks_per_rank;
  const int vb = blockIdx.x % pk.blocks_per_rank;
  a.m = pk.m[vr];
  a.v = pk.v[vr];
  a.stage_in = pk.stage_in[vr];
  a.stage_out = pk.stage_out[vr];
  allreduce_body<FUSE, false, 1, FB_MAX_RANKS>(pk.c[vr], vb, pk.blocks_per_rank, a, &s_fail);
}

// ------------------------------------------------------------- one-shot all-reduce (small messages)
// Latency form for messages of a few hundred KB at most: every rank puts its tensor into its own arena region,
// ONE handshake follows, then every rank reads all regions and reduces for itself, straight into its result
// tensor.  The two-shot form above needs a second trip over the link (publication of the reduced shards) and a
// second handshake.  No exit handshake is needed because the region alternates between two slots from call to
// call: a slot is rewritten only after the next collective's handshake has been passed, and a peer that has
// arrived at that collective has finished the kernel that read the slot (kernels of a stream run in order).
// Block b stages and reads the same contiguous slice of positions on every rank.
struct OneShotArgs {
  int channel;
  uint32_t epoch;
  long long region_off;  // byte offset of the slot used by this call
  long long n;           // elements (floats)
  int op;
  float scale;
  const float* in;
  float* out;
};

template <int W>
__device__ void oneshot_body(const fb_dist_ctx& c, int vblock, int nvblocks, const OneShotArgs& a, const float* in,
                             float* out, int* s_fail) {
  const long long per = (a.n + nvblocks - 1) / nvblocks;
  const long long lo = min(a.n, per * vblock), hi = min(a.n, lo + per);
  float* mine = reinterpret_cast<float*>(c.arena[c.rank] + a.region_off);
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) mine[i] = in[i];
  if (!block_handshake(c, a.channel, vblock, a.epoch, s_fail, 500)) return;
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float part[W];
#pragma unroll
    for (int r = 0; r < W; ++r)
      if (r < c.world) part[r] = *reinterpret_cast<const volatile float*>(c.arena[r] + a.region_off + i * 4);
    float acc = part[0];
#pragma unroll
    for (int r = 1; r < W; ++r)
      if (r < c.world) {
        if (a.op == FB_OP_PROD) acc *= part[r];
        else if (a.op == FB_OP_MIN) acc = fminf(acc, part[r]);
        else if (a.op == FB_OP_MAX) acc = fmaxf(acc, part[r]);
        else acc += part[r];
      }
    out[i] = acc * a.scale;
  }
}

__global__ void __launch_bounds__(256)
oneshot_kernel(const fb_dist_ctx c, const OneShotArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  oneshot_body<FB_MAX_RANKS>(c, blockIdx.x, gridDim.x, a, a.in, a.out, &s_fail);
}

struct EmuOneShot {
  fb_dist_ctx c[FB_MAX_RANKS];
  const float* in[FB_MAX_RANKS];
  float* out[FB_MAX_RANKS];
  int blocks_per_rank;
};
__global__ void __launch_bounds__(256)
oneshot_emulated_kernel(const EmuOneShot pk, const OneShotArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int vr = blockIdx.x / pk.blocks_per_rank;
  oneshot_body<FB_MAX_RANKS>(pk.c[vr], blockIdx.x % pk.blocks_per_rank, pk.blocks_per_rank, a, pk.in[vr], pk.out[vr],
                             &s_fail);
}

// ------------------------------------------------------------- pull collectives
struct CollArgs {
  int mode;
  int channel;
  uint32_t epoch;
  int root;
  long long in_off, out_off;  // byte offsets into the arena
  long long n_bytes;          // bytes per chunk
  int op;
  float scale;
  // Tensors outside the arena (optional).  stage_in: this rank's contribution, copied into the arena's input
  // region by the kernel itself before the entry handshake; direct_out: where this rank's result goes instead
  // of the arena's output region (results are always local, so any device pointer works).
  const unsigned char* stage_in;
  unsigned char* direct_out;
};

// Which bytes a thread moves is decided by the ARENA-side address and the length only, so the block that stages a
// chunk and the peer block of the same index that later pulls it cover exactly the same bytes; the alignment of the
// pointer outside the arena only changes how a thread loads or stores its unit.
__device__ __forceinline__ bool arena_vec_ok(const unsigned char* arena_ptr) {
  return (reinterpret_cast<uintptr_t>(arena_ptr) & 15) == 0;
}

// peer (or own) arena -> any local pointer
__device__ __forceinline__ void copy_bytes(const unsigned char* src, unsigned char* dst, long long nbytes,
                                           long long tid, long long stride) {
  if (arena_vec_ok(src)) {
    const long long nv = nbytes >> 4;
    const uintptr_t da = reinterpret_cast<uintptr_t>(dst);
    long long i = tid;
    if ((da & 15) == 0) {  // eight independent 16-byte loads in flight per thread (a peer load is a round trip)
      constexpr int kU = 8;
      for (; i + (kU - 1) * stride < nv; i += stride * kU) {
        float4 v[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) v[u] = ptx::ld_relaxed_sys_f4(reinterpret_cast<const float4*>(src) + i + u * stride);
#pragma unroll
        for (int u = 0; u < kU; ++u) reinterpret_cast<float4*>(dst)[i + u * stride] = v[u];
      }
    }
    for (; i < nv; i += stride) {
      const float4 v = ptx::ld_relaxed_sys_f4(reinterpret_cast<const float4*>(src) + i);
      if ((da & 15) == 0) {
        reinterpret_cast<float4*>(dst)[i] = v;
      } else if ((da & 3) == 0) {
        float* d = reinterpret_cast<float*>(dst) + i * 4;
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
      } else {
        const unsigned char* b = reinterpret_cast<const unsigned char*>(&v);
        for (int k = 0; k < 16; ++k) dst[i * 16 + k] = b[k];
      }
    }
    for (long long i = (nv << 4) + tid; i < nbytes; i += stride)
      dst[i] = *reinterpret_cast<const volatile unsigned char*>(src + i);
  } else {
    for (long long i = tid; i < nbytes; i += stride) dst[i] = *reinterpret_cast<const volatile unsigned char*>(src + i);
  }
}

// any local pointer -> own arena, same byte ownership as copy_bytes reading that arena address
__device__ __forceinline__ void stage_bytes(const unsigned char* src, unsigned char* arena_dst, long long nbytes,
                                            long long tid, long long stride) {
  if (arena_vec_ok(arena_dst)) {
    const long long nv = nbytes >> 4;
    const uintptr_t sa = reinterpret_cast<uintptr_t>(src);
    long long i = tid;
    if ((sa & 15) == 0) {
      constexpr int kU = 8;
      for (; i + (kU - 1) * stride < nv; i += stride * kU) {
        float4 v[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) v[u] = reinterpret_cast<const float4*>(src)[i + u * stride];
#pragma unroll
        for (int u = 0; u < kU; ++u) reinterpret_cast<float4*>(arena_dst)[i + u * stride] = v[u];
      }
    }
    for (; i < nv; i += stride) {
      float4 v;
      if ((sa & 15) == 0) {
        v = reinterpret_cast<const float4*>(src)[i];
      } else if ((sa & 3) == 0) {
        const float* f = reinterpret_cast<const float*>(src) + i * 4;
        v = make_float4(f[0], f[1], f[2], f[3]);
      } else {
        unsigned char* b = reinterpret_cast<unsigned char*>(&v);
        for (int k = 0; k < 16; ++k) b[k] = src[i * 16 + k];
      }
      reinterpret_cast<float4*>(arena_dst)[i] = v;
    }
    for (long long i = (nv << 4) + tid; i < nbytes; i += stride) arena_dst[i] = src[i];
  } else {
    for (long long i = tid; i < nbytes; i += stride) arena_dst[i] = src[i];
  }
}

// The reductions own data per float: float i of a chunk belongs to thread i mod stride, on both sides.
__device__ __forceinline__ void stage_floats(const unsigned char* src, unsigned char* arena_dst, long long nfloats,
                                             long long tid, long long stride) {
  for (long long i = tid; i < nfloats; i += stride)
    reinterpret_cast<float*>(arena_dst)[i] = reinterpret_cast<const float*>(src)[i];
}

__device__ void reduce_floats(const fb_dist_ctx& c, long long src_off, unsigned char* dst, long long nfloats,
                              int op, float scale, long long tid, long long stride) {
  for (long long i = tid; i < nfloats; i += stride) {
    float acc = 0.f;
    for (int r = 0; r < c.world; ++r) {
      const float x = *reinterpret_cast<const volatile float*>(c.arena[r] + src_off + i * 4);
      if (r == 0) acc = x;
      else if (op == FB_OP_PROD) acc *= x;
      else if (op == FB_OP_MIN) acc = fminf(acc, x);
      else if (op == FB_OP_MAX) acc = fmaxf(acc, x);
      else acc += x;
    }
    reinterpret_cast<float*>(dst)[i] = acc * scale;
  }
}

__device__ void collective_body(const fb_dist_ctx& c, int vblock, int nvblocks, const CollArgs& a, int* s_fail) {
  const long long tid = static_cast<long long>(vblock) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(nvblocks) * blockDim.x;
  unsigned char* self = c.arena[c.rank];
  if (a.stage_in != nullptr) {
    // every block brings the bytes its peers' blocks of the same index will ask for
    switch (a.mode) {
      case FB_COLL_BROADCAST:
        if (c.rank == a.root) stage_bytes(a.stage_in, self + a.in_off, a.n_bytes, tid, stride);
        break;
      case FB_COLL_SCATTER:
        if (c.rank == a.root)
          for (int q = 0; q < c.world; ++q)
            stage_bytes(a.stage_in + q * a.n_bytes, self + a.in_off + q * a.n_bytes, a.n_bytes, tid, stride);
        break;
      case FB_COLL_GATHER:
      case FB_COLL_ALL_GATHER:
        stage_bytes(a.stage_in, self + a.in_off, a.n_bytes, tid, stride);
        break;
      case FB_COLL_REDUCE_SCATTER:
        for (int q = 0; q < c.world; ++q)
          stage_floats(a.stage_in + q * a.n_bytes, self + a.in_off + q * a.n_bytes, a.n_bytes >> 2, tid, stride);
        break;
      case FB_COLL_REDUCE:
        stage_floats(a.stage_in, self + a.in_off, a.n_bytes >> 2, tid, stride);
        break;
      default:
        break;
    }
  }
  if (!block_handshake(c, a.channel, vblock, a.epoch, s_fail, 200)) return;
  unsigned char* out = a.direct_out != nullptr ? a.direct_out : self + a.out_off;
  switch (a.mode) {
    case FB_COLL_BROADCAST:
      if (c.rank != a.root)
        copy_bytes(c.arena[a.root] + a.in_off, a.direct_out != nullptr ? a.direct_out : self + a.in_off, a.n_bytes,
                   tid, stride);
      break;
    case FB_COLL_GATHER:
      if (c.rank != a.root) break;
      // fallthrough
    case FB_COLL_ALL_GATHER:
      // every rank starts with a different source (its right-hand neighbour), so that at any moment each GPU's
      // outbound links serve one reader instead of all of them at once
      for (int i = 0; i < c.world; ++i) {
        const int p = (c.rank + 1 + i) % c.world;
        copy_bytes(c.arena[p] + a.in_off, out + p * a.n_bytes, a.n_bytes, tid, stride);
      }
      break;
    case FB_COLL_ALL_GATHER_INPLACE:
      for (int i = 0; i + 1 < c.world; ++i) {
        const int p = (c.rank + 1 + i) % c.world;
        copy_bytes(c.arena[p] + a.in_off + p * a.n_bytes, self + a.in_off + p * a.n_bytes, a.n_bytes, tid, stride);
      }
      break;
    case FB_COLL_SCATTER:
      copy_bytes(c.arena[a.root] + a.in_off + c.rank * a.n_bytes, out, a.n_bytes, tid, stride);
      break;
    case FB_COLL_REDUCE_SCATTER:
      reduce_floats(c, a.in_off + c.rank * a.n_bytes, out, a.n_bytes >> 2, a.op, a.scale, tid, stride);
      break;
    case FB_COLL_REDUCE:
      if (c.rank == a.root) reduce_floats(c, a.in_off, out, a.n_bytes >> 2, a.op, a.scale, tid, stride);
      break;
    default:
      break;
  }
  block_handshake(c, a.channel, vblock, a.epoch + 1, s_fail, 201);
}

__global__ void __launch_bounds__(512)
collective_kernel(const fb_dist_ctx c, const CollArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  collective_body(c, blockIdx.x, gridDim.x, a, &s_fail);
}

struct EmuCtxPack {
  fb_dist_ctx c[FB_MAX_RANKS];
  const unsigned char* stage_in[FB_MAX_RANKS];  // per virtual rank (NULL = data already in the arena)
  unsigned char* direct_out[FB_MAX_RANKS];
  int blocks_per_rank;
};
__global__ void __launch_bounds__(512)
collective_emulated_kernel(const EmuCtxPack pk, CollArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int vr = blockIdx.x / pk.blocks_per_rank;
  a.stage_in = pk.stage_in[vr];
  a.direct_out = pk.direct_out[vr];
  collective_body(pk.c[vr], blockIdx.x % pk.blocks_per_rank, pk.blocks_per_rank, a, &s_fail);
}

__global__ void barrier_kernel(const fb_dist_ctx c, int channel, uint32_t epoch) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  block_handshake(c, channel, 0, epoch, &s_fail, 300);
}

__global__ void epoch_advance_kernel(unsigned* ctr, unsigned inc) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *ctr += inc;
}

template <int FUSE>
int launch_ar(const fb_dist_ctx& c, const ArArgs& a, int use_mc, int nblocks, int nthreads, cudaStream_t st) {
  // bytes in flight per thread = U * world * 16 (peer loads) = 128: deeper unrolling for small worlds
  if (use_mc)
    allreduce_kernel<FUSE, true, 4, FB_MAX_RANKS><<<nblocks, nthreads, 0, st>>>(c, a);
  else if (c.world <= 2)
    allreduce_kernel<FUSE, false, 4, 2><<<nblocks, nthreads, 0, st>>>(c, a);
  else if (c.world <= 4)
    allreduce_kernel<FUSE, false, 2, 4><<<nblocks, nthreads, 0, st>>>(c, a);
  else
    allreduce_kernel<FUSE, false, 1, FB_MAX_RANKS><<<nblocks, nthreads, 0, st>>>(c, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" int fb_dist_query_flag_bytes() { return FB_FLAG_BYTES; }
extern "C" int fb_dist_query_max_blocks() { return FB_FLAG_BLOCKS; }
extern "C" int fb_dist_query_channels() { return FB_FLAG_CHANNELS; }

// Ranges of the NEXT fused all-reduce launched from this host thread whose gradients were pushed into the shard
// owners' memory by the producing GEMMs (see ArArgs::pushed_lo).  Consumed by that launch.
static thread_local int g_pending_pushed = 0;
static thread_local long long g_pending_lo[4], g_pending_hi[4];
extern "C" int fb_dist_set_pushed_ranges(int n, const long long* lo, const long long* hi) {
  if (n < 0 || n > 4) return -1;
  for (int i = 0; i < n; ++i) {
    if ((lo[i] & 3) || (hi[i] & 3) || lo[i] < 0 || hi[i] < lo[i]) return -1;
    g_pending_lo[i] = lo[i];
    g_pending_hi[i] = hi[i];
  }
  g_pending_pushed = n;
  return 0;
}

// Fused all-reduce of one gradient bucket.  `epoch` and `epoch + 1` are consumed on `channel`.
// fuse: FB_FUSE_NONE (in-place all-reduce of the region at grad_off), FB_FUSE_SGD, FB_FUSE_ADAM.
static int allreduce_impl(const fb_dist_ctx* ctx, int fuse, int use_mc, int channel, unsigned epoch,
                          long long grad_off, long long param_off, long long shadow_off, long long n, int op,
                          float scale, const fb_adam_hparams* adam, const fb_sgd_hparams* sgd, float* m, float* v,
                          int publish_master, int nblocks, int nthreads, const unsigned* dev_epoch, const float* dyn,
                          cudaStream_t stream, const float* stage_in = nullptr, float* stage_out = nullptr,
                          long long n_valid = 0) {
  if (!ctx_ok(ctx) || n <= 0 || (n & 3) || nblocks < 1 || nblocks > FB_FLAG_BLOCKS || nthreads < 32 ||
      nthreads > 256 || channel < 0 || channel >= FB_FLAG_CHANNELS)
    return -1;
  if (use_mc && (ctx->mc_arena == nullptr || (op != FB_OP_SUM && op != FB_OP_AVG))) return -2;
  ArArgs a{};
  a.channel = channel;
  a.epoch = epoch;
  a.grad_off = grad_off;
  a.param_off = param_off;
  a.shadow_off = shadow_off;
  a.n = n;
  a.op = op;
  a.scale = scale;
  if (adam) a.adam = *adam;
  if (sgd) a.sgd = *sgd;
  a.m = m;
  a.v = v;
  a.publish_master = publish_master;
  a.dev_epoch = dev_epoch;
  a.dyn = dyn;
  a.stage_in = stage_in;
  a.stage_out = stage_out;
  a.n_valid = n_valid;
  a.n_pushed = g_pending_pushed;
  for (int i = 0; i < g_pending_pushed; ++i) {
    a.pushed_lo[i] = g_pending_lo[i];
    a.pushed_hi[i] = g_pending_hi[i];
  }
  g_pending_pushed = 0;
  if (a.n_pushed > 0) {
    if (n % (4LL * ctx->world) != 0) return -4;  // slots of equal length need n = world * per
    use_mc = 0;                                   // the switch-side reduction reads every rank's copy of the shard
  }
  {
    static int streaming = -1;
    if (streaming < 0) {
      const char* e = getenv("FERRUM_COMM_STREAMING");
      streaming = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    a.streaming = streaming;
  }
  switch (fuse) {
    case FB_FUSE_NONE: return launch_ar<FB_FUSE_NONE>(*ctx, a, use_mc, nblocks, nthreads, stream);
    case FB_FUSE_SGD: return launch_ar<FB_FUSE_SGD>(*ctx, a, use_mc, nblocks, nthreads, stream);
    case FB_FUSE_ADAM:
      if (m == nullptr || v == nullptr) return -3;
      return launch_ar<FB_FUSE_ADAM>(*ctx, a, use_mc, nblocks, nthreads, stream);
    default: return -1;
  }
}

extern "C" int fb_dist_allreduce(const fb_dist_ctx* ctx, int fuse, int use_mc, int channel, unsigned epoch,
                                 long long grad_off, long long param_off, long long shadow_off, long long n,
                                 int op, float scale, const fb_adam_hparams* adam, const fb_sgd_hparams* sgd,
                                 float* m, float* v, int publish_master, int nblocks, int nthreads,
                                 cudaStream_t stream) {
  return allreduce_impl(ctx, fuse, use_mc, channel, epoch, grad_off, param_off, shadow_off, n, op, scale, adam, sgd, m,
                        v, publish_master, nblocks, nthreads, nullptr, nullptr, stream);
}

// In-place all-reduce of a local fp32 tensor of n_valid elements through the arena region at region_off
// (n elements, a multiple of 4 * world, n >= n_valid): staging in and out happens inside the one kernel.
extern "C" int fb_dist_allreduce_staged(const fb_dist_ctx* ctx, int use_mc, int channel, unsigned epoch,
                                        long long region_off, long long n, int op, float scale, const float* in,
                                        float* out, long long n_valid, int nblocks, int nthreads,
                                        cudaStream_t stream) {
  if (in == nullptr || out == nullptr || n_valid <= 0 || n_valid > n) return -1;
  if ((reinterpret_cast<uintptr_t>(in) & 3) || (reinterpret_cast<uintptr_t>(out) & 3)) return -1;
  return allreduce_impl(ctx, FB_FUSE_NONE, use_mc, channel, epoch, region_off, 0, -1, n, op, scale, nullptr, nullptr,
                        nullptr, nullptr, 1, nblocks, nthreads, nullptr, nullptr, stream, in, out, n_valid);
}

// Graph-capturable form: the handshake epoch is read from *dev_epoch (every rank keeps its own counter; they move
// in lockstep) and advanced by 2 on the stream after the launch; lr / bias corrections come from `dyn` when given.
extern "C" int fb_dist_allreduce_dyn(const fb_dist_ctx* ctx, int fuse, int use_mc, int channel, unsigned* dev_epoch,
                                     long long grad_off, long long param_off, long long shadow_off, long long n,
                                     int op, float scale, const fb_adam_hparams* adam, const fb_sgd_hparams* sgd,
                                     float* m, float* v, int publish_master, int nblocks, int nthreads,
                                     const float* dyn, cudaStream_t stream) {
  if (dev_epoch == nullptr) return -1;
  const int rc = allreduce_impl(ctx, fuse, use_mc, channel, 0u, grad_off, param_off, shadow_off, n, op, scale, adam,
                                sgd, m, v, publish_master, nblocks, nthreads, dev_epoch, dyn, stream);
  if (rc != 0) return rc;
  epoch_advance_kernel<<<1, 32, 0, stream>>>(dev_epoch, 2u);
  return static_cast<int>(cudaGetLastError());
}

// Same computation with all `world` ranks emulated on the current GPU in one cooperative launch.
extern "C" int fb_dist_allreduce_emulated(const fb_dist_ctx* ctxs, int world, int fuse, int channel,
                                          unsigned epoch, long long grad_off, long long param_off,
                                          long long shadow_off, long long n, int op, float scale,
                                          const fb_adam_hparams* adam, const fb_sgd_hparams* sgd, float* const* m,
                                          float* const* v, int publish_master, int nblocks, int nthreads,
                                          cudaStream_t stream) {
  if (world < 1 || world > FB_MAX_RANKS || n <= 0 || (n & 3) || nblocks < 1 || nblocks > FB_FLAG_BLOCKS) return -1;
  EmuPack pk{};
  for (int r = 0; r < world; ++r) {
    if (!ctx_ok(&ctxs[r]) || ctxs[r].world != world || ctxs[r].rank != r) return -1;
    pk.c[r] = ctxs[r];
    pk.m[r] = m ? m[r] : nullptr;
    pk.v[r] = v ? v[r] : nullptr;
  }
  pk.blocks_per_rank = nblocks;
  ArArgs a{};
  a.channel = channel;
  a.epoch = epoch;
  a.grad_off = grad_off;
  a.param_off = param_off;
  a.shadow_off = shadow_off;
  a.n = n;
  a.op = op;
  a.scale = scale;
  if (adam) a.adam = *adam;
  if (sgd) a.sgd = *sgd;
  a.publish_master = publish_master;
  a.n_pushed = g_pending_pushed;
  for (int i = 0; i < g_pending_pushed; ++i) {
    a.pushed_lo[i] = g_pending_lo[i];
    a.pushed_hi[i] = g_pending_hi[i];
  }
  g_pending_pushed = 0;
  if (a.n_pushed > 0 && n % (4LL * world) != 0) return -4;
  void* args[] = {&pk, &a};
  const dim3 grid(world * nblocks), block(nthreads);
  const void* fn = fuse == FB_FUSE_ADAM  ? reinterpret_cast<const void*>(allreduce_emulated_kernel<FB_FUSE_ADAM>)
                   : fuse == FB_FUSE_SGD ? reinterpret_cast<const void*>(allreduce_emulated_kernel<FB_FUSE_SGD>)
                                         : reinterpret_cast<const void*>(allreduce_emulated_kernel<FB_FUSE_NONE>);
  return static_cast<int>(cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream));
}

// The staged all-reduce with every rank emulated in one cooperative launch: in[r] / out[r] are rank r's tensors.
extern "C" int fb_dist_allreduce_staged_emulated(const fb_dist_ctx* ctxs, int world, int channel, unsigned epoch,
                                                 long long region_off, long long n, int op, float scale,
                                                 const float* const* in, float* const* out, long long n_valid,
                                                 int nblocks, int nthreads, cudaStream_t stream) {
  if (world < 1 || world > FB_MAX_RANKS || n <= 0 || (n & 3) || nblocks < 1 || nblocks > FB_FLAG_BLOCKS ||
      in == nullptr || out == nullptr || n_valid <= 0 || n_valid > n)
    return -1;
  EmuPack pk{};
  for (int r = 0; r < world; ++r) {
    if (!ctx_ok(&ctxs[r]) || ctxs[r].world != world || ctxs[r].rank != r) return -1;
    pk.c[r] = ctxs[r];
    pk.stage_in[r] = in[r];
    pk.stage_out[r] = out[r];
  }
  pk.blocks_per_rank = nblocks;
  ArArgs a{};
  a.channel = channel;
  a.epoch = epoch;
  a.grad_off = region_off;
  a.shadow_off = -1;
  a.n = n;
  a.n_valid = n_valid;
  a.op = op;
  a.scale = scale;
  a.publish_master = 1;
  void* args[] = {&pk, &a};
  return static_cast<int>(cudaLaunchCooperativeKernel(
      reinterpret_cast<const void*>(allreduce_emulated_kernel<FB_FUSE_NONE>), dim3(world * nblocks), dim3(nthreads),
      args, 0, stream));
}

extern "C" int fb_dist_collective(const fb_dist_ctx* ctx, int mode, int channel, unsigned epoch, int root,
                                  long long in_off, long long out_off, long long n_bytes, int op, float scale,
                                  int nblocks, cudaStream_t stream) {
  if (!ctx_ok(ctx) || n_bytes < 0 || nblocks < 1 || nblocks > FB_FLAG_BLOCKS || channel < 0 ||
      channel >= FB_FLAG_CHANNELS || root < 0 || root >= ctx->world)
    return -1;
  CollArgs a{mode, channel, epoch, root, in_off, out_off, n_bytes, op, scale, nullptr, nullptr};
  collective_kernel<<<nblocks, 512, 0, stream>>>(*ctx, a);
  return static_cast<int>(cudaGetLastError());
}

// The same collectives on tensors OUTSIDE the arena, in one launch: `in` (this rank's contribution; may be NULL
// where the rank contributes nothing, e.g. a non-root of broadcast / scatter) is staged into the arena region at
// in_off by the kernel, and the result is written straight to `out` (NULL where the rank receives nothing).
// Reductions need 4-byte aligned pointers.
extern "C" int fb_dist_collective_staged(const fb_dist_ctx* ctx, int mode, int channel, unsigned epoch, int root,
                                         long long in_off, long long n_bytes, int op, float scale, const void* in,
                                         void* out, int nblocks, cudaStream_t stream) {
  if (!ctx_ok(ctx) || n_bytes < 0 || nblocks < 1 || nblocks > FB_FLAG_BLOCKS || channel < 0 ||
      channel >= FB_FLAG_CHANNELS || root < 0 || root >= ctx->world || mode == FB_COLL_ALL_GATHER_INPLACE)
    return -1;
  const bool reduces = mode == FB_COLL_REDUCE_SCATTER || mode == FB_COLL_REDUCE;
  if (reduces && ((n_bytes & 3) || (reinterpret_cast<uintptr_t>(in) & 3) || (reinterpret_cast<uintptr_t>(out) & 3)))
    return -1;
  const bool receives = mode == FB_COLL_GATHER || mode == FB_COLL_REDUCE ? ctx->rank == root
                        : mode == FB_COLL_BROADCAST                     ? ctx->rank != root
                                                                        : true;
  if (receives && out == nullptr) return -1;
  CollArgs a{mode, channel, epoch, root, in_off, 0, n_bytes, op, scale, static_cast<const unsigned char*>(in),
             static_cast<unsigned char*>(out)};
  collective_kernel<<<nblocks, 512, 0, stream>>>(*ctx, a);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_dist_collective_emulated(const fb_dist_ctx* ctxs, int world, int mode, int channel,
                                           unsigned epoch, int root, long long in_off, long long out_off,
                                           long long n_bytes, int op, float scale, int nblocks,
                                           cudaStream_t stream) {
  if (world < 1 || world > FB_MAX_RANKS || nblocks < 1 || nblocks > FB_FLAG_BLOCKS) return -1;
  EmuCtxPack pk{};
  for (int r = 0; r < world; ++r) pk.c[r] = ctxs[r];
  pk.blocks_per_rank = nblocks;
  CollArgs a{mode, channel, epoch, root, in_off, out_off, n_bytes, op, scale, nullptr, nullptr};
  void* args[] = {&pk, &a};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(collective_emulated_kernel),
                                                      dim3(world * nblocks), dim3(512), args, 0, stream));
}

// fb_dist_collective_staged with every rank emulated in one cooperative launch; in[r] / out[r] may be NULL.
extern "C" int fb_dist_collective_staged_emulated(const fb_dist_ctx* ctxs, int world, int mode, int channel,
                                                  unsigned epoch, int root, long long in_off, long long n_bytes,
                                                  int op, float scale, const void* const* in, void* const* out,
                                                  int nblocks, cudaStream_t stream) {
  if (world < 1 || world > FB_MAX_RANKS || nblocks < 1 || nblocks > FB_FLAG_BLOCKS || in == nullptr ||
      out == nullptr || mode == FB_COLL_ALL_GATHER_INPLACE)
    return -1;
  EmuCtxPack pk{};
  for (int r = 0; r < world; ++r) {
    pk.c[r] = ctxs[r];
    pk.stage_in[r] = static_cast<const unsigned char*>(in[r]);
    pk.direct_out[r] = static_cast<unsigned char*>(out[r]);
  }
  pk.blocks_per_rank = nblocks;
  CollArgs a{mode, channel, epoch, root, in_off, 0, n_bytes, op, scale, nullptr, nullptr};
  void* args[] = {&pk, &a};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(collective_emulated_kernel),
                                                      dim3(world * nblocks), dim3(512), args, 0, stream));
}

extern "C" int fb_dist_barrier(const fb_dist_ctx* ctx, int channel, unsigned epoch, cudaStream_t stream) {
  if (!ctx_ok(ctx) || channel < 0 || channel >= FB_FLAG_CHANNELS) return -1;
  barrier_kernel<<<1, 32, 0, stream>>>(*ctx, channel, epoch);
  return static_cast<int>(cudaGetLastError());
}

// One-shot all-reduce of a local fp32 tensor of n elements (in and out may be the same pointer) through the
// arena slot at region_off (n * 4 bytes): one launch, one handshake.  The caller alternates between two slots
// from call to call and uses slots that no other collective writes (see the kernel's comment).
extern "C" int fb_dist_allreduce_oneshot(const fb_dist_ctx* ctx, int channel, unsigned epoch, long long region_off,
                                         long long n, int op, float scale, const float* in, float* out,
                                         int nblocks, int nthreads, cudaStream_t stream) {
  if (!ctx_ok(ctx) || n <= 0 || in == nullptr || out == nullptr || nblocks < 1 || nblocks > FB_FLAG_BLOCKS ||
      nthreads < 32 || nthreads > 256 || channel < 0 || channel >= FB_FLAG_CHANNELS || (region_off & 3))
    return -1;
  OneShotArgs a{channel, epoch, region_off, n, op, scale, in, out};
  oneshot_kernel<<<nblocks, nthreads, 0, stream>>>(*ctx, a);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_dist_allreduce_oneshot_emulated(const fb_dist_ctx* ctxs, int world, int channel, unsigned epoch,
                                                  long long region_off, long long n, int op, float scale,
                                                  const float* const* in, float* const* out, int nblocks,
                                                  int nthreads, cudaStream_t stream) {
  if (world < 1 || world > FB_MAX_RANKS || n <= 0 || in == nullptr || out == nullptr || nblocks < 1 ||
      nblocks > FB_FLAG_BLOCKS)
    return -1;
  EmuOneShot pk{};
  for (int r = 0; r < world; ++r) {
    if (!ctx_ok(&ctxs[r]) || ctxs[r].world != world || ctxs[r].rank != r) return -1;
    pk.c[r] = ctxs[r];
    pk.in[r] = in[r];
    pk.out[r] = out[r];
  }
  pk.blocks_per_rank = nblocks;
  OneShotArgs a{channel, epoch, region_off, n, op, scale, nullptr, nullptr};
  void* args[] = {&pk, &a};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(oneshot_emulated_kernel),
                                                      dim3(world * nblocks), dim3(nthreads), args, 0, stream));
}
