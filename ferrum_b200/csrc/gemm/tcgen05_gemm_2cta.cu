// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 computes a 256 x 256 output tile
// per cluster of two CTAs (two SMs).  Each CTA stages only ITS half of the operands
// — 128 rows of A and 128 rows of B per 64-deep k-block, 32 KB — so a stage costs a
// third less L2 -> shared-memory traffic per SM than the single-CTA kernel's
// 128 x 256 tile and six stages fit where that kernel has four; both matter because
// the single-CTA kernel is limited by operand-fetch latency, not by the tensor pipe.
// The accumulator of a CTA (its 128 rows x 256 columns, fp32) lives in that CTA's
// tensor memory, double-buffered (2 x 256 of the 512 columns).
//
// Same contract and operand layouts as fb_gemm_bf16 (tcgen05_gemm.cu); the reference
// loops it replaces are ferrum-core/src/tensor.rs:2487-2558.
//
// Roles (192 threads per CTA):
//   warp 0      TMA producer of this CTA's halves; the byte counts of BOTH CTAs land
//               on the leader's "full" mbarrier (plain cta_group::2 loads, no multicast)
//   warp 1      TMEM allocation (both CTAs); in the leader (cluster rank 0) one lane
//               issues every MMA and commits to the mbarriers of both CTAs
//   warps 2..5  epilogue of this CTA's 128 rows (eight warps, two per TMEM lane quarter, measured slower: the
//               value + derivative epilogue dropped from 1500 to 1413 TFLOP/s); "accumulator drained" is signalled
//               to the leader's mbarrier from both CTAs
//
// Epilogue.  A warp reads its 32 accumulator rows from tensor memory 32 columns at a time (tcgen05.ld), applies
// bias / activation in registers, writes the 32 x 128-byte slab into 128-byte-swizzled shared memory (conflict-free
// 16-byte stores) and one lane hands the slab to the TMA unit (cp.async.bulk.tensor store; cp.reduce...add when the
// result is accumulated into an existing fp32 matrix).  Global memory therefore sees whole 128-byte lines instead of
// 16-byte pieces of 32 different rows, and the warp is free for the next slab while the copy drains; each warp
// double-buffers its slab (bulk groups, wait_group.read before a buffer is rewritten).  Results whose base or row
// pitch is not 16-byte aligned leave through plain register stores.
// Every wait is bounded; the two cluster barriers (after set-up, before exit) are
// reached on every path, including the abort path.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>

#include "../common/ptx.cuh"
#include "../common/status.h"
#include "../dist/dist_ctx.h"
#include "../include/ferrum_kernels.h"
#include "epilogue.cuh"

namespace fb {
namespace {

constexpr int kBM = 128;       // rows per CTA; the pair covers 256
constexpr int kRowBytes = 128;  // one swizzled shared-memory row = one k-block of a K-major operand
constexpr int kThreads = 192;
constexpr int kEpilogueWarps = 4;
constexpr int kABytes = kBM * kRowBytes;        // 16 KB
constexpr int kSlabBytes = 32 * kRowBytes;      // one output slab of a warp: 32 rows x 128 bytes

// BN = columns per pair (each CTA stages half of them).  256 is the high-intensity shape; 128 halves the
// tile for small outputs that would otherwise occupy less than half of the CTA pairs.
template <int BN>
struct Cfg2 {
  static constexpr int kBBytes = (BN / 2) * kRowBytes;        // 16 KB / 8 KB
  static constexpr int kStageBytes = kABytes + kBBytes;       // 32 KB / 24 KB per CTA
  static constexpr int kStages = BN == 256 ? 6 : 8;
  // two output slabs per epilogue warp (the push mode uses a warp's 8 KB as a 32 x 33 fp32 transposing buffer)
  static constexpr int kStoreBytes = kEpilogueWarps * 2 * kSlabBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 256;
  static constexpr int kTmemCols = 2 * BN;                    // two accumulators
};

enum : int { kOutRegs = 0, kOutTma = 1, kOutPush = 2 };

struct Args2 {
  void* out;
  void* out2;  // optional: act'(z) in the layout and dtype of out (bf16 outputs only)
  const float* bias;
  int M, N, K;
  long long ldc;
  int a_mn_major, b_mn_major;
  int out_bf16;
  int act;
  int beta;
  int out_mode;  // kOutTma: slabs leave through the TMA unit; kOutRegs: register stores (unaligned results); kOutPush
  int group_m;   // pair-tiles (256 rows) per rasterisation group
  int32_t* status;
  unsigned long long timeout_ns;
  // Optional per-pair timing record (4 x 64-bit per pair, nanoseconds): MMA thread waiting for a drained
  // accumulator, MMA thread waiting for operands, one epilogue warp busy, whole kernel.  NULL = off.
  unsigned long long* prof;
  // Push mode (weight gradients of a data-parallel job): instead of a local fp32 matrix, every piece of the
  // result goes straight to the rank that OWNS it — element e of the bucket belongs to shard o = e / per, and
  // source rank s deposits its value at element s * per + (e - o * per) of rank o's bucket region — over NVLink
  // peer stores issued from this epilogue, so the gradient reduce-scatter travels while the next tiles are
  // multiplied and the bucket kernel finds all contributions in local memory.  The 32 x 32 block of a warp is
  // turned through shared memory so that one store instruction writes 128 contiguous bytes of ONE row.
  int push_world, push_rank;
  unsigned char* push_arena[8];
  long long push_bucket_off;  // byte offset of the bucket's gradient region inside every arena
  long long push_rel;         // bucket-relative element index of out[0][0] (multiple of 4)
  long long push_per;         // elements per shard (multiple of 4)
};

unsigned long long* g_prof_buffer = nullptr;
int g_group_m = 8;

__device__ __forceinline__ void tile_coords2(int t, int num_m, int num_n, int group_m, int& m_blk, int& n_blk) {
  const int per_group = group_m * num_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsize = min(num_m - first_m, group_m);
  const int r = t - g * per_group;
  m_blk = first_m + (r % gsize);
  n_blk = r / gsize;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&b2);
}

// kTf32: fp32 operands multiplied as TF32 (kind::tf32).  A k-block is always one 128-byte row, so it holds 32
// fp32 or 64 bf16 K elements, one MMA covers 32 bytes of K (8 / 16 elements), and an MN-major operand arrives in
// chunks of 32 / 64 MN elements; the byte geometry of a stage is the same for both element types.
template <int BN, bool kTf32 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_c2,
                      const Args2 p) {
  constexpr int kBN = BN;
  constexpr int kBK = kTf32 ? 32 : 64, kUmmaK = kTf32 ? 8 : 16, kChunk = kTf32 ? 32 : 64;
  constexpr int kStages = Cfg2<BN>::kStages;
  constexpr int kStageBytes = Cfg2<BN>::kStageBytes;
  constexpr int kTmemCols = Cfg2<BN>::kTmemCols;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* slab_base = smem + kStages * kStageBytes;             // 1024-byte aligned (swizzle atom of the stores)
  uint8_t* bar_base = slab_base + Cfg2<BN>::kStoreBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);   // used in the leader only
  uint64_t* empty_bar = full_bar + kStages;                     // one set per CTA
  uint64_t* tmem_full = empty_bar + kStages;                    // one set per CTA
  uint64_t* tmem_empty = tmem_full + 2;                         // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int num_m = (p.M + 2 * kBM - 1) / (2 * kBM);
  const int num_n = (p.N + kBN - 1) / kBN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);   // the leader's arrive.expect_tx; bytes of both CTAs are counted on it
      ptx::mbar_init(&empty_bar[s], 1);  // one commit arrival per CTA
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&tmem_full[a], 1);
      ptx::mbar_init(&tmem_empty[a], 2 * kEpilogueWarps);  // the epilogue warps of both CTAs
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tma_a);
    ptx::prefetch_tensormap(&tma_b);
    if (p.out_mode == kOutTma) {
      ptx::prefetch_tensormap(&tma_c);
      if (p.out2 != nullptr) ptx::prefetch_tensormap(&tma_c2);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc_2cta(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_2cta();
  }
  ptx::tc_fence_before();
  __syncthreads();
  // the peer's mbarriers must exist before anything arrives on them remotely
  ptx::cluster_arrive();
  ptx::cluster_wait();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int m_blk, n_blk;
        tile_coords2(t, num_m, num_n, p.group_m, m_blk, n_blk);
        const int m0 = m_blk * 2 * kBM + static_cast<int>(rank) * kBM;        // this CTA's 128 rows of A
        const int n0 = n_blk * kBN + static_cast<int>(rank) * (kBN / 2);      // this CTA's 128 rows of B
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.timeout_ns)) {
            report_status(p.status, kStatusGemmTimeout, 11, blockIdx.x, stage);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          if (rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[stage], 2 * kStageBytes);
          const uint32_t bar = ptx::smem_u32(&full_bar[stage]) & ptx::kPeerBitMask;  // the leader's barrier
          const int k0 = kb * kBK;
          if (p.a_mn_major) {
#pragma unroll
            for (int c = 0; c < kBM / kChunk; ++c)
              ptx::tma_load_2d_2cta(sa + c * (kBK * 128), &tma_a, bar, m0 + c * kChunk, k0);
          } else {
            ptx::tma_load_2d_2cta(sa, &tma_a, bar, k0, m0);
          }
          if (p.b_mn_major) {
#pragma unroll
            for (int c = 0; c < (kBN / 2) / kChunk; ++c)
              ptx::tma_load_2d_2cta(sb + c * (kBK * 128), &tma_b, bar, n0 + c * kChunk, k0);
          } else {
            ptx::tma_load_2d_2cta(sb, &tma_b, bar, k0, n0);
          }
          // (A TMA prefetch into L2 a few k-blocks ahead of the ring was measured and removed: the prefetches
          // queue in front of the real loads, operand waits grew from 32 us to 117 us, 1534 -> 1082 TFLOP/s.)
          ++issued;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // give copies already in flight time to land before shared memory is released
        const uint64_t t0 = ptx::globaltimer();
        while (issued > 0 && ptx::globaltimer() - t0 < 200000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && lane == 0) {
      const uint32_t idesc = ptx::make_idesc(kTf32 ? 2u : 1u, 2 * kBM, kBN, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? kBK * 128 : 16;
      const uint32_t b_lbo = p.b_mn_major ? kBK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? kUmmaK * 128 : 32;
      const uint32_t b_kstep = p.b_mn_major ? kUmmaK * 128 : 32;
      // MN-major fp32 operands sit in shared memory with the 32-byte-chunk swizzle (4-row groups, 512 B apart)
      const uint32_t a_layout = (kTf32 && p.a_mn_major) ? 1u : 2u, a_sbo = (kTf32 && p.a_mn_major) ? 512u : 1024u;
      const uint32_t b_layout = (kTf32 && p.b_mn_major) ? 1u : 2u, b_sbo = (kTf32 && p.b_mn_major) ? 512u : 1024u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      unsigned long long w_acc = 0, w_ops = 0;
      const unsigned long long k_start = p.prof ? ptx::globaltimer() : 0;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        unsigned long long t0 = p.prof ? ptx::globaltimer() : 0;
        if (!ptx::mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, p.timeout_ns)) {
          report_status(p.status, kStatusGemmTimeout, 12, blockIdx.x, acc);
          break;
        }
        if (p.prof) w_acc += ptx::globaltimer() - t0;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          t0 = p.prof ? ptx::globaltimer() : 0;
          if (!ptx::mbar_wait(&full_bar[stage], phase, abort_flag, p.timeout_ns)) {
            report_status(p.status, kStatusGemmTimeout, 13, blockIdx.x, stage);
            ok = false;
            break;
          }
          if (p.prof) w_ops += ptx::globaltimer() - t0;
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(smem + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t adesc = ptx::make_smem_desc_sw128(sa + k * a_kstep, a_lbo, a_sbo, a_layout);
            const uint64_t bdesc = ptx::make_smem_desc_sw128(sb + k * b_kstep, b_lbo, b_sbo, b_layout);
            if constexpr (kTf32)
              ptx::umma_tf32_2cta(d_tmem, adesc, bdesc, idesc, (kb != 0 || k != 0) ? 1u : 0u);
            else
              ptx::umma_f16_2cta(d_tmem, adesc, bdesc, idesc, (kb != 0 || k != 0) ? 1u : 0u);
          }
          ptx::umma_commit_2cta(&empty_bar[stage], 0x3);  // frees the slot in both CTAs
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        ptx::umma_commit_2cta(&tmem_full[acc], 0x3);  // accumulator complete -> both epilogues
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (p.prof) {
        p.prof[pair * 4 + 0] = w_acc;
        p.prof[pair * 4 + 1] = w_ops;
        p.prof[pair * 4 + 3] = ptx::globaltimer() - k_start;
      }
    }
  } else {
    // ------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int quarter = warp & 3;          // TMEM lanes a warp may read: 32 * (warp % 4) ...
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = ((p.ldc * (p.out_bf16 ? 2 : 4)) % 16 == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    uint8_t* my_slabs = slab_base + (warp - 2) * (2 * kSlabBytes);
    const uint32_t slab_u32 = ptx::smem_u32(my_slabs);
    const uint32_t row_off = static_cast<uint32_t>(lane) * kRowBytes;  // this lane's row inside a slab
    const uint32_t sw = static_cast<uint32_t>(lane) & 7u;              // 128-byte swizzle: chunk ^= row % 8
    const bool dual = p.out2 != nullptr;
    int slot = 0;  // slab the next single-output store fills (the other one may still be read by the TMA unit)
    unsigned long long e_busy = 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int m_blk, n_blk;
      tile_coords2(t, num_m, num_n, p.group_m, m_blk, n_blk);
      const int row_base = m_blk * 2 * kBM + static_cast<int>(rank) * kBM + quarter * 32;  // first of this warp's rows
      const int row = row_base + lane;
      const int n0 = n_blk * kBN;
      const bool ready = ptx::mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.timeout_ns);
      const unsigned long long e0 = p.prof ? ptx::globaltimer() : 0;
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) report_status(p.status, kStatusGemmTimeout, 14, blockIdx.x, acc);
        break;
      }
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kBN;
#pragma unroll 1
      for (int j = 0; j < kBN / 32; ++j) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(taddr + j * 32, r);
        ptx::tmem_wait_ld();
        const int col0 = n0 + j * 32;
        if (p.out_mode == kOutPush) {
          // every lane takes part (rows past M are skipped at the store)
          if (col0 < p.N) {
            float* tb = reinterpret_cast<float*>(my_slabs);
#pragma unroll
            for (int i = 0; i < 32; ++i) tb[lane * 33 + i] = __uint_as_float(r[i]);
            __syncwarp();
            long long rel = p.push_rel + static_cast<long long>(row_base) * p.ldc + col0;
            int owner = static_cast<int>(rel / p.push_per);
            long long jj = rel - static_cast<long long>(owner) * p.push_per;
            const bool col_ok = col0 + lane < p.N;
#pragma unroll 4
            for (int rr = 0; rr < 32; ++rr) {
              if (row_base + rr < p.M && col_ok) {
                int o2 = owner;
                long long j2 = jj + lane;
                if (j2 >= p.push_per) {
                  j2 -= p.push_per;
                  ++o2;
                }
                float* dst = reinterpret_cast<float*>(p.push_arena[o2] + p.push_bucket_off) +
                             static_cast<long long>(p.push_rank) * p.push_per + j2;
                asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(dst), "f"(tb[rr * 33 + lane]) : "memory");
              }
              jj += p.ldc;
              while (jj >= p.push_per) {
                jj -= p.push_per;
                ++owner;
              }
            }
            __syncwarp();
          }
          continue;
        }
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (p.bias != nullptr && col0 < p.N) {
          if (col0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(p.bias + col0) & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {  // eight 16-byte loads instead of 32 guarded scalar ones
              const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.bias + col0) + q);
              v[4 * q] += b4.x; v[4 * q + 1] += b4.y; v[4 * q + 2] += b4.z; v[4 * q + 3] += b4.w;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += __ldg(p.bias + col0 + i);
          }
        }
        if (p.out_mode == kOutTma) {
          // Columns or rows past the edge of the matrix are computed like the rest (the operand tiles were
          // zero-filled there) and clipped by the TMA unit.
          if (p.out_bf16) {
            // two 32-column chunks (64 bf16 = 128 bytes per row) fill one slab
            const int half = j & 1;
            const uint32_t s_val = slab_u32 + (dual ? 0u : static_cast<uint32_t>(slot) * kSlabBytes) + row_off;
            const uint32_t s_der = slab_u32 + kSlabBytes + row_off;
            float dv[32];
            if (dual) act_both_chunk(v, dv, p.act);
            else if (p.act != FB_ACT_NONE) act_chunk(v, p.act);
            if (half == 0) {
              // the slab(s) about to be rewritten must have been read by the store issued from them
              if (lane == 0) {
                if (dual) ptx::tma_store_wait_read<0>();
                else ptx::tma_store_wait_read<1>();
              }
              __syncwarp();
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t off = ((static_cast<uint32_t>(half * 4 + q)) ^ sw) << 4;
              ptx::st_shared_v4(s_val + off, pack_bf16(v[q * 8], v[q * 8 + 1]), pack_bf16(v[q * 8 + 2], v[q * 8 + 3]),
                                pack_bf16(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16(v[q * 8 + 6], v[q * 8 + 7]));
              if (dual)
                ptx::st_shared_v4(s_der + off, pack_bf16(dv[q * 8], dv[q * 8 + 1]),
                                  pack_bf16(dv[q * 8 + 2], dv[q * 8 + 3]), pack_bf16(dv[q * 8 + 4], dv[q * 8 + 5]),
                                  pack_bf16(dv[q * 8 + 6], dv[q * 8 + 7]));
            }
            if (half == 1) {
              ptx::fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (row_base < p.M && col0 - 32 < p.N) {
                  ptx::tma_store_2d(&tma_c, my_slabs + (dual ? 0 : slot * kSlabBytes), col0 - 32, row_base);
                  if (dual) ptx::tma_store_2d(&tma_c2, my_slabs + kSlabBytes, col0 - 32, row_base);
                }
                ptx::tma_store_commit();  // always, so that the group count stays in step with `slot`
              }
              slot ^= 1;
            }
          } else {
            if (p.act != FB_ACT_NONE) act_chunk(v, p.act);
            const uint32_t s_val = slab_u32 + static_cast<uint32_t>(slot) * kSlabBytes + row_off;
            if (lane == 0) ptx::tma_store_wait_read<1>();
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 8; ++q)
              ptx::st_shared_v4(s_val + ((static_cast<uint32_t>(q) ^ sw) << 4), __float_as_uint(v[q * 4]),
                                __float_as_uint(v[q * 4 + 1]), __float_as_uint(v[q * 4 + 2]),
                                __float_as_uint(v[q * 4 + 3]));
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (row_base < p.M && col0 < p.N) {
                if (p.beta) ptx::tma_reduce_add_2d(&tma_c, my_slabs + slot * kSlabBytes, col0, row_base);
                else ptx::tma_store_2d(&tma_c, my_slabs + slot * kSlabBytes, col0, row_base);
              }
              ptx::tma_store_commit();
            }
            slot ^= 1;
          }
          continue;
        }
        // ---- register stores (results the TMA unit cannot address)
        if (row < p.M && col0 < p.N) {
          const bool full = (col0 + 32 <= p.N) && vec_ok;
          if (dual) {
            // value and derivative of the activation, both stored as bf16
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldc + col0;
            __nv_bfloat16* o2 = reinterpret_cast<__nv_bfloat16*>(p.out2) + static_cast<long long>(row) * p.ldc + col0;
            float dv[32];
            act_both_chunk(v, dv, p.act);
            if (full) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                reinterpret_cast<uint4*>(o)[q] =
                    make_uint4(pack_bf16(v[q * 8], v[q * 8 + 1]), pack_bf16(v[q * 8 + 2], v[q * 8 + 3]),
                               pack_bf16(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16(v[q * 8 + 6], v[q * 8 + 7]));
                reinterpret_cast<uint4*>(o2)[q] =
                    make_uint4(pack_bf16(dv[q * 8], dv[q * 8 + 1]), pack_bf16(dv[q * 8 + 2], dv[q * 8 + 3]),
                               pack_bf16(dv[q * 8 + 4], dv[q * 8 + 5]), pack_bf16(dv[q * 8 + 6], dv[q * 8 + 7]));
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) {
                  o[i] = __float2bfloat16_rn(v[i]);
                  o2[i] = __float2bfloat16_rn(dv[i]);
                }
            }
          } else {
            if (p.act != FB_ACT_NONE) act_chunk(v, p.act);
            if (p.out_bf16) {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldc + col0;
              if (full) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  reinterpret_cast<uint4*>(o)[q] =
                      make_uint4(pack_bf16(v[q * 8], v[q * 8 + 1]), pack_bf16(v[q * 8 + 2], v[q * 8 + 3]),
                                 pack_bf16(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16(v[q * 8 + 6], v[q * 8 + 7]));
              } else {
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < p.N) o[i] = __float2bfloat16_rn(v[i]);
              }
            } else {
              float* o = reinterpret_cast<float*>(p.out) + static_cast<long long>(row) * p.ldc + col0;
              if (full) {
                float4* o4 = reinterpret_cast<float4*>(o);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  float4 x = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                  if (p.beta) {
                    const float4 old = o4[q];
                    x.x += old.x; x.y += old.y; x.z += old.z; x.w += old.w;
                  }
                  o4[q] = x;
                }
              } else {
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < p.N) o[i] = p.beta ? o[i] + v[i] : v[i];
              }
            }
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      // "drained" goes to the leader's barrier from both CTAs
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::smem_u32(&tmem_empty[acc]) & ptx::kPeerBitMask);
      if (p.prof) e_busy += ptx::globaltimer() - e0;
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    // the slabs belong to the TMA unit until its stores have completed (reached on the abort path too)
    if (lane == 0) ptx::tma_store_wait<0>();
    if (p.prof && warp == 2 && lane == 0 && rank == 0) p.prof[pair * 4 + 2] = e_busy;
  }

  // Teardown: nobody leaves while the peer may still read this CTA's shared memory (the leader's MMAs
  // read both) or arrive on its mbarriers.
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_2cta(tmem_base, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn2 encode_fn2() {
  // The driver's encoder wants a current context; a thread that has made no runtime call yet (an autograd
  // worker entering its first backward) has none, and the encoder then fails with CUDA_ERROR_INVALID_CONTEXT.
  static thread_local bool bound = false;
  if (!bound) {  // cudaSetDevice binds the primary context to the thread and is legal during stream capture
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
    bound = true;
  }
  static EncodeTiledFn2 fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn2>(sym);
  }
  return fn;
}

bool make_map2(CUtensorMap* map, const void* ptr, long long inner, long long outer, long long ld, int box_outer,
               int elem_bytes, bool atom32 = false) {
  EncodeTiledFn2 enc = encode_fn2();
  if (enc == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ld * elem_bytes) % 16 != 0) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kRowBytes / elem_bytes), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
             const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Number of CTA pairs that can be resident at once (0 if cluster launch is unavailable).
template <int BN, bool kTf32 = false>
int max_pairs() {
  constexpr int kSmemBytes = Cfg2<BN>::kSmemBytes;
  static int n = -1;
  if (n < 0) {
    n = 0;
    if (cudaFuncSetAttribute(gemm_bf16_2cta_kernel<BN, kTf32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
        cudaSuccess) {
      cudaGetLastError();
      return n;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_bf16_2cta_kernel<BN, kTf32>, &cfg) == cudaSuccess) n = clusters;
    else cudaGetLastError();
  }
  return n;
}

template <int BN, bool kTf32 = false>
int launch2(const void* a, const void* b, Args2& args, long long lda, long long ldb, int pairs, long long num_tiles,
            cudaStream_t stream) {
  constexpr int kEb = kTf32 ? 4 : 2, kChunk = kRowBytes / kEb;
  CUtensorMap ma, mb, mc, mc2;
  // MN-major fp32 tiles are written with the 32-byte-chunk swizzle the tensor core requires for them
  bool ok = args.a_mn_major ? make_map2(&ma, a, args.M, args.K, lda, kChunk, kEb, kTf32)
                            : make_map2(&ma, a, args.K, args.M, lda, kBM, kEb);
  if (!ok) return -2;
  ok = args.b_mn_major ? make_map2(&mb, b, args.N, args.K, ldb, kChunk, kEb, kTf32)
                       : make_map2(&mb, b, args.K, args.N, ldb, BN / 2, kEb);
  if (!ok) return -2;
  // Result maps: 32-row x 128-byte slabs.  A result the TMA unit cannot address (base or pitch not 16-byte
  // aligned) is stored from registers instead.
  mc = ma;
  mc2 = ma;
  if (args.out_mode != kOutPush) {
    const int eb = args.out_bf16 ? 2 : 4;
    bool tma = make_map2(&mc, args.out, args.N, args.M, args.ldc, 32, eb);
    if (tma && args.out2 != nullptr) tma = make_map2(&mc2, args.out2, args.N, args.M, args.ldc, 32, eb);
    if (!tma) mc = mc2 = ma;
    args.out_mode = tma ? kOutTma : kOutRegs;
  }
  if (num_tiles < pairs) pairs = static_cast<int>(num_tiles);
  gemm_bf16_2cta_kernel<BN, kTf32><<<2 * pairs, kThreads, Cfg2<BN>::kSmemBytes, stream>>>(ma, mb, mc, mc2, args);
  return static_cast<int>(cudaGetLastError());
}

// Arguments every entry point fills the same way.
void fill_common(Args2& args, int32_t* status) {
  args.out_mode = kOutTma;  // launch2 falls back to register stores where no map can be built
  args.group_m = g_group_m;
  args.push_world = 0;
  args.push_rank = 0;
  args.push_bucket_off = args.push_rel = 0;
  args.push_per = 4;
  for (int i = 0; i < 8; ++i) args.push_arena[i] = nullptr;
  args.status = status;
  args.timeout_ns = 2000000000ull;
  args.prof = g_prof_buffer;
}

}  // namespace
}  // namespace fb

extern "C" int fb_gemm_bf16_2cta_pairs() { return fb::max_pairs<256>(); }

// Device buffer of 4 x 64-bit words per CTA pair that subsequent launches fill with their wait / busy times
// (see Args2::prof); NULL switches the record off again.
extern "C" void fb_gemm_bf16_2cta_set_profile(unsigned long long* buffer) { fb::g_prof_buffer = buffer; }

// Rasterisation: tiles are walked in groups of `group_m` 256-row blocks x all column blocks, so that the pairs
// working at the same time share operand tiles in L2.  Returns the previous value; values < 1 only query.
extern "C" int fb_gemm_bf16_2cta_set_group_m(int group_m) {
  const int prev = fb::g_group_m;
  if (group_m >= 1) fb::g_group_m = group_m;
  return prev;
}

// Same arguments as fb_gemm_bf16.  Returns -3 when CTA pairs cannot be launched on this device.
// Small outputs use the 128-column tile, everything else the 256-column one.
extern "C" int fb_gemm_bf16_2cta(const void* a, const void* b, void* out, void* out2, const float* bias, int M, int N,
                                 int K,
                                 long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major,
                                 int out_bf16, int act, int beta, int max_ctas, int32_t* status,
                                 cudaStream_t stream) {
  using namespace fb;
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if (out2 != nullptr && (!out_bf16 || beta)) return -1;
  const int pairs_avail = max_pairs<256>();
  if (pairs_avail <= 0) return -3;
  Args2 args;
  args.out = out;
  args.out2 = out2;
  args.bias = bias;
  args.M = M;
  args.N = N;
  args.K = K;
  args.ldc = ldc;
  args.a_mn_major = a_mn_major;
  args.b_mn_major = b_mn_major;
  args.out_bf16 = out_bf16;
  args.act = act;
  args.beta = beta;
  fill_common(args, status);
  int pairs = pairs_avail;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  const long long m_tiles = (M + 2 * kBM - 1) / (2 * kBM);
  const long long tiles256 = m_tiles * ((N + 255) / 256), tiles128 = m_tiles * ((N + 127) / 128);
  // The 256 x 128 tile moves a third more operand bytes per flop through shared memory and measured ~0.6 of the
  // wide tile's rate on large problems, so it only pays where the wide tiling leaves at least half of the pairs
  // without any tile at all.
  const bool narrow = max_pairs<128>() >= pairs && 2 * tiles256 <= pairs;
  return narrow ? launch2<128>(a, b, args, lda, ldb, pairs, tiles128, stream)
                : launch2<256>(a, b, args, lda, ldb, pairs, tiles256, stream);
}

// fp32 operands as TF32 on CTA pairs, fp32 result; same arguments as fb_gemm_tf32 (256 x 256 pair tiles only).
extern "C" int fb_gemm_tf32_2cta(const float* a, const float* b, float* out, const float* bias, int M, int N, int K,
                                 long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major,
                                 int act, int beta, int max_ctas, int32_t* status, cudaStream_t stream) {
  using namespace fb;
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  const int pairs_avail = max_pairs<256, true>();
  if (pairs_avail <= 0) return -3;
  Args2 args;
  args.out = out;
  args.out2 = nullptr;
  args.bias = bias;
  args.M = M;
  args.N = N;
  args.K = K;
  args.ldc = ldc;
  args.a_mn_major = a_mn_major;
  args.b_mn_major = b_mn_major;
  args.out_bf16 = 0;
  args.act = act;
  args.beta = beta;
  fill_common(args, status);
  int pairs = pairs_avail;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  const long long tiles = static_cast<long long>((M + 2 * kBM - 1) / (2 * kBM)) * ((N + 255) / 256);
  return launch2<256, true>(a, b, args, lda, ldb, pairs, tiles, stream);
}

// Weight-gradient GEMM of a data-parallel job with the reduce-scatter fused into the epilogue (see Args2::push_*):
// result[M, N] = A * B^T in fp32, every row piece stored into the bucket region of the rank that owns it.
// ctx: this rank's view of all arenas; bucket_off: byte offset of the bucket's gradient region in every arena;
// out_rel: bucket-relative element index of result[0][0]; ldc: row pitch of the result inside the bucket (elements);
// per: elements per shard (bucket length / world).  N, ldc, out_rel and per must be multiples of 4 and the result
// must lie inside the bucket.  Returns -3 where CTA pairs cannot be launched.
extern "C" int fb_gemm_bf16_2cta_push(const void* a, const void* b, int M, int N, int K, long long lda, long long ldb,
                                      long long ldc, int a_mn_major, int b_mn_major, const fb_dist_ctx* ctx,
                                      long long bucket_off, long long out_rel, long long per, long long bucket_len,
                                      int max_ctas, int32_t* status, cudaStream_t stream) {
  using namespace fb;
  if (M <= 0 || N <= 0 || K <= 0 || ctx == nullptr || ctx->world < 2 || ctx->world > FB_MAX_RANKS ||
      ctx->rank < 0 || ctx->rank >= ctx->world)
    return -1;
  if ((N & 3) || (ldc & 3) || (out_rel & 3) || (per & 3) || per <= 0 || (bucket_off & 15) || out_rel < 0 ||
      ldc < N || bucket_len != per * ctx->world || out_rel + static_cast<long long>(M - 1) * ldc + N > bucket_len)
    return -1;
  for (int r = 0; r < ctx->world; ++r)
    if (ctx->arena[r] == nullptr) return -1;
  const int pairs_avail = max_pairs<256>();
  if (pairs_avail <= 0) return -3;
  Args2 args;
  args.out = nullptr;
  args.out2 = nullptr;
  args.bias = nullptr;
  args.M = M;
  args.N = N;
  args.K = K;
  args.ldc = ldc;
  args.a_mn_major = a_mn_major;
  args.b_mn_major = b_mn_major;
  args.out_bf16 = 0;
  args.act = FB_ACT_NONE;
  args.beta = 0;
  fill_common(args, status);
  args.out_mode = kOutPush;
  args.push_world = ctx->world;
  args.push_rank = ctx->rank;
  for (int r = 0; r < ctx->world; ++r) args.push_arena[r] = ctx->arena[r];
  args.push_bucket_off = bucket_off;
  args.push_rel = out_rel;
  args.push_per = per;
  int pairs = pairs_avail;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  const long long tiles = static_cast<long long>((M + 2 * kBM - 1) / (2 * kBM)) * ((N + 255) / 256);
  return launch2<256>(a, b, args, lda, ldb, pairs, tiles, stream);
}
