// Blockwise attention backward on the tcgen05 tensor cores, head dimension 64, bf16: dQ, dK, dV from Q, K, V, dO,
// the row log-sum-exp the forward kernel saved and delta = rowsum(dO * O).  Nothing of size S x S is read from or
// written to memory: the probabilities are recomputed tile by tile from the scores, as in the forward kernel
// (attention.cu).  The reference keeps the whole [S, S] matrix per head (ferrum-nn/src/transformer.rs:127-220).
//
// Two kernels, both shaped like the forward kernel (same operand layouts, same roles), so that neither needs an
// atomic or a cross-CTA reduction:
//
// Roles of a CTA (320 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 the elementwise work — two
// warps per tensor-memory lane quarter, each taking 64 of a tile's 128 columns, because that work (two
// tensor-memory reads, an exponential and half a dozen multiply-adds per score) and not the MMAs bounds a tile.
//
//   attn_bwd_dq_kernel    a CTA owns 128 query rows and walks the key / value tiles:
//                           S = Q K_j^T, dP = dO V_j^T            (tensor memory, 2 x 128 columns)
//                           dS = P * (dP - delta) * scale          (thread = query row; bf16 into shared memory)
//                           dQ += dS K_j                           (accumulates in tensor memory over all tiles)
//   attn_bwd_dkv_kernel   a CTA owns 128 keys and walks the query tiles, everything transposed:
//                           S^T = K Q_i^T, dP^T = V dO_i^T
//                           P^T, dS^T                              (thread = key row; lse / delta of the tile's
//                                                                   queries come through shared memory)
//                           dV += P^T dO_i,  dK += dS^T Q_i        (accumulate in tensor memory)
//
// The scores are computed twice (once per kernel): 7 tile GEMMs per pair of tiles instead of 5, in exchange for
// kernels without atomics whose every MMA operand layout is one the forward kernel already uses.  Causal masks
// skip the tiles on the far side of the diagonal in both kernels.  Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../common/ptx.cuh"
#include "../common/status.h"
#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

constexpr int kT = 128;                     // rows of a query tile = rows of a key tile
constexpr int kBlk = kT * 128;              // 16 KB: 128 rows of 64 bf16 = one 128-byte-swizzled block
constexpr int kPBytes = 2 * kBlk;           // a 128 x 128 bf16 matrix: two k-blocks of 128 rows x 128 bytes
constexpr int kBwdThreads = 320;            // TMA warp, MMA warp, eight softmax warps
constexpr int kSoftmaxWarps = 8;            // two per tensor-memory lane quarter, 64 of the tile's 128 columns each
constexpr int kTmemBwd = 512;
// D = head dimension (64 or 128).  An operand tile (128 rows x D) is D / 64 blocks side by side.  With D = 64 the
// tiles that change per iteration sit in a two-stage ring; with D = 128 shared memory (160 KB / 206 KB) and tensor
// memory (dK/dV: all 512 columns) leave room for one stage only.
template <int D>
struct BwdCfg {
  static constexpr int kNB = D / 64;
  static constexpr int kTile = kNB * kBlk;
  static constexpr int kStages = D == 64 ? 2 : 1;
  static constexpr int kSmemDq = 2 * kTile + 2 * kStages * kTile + kPBytes + 1024 + 256;  // Q dO | K | V | dS
  static constexpr int kSmemDkv = 2 * kTile + 2 * kStages * kTile + 2 * kPBytes + 8192 + 1024 + 256;  // K V | Q | dO | P^T dS^T | lse, delta
};

// One operand tile: D / 64 boxes of 64 columns x 128 rows.
template <int D>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int row0, int h, int b) {
#pragma unroll
  for (int nb = 0; nb < D / 64; ++nb) ptx::tma_load_4d(dst + nb * kBlk, map, bar, nb * 64, row0, h, b);
}
constexpr float kLog2e = 1.4426950408889634f;

struct BwdArgs {
  __nv_bfloat16* dq;   // [B, Sq, H, D]
  __nv_bfloat16* dk;   // [B, Skv, H, D]
  __nv_bfloat16* dv;   // [B, Skv, H, D]
  const float* lse;    // [B, H, Sq] natural log
  const float* delta;  // [B, H, Sq]
  int B, H, Sq, Skv;
  float scale, scale_log2;
  int causal;
  int32_t* status;
  unsigned long long timeout_ns;
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 128 x 128 x D product of two K-major tiles (rows x D): the score shape.
template <int D>
__device__ __forceinline__ void mma_scores(uint32_t tmem, uint32_t a, uint32_t b, uint32_t idesc) {
#pragma unroll
  for (int k = 0; k < D / 16; ++k)
    ptx::umma_f16(tmem, ptx::make_smem_desc_sw128(a + (k >> 2) * kBlk + (k & 3) * 32, 16, 1024),
                  ptx::make_smem_desc_sw128(b + (k >> 2) * kBlk + (k & 3) * 32, 16, 1024), idesc, k != 0 ? 1u : 0u);
}
// 128 x D x 128 product: A = a 128 x 128 matrix in two K-major k-blocks, B = a 128 x D tile whose D columns are
// contiguous (MN-major; its 64-column blocks lie kBlk apart): the P V shape of the forward kernel.
__device__ __forceinline__ void mma_pv(uint32_t tmem, uint32_t a, uint32_t b, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int k = 0; k < kT / 16; ++k)
    ptx::umma_f16(tmem, ptx::make_smem_desc_sw128(a + (k >> 2) * kBlk + (k & 3) * 32, 16, 1024),
                  ptx::make_smem_desc_sw128(b + k * 2048, kBlk, 1024), idesc, (accumulate || k != 0) ? 1u : 0u);
}

// 16 columns (8 bf16 pairs) of one row, starting at column col (a multiple of 16): two 16-byte chunks of the row's
// 128-byte line in k-block (col >> 6), swizzled.
__device__ __forceinline__ void store_cols16(uint8_t* mat, int row, int col, const uint32_t (&w)[8]) {
  uint8_t* blk = mat + (col >> 6) * kBlk + row * 128;
  const int chunk = (col & 63) >> 3;
  *reinterpret_cast<uint4*>(blk + (((chunk) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint4*>(blk + (((chunk + 1) ^ (row & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
}

// Chunks c_lo .. c_hi - 1 (32 columns each) of an accumulator row from tensor memory to bf16 in global memory.  The tensor-memory loads are
// warp-wide (.sync.aligned): EVERY lane of the warp must call this, `valid` only predicates the stores.
__device__ __forceinline__ void store_row_bf16(__nv_bfloat16* dst, uint32_t tmem_row, bool valid, int c_lo,
                                               int c_hi) {
#pragma unroll 1
  for (int c = c_lo; c < c_hi; ++c) {
    uint32_t r[32];
    ptx::tmem_ld_32x32b_x32(tmem_row + c * 32, r);
    ptx::tmem_wait_ld();
    if (!valid) continue;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(r[q * 8 + e * 2]),
                                                        __uint_as_float(r[q * 8 + e * 2 + 1]));
        w[e] = *reinterpret_cast<const uint32_t*>(&pk);
      }
      reinterpret_cast<uint4*>(dst)[c * 4 + q] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ dQ
template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                   const BwdArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kTile = BwdCfg<D>::kTile, kStages = BwdCfg<D>::kStages;
  uint8_t* sq = smem;
  uint8_t* sdo = sq + kTile;
  uint8_t* sk = sdo + kTile;             // kStages stages
  uint8_t* sv = sk + kStages * kTile;    // kStages stages
  uint8_t* sds = sv + kStages * kTile;   // dS: 128 x 128 bf16
  uint8_t* bar_base = sds + kPBytes;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* kv_full = q_full + 1;    // [2]
  uint64_t* kv_empty = kv_full + 2;  // [2]
  uint64_t* sp_full = kv_empty + 2;  // S and dP of a tile are complete
  uint64_t* ds_full = sp_full + 1;   // dS written (and S, dP read) by the four softmax warps
  uint64_t* ds_empty = ds_full + 1;  // the dQ MMAs have read dS
  uint64_t* dq_full = ds_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * kT;
  const int h = blockIdx.y % p.H, b = blockIdx.y / p.H;
  const int off = p.Skv - p.Sq;
  const int kv_end = p.causal ? min(p.Skv, q0 + kT + off) : p.Skv;
  const int n_tiles = (kv_end + kT - 1) / kT;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&kv_full[s], 1);
      ptx::mbar_init(&kv_empty[s], 1);
    }
    ptx::mbar_init(sp_full, 1);
    ptx::mbar_init(ds_full, kSoftmaxWarps);
    ptx::mbar_init(ds_empty, 1);
    ptx::mbar_init(dq_full, 1);
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
    ptx::prefetch_tensormap(&map_do);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemBwd);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dq = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      ptx::mbar_arrive_expect_tx(q_full, 2 * kTile);
      load_tile<D>(sq, &map_q, q_full, q0, h, b);
      load_tile<D>(sdo, &map_do, q_full, q0, h, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % kStages;
        const uint32_t round = static_cast<uint32_t>(j / kStages) & 1u;
        if (!ptx::mbar_wait(&kv_empty[st], round ^ 1u, abort_flag, p.timeout_ns)) {
          report_status(p.status, kStatusGemmTimeout, 61, blockIdx.x, j);
          break;
        }
        ptx::mbar_arrive_expect_tx(&kv_full[st], 2 * kTile);
        load_tile<D>(sk + st * kTile, &map_k, &kv_full[st], j * kT, h, b);
        load_tile<D>(sv + st * kTile, &map_v, &kv_full[st], j * kT, h, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = ptx::make_idesc(1u, kT, kT, 0, 0);
      const uint32_t idesc_o = ptx::make_idesc(1u, kT, D, 0, 1);
      const uint32_t sq_a = ptx::smem_u32(sq), sdo_a = ptx::smem_u32(sdo), sds_a = ptx::smem_u32(sds);
      bool ok = ptx::mbar_wait(q_full, 0, abort_flag, p.timeout_ns);
      if (!ok) report_status(p.status, kStatusGemmTimeout, 62, blockIdx.x, 0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int st = j % kStages;
        const uint32_t sk_a = ptx::smem_u32(sk + st * kTile), sv_a = ptx::smem_u32(sv + st * kTile);
        if (!ptx::mbar_wait(&kv_full[st], static_cast<uint32_t>(j / kStages) & 1u, abort_flag, p.timeout_ns)) {
          report_status(p.status, kStatusGemmTimeout, 63, blockIdx.x, j);
          break;
        }
        ptx::tc_fence_after();
        // (S and dP of the previous tile were read before its ds_full, which the previous iteration waited for)
        mma_scores<D>(t_s, sq_a, sk_a, idesc_s);
        mma_scores<D>(t_dp, sdo_a, sv_a, idesc_s);
        ptx::umma_commit(sp_full);
        if (!ptx::mbar_wait(ds_full, j & 1, abort_flag, p.timeout_ns)) {
          report_status(p.status, kStatusGemmTimeout, 64, blockIdx.x, j);
          break;
        }
        ptx::tc_fence_after();
        mma_pv(t_dq, sds_a, sk_a, idesc_o, j != 0);
        ptx::umma_commit(&kv_empty[st]);
        ptx::umma_commit(ds_empty);
        if (j + 1 == n_tiles) ptx::umma_commit(dq_full);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;      // which 64 columns of a tile this warp handles
    const int row = quarter * 32 + lane;
    const int qrow = q0 + row;
    const uint32_t t_row = (static_cast<uint32_t>(quarter * 32) << 16);
    const long long stat = (static_cast<long long>(b) * p.H + h) * p.Sq + qrow;
    // a row past the end contributes nothing: +inf makes every probability zero
    const float lse2 = qrow < p.Sq ? p.lse[stat] * kLog2e : INFINITY;
    const float delta = qrow < p.Sq ? p.delta[stat] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const bool ready = ptx::mbar_wait(sp_full, j & 1, abort_flag, p.timeout_ns);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) report_status(p.status, kStatusGemmTimeout, 65, blockIdx.x, j);
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      if (j > 0) {  // the dQ MMAs of the previous tile have read dS
        const bool freed = ptx::mbar_wait(ds_empty, (j - 1) & 1, abort_flag, p.timeout_ns);
        if (!__all_sync(0xffffffffu, freed)) {
          if (lane == 0) report_status(p.status, kStatusGemmTimeout, 66, blockIdx.x, j);
          ok = false;
          break;
        }
      }
      int valid = min(kT, p.Skv - j * kT);
      if (p.causal) valid = max(0, min(valid, qrow + off + 1 - j * kT));
      // The warp's 64 columns in four batches of 16: the tensor-memory loads of batch k + 1 are in flight while
      // batch k is computed (tcgen05.wait::ld waits for every load issued before it, so the wait for a batch comes
      // after the arithmetic of the previous one).
      {
        const float2 sl2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(-lse2, -lse2);
        const float2 sc2 = make_float2(p.scale, p.scale), nd2 = make_float2(-delta * p.scale, -delta * p.scale);
        auto batch = [&](int col, const uint32_t (&rs)[16], const uint32_t (&rp)[16]) {
          uint32_t w[8];
          // packed path (two scores per instruction) unless the causal diagonal or the end of the keys cuts a row
          if (__all_sync(0xffffffffu, col + 16 <= valid)) {
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const float2 e = __ffma2_rn(make_float2(__uint_as_float(rs[i]), __uint_as_float(rs[i + 1])), sl2, nl2);
              const float2 t = __ffma2_rn(make_float2(__uint_as_float(rp[i]), __uint_as_float(rp[i + 1])), sc2, nd2);
              const float2 d = __fmul2_rn(make_float2(ex2f(e.x), ex2f(e.y)), t);
              const __nv_bfloat162 pk = __floats2bfloat162_rn(d.x, d.y);
              w[i >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              float d0 = 0.f, d1 = 0.f;
              if (col + i < valid)
                d0 = ex2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse2)) * (__uint_as_float(rp[i]) - delta) * p.scale;
              if (col + i + 1 < valid)
                d1 = ex2f(fmaf(__uint_as_float(rs[i + 1]), p.scale_log2, -lse2)) *
                     (__uint_as_float(rp[i + 1]) - delta) * p.scale;
              const __nv_bfloat162 pk = __floats2bfloat162_rn(d0, d1);
              w[i >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
            }
          }
          store_cols16(sds, row, col, w);
        };
        const int c0 = half * 64;
        uint32_t sa[16], pa[16], sb[16], pb[16];
        ptx::tmem_ld_32x32b_x16(t_s + t_row + c0, sa);
        ptx::tmem_ld_32x32b_x16(t_dp + t_row + c0, pa);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_32x32b_x16(t_s + t_row + c0 + 16, sb);
        ptx::tmem_ld_32x32b_x16(t_dp + t_row + c0 + 16, pb);
        batch(c0, sa, pa);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_32x32b_x16(t_s + t_row + c0 + 32, sa);
        ptx::tmem_ld_32x32b_x16(t_dp + t_row + c0 + 32, pa);
        batch(c0 + 16, sb, pb);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_32x32b_x16(t_s + t_row + c0 + 48, sb);
        ptx::tmem_ld_32x32b_x16(t_dp + t_row + c0 + 48, pb);
        batch(c0 + 32, sa, pa);
        ptx::tmem_wait_ld();
        batch(c0 + 48, sb, pb);
      }
      ptx::tc_fence_before();
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ds_full);
    }
    if (ok) {
      const bool done = n_tiles > 0 ? ptx::mbar_wait(dq_full, 0, abort_flag, p.timeout_ns) : true;
      if (!__all_sync(0xffffffffu, done)) {
        if (lane == 0) report_status(p.status, kStatusGemmTimeout, 67, blockIdx.x, 0);
      } else {
        ptx::tc_fence_after();
        __nv_bfloat16* dst = p.dq + ((static_cast<long long>(b) * p.Sq + qrow) * p.H + h) * D;
        if (n_tiles > 0) {  // uniform over the CTA; each warp of a quarter stores half of the D columns
          store_row_bf16(dst, t_dq + t_row, qrow < p.Sq, half * (D / 64), (half + 1) * (D / 64));
        } else if (qrow < p.Sq && half == 0) {
#pragma unroll
          for (int q = 0; q < D / 8; ++q) reinterpret_cast<uint4*>(dst)[q] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemBwd);
  }
}

// ------------------------------------------------------------------------------------------------ dK, dV
template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                    const BwdArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kTile = BwdCfg<D>::kTile, kStages = BwdCfg<D>::kStages;
  uint8_t* sk = smem;
  uint8_t* sv = sk + kTile;
  uint8_t* sq = sv + kTile;              // kStages stages
  uint8_t* sdo = sq + kStages * kTile;   // kStages stages
  uint8_t* spt = sdo + kStages * kTile;  // P^T: 128 keys x 128 queries bf16
  uint8_t* sdst = spt + kPBytes;   // dS^T
  float* s_stat = reinterpret_cast<float*>(sdst + kPBytes);  // per softmax warp: [lse2 | delta][128]
  uint8_t* bar_base = reinterpret_cast<uint8_t*>(s_stat) + 8192;
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* qd_full = kv_full + 1;    // [2]
  uint64_t* qd_empty = qd_full + 2;   // [2]
  uint64_t* sp_full = qd_empty + 2;
  uint64_t* pt_full = sp_full + 1;
  uint64_t* pt_empty = pt_full + 1;
  uint64_t* acc_full = pt_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * kT;
  const int h = blockIdx.y % p.H, b = blockIdx.y / p.H;
  const int off = p.Skv - p.Sq;
  const int n_qtiles = (p.Sq + kT - 1) / kT;
  // causal: query q sees key k when k <= q + off, so the first query that sees this tile's first key is k0 - off
  const int i_begin = p.causal ? max(0, k0 - off) / kT : 0;
  const int n_iter = max(0, n_qtiles - i_begin);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    ptx::mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&qd_full[s], 1);
      ptx::mbar_init(&qd_empty[s], 1);
    }
    ptx::mbar_init(sp_full, 1);
    ptx::mbar_init(pt_full, kSoftmaxWarps);
    ptx::mbar_init(pt_empty, 1);
    ptx::mbar_init(acc_full, 1);
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
    ptx::prefetch_tensormap(&map_do);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemBwd);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 256 + D;

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      ptx::mbar_arrive_expect_tx(kv_full, 2 * kTile);
      load_tile<D>(sk, &map_k, kv_full, k0, h, b);
      load_tile<D>(sv, &map_v, kv_full, k0, h, b);
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % kStages, i = i_begin + it;
        const uint32_t round = static_cast<uint32_t>(it / kStages) & 1u;
        if (!ptx::mbar_wait(&qd_empty[st], round ^ 1u, abort_flag, p.timeout_ns)) {
          report_status(p.status, kStatusGemmTimeout, 71, blockIdx.x, it);
          break;
        }
        ptx::mbar_arrive_expect_tx(&qd_full[st], 2 * kTile);
        load_tile<D>(sq + st * kTile, &map_q, &qd_full[st], i * kT, h, b);
        load_tile<D>(sdo + st * kTile, &map_do, &qd_full[st], i * kT, h, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_s = ptx::make_idesc(1u, kT, kT, 0, 0);
      const uint32_t idesc_o = ptx::make_idesc(1u, kT, D, 0, 1);
      const uint32_t sk_a = ptx::smem_u32(sk), sv_a = ptx::smem_u32(sv);
      const uint32_t spt_a = ptx::smem_u32(spt), sdst_a = ptx::smem_u32(sdst);
      bool ok = ptx::mbar_wait(kv_full, 0, abort_flag, p.timeout_ns);
      if (!ok) report_status(p.status, kStatusGemmTimeout, 72, blockIdx.x, 0);
      for (int it = 0; ok && it < n_iter; ++it) {
        const int st = it % kStages;
        const uint32_t sq_a = ptx::smem_u32(sq + st * kTile), sdo_a = ptx::smem_u32(sdo + st * kTile);
        if (!ptx::mbar_wait(&qd_full[st], static_cast<uint32_t>(it / kStages) & 1u, abort_flag, p.timeout_ns)) {
          report_status(p.status, kStatusGemmTimeout, 73, blockIdx.x, it);
          break;
        }
        ptx::tc_fence_after();
        mma_scores<D>(t_s, sk_a, sq_a, idesc_s);     // S^T  = K Q_i^T
        mma_scores<D>(t_dp, sv_a, sdo_a, idesc_s);   // dP^T = V dO_i^T
        ptx::umma_commit(sp_full);
        if (!ptx::mbar_wait(pt_full, it & 1, abort_flag, p.timeout_ns)) {
          report_status(p.status, kStatusGemmTimeout, 74, blockIdx.x, it);
          break;
        }
        ptx::tc_fence_after();
        mma_pv(t_dv, spt_a, sdo_a, idesc_o, it != 0);   // dV += P^T dO_i
        mma_pv(t_dk, sdst_a, sq_a, idesc_o, it != 0);   // dK += dS^T Q_i
        ptx::umma_commit(&qd_empty[st]);
        ptx::umma_commit(pt_empty);
        if (it + 1 == n_iter) ptx::umma_commit(acc_full);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;      // which 64 query columns of a tile this warp handles
    const int row = quarter * 32 + lane;   // key row of this thread
    const int krow = k0 + row;
    const uint32_t t_row = (static_cast<uint32_t>(quarter * 32) << 16);
    const long long stat_base = (static_cast<long long>(b) * p.H + h) * p.Sq;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int i = i_begin + it;
      // Every warp keeps its own copy of the tile's 128 (lse, delta) pairs, so that no barrier between warps is
      // needed (a warp that gave up on a wait must not leave the others stuck at one).
      float* slot = s_stat + (warp - 2) * 256;
      __syncwarp();  // the previous iteration's reads are done
#pragma unroll
      for (int x = 2 * half; x < 2 * half + 2; ++x) {  // only the columns this warp handles
        const int ql = x * 32 + lane, q = i * kT + ql;
        // negated, so that one fused multiply-add forms the exponent; -inf: a query past the end sees nothing
        slot[ql] = q < p.Sq ? -p.lse[stat_base + q] * kLog2e : -INFINITY;
        slot[128 + ql] = q < p.Sq ? -p.delta[stat_base + q] * p.scale : 0.f;
      }
      __syncwarp();
      const bool ready = ptx::mbar_wait(sp_full, it & 1, abort_flag, p.timeout_ns);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) report_status(p.status, kStatusGemmTimeout, 75, blockIdx.x, it);
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      if (it > 0) {
        const bool freed = ptx::mbar_wait(pt_empty, (it - 1) & 1, abort_flag, p.timeout_ns);
        if (!__all_sync(0xffffffffu, freed)) {
          if (lane == 0) report_status(p.status, kStatusGemmTimeout, 76, blockIdx.x, it);
          ok = false;
          break;
        }
      }
      // queries of this tile that may see this key: all of them, or (causal) those with q + off >= key
      const int q_first = p.causal ? max(0, krow - off - i * kT) : 0;  // first local query column that sees the key
      // Four batches of 16 query columns, tensor-memory loads of the next batch in flight during the arithmetic.
      // Keys past the end need no mask (their rows of dK / dV are never stored and no other row depends on them);
      // only the causal diagonal does.
      {
        const float2 sl2 = make_float2(p.scale_log2, p.scale_log2), sc2 = make_float2(p.scale, p.scale);
        auto batch = [&](int col, const uint32_t (&rs)[16], const uint32_t (&rp)[16]) {
          uint32_t wp[8], wd[8];
          if (__all_sync(0xffffffffu, q_first <= col)) {
#pragma unroll
            for (int x = 0; x < 16; x += 4) {
              const float4 nl = *reinterpret_cast<const float4*>(slot + col + x);
              const float4 nd = *reinterpret_cast<const float4*>(slot + 128 + col + x);
              const float2 e0 = __ffma2_rn(make_float2(__uint_as_float(rs[x]), __uint_as_float(rs[x + 1])), sl2,
                                           make_float2(nl.x, nl.y));
              const float2 e1 = __ffma2_rn(make_float2(__uint_as_float(rs[x + 2]), __uint_as_float(rs[x + 3])), sl2,
                                           make_float2(nl.z, nl.w));
              const float2 t0 = __ffma2_rn(make_float2(__uint_as_float(rp[x]), __uint_as_float(rp[x + 1])), sc2,
                                           make_float2(nd.x, nd.y));
              const float2 t1 = __ffma2_rn(make_float2(__uint_as_float(rp[x + 2]), __uint_as_float(rp[x + 3])), sc2,
                                           make_float2(nd.z, nd.w));
              const float2 p0 = make_float2(ex2f(e0.x), ex2f(e0.y)), p1 = make_float2(ex2f(e1.x), ex2f(e1.y));
              const float2 d0 = __fmul2_rn(p0, t0), d1 = __fmul2_rn(p1, t1);
              const __nv_bfloat162 a0 = __floats2bfloat162_rn(p0.x, p0.y), a1 = __floats2bfloat162_rn(p1.x, p1.y);
              const __nv_bfloat162 b0 = __floats2bfloat162_rn(d0.x, d0.y), b1 = __floats2bfloat162_rn(d1.x, d1.y);
              wp[x >> 1] = *reinterpret_cast<const uint32_t*>(&a0);
              wp[(x >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&a1);
              wd[x >> 1] = *reinterpret_cast<const uint32_t*>(&b0);
              wd[(x >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&b1);
            }
          } else {
#pragma unroll
            for (int x = 0; x < 16; x += 2) {
              float p0 = 0.f, p1 = 0.f, d0 = 0.f, d1 = 0.f;
              const int qa = col + x;
              if (qa >= q_first) {
                p0 = ex2f(fmaf(__uint_as_float(rs[x]), p.scale_log2, slot[qa]));
                d0 = p0 * fmaf(__uint_as_float(rp[x]), p.scale, slot[128 + qa]);
              }
              if (qa + 1 >= q_first) {
                p1 = ex2f(fmaf(__uint_as_float(rs[x + 1]), p.scale_log2, slot[qa + 1]));
                d1 = p1 * fmaf(__uint_as_float(rp[x + 1]), p.scale, slot[128 + qa + 1]);
              }
              const __nv_bfloat162 a = __floats2bfloat162_rn(p0, p1), d = __floats2bfloat162_rn(d0, d1);
              wp[x >> 1] = *reinterpret_cast<const uint32_t*>(&a);
              wd[x >> 1] = *reinterpret_cast<const uint32_t*>(&d);
            }
          }
          store_cols16(spt, row, col, wp);
          store_cols16(sdst, row, col, wd);
        };
        const int c0 = half * 64;
        uint32_t sa[16], pa[16], sb[16], pb[16];
        ptx::tmem_ld_32x32b_x16(t_s + t_row + c0, sa);
        ptx::tmem_ld_32x32b_x16(t_dp + t_row + c0, pa);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_32x32b_x16(t_s + t_row + c0 + 16, sb);
        ptx::tmem_ld_32x32b_x16(t_dp + t_row + c0 + 16, pb);
        batch(c0, sa, pa);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_32x32b_x16(t_s + t_row + c0 + 32, sa);
        ptx::tmem_ld_32x32b_x16(t_dp + t_row + c0 + 32, pa);
        batch(c0 + 16, sb, pb);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_32x32b_x16(t_s + t_row + c0 + 48, sb);
        ptx::tmem_ld_32x32b_x16(t_dp + t_row + c0 + 48, pb);
        batch(c0 + 32, sa, pa);
        ptx::tmem_wait_ld();
        batch(c0 + 48, sb, pb);
      }
      ptx::tc_fence_before();
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(pt_full);
    }
    if (n_iter == 0 && krow < p.Skv && half == 0) {  // no query sees these keys
      __nv_bfloat16* dv = p.dv + ((static_cast<long long>(b) * p.Skv + krow) * p.H + h) * D;
      __nv_bfloat16* dk = p.dk + ((static_cast<long long>(b) * p.Skv + krow) * p.H + h) * D;
#pragma unroll
      for (int q = 0; q < D / 8; ++q) {
        reinterpret_cast<uint4*>(dv)[q] = make_uint4(0u, 0u, 0u, 0u);
        reinterpret_cast<uint4*>(dk)[q] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (n_iter > 0 && ok) {  // both uniform over the warp
      const bool done = ptx::mbar_wait(acc_full, 0, abort_flag, p.timeout_ns);
      if (!__all_sync(0xffffffffu, done)) {
        if (lane == 0) report_status(p.status, kStatusGemmTimeout, 77, blockIdx.x, 0);
      } else {
        ptx::tc_fence_after();
        // the two warps of a lane quarter share the work: one stores the dV rows, the other the dK rows
        if (half == 0)
          store_row_bf16(p.dv + ((static_cast<long long>(b) * p.Skv + krow) * p.H + h) * D, t_dv + t_row,
                         krow < p.Skv, 0, D / 32);
        else
          store_row_bf16(p.dk + ((static_cast<long long>(b) * p.Skv + krow) * p.H + h) * D, t_dk + t_row,
                         krow < p.Skv, 0, D / 32);
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemBwd);
  }
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]  (both [B, S, H, D] contiguous bf16); warp per row.
template <int D>
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int B, int H, int S) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;  // over B * S * H
  const int lane = threadIdx.x & 31;
  const long long rows = static_cast<long long>(B) * S * H;
  if (row >= rows) return;
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < D / 64; ++i) {
    const __nv_bfloat162 a = reinterpret_cast<const __nv_bfloat162*>(o + row * D)[lane + 32 * i];
    const __nv_bfloat162 g = reinterpret_cast<const __nv_bfloat162*>(d_o + row * D)[lane + 32 * i];
    acc += __bfloat162float(a.x) * __bfloat162float(g.x) + __bfloat162float(a.y) * __bfloat162float(g.y);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) {
    const int hh = static_cast<int>(row % H);
    const long long bs = row / H;
    const int ss = static_cast<int>(bs % S);
    const long long bb = bs / S;
    delta[(bb * H + hh) * S + ss] = acc;
  }
}

typedef CUresult (*EncodeTiledFnB)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFnB encode_fn_b() {
  // The driver's encoder wants a current context; a thread that has made no runtime call yet (an autograd
  // worker entering its first backward) has none, and the encoder then fails with CUDA_ERROR_INVALID_CONTEXT.
  static thread_local bool bound = false;
  if (!bound) {  // cudaSetDevice binds the primary context to the thread and is legal during stream capture
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
    bound = true;
  }
  static EncodeTiledFnB fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFnB>(sym);
  }
  return fn;
}

// [B, H, S, D] bf16 view with element strides (sb, sh, ss): 4-D map, 64 x 128 x 1 x 1 box, rows past S read zeros.
int g_map_error = 0;  // why the last map_bhsd failed: -1 no driver entry point, -2 / -3 alignment, > 0 the driver's code

bool map_bhsd(CUtensorMap* map, const void* ptr, int B, int H, int S, int kD, long long sb, long long sh,
              long long ss) {
  EncodeTiledFnB enc = encode_fn_b();
  g_map_error = -1;
  if (enc == nullptr) return false;
  g_map_error = -2;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || ss % 8 || ss < kD) return false;
  g_map_error = -3;
  if ((H > 1 && (sh % 8 || sh <= 0)) || (B > 1 && (sb % 8 || sb <= 0))) return false;
  const long long sh_ok = H > 1 ? sh : ss * S + ((8 - (ss * S) % 8) % 8);
  const long long sb_ok = B > 1 ? sb : sh_ok * H;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(kD), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ss) * 2, static_cast<cuuint64_t>(sh_ok) * 2,
                           static_cast<cuuint64_t>(sb_ok) * 2};
  cuuint32_t box[4] = {64, 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  g_map_error = static_cast<int>(enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides,
                                       box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return g_map_error == 0;
}

}  // namespace
}  // namespace fb

// Reason of the last -2 ... -5 of fb_attention_bwd (see g_map_error).
extern "C" int fb_attention_bwd_map_error() { return fb::g_map_error; }

namespace fb {
namespace {
template <int D>
int launch_bwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
               const void* out, const void* d_out, const BwdArgs& a, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             BwdCfg<D>::kSmemDq) != cudaSuccess ||
        cudaFuncSetAttribute(attn_bwd_dkv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             BwdCfg<D>::kSmemDkv) != cudaSuccess)
      return static_cast<int>(cudaGetLastError());
    attr_set = true;
  }
  const long long rows = static_cast<long long>(a.B) * a.Sq * a.H;
  attn_delta_kernel<D><<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(d_out),
      const_cast<float*>(a.delta), a.B, a.H, a.Sq);
  attn_bwd_dq_kernel<D><<<dim3((a.Sq + kT - 1) / kT, a.B * a.H), kBwdThreads, BwdCfg<D>::kSmemDq, stream>>>(
      mq, mk, mv, mdo, a);
  attn_bwd_dkv_kernel<D><<<dim3((a.Skv + kT - 1) / kT, a.B * a.H), kBwdThreads, BwdCfg<D>::kSmemDkv, stream>>>(
      mq, mk, mv, mdo, a);
  return static_cast<int>(cudaGetLastError());
}
}  // namespace
}  // namespace fb

// Gradients of out = softmax(scale q k^T) v (head dimension D = 64 or 128, bf16).  q, k, v: [B, H, S, D] views with
// element strides (last dimension contiguous, strides multiples of 8); out, d_out: [B, Sq, H, D] contiguous (the
// forward kernel's output layout); lse: [B, H, Sq] fp32 as written by fb_attention_fwd; delta: [B, H, Sq] fp32
// scratch that this call fills.  dq: [B, Sq, H, D], dk, dv: [B, Skv, H, D], contiguous bf16.  Returns -2 ... -5
// when q / k / v / d_out cannot be described by a TMA map.
extern "C" int fb_attention_bwd(const void* q, const void* k, const void* v, const void* out, const void* d_out,
                                const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int H, int Sq,
                                int Skv, int D, long long q_sb, long long q_sh, long long q_ss, long long k_sb,
                                long long k_sh, long long k_ss, long long v_sb, long long v_sh, long long v_ss,
                                float scale, int causal, int32_t* status, cudaStream_t stream) {
  using namespace fb;
  if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0 || (causal && Skv < Sq) || (D != 64 && D != 128)) return -1;
  if (lse == nullptr || delta == nullptr || out == nullptr || d_out == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv) |
       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(d_out)) & 15)
    return -1;
  CUtensorMap mq, mk, mv, mdo;
  const long long o_sb = static_cast<long long>(Sq) * H * D, o_sh = D, o_ss = static_cast<long long>(H) * D;
  if (!map_bhsd(&mq, q, B, H, Sq, D, q_sb, q_sh, q_ss)) return -2;
  if (!map_bhsd(&mk, k, B, H, Skv, D, k_sb, k_sh, k_ss)) return -3;
  if (!map_bhsd(&mv, v, B, H, Skv, D, v_sb, v_sh, v_ss)) return -4;
  if (!map_bhsd(&mdo, d_out, B, H, Sq, D, o_sb, o_sh, o_ss)) return -5;
  BwdArgs a;
  a.dq = static_cast<__nv_bfloat16*>(dq);
  a.dk = static_cast<__nv_bfloat16*>(dk);
  a.dv = static_cast<__nv_bfloat16*>(dv);
  a.lse = lse;
  a.delta = delta;
  a.B = B;
  a.H = H;
  a.Sq = Sq;
  a.Skv = Skv;
  a.scale = scale;
  a.scale_log2 = scale * kLog2e;
  a.causal = causal ? 1 : 0;
  a.status = status;
  a.timeout_ns = 2000000000ull;
  return D == 64 ? launch_bwd<64>(mq, mk, mv, mdo, out, d_out, a, stream)
                 : launch_bwd<128>(mq, mk, mv, mdo, out, d_out, a, stream);
}
