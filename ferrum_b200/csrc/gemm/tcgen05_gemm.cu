// bf16 x bf16 -> fp32-accumulate GEMM for sm_100a on the 5th-generation
// tensor cores: TMA (cp.async.bulk.tensor, 128-byte swizzle) stages operand
// tiles in shared memory, one elected thread issues tcgen05.mma with the
// accumulator in tensor memory (TMEM), and four epilogue warps read the
// accumulator back with tcgen05.ld and apply bias / activation / dtype
// conversion while the next tile's main loop already runs (the 512 TMEM
// columns hold two 128 x 256 fp32 accumulators).
//
// Replaces the reference's scalar i-j-p loop (ferrum-core/src/tensor.rs:2487-2558)
// and the tiled / rayon / BLAS variants (ferrum-ops/src/matmul.rs:27-173).
//
// Computes   D[M,N] = act(A[M,K] * B[N,K]^T + bias[N])   (optionally += D)
// where each operand may be stored K-major (reduction dimension contiguous)
// or MN-major (M resp. N contiguous), which covers the three products of a
// linear layer without a transpose copy:
//   forward  y  = x  W^T : A K-major,  B K-major
//   dgrad    dx = dy W   : A K-major,  B MN-major
//   wgrad    dW = dy^T x : A MN-major, B MN-major
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + MMA issue (one elected lane)
//   warps 2..5  epilogue (TMEM lane quarter = warp_id % 4)
// No cluster launch and no multicast TMA: every CTA loads its own tiles, so
// the same binary is safe in multi-GPU jobs.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../common/ptx.cuh"
#include "../common/status.h"
#include "../include/ferrum_kernels.h"
#include "epilogue.cuh"

namespace fb {
namespace {

constexpr int kBM = 128;
// One 128-byte swizzle row of K per k-block and 32 bytes of K per tcgen05.mma, whatever the element type:
// bf16 (kind::f16): 64 / 16 elements; fp32 read as tf32 (kind::tf32): 32 / 8 elements.
constexpr int kRowBytes = 128;
template <bool kTf32>
struct El {
  static constexpr int kBytes = kTf32 ? 4 : 2;
  static constexpr int kBK = kRowBytes / kBytes;   // K elements per k-block
  static constexpr int kUmmaK = 32 / kBytes;       // K elements per MMA
  static constexpr int kMnChunk = kRowBytes / kBytes;  // MN elements per 128-byte row of an MN-major operand
};
constexpr int kThreads = 192;
constexpr int kGroupM = 16;  // m-blocks per rasterisation group (L2 reuse)

template <int BN>
struct Cfg {
  static constexpr int kABytes = kBM * kRowBytes;
  static constexpr int kBBytes = BN * kRowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + kBarrierBytes;
  static constexpr int kTmemCols = 2 * BN;  // two accumulators
};

struct GemmArgs {
  void* out;
  void* out2;  // optional: act'(z) in the layout and dtype of out (bf16 outputs only)
  const float* bias;
  int M, N, K;
  long long ldc;
  int a_mn_major, b_mn_major;
  int out_bf16;
  int act;
  int beta;
  int32_t* status;
  unsigned long long timeout_ns;
  // Batched form only: batch = batch_outer x batch_inner slices; the operands' slice strides live in
  // the 4-D tensor maps, the output's here (elements).  alpha scales the accumulator before bias / act.
  int batch_inner, batch_total;
  long long sc_outer, sc_inner;
  float alpha;
  // Convolution forms (kConv), stride 1, NHWC bf16 operands read through 4-D tensor maps {channel, x, y, image}:
  //   cv_wgrad == 0 (forward / data gradient): a row tile is a cv_tw x cv_th patch of 128 output pixels of one
  //     image, a k-block is 64 channels of one filter tap, and the A tile is the patch shifted by the tap
  //     (out-of-range pixels read zeros: the padding).
  //   cv_wgrad == 1 (weight gradient): rows = output channels, columns = input channels, and the REDUCTION runs
  //     over output pixels in patches of 64 (one k-block); tile index = ((split * taps + tap) * num_m + m) ...
  //     with the patches of a split summed into slice `split` of the output (sc_outer), tap at sc_inner * tap.
  int cv_wgrad;
  int cv_tw, cv_th, cv_tiles_w, cv_tiles_h, cv_nb;
  int cv_Ho, cv_Wo;
  int cv_kw, cv_taps, cv_cchunks, cv_cp;
  int cv_ph, cv_pw, cv_dh, cv_dw;
  int cv_splits, cv_kb_per_split, cv_total_kb;
};

// Patch index -> (image, first y, first x) of the patch.
__device__ __forceinline__ void conv_patch(const GemmArgs& p, int idx, int& b, int& y0, int& x0) {
  const int per_img = p.cv_tiles_h * p.cv_tiles_w;
  b = idx / per_img;
  const int r = idx - b * per_img;
  const int ty = r / p.cv_tiles_w;
  y0 = ty * p.cv_th;
  x0 = (r - ty * p.cv_tiles_w) * p.cv_tw;
}

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int per_group = kGroupM * num_n;
  const int g = t / per_group;
  const int first_m = g * kGroupM;
  const int gsize = min(num_m - first_m, kGroupM);
  const int r = t - g * per_group;
  m_blk = first_m + (r % gsize);
  n_blk = r / gsize;
}

template <int BN, bool kBatched, bool kTf32, bool kConv = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmArgs p) {
  using C = Cfg<BN>;
  constexpr int kBK = El<kTf32>::kBK, kUmmaK = El<kTf32>::kUmmaK, kMnChunk = El<kTf32>::kMnChunk;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_base = smem + C::kStages * C::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* tmem_full = empty_bar + C::kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const bool conv_rows = kConv && !p.cv_wgrad;   // rows are output pixels
  const bool conv_red = kConv && p.cv_wgrad;     // the reduction runs over output pixels
  const int num_m = conv_rows ? p.cv_nb * p.cv_tiles_h * p.cv_tiles_w : (p.M + kBM - 1) / kBM;
  const int num_n = (p.N + BN - 1) / BN;
  const int tiles_per_slice = num_m * num_n;
  const int num_tiles = kBatched ? tiles_per_slice * p.batch_total
                                 : (conv_red ? tiles_per_slice * p.cv_taps * p.cv_splits : tiles_per_slice);
  const int num_kb = conv_rows ? p.cv_taps * p.cv_cchunks : (p.K + kBK - 1) / kBK;
  // k-blocks [kb_lo, kb_hi) of tile t: everything, or (weight gradient) the pixel patches of the tile's split
  auto kb_range = [&](int t, int& kb_lo, int& kb_hi) {
    kb_lo = 0;
    kb_hi = num_kb;
    if (conv_red) {
      const int split = (t / tiles_per_slice) / p.cv_taps;
      kb_lo = split * p.cv_kb_per_split;
      kb_hi = min(p.cv_total_kb, kb_lo + p.cv_kb_per_split);
    }
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&tmem_full[a], 1);
      ptx::mbar_init(&tmem_empty[a], 4);
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tma_a);
    ptx::prefetch_tensormap(&tma_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        const int slice = (kBatched || conv_red) ? t / tiles_per_slice : 0;
        tile_coords((kBatched || conv_red) ? t - slice * tiles_per_slice : t, num_m, num_n, m_blk, n_blk);
        const int m0 = m_blk * kBM, n0 = n_blk * BN;
        const int bz = kBatched ? slice % p.batch_inner : 0, bw = kBatched ? slice / p.batch_inner : 0;
        int kb_lo, kb_hi;
        kb_range(t, kb_lo, kb_hi);
        int cb = 0, cy0 = 0, cx0 = 0;              // conv, rows = pixels: this tile's patch
        if (conv_rows) conv_patch(p, m_blk, cb, cy0, cx0);
        const int ctap = conv_red ? slice % p.cv_taps : 0;   // conv, weight gradient: this tile's filter tap
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.timeout_ns)) {
            report_status(p.status, kStatusGemmTimeout, 1, blockIdx.x, stage);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          ptx::mbar_arrive_expect_tx(&full_bar[stage], C::kStageBytes);
          const int k0 = kb * kBK;
          if constexpr (kConv) {
            if (!p.cv_wgrad) {
              const int tap = kb / p.cv_cchunks, cc = kb - tap * p.cv_cchunks;
              const int khi = tap / p.cv_kw, kwi = tap - khi * p.cv_kw;
              ptx::tma_load_4d(sa, &tma_a, &full_bar[stage], cc * 64, cx0 - p.cv_pw + kwi * p.cv_dw,
                               cy0 - p.cv_ph + khi * p.cv_dh, cb);
              ptx::tma_load_2d(sb, &tma_b, &full_bar[stage], tap * p.cv_cp + cc * 64, n0);
            } else {
              int pb, py0, px0;
              conv_patch(p, kb, pb, py0, px0);
              const int khi = ctap / p.cv_kw, kwi = ctap - khi * p.cv_kw;
#pragma unroll
              for (int c = 0; c < kBM / 64; ++c)
                ptx::tma_load_4d(sa + c * (64 * 128), &tma_a, &full_bar[stage], m0 + c * 64, px0, py0, pb);
#pragma unroll
              for (int c = 0; c < BN / 64; ++c)
                ptx::tma_load_4d(sb + c * (64 * 128), &tma_b, &full_bar[stage], n0 + c * 64,
                                 px0 - p.cv_pw + kwi * p.cv_dw, py0 - p.cv_ph + khi * p.cv_dh, pb);
            }
          } else if constexpr (kBatched) {
            if (p.a_mn_major) {
#pragma unroll
              for (int c = 0; c < kBM / kMnChunk; ++c)
                ptx::tma_load_4d(sa + c * (kBK * 128), &tma_a, &full_bar[stage], m0 + c * kMnChunk, k0, bz, bw);
            } else {
              ptx::tma_load_4d(sa, &tma_a, &full_bar[stage], k0, m0, bz, bw);
            }
            if (p.b_mn_major) {
#pragma unroll
              for (int c = 0; c < BN / kMnChunk; ++c)
                ptx::tma_load_4d(sb + c * (kBK * 128), &tma_b, &full_bar[stage], n0 + c * kMnChunk, k0, bz, bw);
            } else {
              ptx::tma_load_4d(sb, &tma_b, &full_bar[stage], k0, n0, bz, bw);
            }
          } else {
            if (p.a_mn_major) {
#pragma unroll
              for (int c = 0; c < kBM / kMnChunk; ++c)
                ptx::tma_load_2d(sa + c * (kBK * 128), &tma_a, &full_bar[stage], m0 + c * kMnChunk, k0);
            } else {
              ptx::tma_load_2d(sa, &tma_a, &full_bar[stage], k0, m0);
            }
            if (p.b_mn_major) {
#pragma unroll
              for (int c = 0; c < BN / kMnChunk; ++c)
                ptx::tma_load_2d(sb + c * (kBK * 128), &tma_b, &full_bar[stage], n0 + c * kMnChunk, k0);
            } else {
              ptx::tma_load_2d(sb, &tma_b, &full_bar[stage], k0, n0);
            }
          }
          ++issued;
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Drain: wait (bounded) for the copies this thread already issued so
        // that no bulk copy is still writing shared memory when the CTA exits.
        for (int s = 0; s < C::kStages; ++s) {
          if (issued > s) {
            const long long last = ((issued - 1 - s) / C::kStages) * C::kStages + s;
            const uint32_t par = static_cast<uint32_t>((last / C::kStages) & 1);
            const uint64_t t0 = ptx::globaltimer();
            while (!ptx::mbar_try_wait(&full_bar[s], par)) {
              if (ptx::globaltimer() - t0 > p.timeout_ns) break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = ptx::make_idesc(kTf32 ? 2u : 1u, kBM, BN, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? kBK * 128 : 16;
      const uint32_t b_lbo = p.b_mn_major ? kBK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? kUmmaK * 128 : 32;  // MN-major: kUmmaK rows of 128 B; K-major: 32 B
      const uint32_t b_kstep = p.b_mn_major ? kUmmaK * 128 : 32;
      // MN-major fp32 operands sit in shared memory with the 32-byte-chunk swizzle (4-row groups, 512 B apart)
      const uint32_t a_layout = (kTf32 && p.a_mn_major) ? 1u : 2u, a_sbo = (kTf32 && p.a_mn_major) ? 512u : 1024u;
      const uint32_t b_layout = (kTf32 && p.b_mn_major) ? 1u : 2u, b_sbo = (kTf32 && p.b_mn_major) ? 512u : 1024u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!ptx::mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, p.timeout_ns)) {
          report_status(p.status, kStatusGemmTimeout, 2, blockIdx.x, acc);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        int kb_lo, kb_hi;
        kb_range(t, kb_lo, kb_hi);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase, abort_flag, p.timeout_ns)) {
            report_status(p.status, kStatusGemmTimeout, 3, blockIdx.x, stage);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(smem + stage * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t adesc = ptx::make_smem_desc_sw128(sa + k * a_kstep, a_lbo, a_sbo, a_layout);
            const uint64_t bdesc = ptx::make_smem_desc_sw128(sb + k * b_kstep, b_lbo, b_sbo, b_layout);
            if constexpr (kTf32)
              ptx::umma_tf32(d_tmem, adesc, bdesc, idesc, ((kb - kb_lo) | k) != 0 ? 1u : 0u);
            else
              ptx::umma_f16(d_tmem, adesc, bdesc, idesc, ((kb - kb_lo) | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&empty_bar[stage]);  // frees the smem slot when the MMAs retire
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        ptx::umma_commit(&tmem_full[acc]);  // accumulator complete -> epilogue
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int esz = p.out_bf16 ? 2 : 4;
    const bool vec_ok = ((p.ldc * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        (!(kBatched || kConv) || ((p.sc_outer * esz) % 16 == 0 && (p.sc_inner * esz) % 16 == 0));
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int m_blk, n_blk;
      const int slice = (kBatched || conv_red) ? t / tiles_per_slice : 0;
      tile_coords((kBatched || conv_red) ? t - slice * tiles_per_slice : t, num_m, num_n, m_blk, n_blk);
      int row = m_blk * kBM + quarter * 32 + lane;
      if (conv_rows) {  // accumulator row -> output pixel of the patch (rows outside the image are dropped)
        int cb, cy0, cx0;
        conv_patch(p, m_blk, cb, cy0, cx0);
        const int ml = quarter * 32 + lane;
        const int oy = cy0 + ml / p.cv_tw, ox = cx0 + ml % p.cv_tw;
        row = (oy < p.cv_Ho && ox < p.cv_Wo) ? (cb * p.cv_Ho + oy) * p.cv_Wo + ox : p.M;
      }
      const int n0 = n_blk * BN;
      const long long slice_off =
          kBatched ? (slice / p.batch_inner) * p.sc_outer + (slice % p.batch_inner) * p.sc_inner
                   : (conv_red ? (slice / p.cv_taps) * p.sc_outer + (slice % p.cv_taps) * p.sc_inner : 0);
      // The vote keeps the warp converged for the .sync.aligned TMEM loads below.
      const bool ready = ptx::mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.timeout_ns);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) report_status(p.status, kStatusGemmTimeout, 4, blockIdx.x, acc);
        break;
      }
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int j = 0; j < BN / 32; ++j) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(taddr + j * 32, r);
        ptx::tmem_wait_ld();
        const int col0 = n0 + j * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if constexpr (kBatched) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= p.alpha;
          }
          if (p.bias != nullptr) {
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
          const bool full = (col0 + 32 <= p.N) && vec_ok;
          if (p.out2 != nullptr) {
            // value and derivative of the activation, both stored as bf16
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + slice_off + static_cast<long long>(row) * p.ldc + col0;
            __nv_bfloat16* o2 = reinterpret_cast<__nv_bfloat16*>(p.out2) + slice_off + static_cast<long long>(row) * p.ldc + col0;
            float dv[32];
            act_both_chunk(v, dv, p.act);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t wv[4], wd[4];
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                __nv_bfloat162 pa = __floats2bfloat162_rn(v[q * 8 + h * 2], v[q * 8 + h * 2 + 1]);
                __nv_bfloat162 pd = __floats2bfloat162_rn(dv[q * 8 + h * 2], dv[q * 8 + h * 2 + 1]);
                wv[h] = *reinterpret_cast<uint32_t*>(&pa);
                wd[h] = *reinterpret_cast<uint32_t*>(&pd);
              }
              if (full) {
                reinterpret_cast<uint4*>(o)[q] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                reinterpret_cast<uint4*>(o2)[q] = make_uint4(wd[0], wd[1], wd[2], wd[3]);
              } else {
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                  const int c = q * 8 + h * 2;
                  const __nv_bfloat162 pa = *reinterpret_cast<__nv_bfloat162*>(&wv[h]);
                  const __nv_bfloat162 pd = *reinterpret_cast<__nv_bfloat162*>(&wd[h]);
                  if (col0 + c < p.N) { o[c] = pa.x; o2[c] = pd.x; }
                  if (col0 + c + 1 < p.N) { o[c + 1] = pa.y; o2[c + 1] = pd.y; }
                }
              }
            }
          } else {
          if (p.act != FB_ACT_NONE) act_chunk(v, p.act);
          if (p.out_bf16) {
            __nv_bfloat16* o =
                reinterpret_cast<__nv_bfloat16*>(p.out) + slice_off + static_cast<long long>(row) * p.ldc + col0;
            if (full) {
              uint4* o4 = reinterpret_cast<uint4*>(o);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint32_t w[4];
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                  __nv_bfloat162 b2 = __floats2bfloat162_rn(v[q * 8 + h * 2], v[q * 8 + h * 2 + 1]);
                  w[h] = *reinterpret_cast<uint32_t*>(&b2);
                }
                o4[q] = make_uint4(w[0], w[1], w[2], w[3]);
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) o[i] = __float2bfloat16_rn(v[i]);
            }
          } else {
            float* o = reinterpret_cast<float*>(p.out) + slice_off + static_cast<long long>(row) * p.ldc + col0;
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
          }  // out2 == nullptr
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  // The driver's encoder wants a current context; a thread that has made no runtime call yet (an autograd
  // worker entering its first backward) has none, and the encoder then fails with CUDA_ERROR_INVALID_CONTEXT.
  static thread_local bool bound = false;
  if (!bound) {  // cudaSetDevice binds the primary context to the thread and is legal during stream capture
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
    bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D tensor map of bf16 (elem_bytes 2) or fp32 (4) data: `inner` contiguous elements per row, `outer` rows,
// row pitch `ld` elements, box = one 128-byte row segment x box_outer, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* ptr, long long inner, long long outer, long long ld, int box_outer,
              int elem_bytes = 2, bool atom32 = false) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ld * elem_bytes) % 16 != 0) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kRowBytes / elem_bytes), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 4-D form of the same map for batched operands: dims {inner, outer, batch_inner, batch_outer} with the two slice
// strides in elements; box = 64 x box_outer x 1 x 1, so a tile never crosses a slice and rows past the slice's
// extent read zeros.
bool make_map_batched(CUtensorMap* map, const void* ptr, long long inner, long long outer, long long ld,
                      int box_outer, int batch_inner, int batch_outer, long long s_inner, long long s_outer) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ld * 2) % 16 != 0) return false;
  if (batch_inner > 1 && (s_inner <= 0 || (s_inner * 2) % 16 != 0)) return false;
  if (batch_outer > 1 && (s_outer <= 0 || (s_outer * 2) % 16 != 0)) return false;
  // A dimension of extent 1 still needs a legal (non-zero, 16-byte multiple) stride.
  const long long si = batch_inner > 1 ? s_inner : ld * outer + ((8 - (ld * outer) % 8) % 8);
  const long long so = batch_outer > 1 ? s_outer : si * batch_inner;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer),
                        static_cast<cuuint64_t>(batch_inner), static_cast<cuuint64_t>(batch_outer)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(si) * 2,
                           static_cast<cuuint64_t>(so) * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_outer), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN, bool kBatched, bool kTf32 = false, bool kConv = false>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& args, int max_ctas, cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, kBatched, kTf32, kConv>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  long long tiles = static_cast<long long>((args.M + kBM - 1) / kBM) * ((args.N + BN - 1) / BN) *
                    (kBatched ? args.batch_total : 1);
  if (kConv) {
    const long long num_n = (args.N + BN - 1) / BN;
    tiles = args.cv_wgrad ? static_cast<long long>((args.M + kBM - 1) / kBM) * num_n * args.cv_taps * args.cv_splits
                          : static_cast<long long>(args.cv_nb) * args.cv_tiles_h * args.cv_tiles_w * num_n;
  }
  if (tiles > 0x7fffffffll) return -1;
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = static_cast<int>(tiles);
  gemm_bf16_kernel<BN, kBatched, kTf32, kConv><<<grid, kThreads, C::kSmemBytes, stream>>>(ma, mb, args);
  return static_cast<int>(cudaGetLastError());
}

// 4-D map of an NHWC bf16 tensor [images, height, width, channels] (channels a multiple of 8): dims {channel, x, y,
// image}, box = 64 channels x (bw x bh) pixels of one image, 128-byte swizzle; pixels and channels outside the
// tensor read zeros, which is how a convolution's padding is applied.
bool make_map_nhwc(CUtensorMap* map, const void* ptr, int images, int height, int width, int channels, int bw,
                   int bh) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || channels % 8 != 0 || bw < 1 || bh < 1 || bw > 256 || bh > 256)
    return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(channels), static_cast<cuuint64_t>(width),
                        static_cast<cuuint64_t>(height), static_cast<cuuint64_t>(images)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(channels) * 2, static_cast<cuuint64_t>(width) * channels * 2,
                           static_cast<cuuint64_t>(height) * width * channels * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(bw), static_cast<cuuint32_t>(bh), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Patch of `pixels` (a power of two) output pixels, bw x bh, that wastes the fewest positions on a wo x ho image.
void pick_patch(int pixels, int wo, int ho, int& bw, int& bh) {
  long long best = -1;
  for (int w = 1; w <= pixels; w <<= 1) {
    const int h = pixels / w;
    if (w > 256 || h > 256) continue;
    const long long cost = static_cast<long long>((wo + w - 1) / w) * w * ((ho + h - 1) / h) * h;
    // ties: the wider patch (longer contiguous runs of pixels in memory)
    if (best < 0 || cost < best || (cost == best && w > bw)) {
      best = cost;
      bw = w;
      bh = h;
    }
  }
}

void default_args(GemmArgs& args) {
  args.out2 = nullptr;
  args.bias = nullptr;
  args.act = FB_ACT_NONE;
  args.beta = 0;
  args.timeout_ns = 2000000000ull;
  args.batch_inner = 1;
  args.batch_total = 1;
  args.sc_outer = args.sc_inner = 0;
  args.alpha = 1.f;
  args.cv_wgrad = 0;
  args.cv_splits = 1;
}

}  // namespace
}  // namespace fb

extern "C" int fb_gemm_bf16_supported(const void* a, const void* b, long long lda, long long ldb) {
  return ((reinterpret_cast<uintptr_t>(a) & 15) == 0) && ((reinterpret_cast<uintptr_t>(b) & 15) == 0) &&
         ((lda * 2) % 16 == 0) && ((ldb * 2) % 16 == 0);
}

extern "C" int fb_gemm_bf16(const void* a, const void* b, void* out, void* out2, const float* bias, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major,
                            int out_bf16, int act, int beta, int max_ctas, int32_t* status, cudaStream_t stream) {
  using namespace fb;
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if (out2 != nullptr && (!out_bf16 || beta)) return -1;
  const bool small_n = N <= 128;
  const int bn = small_n ? 128 : 256;
  CUtensorMap ma, mb;
  bool ok;
  if (a_mn_major)
    ok = make_map(&ma, a, M, K, lda, 64);
  else
    ok = make_map(&ma, a, K, M, lda, kBM);
  if (!ok) return -2;
  if (b_mn_major)
    ok = make_map(&mb, b, N, K, ldb, 64);
  else
    ok = make_map(&mb, b, K, N, ldb, bn);
  if (!ok) return -2;
  GemmArgs args;
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
  args.status = status;
  args.timeout_ns = 2000000000ull;
  args.batch_inner = 1;
  args.batch_total = 1;
  args.sc_outer = args.sc_inner = 0;
  args.alpha = 1.f;
  return small_n ? launch<128, false>(ma, mb, args, max_ctas, stream)
                 : launch<256, false>(ma, mb, args, max_ctas, stream);
}

// Batched product over batch_outer x batch_inner slices:  D[s] = alpha * A[s] * B[s]^T  (optionally += D[s]).
// Every operand has its own pair of slice strides (elements), so [B, S, H, D] activations are used in place
// (slice (b, h) at b * S*H*D + h * D with row pitch H*D) as well as plain [batch, rows, cols] arrays.
extern "C" int fb_gemm_bf16_batched(const void* a, const void* b, void* out, int M, int N, int K, long long lda,
                                    long long ldb, long long ldc, int batch_outer, int batch_inner,
                                    long long sa_outer, long long sa_inner, long long sb_outer, long long sb_inner,
                                    long long sc_outer, long long sc_inner, int a_mn_major, int b_mn_major,
                                    int out_bf16, int beta, float alpha, int32_t* status, cudaStream_t stream) {
  using namespace fb;
  if (M <= 0 || N <= 0 || K <= 0 || batch_outer <= 0 || batch_inner <= 0) return -1;
  const bool small_n = N <= 128;
  const int bn = small_n ? 128 : 256;
  CUtensorMap ma, mb;
  bool ok;
  if (a_mn_major)
    ok = make_map_batched(&ma, a, M, K, lda, 64, batch_inner, batch_outer, sa_inner, sa_outer);
  else
    ok = make_map_batched(&ma, a, K, M, lda, kBM, batch_inner, batch_outer, sa_inner, sa_outer);
  if (!ok) return -2;
  if (b_mn_major)
    ok = make_map_batched(&mb, b, N, K, ldb, 64, batch_inner, batch_outer, sb_inner, sb_outer);
  else
    ok = make_map_batched(&mb, b, K, N, ldb, bn, batch_inner, batch_outer, sb_inner, sb_outer);
  if (!ok) return -2;
  GemmArgs args;
  args.out = out;
  args.out2 = nullptr;
  args.bias = nullptr;
  args.M = M;
  args.N = N;
  args.K = K;
  args.ldc = ldc;
  args.a_mn_major = a_mn_major;
  args.b_mn_major = b_mn_major;
  args.out_bf16 = out_bf16;
  args.act = FB_ACT_NONE;
  args.beta = beta;
  args.status = status;
  args.timeout_ns = 2000000000ull;
  args.batch_inner = batch_inner;
  args.batch_total = batch_inner * batch_outer;
  args.sc_outer = sc_outer;
  args.sc_inner = sc_inner;
  args.alpha = alpha;
  return small_n ? launch<128, true>(ma, mb, args, 0, stream) : launch<256, true>(ma, mb, args, 0, stream);
}

// fp32 operands multiplied on the tensor cores as TF32 (tcgen05.mma kind::tf32: 10-bit mantissa inputs, fp32
// accumulate) with an fp32 result: out[M,N] = act(A * B^T + bias) (+= out when beta).  Same operand layouts as
// fb_gemm_bf16 (K-major or MN-major per operand); lda / ldb in elements, multiples of 4.
extern "C" int fb_gemm_tf32(const float* a, const float* b, float* out, const float* bias, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major, int act,
                            int beta, int max_ctas, int32_t* status, cudaStream_t stream) {
  using namespace fb;
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  const bool small_n = N <= 128;
  const int bn = small_n ? 128 : 256;
  constexpr int kChunk = El<true>::kMnChunk;
  CUtensorMap ma, mb;
  // MN-major fp32 tiles are written with the 32-byte-chunk swizzle the tensor core requires for them
  bool ok = a_mn_major ? make_map(&ma, a, M, K, lda, kChunk, 4, true) : make_map(&ma, a, K, M, lda, kBM, 4);
  if (!ok) return -2;
  ok = b_mn_major ? make_map(&mb, b, N, K, ldb, kChunk, 4, true) : make_map(&mb, b, K, N, ldb, bn, 4);
  if (!ok) return -2;
  GemmArgs args;
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
  args.status = status;
  args.timeout_ns = 2000000000ull;
  args.batch_inner = 1;
  args.batch_total = 1;
  args.sc_outer = args.sc_inner = 0;
  args.alpha = 1.f;
  return small_n ? launch<128, false, true>(ma, mb, args, max_ctas, stream)
                 : launch<256, false, true>(ma, mb, args, max_ctas, stream);
}

// Stride-1 convolution as an implicit GEMM on the tensor cores (no window matrix in memory):
//   y[b, oy, ox, o] = bias[o] + sum over (ky, kx, c) of x[b, oy - ph + ky * dh, ox - pw + kx * dw, c] * w[o, ky, kx, c]
// x: NHWC bf16 [B, H, W, Cp]; w: bf16 [O, kh * kw * Cp] (tap-major, channel innermost); Cp a multiple of 8 (pad the
// channels with zeros).  y: NHWC [B, Ho, Wo, ldy] (fp32, or bf16 with out_bf16), Ho = H + 2 ph - dh (kh - 1), Wo alike.
// The data gradient of a stride-1 convolution is the same call with the flipped, transposed filters and padding
// dh (kh - 1) - ph.  Returns -2 when an operand cannot be described by a TMA map.
extern "C" int fb_conv_igemm(const void* x, const void* w, void* y, const float* bias, int B, int H, int W, int Cp,
                             int O, int kh, int kw, int ph, int pw, int dh, int dw, long long ldy, int out_bf16,
                             int32_t* status, cudaStream_t stream) {
  using namespace fb;
  const int Ho = H + 2 * ph - dh * (kh - 1), Wo = W + 2 * pw - dw * (kw - 1);
  if (B <= 0 || H <= 0 || W <= 0 || Cp <= 0 || (Cp & 7) || O <= 0 || kh <= 0 || kw <= 0 || Ho <= 0 || Wo <= 0 ||
      dh <= 0 || dw <= 0 || ldy < O)
    return -1;
  if (static_cast<long long>(B) * Ho * Wo > 0x7fffffffll) return -1;
  GemmArgs args;
  default_args(args);
  pick_patch(128, Wo, Ho, args.cv_tw, args.cv_th);
  const bool small_n = O <= 128;
  CUtensorMap ma, mb;
  if (!make_map_nhwc(&ma, x, B, H, W, Cp, args.cv_tw, args.cv_th)) return -2;
  const long long K = static_cast<long long>(kh) * kw * Cp;
  if (!make_map(&mb, w, K, O, K, small_n ? 128 : 256)) return -2;
  args.out = y;
  args.bias = bias;
  args.M = B * Ho * Wo;
  args.N = O;
  args.K = static_cast<int>(K);
  args.ldc = ldy;
  args.a_mn_major = 0;
  args.b_mn_major = 0;
  args.out_bf16 = out_bf16;
  args.status = status;
  args.cv_tiles_w = (Wo + args.cv_tw - 1) / args.cv_tw;
  args.cv_tiles_h = (Ho + args.cv_th - 1) / args.cv_th;
  args.cv_nb = B;
  args.cv_Ho = Ho;
  args.cv_Wo = Wo;
  args.cv_kw = kw;
  args.cv_taps = kh * kw;
  args.cv_cchunks = (Cp + 63) / 64;
  args.cv_cp = Cp;
  args.cv_ph = ph;
  args.cv_pw = pw;
  args.cv_dh = dh;
  args.cv_dw = dw;
  args.cv_kb_per_split = args.cv_total_kb = 0;
  return small_n ? launch<128, false, false, true>(ma, mb, args, 0, stream)
                 : launch<256, false, false, true>(ma, mb, args, 0, stream);
}

// Number of partial results fb_conv_wgrad writes for this problem (the caller sums them; 1 = final result).
extern "C" int fb_conv_wgrad_splits(int B, int Ho, int Wo, int O, int Cp, int taps) {
  using namespace fb;
  if (B <= 0 || Ho <= 0 || Wo <= 0 || O <= 0 || Cp <= 0 || taps <= 0) return 0;
  int bw = 1, bh = 1;
  pick_patch(64, Wo, Ho, bw, bh);
  const long long total_kb = static_cast<long long>(B) * ((Wo + bw - 1) / bw) * ((Ho + bh - 1) / bh);
  const long long tiles = static_cast<long long>((O + kBM - 1) / kBM) * ((Cp + (Cp <= 128 ? 127 : 255)) / (Cp <= 128 ? 128 : 256)) * taps;
  long long splits = (2ll * sm_count() + tiles - 1) / tiles;
  if (splits > 64) splits = 64;
  if (splits > total_kb) splits = total_kb;
  if (splits < 1) splits = 1;
  const long long per = (total_kb + splits - 1) / splits;
  return static_cast<int>((total_kb + per - 1) / per);
}

// Weight gradient of the convolution above:
//   dw[s][o, (ky, kx), c] = sum over the output pixels of split s of dy[b, oy, ox, o] * x[b, oy - ph + ky * dh, ox - pw + kx * dw, c]
// dy: NHWC bf16 [B, Ho, Wo, Op] (Op >= O, a multiple of 8), x: NHWC bf16 [B, H, W, Cp]; out: fp32
// [fb_conv_wgrad_splits(...)][O][kh * kw * Cp]; the caller adds the splits.
extern "C" int fb_conv_wgrad(const void* dy, const void* x, float* out, int B, int H, int W, int Cp, int O, int Op,
                             int kh, int kw, int ph, int pw, int dh, int dw, int32_t* status, cudaStream_t stream) {
  using namespace fb;
  const int Ho = H + 2 * ph - dh * (kh - 1), Wo = W + 2 * pw - dw * (kw - 1);
  if (B <= 0 || H <= 0 || W <= 0 || Cp <= 0 || (Cp & 7) || O <= 0 || Op < O || (Op & 7) || kh <= 0 || kw <= 0 ||
      Ho <= 0 || Wo <= 0 || dh <= 0 || dw <= 0)
    return -1;
  GemmArgs args;
  default_args(args);
  pick_patch(64, Wo, Ho, args.cv_tw, args.cv_th);
  CUtensorMap ma, mb;
  if (!make_map_nhwc(&ma, dy, B, Ho, Wo, Op, args.cv_tw, args.cv_th)) return -2;
  if (!make_map_nhwc(&mb, x, B, H, W, Cp, args.cv_tw, args.cv_th)) return -2;
  const int taps = kh * kw;
  const bool small_n = Cp <= 128;
  args.out = out;
  args.M = O;
  args.N = Cp;
  args.K = 64;  // not used: the reduction is the list of pixel patches
  args.ldc = static_cast<long long>(taps) * Cp;
  args.a_mn_major = 1;
  args.b_mn_major = 1;
  args.out_bf16 = 0;
  args.status = status;
  args.cv_wgrad = 1;
  args.cv_tiles_w = (Wo + args.cv_tw - 1) / args.cv_tw;
  args.cv_tiles_h = (Ho + args.cv_th - 1) / args.cv_th;
  args.cv_nb = B;
  args.cv_Ho = Ho;
  args.cv_Wo = Wo;
  args.cv_kw = kw;
  args.cv_taps = taps;
  args.cv_cchunks = (Cp + 63) / 64;
  args.cv_cp = Cp;
  args.cv_ph = ph;
  args.cv_pw = pw;
  args.cv_dh = dh;
  args.cv_dw = dw;
  const long long total_kb = static_cast<long long>(B) * args.cv_tiles_w * args.cv_tiles_h;
  if (total_kb > 0x7fffffffll) return -1;
  const int splits = fb_conv_wgrad_splits(B, Ho, Wo, O, Cp, taps);
  args.cv_total_kb = static_cast<int>(total_kb);
  args.cv_kb_per_split = static_cast<int>((total_kb + splits - 1) / splits);
  args.cv_splits = splits;
  args.sc_outer = static_cast<long long>(O) * args.ldc;
  args.sc_inner = Cp;
  return small_n ? launch<128, false, false, true>(ma, mb, args, 0, stream)
                 : launch<256, false, false, true>(ma, mb, args, 0, stream);
}
