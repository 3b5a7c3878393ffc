// Blockwise (flash-style) attention forward on the tcgen05 tensor cores, head dimension 64 or 128, bf16.
//
// The reference materialises the [S, S] score matrix per head on the host (ferrum-nn/src/transformer.rs:127-220).
// This kernel never writes scores to memory: one CTA owns 128 query rows of one (batch, head) and walks the keys /
// values in tiles of 128:
//
//   warp 0      TMA producer: Q once, then K_j into a two-stage shared-memory ring and V_j into a single buffer
//               (128-byte swizzle; a 128-wide head is two 64-column blocks per tile).  Head dimension 64: 97 KB of
//               shared memory and 256 tensor-memory columns, so two CTAs share an SM and one CTA's softmax runs
//               while the other's MMAs and loads are in flight; head dimension 128: 161 KB, one CTA per SM
//   warp 1      one thread issues the MMAs: S = Q K_j^T (128 x 128 x 64) into tensor memory, later
//               O_j = P_j V_j (128 x 64 x 128) into a second tensor-memory region
//   warps 2-5   softmax: thread = query row.  Reads its row of S from tensor memory (tcgen05.ld), keeps the running
//               maximum and sum (online softmax, base-2 exponentials), writes P_j as bf16 into shared memory in the
//               swizzled K-major layout the tensor core reads, rescales its 64 output accumulators kept in
//               registers and adds O_j when the second MMA has finished.
//
// Every mbarrier wait is bounded (status block + abort flag shared by the CTA's roles); nothing traps.
// Output: [B, S, H, 64] contiguous bf16 (so the output projection sees [B, S, H*64]) and, optionally, the
// log-sum-exp of every row (natural log) for a recomputing backward.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../common/ptx.cuh"
#include "../common/status.h"
#include "../include/ferrum_kernels.h"

namespace fb {
namespace {

constexpr int kBQ = 128;          // query rows per CTA
constexpr int kBKV = 128;         // keys per tile
constexpr int kBlk = 128 * 128;   // 16 KB: 128 rows of 64 bf16 = one 128-byte-swizzled block
constexpr int kAttnThreads = 192;
constexpr int kTmemColsAttn = 256;  // S: columns 0..127, O_j: columns 128..(128 + D - 1)
// D = head dimension (64 or 128): an operand tile is D / 64 blocks side by side in the reduction (Q, K) or output (V)
// dimension; P is always 128 x 128 = two blocks.
template <int D>
struct AttnCfg {
  static constexpr int kNB = D / 64;
  static constexpr int kTile = kNB * kBlk;
  static constexpr int kSmem = kTile * (1 + 2 + 1) + 2 * kBlk + 1024 + 256;  // Q, K x2, V, P
  static constexpr int kCtasPerSm = D == 64 ? 2 : 1;
};

struct AttnArgs {
  __nv_bfloat16* out;   // [B, Sq, H, D]
  float* lse;           // [B, H, Sq] or NULL
  int B, H, Sq, Skv;
  float scale_log2;     // softmax scale * log2(e)
  int causal;           // 1: query i attends keys j <= i + (Skv - Sq) (needs Skv >= Sq)
  int32_t* status;
  unsigned long long timeout_ns;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads, AttnCfg<D>::kCtasPerSm)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const AttnArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kNB = AttnCfg<D>::kNB, kTileBytes = AttnCfg<D>::kTile;
  uint8_t* sq = smem;
  uint8_t* sk = sq + kTileBytes;            // two stages
  uint8_t* sv = sk + 2 * kTileBytes;        // one buffer
  uint8_t* sp = sv + kTileBytes;            // P: two k-blocks of 128 rows x 128 bytes
  uint8_t* bar_base = sp + 2 * kBlk;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* k_full = q_full + 1;    // [2]
  uint64_t* k_empty = k_full + 2;   // [2]
  uint64_t* v_full = k_empty + 2;
  uint64_t* v_empty = v_full + 1;
  uint64_t* s_full = v_empty + 1;
  uint64_t* p_full = s_full + 1;
  uint64_t* o_full = p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * kBQ;
  const int h = blockIdx.y % p.H, b = blockIdx.y / p.H;
  // causal: this tile's last query row bounds the keys any of its rows may see
  const int kv_end = p.causal ? min(p.Skv, q0 + kBQ + (p.Skv - p.Sq)) : p.Skv;
  const int n_tiles = (kv_end + kBKV - 1) / kBKV;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&k_full[s], 1);
      ptx::mbar_init(&k_empty[s], 1);
    }
    ptx::mbar_init(v_full, 1);
    ptx::mbar_init(v_empty, 1);
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(p_full, 4);  // one arrival per softmax warp
    ptx::mbar_init(o_full, 1);
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemColsAttn);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      ptx::mbar_arrive_expect_tx(q_full, kTileBytes);
#pragma unroll
      for (int nb = 0; nb < kNB; ++nb) ptx::tma_load_4d(sq + nb * kBlk, &map_q, q_full, nb * 64, q0, h, b);
      uint32_t phase = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        if (!ptx::mbar_wait(&k_empty[st], phase ^ 1u, abort_flag, p.timeout_ns)) {  // S_(j-2) has read the slot
          report_status(p.status, kStatusGemmTimeout, 51, blockIdx.x, j);
          break;
        }
        ptx::mbar_arrive_expect_tx(&k_full[st], kTileBytes);
#pragma unroll
        for (int nb = 0; nb < kNB; ++nb)
          ptx::tma_load_4d(sk + st * kTileBytes + nb * kBlk, &map_k, &k_full[st], nb * 64, j * kBKV, h, b);
        if (!ptx::mbar_wait(v_empty, (j & 1) ^ 1u, abort_flag, p.timeout_ns)) {        // P_(j-1) V_(j-1) is done
          report_status(p.status, kStatusGemmTimeout, 57, blockIdx.x, j);
          break;
        }
        ptx::mbar_arrive_expect_tx(v_full, kTileBytes);
#pragma unroll
        for (int nb = 0; nb < kNB; ++nb) ptx::tma_load_4d(sv + nb * kBlk, &map_v, v_full, nb * 64, j * kBKV, h, b);
        if (st == 1) phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = ptx::make_idesc(1u, kBQ, kBKV, 0, 0);   // Q, K both K-major
      const uint32_t idesc_o = ptx::make_idesc(1u, kBQ, D, 0, 1);      // P K-major, V with d contiguous (MN-major)
      const uint32_t t_s = tmem_base, t_o = tmem_base + 128;
      const uint32_t sq_a = ptx::smem_u32(sq), sp_a = ptx::smem_u32(sp);
      auto issue_s = [&](int st) {
        const uint32_t sk_a = ptx::smem_u32(sk + st * kTileBytes);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          ptx::umma_f16(t_s, ptx::make_smem_desc_sw128(sq_a + (k >> 2) * kBlk + (k & 3) * 32, 16, 1024),
                        ptx::make_smem_desc_sw128(sk_a + (k >> 2) * kBlk + (k & 3) * 32, 16, 1024), idesc_s,
                        k != 0 ? 1u : 0u);
        ptx::umma_commit(s_full);
        ptx::umma_commit(&k_empty[st]);  // the K slot is free once these MMAs have read it
      };
      bool ok = ptx::mbar_wait(q_full, 0, abort_flag, p.timeout_ns) &&
                ptx::mbar_wait(&k_full[0], 0, abort_flag, p.timeout_ns);
      if (!ok) report_status(p.status, kStatusGemmTimeout, 52, blockIdx.x, 0);
      if (ok) {
        ptx::tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (!ptx::mbar_wait(p_full, j & 1, abort_flag, p.timeout_ns) ||
            !ptx::mbar_wait(v_full, j & 1, abort_flag, p.timeout_ns)) {
          report_status(p.status, kStatusGemmTimeout, 53, blockIdx.x, j);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t sv_a = ptx::smem_u32(sv);
#pragma unroll
        for (int k = 0; k < kBKV / 16; ++k)
          // V: 16 keys (rows of 128 bytes) per MMA; its 64-column blocks lie kBlk apart (the leading-dimension offset)
          ptx::umma_f16(t_o, ptx::make_smem_desc_sw128(sp_a + (k >> 2) * kBlk + (k & 3) * 32, 16, 1024),
                        ptx::make_smem_desc_sw128(sv_a + k * 2048, kBlk, 1024), idesc_o, k != 0 ? 1u : 0u);
        ptx::umma_commit(o_full);
        ptx::umma_commit(v_empty);
        if (j + 1 < n_tiles) {
          const int sn = (j + 1) & 1;
          if (!ptx::mbar_wait(&k_full[sn], ((j + 1) >> 1) & 1, abort_flag, p.timeout_ns)) {
            report_status(p.status, kStatusGemmTimeout, 54, blockIdx.x, j);
            break;
          }
          ptx::tc_fence_after();
          issue_s(sn);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output (thread = query row)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float m = -INFINITY, l = 0.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const bool ready = ptx::mbar_wait(s_full, j & 1, abort_flag, p.timeout_ns);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) report_status(p.status, kStatusGemmTimeout, 55, blockIdx.x, j);
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      int valid = min(kBKV, p.Skv - j * kBKV);  // columns past it are padding
      if (p.causal) valid = max(0, min(valid, q0 + row + (p.Skv - p.Sq) + 1 - j * kBKV));  // this row's keys only
      // (0 is possible from the second tile on — all of the row's keys lie in earlier tiles — and harmless: the
      // running maximum is finite by then, so alpha = 1 and every p = 0; the first tile always holds key 0)
      const bool full_tile = valid == kBKV;
      // pass 1: row maximum of the raw scores (the scale is positive, applied once afterwards)
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(t_row + c * 32, r);
        ptx::tmem_wait_ld();
        if (full_tile) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < valid) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float alpha = ex2(m - m_new);  // 0 for the first tile (m = -inf)
      l *= alpha;
#pragma unroll
      for (int i = 0; i < D; ++i) o[i] *= alpha;
      // pass 2: p = 2^(s * scale - m_new), row sum, bf16 P into shared memory (K-major, 128-byte swizzle)
      const float neg_m = -m_new;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(t_row + c * 32, r);
        ptx::tmem_wait_ld();
        uint32_t packed[16];
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2(fmaf(__uint_as_float(r[i]), p.scale_log2, neg_m));
          float p1 = ex2(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, neg_m));
          if (!full_tile) {
            if (c * 32 + i >= valid) p0 = 0.f;
            if (c * 32 + i + 1 >= valid) p1 = 0.f;
          }
          part += p0 + p1;
          const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
        }
        l += part;
        // 32 columns = four 16-byte chunks; chunk index inside the 64-column k-block: (c & 1) * 4 + q
        uint8_t* blk = sp + (c >> 1) * kBlk + row * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = (c & 1) * 4 + q;
          *reinterpret_cast<uint4*>(blk + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
        }
      }
      m = m_new;
      ptx::tc_fence_before();          // the reads of S are ordered before the MMA that overwrites it
      ptx::fence_proxy_async_smem();   // P becomes visible to the tensor core's (async-proxy) reads
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(p_full);
      // O_j = P_j V_j
      const bool done = ptx::mbar_wait(o_full, j & 1, abort_flag, p.timeout_ns);
      if (!__all_sync(0xffffffffu, done)) {
        if (lane == 0) report_status(p.status, kStatusGemmTimeout, 56, blockIdx.x, j);
        ok = false;
        break;
      }
      ptx::tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(t_row + 128 + c * 32, r);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(r[i]);
      }
      ptx::tc_fence_before();
    }
    const int qrow = q0 + row;
    if (ok && qrow < p.Sq) {
      const float inv = 1.f / l;
      __nv_bfloat16* dst = p.out + ((static_cast<long long>(b) * p.Sq + qrow) * p.H + h) * D;
#pragma unroll
      for (int q = 0; q < D / 8; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __nv_bfloat162 pk = __floats2bfloat162_rn(o[q * 8 + e * 2] * inv, o[q * 8 + e * 2 + 1] * inv);
          w[e] = *reinterpret_cast<const uint32_t*>(&pk);
        }
        reinterpret_cast<uint4*>(dst)[q] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (p.lse != nullptr)
        p.lse[(static_cast<long long>(b) * p.H + h) * p.Sq + qrow] = (m + log2f(l)) * 0.6931471805599453f;
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemColsAttn);
  }
}

typedef CUresult (*EncodeTiledFnA)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFnA encode_fn_a() {
  // The driver's encoder wants a current context; a thread that has made no runtime call yet (an autograd
  // worker entering its first backward) has none, and the encoder then fails with CUDA_ERROR_INVALID_CONTEXT.
  static thread_local bool bound = false;
  if (!bound) {  // cudaSetDevice binds the primary context to the thread and is legal during stream capture
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
    bound = true;
  }
  static EncodeTiledFnA fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFnA>(sym);
  }
  return fn;
}

// [B, H, S, D] bf16 view with element strides (sb, sh, ss), last dimension contiguous: a 4-D map with a
// 64 x 128 x 1 x 1 box (one 64-column block of 128 rows); rows past S read zeros.
bool make_map_bhsd(CUtensorMap* map, const void* ptr, int B, int H, int S, int kD, long long sb, long long sh,
                   long long ss) {
  EncodeTiledFnA enc = encode_fn_a();
  if (enc == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || ss % 8 || ss < kD) return false;
  if ((H > 1 && (sh % 8 || sh <= 0)) || (B > 1 && (sb % 8 || sb <= 0))) return false;
  // a dimension of extent 1 still needs a legal stride
  const long long sh_ok = H > 1 ? sh : ss * S + ((8 - (ss * S) % 8) % 8);
  const long long sb_ok = B > 1 ? sb : sh_ok * H;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(kD), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ss) * 2, static_cast<cuuint64_t>(sh_ok) * 2,
                           static_cast<cuuint64_t>(sb_ok) * 2};
  cuuint32_t box[4] = {64, 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D>
int launch_attn(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& a,
                cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnCfg<D>::kSmem) !=
        cudaSuccess)
      return static_cast<int>(cudaGetLastError());
    attr_set = true;
  }
  const dim3 grid((a.Sq + kBQ - 1) / kBQ, a.B * a.H);
  attn_fwd_kernel<D><<<grid, kAttnThreads, AttnCfg<D>::kSmem, stream>>>(mq, mk, mv, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
}  // namespace fb

// out[b, s, h, :] = softmax(scale * q[b,h,s,:] . k[b,h,:,:]^T) v[b,h,:,:]  for head dimension D = 64 or 128, bf16
// operands given as [B, H, S, D] views with element strides (last dimension contiguous, strides multiples of 8).
// out is [B, Sq, H, D] contiguous; lse (optional) [B, H, Sq] fp32.  Returns -2 when an operand cannot be described
// by a TMA map.  causal: query i sees keys j <= i + (Skv - Sq); key tiles past the diagonal are skipped.
extern "C" int fb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H,
                                int Sq, int Skv, int D, long long q_sb, long long q_sh, long long q_ss,
                                long long k_sb, long long k_sh, long long k_ss, long long v_sb, long long v_sh,
                                long long v_ss, float scale, int causal, int32_t* status, cudaStream_t stream) {
  using namespace fb;
  if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0 || (causal && Skv < Sq) || (D != 64 && D != 128)) return -1;
  if (reinterpret_cast<uintptr_t>(out) & 15) return -1;
  CUtensorMap mq, mk, mv;
  if (!make_map_bhsd(&mq, q, B, H, Sq, D, q_sb, q_sh, q_ss) || !make_map_bhsd(&mk, k, B, H, Skv, D, k_sb, k_sh, k_ss) ||
      !make_map_bhsd(&mv, v, B, H, Skv, D, v_sb, v_sh, v_ss))
    return -2;
  AttnArgs a;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.B = B;
  a.H = H;
  a.Sq = Sq;
  a.Skv = Skv;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal ? 1 : 0;
  a.status = status;
  a.timeout_ns = 2000000000ull;
  return D == 64 ? launch_attn<64>(mq, mk, mv, a, stream) : launch_attn<128>(mq, mk, mv, a, stream);
}
