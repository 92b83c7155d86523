// Fused causal self-attention (flash-attention style) on tcgen05 tensor cores.
//
// Replaces the reference's attention chain -- QKV split, four transposes, a batched
// matmul that materialises the [B,H,T,T] scores, scale, mask, softmax, a second
// batched matmul and a transpose back (example/gpt2/net.cc:77-108; kernels
// split.cu, transform.cu, softmax.cu, linear.cu) -- with one forward and one
// backward kernel that keep the score tile in tensor memory:
//
//   forward, one CTA per (128 query rows, head, batch), loop over key blocks j <= i:
//     S = Q K_j^T          tcgen05.mma, A/B from TMA-loaded swizzled smem, D in TMEM
//     online softmax       128 threads, one score row each, read with tcgen05.ld
//     P -> smem (bf16)     written in the 128-byte-swizzle layout the MMA expects
//     O_blk = P V_j        tcgen05.mma with V as an MN-major operand (no transpose)
//     O = O * alpha + O_blk in registers; finally O / l and the log-sum-exp row.
//
//   backward, one CTA per (128 key rows, kv head, batch), loop over query blocks i >= j
//   and over the query heads that share the kv head (GQA):
//     S = Q_i K_j^T, dP = dO_i V_j^T            -> TMEM
//     P = exp(S - lse), dS = P (dP - delta)     -> smem (bf16), both stored once and read
//                                                  as K-major and as MN-major operands
//     dV += P^T dO_i, dK += dS^T Q_i            accumulate in TMEM over the whole loop
//     dQ_i += dS K_j                            TMEM -> fp32 vector reductions in HBM
//
// q/k/v are addressed in place inside a fused projection buffer through TMA tensor
// maps (row stride = token stride), so no split/transpose kernel runs.  All waits
// are bounded (ptx_sm100.cuh).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "api.h"
#include "ptx_sm100.cuh"

namespace titb {

bool make_tmap_bf16_2d(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                       uint32_t box_inner, uint32_t box_outer);
bool make_tmap_f32_2d(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

constexpr int kAttnThreads = 192;
constexpr int kBlk = 128;             // query rows per CTA tile and keys per step
constexpr int kChunkBytes = kBlk * 128;  // one [128 rows x 64 bf16] swizzled sub-tile
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 8 consecutive bf16 (one 16-byte unit) in a [128 x 128] tile stored as two
// [128 rows x 128 B] sub-tiles with the 128-byte swizzle: unit index u = col / 8 in 0..15.
__device__ __forceinline__ uint32_t swz_off(int row, int u) {
  return static_cast<uint32_t>((u >> 3) * kChunkBytes + row * 128 + (((u & 7) ^ (row & 7)) << 4));
}

// A shared-memory descriptor whose start address is moved by `bytes` (a multiple of 16 that stays inside the CTA's
// shared memory): only the 14-bit address field changes, so one add replaces rebuilding the descriptor.
__device__ __forceinline__ uint64_t desc_add(uint64_t desc, uint32_t bytes) { return desc + (bytes >> 4); }

struct AttnArgs {
  int B, T, Hq, Hkv, hd;
  float scale;
  bf16* o;
  float* lse;
  long long o_stride_t;
  // backward
  const float* delta;
  float* dq_accum;  // fp32 [B, T, Hq, hd]
  bf16* dk;
  bf16* dv;
  long long dk_stride_t, dv_stride_t;
  int* status;
};

// ------------------------------------------------------------------------- forward
template <int HD>
struct FwdCfg {
  static constexpr int kTileBytes = kBlk * HD * 2;  // Q, K or V tile
  static constexpr int kStages = 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;
  static constexpr int kV = kK + kStages * kTileBytes;
  static constexpr int kP = kV + kStages * kTileBytes;
  static constexpr int kBar = kP + kBlk * kBlk * 2;
  static constexpr int kSmem = kBar + 128;
  static constexpr int kTmemCols = 256;  // S: [0,128)  O_blk: [128, 128+HD)
};

// Forward pipeline.  Per key block j the CTA runs
//   MMA warp:      S(j+1) = Q K(j+1)^T is issued as soon as the softmax warps have copied S(j) out of tensor
//                  memory (s_free), i.e. it runs underneath the exponentials of block j; O += P(j) V(j) is issued
//                  when P(j) has been written (p_full) and accumulates in tensor memory over the whole loop.
//   softmax warps: one score row per thread, read from tensor memory ONCE (128 registers), row maximum, then the
//                  exponentials straight from registers.  The running maximum `m_ref` that the exponentials refer
//                  to is only advanced when a block's maximum exceeds it by more than 2^8 (P stays within bf16
//                  range, the row sum is fp32); only then is the O accumulator rescaled, in place in tensor
//                  memory, after the previous P V product has finished.  P(j) is stored to shared memory after
//                  P(j-1) V(j-1) has finished reading the buffer.
template <int HD>
__global__ void __launch_bounds__(kAttnThreads, (HD == 64) ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const AttnArgs p) {
  using Cfg = FwdCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBar);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]  a K tile is free as soon as its S product has finished ...
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]  ... a V tile only after its P V product: K runs a block further ahead
  uint64_t* s_full = bars + 9;
  uint64_t* p_full = bars + 10;
  uint64_t* o_full = bars + 11;
  uint64_t* s_free = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.T + kBlk - 1) / kBlk;
  const int qb = nqb - 1 - blockIdx.x;  // heaviest tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * kBlk;
  const int nblk = qb + 1;

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&k_full[s], 1); ptx::mbar_init(&k_empty[s], 1);
      ptx::mbar_init(&v_full[s], 1); ptx::mbar_init(&v_empty[s], 1);
    }
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(p_full, 4);
    ptx::mbar_init(o_full, 1);
    ptx::mbar_init(s_free, 4);
    *abort_flag = (ptx::smem_u32(smem) & 1023u) ? 1u : 0u;  // swizzled tiles need a 1024-byte aligned base
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tq);
    ptx::tma_prefetch_desc(&tk);
    ptx::tma_prefetch_desc(&tv);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + 128;
  const bool bad_align = (*abort_flag != 0);

  if (bad_align) {
    // fall through to the common exit
  } else if (warp == 0) {
    if (lane == 0) {
      ptx::mbar_expect_tx(q_full, Cfg::kTileBytes);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c)
        ptx::tma_load_2d(smem + Cfg::kQ + c * kChunkBytes, &tq, q_full, h * HD + c * 64, b * p.T + q0);
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1;
        if (!ptx::mbar_wait(&k_empty[st], ((j >> 1) & 1) ^ 1u, abort_flag)) break;
        ptx::mbar_expect_tx(&k_full[st], Cfg::kTileBytes);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          ptx::tma_load_2d(smem + Cfg::kK + st * Cfg::kTileBytes + c * kChunkBytes, &tk, &k_full[st],
                           hk * HD + c * 64, b * p.T + j * kBlk);
        if (!ptx::mbar_wait(&v_empty[st], ((j >> 1) & 1) ^ 1u, abort_flag)) break;
        ptx::mbar_expect_tx(&v_full[st], Cfg::kTileBytes);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          ptx::tma_load_2d(smem + Cfg::kV + st * Cfg::kTileBytes + c * kChunkBytes, &tv, &v_full[st],
                           hk * HD + c * 64, b * p.T + j * kBlk);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = ptx::make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = ptx::make_idesc_bf16(128, HD, 0, 1);
      const uint32_t q_base = ptx::smem_u32(smem + Cfg::kQ);
      const uint32_t p_base = ptx::smem_u32(smem + Cfg::kP);
      const uint64_t q_desc = ptx::make_smem_desc(q_base, 16, 1024);
      const uint64_t k_desc0 = ptx::make_smem_desc(ptx::smem_u32(smem + Cfg::kK), 16, 1024);
      const uint64_t p_desc = ptx::make_smem_desc(p_base, 16, 1024);
      const uint64_t v_desc0 = ptx::make_smem_desc(ptx::smem_u32(smem + Cfg::kV), kChunkBytes, 1024);
      auto issue_s = [&](int j) {
        const uint64_t k_desc = desc_add(k_desc0, (j & 1) * Cfg::kTileBytes);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * kChunkBytes + (k & 3) * 32;
          ptx::mma_f16_ss(tS, desc_add(q_desc, off), desc_add(k_desc, off), idesc_s, k > 0);
        }
        ptx::tc_commit(s_full);
        ptx::tc_commit(&k_empty[j & 1]);   // the K tile may be refilled once this product has finished
      };
      bool ok = ptx::mbar_wait(q_full, 0, abort_flag) && ptx::mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        ptx::tc_fence_after_sync();
        issue_s(0);
      }
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          // S(j+1) goes into the score columns as soon as S(j) has been copied to registers
          if (!ptx::mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag)) break;
          if (!ptx::mbar_wait(s_free, j & 1, abort_flag)) break;
          ptx::tc_fence_after_sync();
          issue_s(j + 1);
        }
        if (!ptx::mbar_wait(&v_full[j & 1], (j >> 1) & 1, abort_flag)) break;
        if (!ptx::mbar_wait(p_full, j & 1, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const uint64_t v_desc = desc_add(v_desc0, (j & 1) * Cfg::kTileBytes);
#pragma unroll
        for (int k = 0; k < kBlk / 16; ++k) {
          const uint32_t a_off = (k >> 2) * kChunkBytes + (k & 3) * 32;
          ptx::mma_f16_ss(tO, desc_add(p_desc, a_off), desc_add(v_desc, k * 2048), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        ptx::tc_commit(o_full);
        ptx::tc_commit(&v_empty[j & 1]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int q_idx = q0 + row;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const float sc = p.scale * kLog2e;
    constexpr float kLazy = 8.f;   // log2 of the largest P value tolerated before the reference maximum moves
    float m_ref = -INFINITY, l = 0.f;
    uint8_t* p_smem = smem + Cfg::kP;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      if (!ptx::mbar_wait(s_full, j & 1, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      uint32_t r0[32], r1[32], r2[32], r3[32];
      ptx::tmem_ld32(tS + lane_sel + 0, r0);
      ptx::tmem_ld32(tS + lane_sel + 32, r1);
      ptx::tmem_ld32(tS + lane_sel + 64, r2);
      ptx::tmem_ld32(tS + lane_sel + 96, r3);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(s_free);   // the score columns may be overwritten by S(j+1)
      const int kv0 = j * kBlk;
      if (j == qb) {  // diagonal block: keys after the query are masked
        const uint32_t ninf = __float_as_uint(-INFINITY);
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          if (kv0 + e > q_idx) r0[e] = ninf;
          if (kv0 + 32 + e > q_idx) r1[e] = ninf;
          if (kv0 + 64 + e > q_idx) r2[e] = ninf;
          if (kv0 + 96 + e > q_idx) r3[e] = ninf;
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        mx0 = fmaxf(mx0, __uint_as_float(r0[e]));
        mx1 = fmaxf(mx1, __uint_as_float(r1[e]));
        mx2 = fmaxf(mx2, __uint_as_float(r2[e]));
        mx3 = fmaxf(mx3, __uint_as_float(r3[e]));
      }
      const float m_blk = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sc;
      bool waited_o = (j == 0);
      if (j == 0) {
        m_ref = m_blk;
      } else {
        const bool need = m_blk > m_ref + kLazy;
        if (__any_sync(0xffffffffu, need)) {
          // the previous P V product must have landed before O is rescaled in place
          if (!ptx::mbar_wait(o_full, (j - 1) & 1, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          waited_o = true;
          const float alpha = need ? ex2(m_ref - m_blk) : 1.f;
#pragma unroll 1
          for (int c = 0; c < HD / 16; ++c) {
            uint32_t t[16];
            ptx::tmem_ld16(tO + lane_sel + c * 16, t);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) t[e] = __float_as_uint(__uint_as_float(t[e]) * alpha);
            ptx::tmem_st16(tO + lane_sel + c * 16, t);
          }
          ptx::tmem_st_wait();
          l *= alpha;
          if (need) m_ref = m_blk;
        }
      }
      const float neg = -m_ref;
      float rs0 = 0.f, rs1 = 0.f;
      auto exp_chunk = [&](uint32_t (&r)[32], int c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = ex2(fmaf(__uint_as_float(r[e]), sc, neg));
          const float p1 = ex2(fmaf(__uint_as_float(r[e + 1]), sc, neg));
          rs0 += p0;
          rs1 += p1;
          pk[e >> 1] = pack_bf16x2(p0, p1);
        }
        if (c == 0 && !waited_o) {
          // P(j-1) V(j-1) must have finished reading the P buffer before it is overwritten
          if (!ptx::mbar_wait(o_full, (j - 1) & 1, abort_flag)) ok = false;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          *reinterpret_cast<uint4*>(p_smem + swz_off(row, c * 4 + u)) =
              make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
      };
      exp_chunk(r0, 0);
      if (!ok) break;
      exp_chunk(r1, 1);
      exp_chunk(r2, 2);
      exp_chunk(r3, 3);
      l += rs0 + rs1;
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(p_full);
    }
    if (ok) ok = ptx::mbar_wait(o_full, (nblk - 1) & 1, abort_flag);
    if (ok) {
      ptx::tc_fence_after_sync();
      const float inv = 1.f / l;
      bf16* dst = p.o + (static_cast<long long>(b) * p.T + q_idx) * p.o_stride_t + h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld32(tO + lane_sel + c * 32, r);
        ptx::tmem_ld_wait();
        if (q_idx < p.T) {
#pragma unroll
          for (int d = 0; d < 32; d += 8) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(r[d]) * inv, __uint_as_float(r[d + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(r[d + 2]) * inv, __uint_as_float(r[d + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(r[d + 4]) * inv, __uint_as_float(r[d + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(r[d + 6]) * inv, __uint_as_float(r[d + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + d) = u;
          }
        }
      }
      if (q_idx < p.T)
        p.lse[(static_cast<long long>(b) * p.Hq + h) * p.T + q_idx] = (m_ref + log2f(l)) * 0.6931471805599453f;
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, kStatusMbarTimeout);
}

// ------------------------------------------------------------------------ backward
template <int HD>
struct BwdCfg {
  static constexpr int kTileBytes = kBlk * HD * 2;
  // Q / dO tiles of the coming iterations: with three stages a load is issued a whole iteration before its tile is
  // needed (two stages left no lead at all: the slot of iteration it+1 is only released by iteration it-1)
  static constexpr int kStages = (HD == 64) ? 3 : 1;
  static constexpr bool kAliasDq = (HD > 64);  // dQ partial reuses the S columns when TMEM is full
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTileBytes;
  static constexpr int kQ = kV + kTileBytes;
  static constexpr int kDO = kQ + kStages * kTileBytes;
  static constexpr int kP = kDO + kStages * kTileBytes;
  static constexpr int kDS = kP + kBlk * kBlk * 2;
  // hd 64: two [128 rows x 32 fp32] staging tiles from which dQ leaves by TMA reduce-add (hd 128 has no room and
  // flushes dQ with vector reductions from registers)
  static constexpr int kDQ = kDS + kBlk * kBlk * 2;
  static constexpr int kDQBytes = kAliasDq ? 0 : 2 * kBlk * 128;
  static constexpr int kBar = kDQ + kDQBytes;
  static constexpr int kSmem = kBar + 128;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS = 0, kColDP = 128, kColDV = 256, kColDK = 256 + HD;
  static constexpr int kColDQ = kAliasDq ? 0 : 256 + 2 * HD;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Backward pipeline.  Warps 2..9 are the element-wise warps: a score row is shared by two warps (warps 2..5 take
// key columns 0..63 and the first half of the head dimension, warps 6..9 the second halves; both sets sit on the
// TMEM lane quarter `warp & 3`).  Per (query head, query block) iteration `it`:
//   MMA warp:  S(it+1), dP(it+1) are issued as soon as the element-wise warps have copied S(it), dP(it) out of
//              tensor memory (sdp_free), so they run underneath the exponentials of iteration it; dV, dK
//              accumulate over the whole loop; dQ(it) is issued when the element-wise warps have flushed dQ(it-1).
//   EW warps:  S and dP of their 64 columns are read from tensor memory once (128 registers), P and dS are
//              computed from registers, stored to shared memory once MMA group 2 of iteration it-1 has finished
//              reading the buffers, and only then is dQ(it-1) flushed to HBM -- underneath dV(it), dK(it).
// With hd = 128 tensor memory is full and dQ shares the S columns, so S(it+1) has to wait for the dQ(it) flush:
// that instantiation keeps the order S, dP -> P, dS -> dV, dK, dQ -> flush.
template <int HD>
__global__ void __launch_bounds__(320, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                const __grid_constant__ CUtensorMap tdq, const AttnArgs p) {
  using Cfg = BwdCfg<HD>;
  constexpr int S = Cfg::kStages;
  constexpr bool kPipe = !Cfg::kAliasDq;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBar);
  uint64_t* kv_full = bars;            // 1
  uint64_t* qdo_full = bars + 1;       // [3]
  uint64_t* qdo_empty = bars + 4;      // [3]
  uint64_t* sdp_full = bars + 7;
  uint64_t* pds_full = bars + 8;
  uint64_t* dq_full = bars + 9;
  uint64_t* dq_free = bars + 10;
  uint64_t* sdp_free = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.T + kBlk - 1) / kBlk;
  const int jb = blockIdx.x;  // key block
  const int hk = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int nq = nqb - jb;     // query blocks jb .. nqb-1
  const int niter = G * nq;

  if (threadIdx.x == 0) {
    ptx::mbar_init(kv_full, 1);
    for (int s = 0; s < 3; ++s) { ptx::mbar_init(&qdo_full[s], 1); ptx::mbar_init(&qdo_empty[s], 1); }
    ptx::mbar_init(sdp_full, 1);
    ptx::mbar_init(pds_full, 8);
    ptx::mbar_init(dq_full, 1);
    ptx::mbar_init(dq_free, 8);
    ptx::mbar_init(sdp_free, 8);
    *abort_flag = (ptx::smem_u32(smem) & 1023u) ? 1u : 0u;
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tq);
    ptx::tma_prefetch_desc(&tk);
    ptx::tma_prefetch_desc(&tv);
    ptx::tma_prefetch_desc(&tdo);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool bad_align = (*abort_flag != 0);

  if (bad_align) {
  } else if (warp == 0) {
    if (lane == 0) {
      ptx::mbar_expect_tx(kv_full, 2 * Cfg::kTileBytes);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        ptx::tma_load_2d(smem + Cfg::kK + c * kChunkBytes, &tk, kv_full, hk * HD + c * 64, b * p.T + jb * kBlk);
        ptx::tma_load_2d(smem + Cfg::kV + c * kChunkBytes, &tv, kv_full, hk * HD + c * 64, b * p.T + jb * kBlk);
      }
      for (int it = 0; it < niter; ++it) {
        const int g = it / nq, i = jb + (it - g * nq);
        const int h = hk * G + g;
        const int st = it % S;
        if (!ptx::mbar_wait(&qdo_empty[st], ((it / S) & 1) ^ 1u, abort_flag)) break;
        ptx::mbar_expect_tx(&qdo_full[st], 2 * Cfg::kTileBytes);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          ptx::tma_load_2d(smem + Cfg::kQ + st * Cfg::kTileBytes + c * kChunkBytes, &tq, &qdo_full[st],
                           h * HD + c * 64, b * p.T + i * kBlk);
          ptx::tma_load_2d(smem + Cfg::kDO + st * Cfg::kTileBytes + c * kChunkBytes, &tdo, &qdo_full[st],
                           h * HD + c * 64, b * p.T + i * kBlk);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = ptx::make_idesc_bf16(128, 128, 0, 0);   // S, dP : K-major x K-major
      const uint32_t idesc_t = ptx::make_idesc_bf16(128, HD, 1, 1);    // dV, dK: MN-major x MN-major
      const uint32_t idesc_q = ptx::make_idesc_bf16(128, HD, 0, 1);    // dQ    : K-major x MN-major
      const uint32_t k_base = ptx::smem_u32(smem + Cfg::kK), v_base = ptx::smem_u32(smem + Cfg::kV);
      const uint32_t p_base = ptx::smem_u32(smem + Cfg::kP), ds_base = ptx::smem_u32(smem + Cfg::kDS);
      // descriptors of the fixed tiles, and of stage 0 of the Q / dO ring, in both operand layouts
      const uint64_t k_kmaj = ptx::make_smem_desc(k_base, 16, 1024), v_kmaj = ptx::make_smem_desc(v_base, 16, 1024);
      const uint64_t k_mn = ptx::make_smem_desc(k_base, kChunkBytes, 1024);
      const uint64_t p_mn = ptx::make_smem_desc(p_base, kChunkBytes, 1024), ds_mn = ptx::make_smem_desc(ds_base, kChunkBytes, 1024);
      const uint64_t ds_kmaj = ptx::make_smem_desc(ds_base, 16, 1024);
      const uint32_t q_base0 = ptx::smem_u32(smem + Cfg::kQ), do_base0 = ptx::smem_u32(smem + Cfg::kDO);
      const uint64_t q_kmaj0 = ptx::make_smem_desc(q_base0, 16, 1024), do_kmaj0 = ptx::make_smem_desc(do_base0, 16, 1024);
      const uint64_t q_mn0 = ptx::make_smem_desc(q_base0, kChunkBytes, 1024), do_mn0 = ptx::make_smem_desc(do_base0, kChunkBytes, 1024);
      auto issue_sdp = [&](int it) {
        const uint32_t st_off = (it % S) * Cfg::kTileBytes;
        const uint64_t q_d = desc_add(q_kmaj0, st_off), do_d = desc_add(do_kmaj0, st_off);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * kChunkBytes + (k & 3) * 32;
          ptx::mma_f16_ss(tmem_base + Cfg::kColS, desc_add(q_d, off), desc_add(k_kmaj, off), idesc_s, k > 0);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * kChunkBytes + (k & 3) * 32;
          ptx::mma_f16_ss(tmem_base + Cfg::kColDP, desc_add(do_d, off), desc_add(v_kmaj, off), idesc_s, k > 0);
        }
        ptx::tc_commit(sdp_full);
      };
      bool ok = ptx::mbar_wait(kv_full, 0, abort_flag);
      if (ok && niter > 0) {
        ok = ptx::mbar_wait(&qdo_full[0], 0, abort_flag);
        if (ok) {
          ptx::tc_fence_after_sync();
          issue_sdp(0);
        }
      }
      for (int it = 0; it < niter && ok; ++it) {
        const int st = it % S;
        const uint64_t q_m = desc_add(q_mn0, st * Cfg::kTileBytes), do_m = desc_add(do_mn0, st * Cfg::kTileBytes);
        if (kPipe && it + 1 < niter) {
          // next S / dP: operands loaded, and the score columns copied out by the element-wise warps
          if (!ptx::mbar_wait(&qdo_full[(it + 1) % S], ((it + 1) / S) & 1, abort_flag)) break;
          if (!ptx::mbar_wait(sdp_free, it & 1, abort_flag)) break;
          ptx::tc_fence_after_sync();
          issue_sdp(it + 1);
        }
        if (!ptx::mbar_wait(pds_full, it & 1, abort_flag)) break;
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < kBlk / 16; ++k) {  // reduction over the 128 query rows
          ptx::mma_f16_ss(tmem_base + Cfg::kColDV, desc_add(p_mn, k * 2048), desc_add(do_m, k * 2048), idesc_t, (it > 0 || k > 0));
        }
#pragma unroll
        for (int k = 0; k < kBlk / 16; ++k) {
          ptx::mma_f16_ss(tmem_base + Cfg::kColDK, desc_add(ds_mn, k * 2048), desc_add(q_m, k * 2048), idesc_t, (it > 0 || k > 0));
        }
        if (kPipe && it > 0) {
          // dQ(it-1) has left tensor memory
          if (!ptx::mbar_wait(dq_free, (it - 1) & 1, abort_flag)) break;
          ptx::tc_fence_after_sync();
        }
#pragma unroll
        for (int k = 0; k < kBlk / 16; ++k) {  // reduction over the 128 keys
          const uint32_t a_off = (k >> 2) * kChunkBytes + (k & 3) * 32;
          ptx::mma_f16_ss(tmem_base + Cfg::kColDQ, desc_add(ds_kmaj, a_off), desc_add(k_mn, k * 2048), idesc_q, k > 0);
        }
        ptx::tc_commit(dq_full);
        ptx::tc_commit(&qdo_empty[st]);
        if (!kPipe && it + 1 < niter) {
          // dQ shares the S columns: the next S / dP wait for the flush of dQ(it)
          if (!ptx::mbar_wait(&qdo_full[(it + 1) % S], ((it + 1) / S) & 1, abort_flag)) break;
          if (!ptx::mbar_wait(dq_free, it & 1, abort_flag)) break;
          ptx::tc_fence_after_sync();
          issue_sdp(it + 1);
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const float sc = p.scale * kLog2e;
    uint8_t* p_smem = smem + Cfg::kP;
    uint8_t* ds_smem = smem + Cfg::kDS;
    bool ok = true;
    // (lse, delta) of this thread's query row in iteration `it2`; rows past the end of the sequence get lse = +inf,
    // which turns their probabilities into exact zeros
    auto load_stats = [&](int it2, float& l, float& d) {
      const int g2 = it2 / nq, i2 = jb + (it2 - g2 * nq);
      const int q2 = i2 * kBlk + row;
      const long long stat2 = (static_cast<long long>(b) * p.Hq + (hk * G + g2)) * p.T + q2;
      // raw values: the conversion to base 2 happens where lse is used, so that nothing here waits for the loads
      l = q2 < p.T ? p.lse[stat2] : INFINITY;
      d = q2 < p.T ? p.delta[stat2] : 0.f;
    };
    // dQ of iteration `it2`, this warp's half of the head dimension, leaves tensor memory and is added to the fp32
    // accumulator in HBM.  hd 64: through a swizzled shared-memory tile and one TMA reduce-add per half (rows past the
    // end of the sequence are exact zeros, so adding them is harmless); hd 128: vector reductions from registers.
    auto flush_dq = [&](int it2) {
      const int g2 = it2 / nq, i2 = jb + (it2 - g2 * nq);
      const int q2 = i2 * kBlk + row;
      if constexpr (kPipe) {
        uint8_t* stg = smem + Cfg::kDQ + half * (kBlk * 128);
        const bool elected = (warp == 2 && lane == 0);
        // the reduce-adds of the previous flush have finished reading the staging tiles
        if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync 2, 256;" ::: "memory");
        uint32_t r[32];
        ptx::tmem_ld32(tmem_base + Cfg::kColDQ + lane_sel + half * 32, r);
        ptx::tmem_ld_wait();
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(dq_free);       // the dQ columns may be overwritten
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<uint4*>(stg + row * 128 + ((u ^ (row & 7)) << 4)) =
              make_uint4(r[u * 4], r[u * 4 + 1], r[u * 4 + 2], r[u * 4 + 3]);
        ptx::fence_proxy_async_smem();
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (elected) {
          const int x = (hk * G + g2) * HD, y = b * p.T + i2 * kBlk;
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2)
            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                             reinterpret_cast<uint64_t>(&tdq)),
                         "r"(ptx::smem_u32(smem + Cfg::kDQ + h2 * (kBlk * 128))), "r"(x + h2 * 32), "r"(y)
                         : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      } else {
        float* dq_row = p.dq_accum + ((static_cast<long long>(b) * p.T + q2) * p.Hq + (hk * G + g2)) * HD;
#pragma unroll 1
        for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); ++c) {
          uint32_t r[32];
          ptx::tmem_ld32(tmem_base + Cfg::kColDQ + lane_sel + c * 32, r);
          ptx::tmem_ld_wait();
          if (q2 < p.T) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              red_add_v4(dq_row + c * 32 + e, __uint_as_float(r[e]), __uint_as_float(r[e + 1]), __uint_as_float(r[e + 2]),
                         __uint_as_float(r[e + 3]));
          }
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(dq_free);
      }
    };
    float pre_lse = 0.f, pre_dlt = 0.f;
    if (niter > 0) load_stats(0, pre_lse, pre_dlt);
    for (int it = 0; it < niter; ++it) {
      const int i = jb + (it % nq);
      const int q_idx = i * kBlk + row;
      const float lse2 = pre_lse, dlt = pre_dlt;       // requested one iteration ahead
      if (it + 1 < niter) load_stats(it + 1, pre_lse, pre_dlt);
      if (!ptx::mbar_wait(sdp_full, it & 1, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      uint32_t s0[32], s1[32], d0[32], d1[32];
      ptx::tmem_ld32(tmem_base + Cfg::kColS + lane_sel + half * 64, s0);
      ptx::tmem_ld32(tmem_base + Cfg::kColS + lane_sel + half * 64 + 32, s1);
      ptx::tmem_ld32(tmem_base + Cfg::kColDP + lane_sel + half * 64, d0);
      ptx::tmem_ld32(tmem_base + Cfg::kColDP + lane_sel + half * 64 + 32, d1);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(sdp_free);       // S / dP columns may be overwritten
      if (i == jb) {  // diagonal block: keys after the query get probability zero
        const uint32_t ninf = __float_as_uint(-INFINITY);
        const int kv0 = jb * kBlk + half * 64;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          if (kv0 + e > q_idx) s0[e] = ninf;
          if (kv0 + 32 + e > q_idx) s1[e] = ninf;
        }
      }
      const float neg = -lse2 * kLog2e;
      auto ew_chunk = [&](uint32_t (&rs)[32], uint32_t (&rd)[32], int c) {
        uint32_t pk[16], dk_[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = ex2(fmaf(__uint_as_float(rs[e]), sc, neg));
          const float p1 = ex2(fmaf(__uint_as_float(rs[e + 1]), sc, neg));
          const float g0 = p0 * (__uint_as_float(rd[e]) - dlt) * p.scale;
          const float g1 = p1 * (__uint_as_float(rd[e + 1]) - dlt) * p.scale;
          pk[e >> 1] = pack_bf16x2(p0, p1);
          dk_[e >> 1] = pack_bf16x2(g0, g1);
        }
        if (kPipe && c == 0 && it > 0) {
          // MMA group 2 of the previous iteration must have finished reading P / dS (and produced dQ(it-1))
          if (!ptx::mbar_wait(dq_full, (it - 1) & 1, abort_flag)) ok = false;
          ptx::tc_fence_after_sync();
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t off = swz_off(row, half * 8 + c * 4 + u);
          *reinterpret_cast<uint4*>(p_smem + off) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
          *reinterpret_cast<uint4*>(ds_smem + off) = make_uint4(dk_[u * 4], dk_[u * 4 + 1], dk_[u * 4 + 2], dk_[u * 4 + 3]);
        }
      };
      ew_chunk(s0, d0, 0);
      if (!ok) break;
      ew_chunk(s1, d1, 1);
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(pds_full);
      if (kPipe) {
        if (it > 0) flush_dq(it - 1);                   // underneath dV(it), dK(it)
      } else {
        // dQ shares the S columns: flush dQ(it) before the next S / dP may be issued
        if (!ptx::mbar_wait(dq_full, it & 1, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        flush_dq(it);
      }
    }
    if (kPipe && ok && niter > 0) {
      ok = ptx::mbar_wait(dq_full, (niter - 1) & 1, abort_flag);
      if (ok) {
        ptx::tc_fence_after_sync();
        flush_dq(niter - 1);
      }
    }
    if (kPipe && warp == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all reduce-adds done
    // The last dq_full arrival also covers every dV/dK accumulation issued before it.
    const int kv_idx = jb * kBlk + row;
    if (ok && niter > 0) {
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        bf16* base = which == 0 ? p.dv : p.dk;
        const long long stride = which == 0 ? p.dv_stride_t : p.dk_stride_t;
        const uint32_t col = which == 0 ? Cfg::kColDV : Cfg::kColDK;
        bf16* dst = base + (static_cast<long long>(b) * p.T + kv_idx) * stride + hk * HD;
#pragma unroll 1
        for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); ++c) {
          uint32_t r[32];
          ptx::tmem_ld32(tmem_base + col + lane_sel + c * 32, r);
          ptx::tmem_ld_wait();
          if (kv_idx < p.T) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(r[e]), __uint_as_float(r[e + 1]));
              u.y = pack_bf16x2(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
              u.z = pack_bf16x2(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
              u.w = pack_bf16x2(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
              *reinterpret_cast<uint4*>(dst + c * 32 + e) = u;
            }
          }
        }
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, kStatusMbarTimeout);
}

// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; one thread per (b,t,h) row.
__global__ void attn_delta_kernel(const bf16* __restrict__ d_o, const bf16* __restrict__ o, float* __restrict__ delta,
                                  int B, int T, int H, int hd, long long do_stride_t, long long o_stride_t) {
  const long long n = static_cast<long long>(B) * T * H;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int h = static_cast<int>(i % H);
    const long long bt = i / H;
    const bf16* a = d_o + bt * do_stride_t + h * hd;
    const bf16* c = o + bt * o_stride_t + h * hd;
    float s = 0.f;
    for (int d = 0; d < hd; d += 8) {
      uint4 ua = *reinterpret_cast<const uint4*>(a + d), uc = *reinterpret_cast<const uint4*>(c + d);
      float2 a0 = unpack_bf16x2(ua.x), a1 = unpack_bf16x2(ua.y), a2 = unpack_bf16x2(ua.z), a3 = unpack_bf16x2(ua.w);
      float2 c0 = unpack_bf16x2(uc.x), c1 = unpack_bf16x2(uc.y), c2 = unpack_bf16x2(uc.z), c3 = unpack_bf16x2(uc.w);
      s += a0.x * c0.x + a0.y * c0.y + a1.x * c1.x + a1.y * c1.y + a2.x * c2.x + a2.y * c2.y + a3.x * c3.x + a3.y * c3.y;
    }
    const long long b = bt / T, t = bt - b * T;
    delta[(b * H + h) * T + t] = s;
  }
}

// dq (bf16, token stride dq_stride_t) = dq_accum (fp32 [B*T, H*hd])
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, long long BT, int width,
                                       long long dq_stride_t) {
  const int wv = width / 8;
  const long long n = BT * wv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long bt = i / wv;
    const int c = static_cast<int>(i - bt * wv) * 8;
    const float4 f0 = *reinterpret_cast<const float4*>(acc + bt * width + c);
    const float4 f1 = *reinterpret_cast<const float4*>(acc + bt * width + c + 4);
    uint4 u;
    u.x = pack_bf16x2(f0.x, f0.y); u.y = pack_bf16x2(f0.z, f0.w);
    u.z = pack_bf16x2(f1.x, f1.y); u.w = pack_bf16x2(f1.z, f1.w);
    *reinterpret_cast<uint4*>(dq + bt * dq_stride_t + c) = u;
  }
}

static bool attn_check(const TitbAttnDesc* d) {
  if (d->hd != 64 && d->hd != 128) return false;
  if (d->Hq % d->Hkv) return false;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al(d->q) || !al(d->k) || !al(d->v) || !al(d->o)) return false;
  if ((d->q_stride_t & 7) || (d->k_stride_t & 7) || (d->v_stride_t & 7) || (d->o_stride_t & 7)) return false;
  return true;
}

template <int HD>
static int attn_fwd_launch(const TitbAttnDesc* d, cudaStream_t st) {
  using Cfg = FwdCfg<HD>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  const uint64_t rows = static_cast<uint64_t>(d->B) * d->T;
  CUtensorMap tq, tk, tv;
  if (!make_tmap_bf16_2d(&tq, d->q, static_cast<uint64_t>(d->Hq) * HD, rows, d->q_stride_t, 64, kBlk) ||
      !make_tmap_bf16_2d(&tk, d->k, static_cast<uint64_t>(d->Hkv) * HD, rows, d->k_stride_t, 64, kBlk) ||
      !make_tmap_bf16_2d(&tv, d->v, static_cast<uint64_t>(d->Hkv) * HD, rows, d->v_stride_t, 64, kBlk))
    return TITB_ERR_TENSOR_MAP;
  AttnArgs a{};
  a.B = d->B; a.T = d->T; a.Hq = d->Hq; a.Hkv = d->Hkv; a.hd = HD;
  a.scale = d->scale;
  a.o = static_cast<bf16*>(d->o); a.lse = d->lse; a.o_stride_t = d->o_stride_t;
  a.status = titb_status_ptr();
  dim3 grid((d->T + kBlk - 1) / kBlk, d->Hq, d->B);
  attn_fwd_kernel<HD><<<grid, kAttnThreads, Cfg::kSmem, st>>>(tq, tk, tv, a);
  return static_cast<int>(cudaGetLastError());
}

template <int HD>
static int attn_bwd_launch(const TitbAttnDesc* d, cudaStream_t st) {
  using Cfg = BwdCfg<HD>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  const uint64_t rows = static_cast<uint64_t>(d->B) * d->T;
  CUtensorMap tq, tk, tv, tdo, tdq;
  if (!make_tmap_bf16_2d(&tq, d->q, static_cast<uint64_t>(d->Hq) * HD, rows, d->q_stride_t, 64, kBlk) ||
      !make_tmap_bf16_2d(&tk, d->k, static_cast<uint64_t>(d->Hkv) * HD, rows, d->k_stride_t, 64, kBlk) ||
      !make_tmap_bf16_2d(&tv, d->v, static_cast<uint64_t>(d->Hkv) * HD, rows, d->v_stride_t, 64, kBlk) ||
      !make_tmap_bf16_2d(&tdo, d->d_o, static_cast<uint64_t>(d->Hq) * HD, rows, d->do_stride_t, 64, kBlk))
    return TITB_ERR_TENSOR_MAP;
  tdq = tq;  // placeholder where the kernel does not use it (hd 128)
  if (!Cfg::kAliasDq && !make_tmap_f32_2d(&tdq, d->dq_accum, static_cast<uint64_t>(d->Hq) * HD, rows,
                                          static_cast<uint64_t>(d->Hq) * HD, 32, kBlk))
    return TITB_ERR_TENSOR_MAP;
  const long long nrows = static_cast<long long>(d->B) * d->T * d->Hq;
  int blocks = static_cast<int>((nrows + 255) / 256);
  if (blocks > device_sm_count() * 8) blocks = device_sm_count() * 8;
  attn_delta_kernel<<<blocks, 256, 0, st>>>(static_cast<const bf16*>(d->d_o), static_cast<const bf16*>(d->o), d->delta,
                                            d->B, d->T, d->Hq, HD, d->do_stride_t, d->o_stride_t);
  cudaError_t e = cudaMemsetAsync(d->dq_accum, 0, sizeof(float) * nrows * HD, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  AttnArgs a{};
  a.B = d->B; a.T = d->T; a.Hq = d->Hq; a.Hkv = d->Hkv; a.hd = HD;
  a.scale = d->scale;
  a.lse = d->lse; a.delta = d->delta; a.dq_accum = d->dq_accum;
  a.dk = static_cast<bf16*>(d->dk); a.dv = static_cast<bf16*>(d->dv);
  a.dk_stride_t = d->dk_stride_t; a.dv_stride_t = d->dv_stride_t;
  a.status = titb_status_ptr();
  dim3 grid((d->T + kBlk - 1) / kBlk, d->Hkv, d->B);
  attn_bwd_kernel<HD><<<grid, 320, Cfg::kSmem, st>>>(tq, tk, tv, tdo, tdq, a);
  const long long bt = static_cast<long long>(d->B) * d->T;
  const int width = d->Hq * HD;
  int cb = static_cast<int>((bt * (width / 8) + 255) / 256);
  if (cb > device_sm_count() * 8) cb = device_sm_count() * 8;
  attn_dq_convert_kernel<<<cb, 256, 0, st>>>(d->dq_accum, static_cast<bf16*>(d->dq), bt, width, d->dq_stride_t);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace titb

using namespace titb;

TITB_API int titb_attn_fwd(const TitbAttnDesc* d, cudaStream_t stream) {
  (void)cudaGetLastError();
  if (d->B <= 0 || d->T <= 0) return 0;
  if (!attn_check(d)) return TITB_ERR_SHAPE;
  return d->hd == 64 ? attn_fwd_launch<64>(d, stream) : attn_fwd_launch<128>(d, stream);
}

TITB_API int titb_attn_bwd(const TitbAttnDesc* d, cudaStream_t stream) {
  (void)cudaGetLastError();
  if (d->B <= 0 || d->T <= 0) return 0;
  if (!attn_check(d)) return TITB_ERR_SHAPE;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al(d->d_o) || !al(d->dq) || !al(d->dk) || !al(d->dv) || (d->do_stride_t & 7) || (d->dq_stride_t & 7) ||
      (d->dk_stride_t & 7) || (d->dv_stride_t & 7))
    return TITB_ERR_ALIGNMENT;
  return d->hd == 64 ? attn_bwd_launch<64>(d, stream) : attn_bwd_launch<128>(d, stream);
}
