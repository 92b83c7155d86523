// bf16 GEMM on the 5th-generation tensor cores: TMA -> shared-memory ring ->
// tcgen05.mma (accumulators in tensor memory) -> tcgen05.ld -> fused epilogue.
//
// Replaces the reference's cuBLAS SGEMM call sites (infini_train/src/kernels/cuda/linear.cu:58-128
// LinearForward, :148-232 LinearBackward, :26-47 Matmul) with one persistent,
// warp-specialised kernel:
//   warp 0 (one lane)  TMA producer, fills a STAGES-deep ring of A/B tiles
//   warp 1 (one lane)  issues tcgen05.mma, 128 x BN x 16 per instruction
//   warps 2..5         epilogue: read the fp32 accumulator from TMEM, apply
//                      bias / GELU / dGELU / residual, store bf16 or fp32
// The accumulator is double buffered in TMEM (2 x BN columns), so the epilogue
// of tile i overlaps the main loop of tile i+1.  Operands may be K-major or
// MN-major, which covers forward, dgrad and wgrad without transposing in HBM.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include <cstdlib>

#include "api.h"
#include "ptx_sm100.cuh"

// This file is compiled twice.  On its own it is the GEMM every training step uses.  gemm_param_gather.cu defines
// TITB_GEMM_PARAM_GATHER (and renames the namespace) before including it: that second copy adds collective mode 3,
// the weight all-gather fused into the consuming GEMM, without changing one token of the first.
#ifdef TITB_GEMM_PARAM_GATHER
#define TITB_GEMM_ENTRY titb_gemm_param_gather_bf16
#else
#define TITB_GEMM_ENTRY titb_gemm_bf16
#endif

namespace titb {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kABytes = kBM * kBK * 2;
constexpr int kGemmThreads = 192;

// Collective fused into the GEMM (tensor parallelism with sequence-sharded activations).
//  mode 1, all-gather -> GEMM: the first `helper_ctas` CTAs copy 128-row chunks of every rank's
//    activation shard from peer memory into the local `gathered` buffer (bulk copies by the TMA
//    engine: peer memory -> shared memory -> local memory, a dozen 16 KB pieces in flight per
//    CTA) and raise a per-chunk flag; the GEMM CTAs visit m-blocks in the same order (local
//    shard first) and their TMA producer waits on the flag of the chunk it is about to load.
//    When their copies are done the helper CTAs join the GEMM: they sit out the first
//    `helper_rounds` rounds of the tile list (the other CTAs share those) and take a full
//    share of every later round.
//  mode 2, GEMM -> reduce-scatter: the epilogue stores each bf16 partial tile straight into the
//    receive buffer of the rank that owns those rows (peer stores over NVLink) and bumps a
//    counter there; the first `helper_ctas` CTAs of the owner wait per 128-row chunk for all
//    partial tiles, sum the `world` slots (+bias +residual) and write the output shard.
#ifdef TITB_GEMM_PARAM_GATHER
//  mode 3, parameter all-gather -> GEMM: the B operand (a weight [N, K], K-major) is sharded by rows over the
//    data-parallel ranks.  `gathered` is this rank's full-size copy of the weight (the tensor map of B points at
//    it), `peers[r]` the rows rank r owns, in r's memory.  The first `helper_ctas` CTAs pull 128-row chunks from
//    their owners (the same bulk-copy role as mode 1; the local shard is already in place when peers[rank] aliases
//    it) and raise the chunk's flag; the GEMM CTAs visit n-blocks shard by shard, local shard first, and their TMA
//    producer waits for the chunks under the B tile it is about to load.  rows_per_rank counts weight rows.
#endif
struct CollArgs {
  int mode, world, rank, helper_ctas, rows_per_rank;
  int helper_rounds;    // modes 1, 3: rounds of the tile list the copying CTAs leave to the others while they copy
  void* peers[16];      // mode 1: shard bases bf16 [Ms, K]; mode 2: receive buffers bf16 [world][Ms][N]
  void* cnt_peers[16];  // mode 2: counter arrays uint32 [Ms / 128] of every rank
  bf16* gathered;       // mode 1: local [M, K] staging buffer (the GEMM's A operand)
  uint32_t* flags;      // mode 1: local chunk flags [M / 128]; mode 2: this rank's counters
  bf16* rs_out;         // mode 2: output shard [Ms, N]
  const bf16* rs_bias;
  const bf16* rs_residual;
};

struct GemmArgs {
  CollArgs coll;
  int M, N, K;
  int a_mn, b_mn;
  int a_box3, b_box3;   // MN-major operand arrives as one 3-D TMA box (64 columns x kBK rows x chunks) per k-block
  void* out;
  long long ldo;
  int out_fp32, accumulate, epi;
  const bf16* bias;
  const bf16* aux_in;
  long long ld_aux_in;
  bf16* aux_out;
  long long ld_aux_out;
  int splits;       // split-K factor; partial tiles go to `out` = workspace [splits, M, N] fp32
  int kb_per_split;
  int vec_ok;       // all row strides / base pointers allow 16-byte accesses
  int tma_store;    // 1: bf16 outputs leave through shared-memory staging + TMA stores; 2: fp32 outputs do
  int f32_red;      // tma_store == 2: tiles are added to the output (TMA reduce-add) instead of stored
  int aux_tma_load; // residual / pre-activation tiles arrive through TMA loads into the aux staging tile
  const float* alpha;  // optional device scalar multiplied into the accumulator
  uint32_t a_lbo, a_sbo, a_kstep, b_lbo, b_sbo, b_kstep;
  int* status;
};

// PAIR: two CTAs of a cluster share one 256 x BN tile (tcgen05 cta_group::2).  Each stages its own 128 rows of A and
// its own half of the B tile, so a k-block costs every SM (128 + BN / 2) x 64 x 2 bytes of operand traffic instead
// of (128 + BN) x 64 x 2: two thirds at BN = 256.  No multicast: every CTA fetches its own tiles.
template <int BN, bool PAIR = false>
struct GemmCfg {
  static constexpr int kBRows = PAIR ? BN / 2 : BN;   // rows of B (output columns) this CTA stages per k-block
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStages = PAIR ? 6 : ((BN == 128) ? 6 : 4);
  static constexpr int kTileM = PAIR ? 2 * kBM : kBM;
  static constexpr int kAccStride = (BN == 128) ? 128 : 256;  // TMEM columns between the two accumulators
  static constexpr int kTmemCols = 2 * kAccStride;            // allocation size must be a power of two
  static constexpr int kRing = kStages * (kABytes + kBBytes);
  static constexpr int kStage = 2 * kBM * 128;  // two [128 rows x 64 bf16] swizzled staging tiles for TMA stores
  static constexpr int kSmem = kRing + kStage + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float gelu_fast(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanh_fast(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_fast(float x) {
  const float k = 0.7978845608028654f;
  float x2 = x * x;
  float t = tanh_fast(k * (x + 0.044715f * x * x2));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 0.134145f * x2);
}

// Epilogue for one thread: 32 consecutive columns [col0, col0+32) of one output row.
__device__ __forceinline__ void epilogue_row32(const GemmArgs& p, float (&v)[32], long long row, int col0,
                                                int split) {
  const int ncols = min(32, p.N - col0);
  const bool full = (ncols == 32) && p.vec_ok;

  if (p.alpha != nullptr && p.splits == 1) {
    const float al = *p.alpha;
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= al;
  }
  if (p.splits > 1) {  // raw fp32 partials, reduced by splitk_reduce_kernel
    float* dst = reinterpret_cast<float*>(p.out) + (static_cast<long long>(split) * p.M + row) * p.N + col0;
    if (ncols == 32 && (p.N & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
      for (int j = 0; j < ncols; ++j) dst[j] = v[j];
    }
    return;
  }

  if (p.epi == TITB_EPI_BIAS || p.epi == TITB_EPI_BIAS_GELU || p.epi == TITB_EPI_BIAS_RESIDUAL) {
    if (p.bias != nullptr) {
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 u = *reinterpret_cast<const uint4*>(p.bias + col0 + j);
          float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
          v[j] += f0.x; v[j + 1] += f0.y; v[j + 2] += f1.x; v[j + 3] += f1.y;
          v[j + 4] += f2.x; v[j + 5] += f2.y; v[j + 6] += f3.x; v[j + 7] += f3.y;
        }
      } else {
        for (int j = 0; j < ncols; ++j) v[j] += __bfloat162float(p.bias[col0 + j]);
      }
    }
  }
  if (p.epi == TITB_EPI_BIAS_GELU) {
    if (p.aux_out != nullptr) {
      bf16* ao = p.aux_out + row * p.ld_aux_out + col0;
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 u;
          u.x = pack_bf16x2(v[j], v[j + 1]); u.y = pack_bf16x2(v[j + 2], v[j + 3]);
          u.z = pack_bf16x2(v[j + 4], v[j + 5]); u.w = pack_bf16x2(v[j + 6], v[j + 7]);
          *reinterpret_cast<uint4*>(ao + j) = u;
        }
      } else {
        for (int j = 0; j < ncols; ++j) ao[j] = __float2bfloat16_rn(v[j]);
      }
    }
    // The activation is evaluated on the bf16-rounded pre-activation so that the
    // backward pass, which only has the stored bf16 copy, differentiates the same point.
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_fast(__bfloat162float(__float2bfloat16_rn(v[j])));
  } else if (p.epi == TITB_EPI_DGELU || p.epi == TITB_EPI_BIAS_RESIDUAL) {
    if (p.aux_in != nullptr) {
      const bf16* ai = p.aux_in + row * p.ld_aux_in + col0;
      float a[32];
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 u = *reinterpret_cast<const uint4*>(ai + j);
          float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
          a[j] = f0.x; a[j + 1] = f0.y; a[j + 2] = f1.x; a[j + 3] = f1.y;
          a[j + 4] = f2.x; a[j + 5] = f2.y; a[j + 6] = f3.x; a[j + 7] = f3.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) a[j] = (j < ncols) ? __bfloat162float(ai[j]) : 0.f;
      }
      if (p.epi == TITB_EPI_DGELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= gelu_grad_fast(a[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += a[j];
      }
    }
  }

  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(p.out) + row * p.ldo + col0;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (p.accumulate) {
          float4 c = *reinterpret_cast<const float4*>(dst + j);
          o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
        }
        *reinterpret_cast<float4*>(dst + j) = o;
      }
    } else {
      for (int j = 0; j < ncols; ++j) dst[j] = p.accumulate ? dst[j] + v[j] : v[j];
    }
  } else {
    bf16* dst = reinterpret_cast<bf16*>(p.out) + row * p.ldo + col0;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        if (p.accumulate) {
          uint4 c = *reinterpret_cast<const uint4*>(dst + j);
          float2 f0 = unpack_bf16x2(c.x), f1 = unpack_bf16x2(c.y), f2 = unpack_bf16x2(c.z), f3 = unpack_bf16x2(c.w);
          v[j] += f0.x; v[j + 1] += f0.y; v[j + 2] += f1.x; v[j + 3] += f1.y;
          v[j + 4] += f2.x; v[j + 5] += f2.y; v[j + 6] += f3.x; v[j + 7] += f3.y;
        }
        uint4 u;
        u.x = pack_bf16x2(v[j], v[j + 1]); u.y = pack_bf16x2(v[j + 2], v[j + 3]);
        u.z = pack_bf16x2(v[j + 4], v[j + 5]); u.w = pack_bf16x2(v[j + 6], v[j + 7]);
        *reinterpret_cast<uint4*>(dst + j) = u;
      }
    } else {
      for (int j = 0; j < ncols; ++j) {
        float o = v[j];
        if (p.accumulate) o += __bfloat162float(dst[j]);
        dst[j] = __float2bfloat16_rn(o);
      }
    }
  }
}

struct TileCoord { int m0, n0, split, mblk; };

__device__ __forceinline__ TileCoord tile_coord(const GemmArgs& p, int tile, int tiles_m, int tiles_n, int bn,
                                                int tile_m = kBM, int row_off = 0) {
  const int tiles_mn = tiles_m * tiles_n;
  TileCoord t;
  t.split = tile / tiles_mn;
  const int mn = tile - t.split * tiles_mn;
  int nblk;
  if (p.coll.mode == 0) {
    t.mblk = mn % tiles_m;
    nblk = mn / tiles_m;
#ifdef TITB_GEMM_PARAM_GATHER
  } else if (p.coll.mode == 3) {
    // n-blocks shard by shard, starting with the rows this rank owns; all m-blocks of an n-block back to back
    t.mblk = mn % tiles_m;
    nblk = (mn / tiles_m + (p.coll.rank * p.coll.rows_per_rank) / bn) % tiles_n;
#endif
  } else {
    // m-blocks are visited shard by shard: all-gather starts with the local shard (already here),
    // reduce-scatter with the next rank's rows so that remote partials leave early.
    const int cpr = p.coll.rows_per_rank / kBM;
    const int start = (p.coll.mode == 1 ? p.coll.rank : p.coll.rank + 1) * cpr;
    t.mblk = (mn / tiles_n + start) % tiles_m;
    nblk = mn % tiles_n;
  }
  t.m0 = t.mblk * tile_m + row_off;   // row_off: second CTA of a pair owns the lower 128 rows of the tile
  t.n0 = nblk * bn;
  return t;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* a) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* a) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* a, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add_u32(uint32_t* a, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add_u32(uint32_t* a, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded spin until *flag >= want (acquire at `sys` or `gpu` scope); false on timeout.
template <bool SYS>
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want) {
  const long long t0 = clock64();
  while (true) {
    const uint32_t v = SYS ? ld_acquire_sys_u32(flag) : ld_acquire_gpu_u32(flag);
    if (v >= want) return true;
    __nanosleep(32);
    if (clock64() - t0 > ptx::kWaitBudgetCycles) return false;
  }
}

// Which tiles a CTA works on, round by round.  Plain launches deal the tiles round-robin over n CTAs (H = 0).  In an
// all-gather -> GEMM launch the first H CTAs are busy copying during the first `skip` rounds, which the other n - H
// CTAs share among themselves; from round `skip` on all n CTAs take part.
struct TileWalk {
  int c, n, H, skip;
  __device__ __forceinline__ int first_round() const { return c < H ? skip : 0; }
  __device__ __forceinline__ int tile(int round) const {
    return round < skip ? round * (n - H) + (c - H) : skip * (n - H) + (round - skip) * n + c;
  }
};

// mode 1 helper CTA: pull 128-row chunks of every rank's shard into the local gathered buffer.  One thread drives
// the TMA engine: 16 KB pieces travel peer (or local) memory -> shared-memory ring -> gathered buffer; of the twelve
// stages eight hold loads in flight and four hold stores that are still being read, so neither latency is exposed
// per piece (plain per-thread loads and stores moved 13-17 GB/s per CTA, one round trip per 48 KB batch).  Returns
// false when a wait ran out (status word set).
// the gather mode this compilation serves: activation rows (mode 1), or weight rows in the parameter-gather build
#ifdef TITB_GEMM_PARAM_GATHER
constexpr int kGatherMode = 3;
#else
constexpr int kGatherMode = 1;
#endif
constexpr int kAgMaxStages = 12;
constexpr int kAgPiece = 16384;
constexpr int kAgStoresInFlight = 5;
// A 128-row chunk of the gathered operand is copied in up to four parts by different CTAs; its flag counts parts.
__device__ __forceinline__ int ag_pieces_per_chunk(int K) { return (kBM * K * 2 + kAgPiece - 1) / kAgPiece; }
__device__ __forceinline__ int ag_pieces_per_part(int K) { return (ag_pieces_per_chunk(K) + 3) / 4; }
__device__ __forceinline__ int ag_parts_per_chunk(int K) {
  return (ag_pieces_per_chunk(K) + ag_pieces_per_part(K) - 1) / ag_pieces_per_part(K);   // no part is empty
}

// The gathered extent is M for the activation gather and N for the weight gather of mode 3, where a part whose source
// already is its destination (the owner's rows of the weight) is published without a copy.
__device__ __noinline__ bool ag_copy_role(const GemmArgs& p, uint8_t* ring, int kAgStages) {
  __shared__ uint64_t ag_bar[kAgMaxStages];
  __shared__ int ag_sig[kAgMaxStages];   // per stage: m-block to publish when that stage's store completes, or -1
  __shared__ int ag_ok;
  const CollArgs& c = p.coll;
  const bool skip_local = c.mode == 3;        // mode 3 gathers rows of B (the weight), mode 1 rows of A
  const int rows = skip_local ? p.N : p.M;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kAgStages; ++s) ptx::mbar_init(&ag_bar[s], 1);
    ptx::mbar_fence_init();
    const int nchunks = rows / kBM, cpr = c.rows_per_rank / kBM;
    const int chunk_bytes = kBM * p.K * 2;
    const int ppc = ag_pieces_per_chunk(p.K);
    const int parts = ag_parts_per_chunk(p.K);
    const int pp = ag_pieces_per_part(p.K);
    const int H = c.helper_ctas;
    volatile uint32_t no_abort = 0;
    // The copying CTAs deal out the parts of all chunks (chunks in the order the GEMM visits them) round-robin, so
    // the first chunks are complete after a quarter of a chunk time.  A cursor walks this CTA's pieces and keeps
    // addresses, ring stage and barrier parity up to date with additions only: one thread issues every copy, so
    // its instruction count per piece bounds the copy rate.
    struct Cursor {
      int pos, part, piece, end, stage, mblk;
      uint32_t parity;
      const uint8_t* src;
      uint8_t* dst;
    };
    auto open_part = [&](Cursor& q) {
      q.mblk = (q.pos + c.rank * cpr) % nchunks;
      const int src_rank = q.mblk / cpr;
      q.src = reinterpret_cast<const uint8_t*>(static_cast<const bf16*>(c.peers[src_rank]) +
                                               static_cast<long long>(q.mblk - src_rank * cpr) * kBM * p.K);
      q.dst = reinterpret_cast<uint8_t*>(c.gathered + static_cast<long long>(q.mblk) * kBM * p.K);
      q.piece = q.part * pp;
      q.end = min(ppc, q.piece + pp);
    };
    auto valid = [&](const Cursor& q) { return q.pos < nchunks; };
    auto next_part = [&](Cursor& q) {
      q.part += H;
      while (q.part >= parts) { q.part -= parts; ++q.pos; }
    };
    // opens the part under the cursor, passing over parts that need no copy (`announce`: the cursor that issues the
    // stores also publishes those parts; the load cursor walks the same sequence silently)
    auto settle = [&](Cursor& q, bool announce) {
      while (valid(q)) {
        open_part(q);
        if (!(skip_local && q.src == q.dst)) break;
        if (announce) red_release_gpu_add_u32(c.flags + q.mblk, 1u);
        next_part(q);
      }
    };
    auto advance = [&](Cursor& q, bool announce) {
      if (++q.piece == q.end) {
        next_part(q);
        settle(q, announce);
      }
      if (++q.stage == kAgStages) { q.stage = 0; q.parity ^= 1u; }
    };
    auto piece_bytes = [&](const Cursor& q) {
      return static_cast<uint32_t>(min(kAgPiece, chunk_bytes - q.piece * kAgPiece));
    };
    const int g0 = static_cast<int>(blockIdx.x);
    Cursor ld{g0 / parts, g0 % parts, 0, 0, 0, 0, 0u, nullptr, nullptr};
    Cursor st = ld;
    settle(ld, false);
    settle(st, true);
    auto issue = [&]() {
      const uint32_t bytes = piece_bytes(ld);
      ptx::mbar_expect_tx(&ag_bar[ld.stage], bytes);
      ptx::bulk_load(ring + ld.stage * kAgPiece, ld.src + ld.piece * kAgPiece, bytes, &ag_bar[ld.stage]);
      advance(ld, false);
    };
    // the store issued from `stage` has completed: if it closed a part, tell the GEMM CTAs
    auto publish = [&](int stage) {
      if (ag_sig[stage] >= 0) {
        fence_proxy_async_all();   // written through the async proxy, read through it again by the GEMM's TMA loads
        red_release_gpu_add_u32(c.flags + ag_sig[stage], 1u);
      }
    };
    bool ok = true;
    // kAgStoresInFlight stages hold stores that have not completed, the others loads in flight
    for (int n = 0; n < kAgStages - kAgStoresInFlight && valid(ld); ++n) issue();
    int i = 0;           // pieces stored so far
    int oldest = 0;      // stage of the oldest store not yet known to be complete
    for (; valid(st); ++i) {
      if (!ptx::mbar_wait(&ag_bar[st.stage], st.parity, &no_abort)) { ok = false; break; }
      ptx::bulk_store(st.dst + st.piece * kAgPiece, ring + st.stage * kAgPiece, piece_bytes(st));
      ptx::bulk_commit();
      ag_sig[st.stage] = (st.piece == st.end - 1) ? st.mblk : -1;
      advance(st, true);
      // all but the newest kAgStoresInFlight - 1 stores are complete: the oldest one can be published and its stage
      // reused (waiting for a store issued several pieces ago costs little; waiting for the newest would serialise
      // the ring on the latency of a store)
      ptx::bulk_wait_all<kAgStoresInFlight - 1>();
      if (i >= kAgStoresInFlight - 1) {
        publish(oldest);
        if (++oldest == kAgStages) oldest = 0;
      }
      if (valid(ld)) issue();
    }
    ptx::bulk_wait_all<0>();
    if (ok) {
      for (int d = max(0, i - (kAgStoresInFlight - 1)); d < i; ++d) {
        publish(oldest);
        if (++oldest == kAgStages) oldest = 0;
      }
    } else {
      atomicExch(p.status, kStatusPeerTimeout);
      // loads already issued still write into the ring: give each a bounded wait before the CTA leaves
      for (int s = 0; s < kAgStages; ++s) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(&ag_bar[s], 0) && !ptx::mbar_try_wait(&ag_bar[s], 1) && clock64() - t0 < 2000000LL) {
        }
      }
    }
    ag_ok = ok ? 1 : 0;
  }
  __syncthreads();
  return ag_ok != 0;
}


// mode 2, second phase: when a CTA has pushed all its partial tiles, its four epilogue warps (128 threads, named
// barrier 1) help to sum the `world` partial slots of this rank's rows.  A work unit is a 128-row chunk x a strip of
// 64 columns; units are dealt round-robin over all CTAs, so the whole GPU streams the reduction.  A unit waits --
// bounded -- until every rank's partial tiles of its chunk have arrived; remote ranks send this rank's rows first,
// so they usually have.  The pass is pure streaming, so what matters is bytes in flight: a thread issues the loads
// of B rows x W slots (16 vectors of 16 bytes) before it sums the first.
__device__ __forceinline__ void rs_add8(float (&acc)[8], const uint4& v) {
  const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
  acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
  acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
}

// W: slots read per row (world rounded up to a power of two); B = 16 / W rows in flight per thread.
template <int W>
__device__ __forceinline__ void rs_sum_unit(const GemmArgs& p, const bf16* recv, long long slot, int ch, int v0, int vn,
                                            int tid) {
  constexpr int B = W >= 8 ? 1 : 8 / W;
  const CollArgs& c = p.coll;
  // 128 rows x vn vectors; consecutive threads take consecutive vectors of a row.  Position tid + 128 j, j < vn:
  // every thread has the same number of positions, so the guards below are uniform.
  for (int j0 = 0; j0 < vn; j0 += B) {
    uint4 part[B][W];
    long long off[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const int i = tid + (j0 + b) * 128;
      const int r = ch * kBM + i / vn, col = (v0 + i % vn) * 8;
      off[b] = static_cast<long long>(r) * p.N + col;
      if (j0 + b < vn) {
#pragma unroll
        for (int s = 0; s < W; ++s)
          if (s < c.world) part[b][s] = *reinterpret_cast<const uint4*>(recv + s * slot + off[b]);
      }
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const int i = tid + (j0 + b) * 128;
      if (j0 + b >= vn) continue;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < W; ++s)
        if (s < c.world) rs_add8(acc, part[b][s]);
      if (c.rs_bias != nullptr) rs_add8(acc, *reinterpret_cast<const uint4*>(c.rs_bias + (v0 + i % vn) * 8));
      if (c.rs_residual != nullptr) rs_add8(acc, *reinterpret_cast<const uint4*>(c.rs_residual + off[b]));
      *reinterpret_cast<uint4*>(c.rs_out + off[b]) =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                     pack_bf16x2(acc[6], acc[7]));
    }
  }
}

__device__ __noinline__ void rs_reduce_phase(const GemmArgs& p, int tiles_n, int worker, int nworkers, int tid) {
  const CollArgs& c = p.coll;
  __shared__ int ok_sh;
  const int cpr = c.rows_per_rank / kBM;
  const uint32_t expected = static_cast<uint32_t>(c.world * tiles_n);  // one arrival per partial tile
  const bf16* recv = static_cast<const bf16*>(c.peers[c.rank]);
  const long long slot = static_cast<long long>(c.rows_per_rank) * p.N;
  const int nv = p.N / 8;
  const int strips = (nv + 7) / 8;
  const int units = cpr * strips;
  int ready_ch = -1;
  for (int u = worker; u < units; u += nworkers) {
    const int ch = u / strips, st = u - ch * strips;
    if (ch != ready_ch) {
      if (tid == 0) {
        ok_sh = wait_flag_ge<true>(c.flags + ch, expected) ? 1 : 0;
        if (!ok_sh) atomicExch(p.status, kStatusPeerTimeout);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const bool ok = ok_sh != 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");   // ok_sh may be rewritten for the next unit
      if (!ok) continue;
      ready_ch = ch;
    }
    const int v0 = st * 8, vn = min(8, nv - v0);
    if (c.world <= 1) rs_sum_unit<1>(p, recv, slot, ch, v0, vn, tid);
    else if (c.world <= 2) rs_sum_unit<2>(p, recv, slot, ch, v0, vn, tid);
    else if (c.world <= 4) rs_sum_unit<4>(p, recv, slot, ch, v0, vn, tid);
    else if (c.world <= 8) rs_sum_unit<8>(p, recv, slot, ch, v0, vn, tid);
    else rs_sum_unit<16>(p, recv, slot, ch, v0, vn, tid);
  }
}

template <int BN, bool PAIR>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                         const __grid_constant__ CUtensorMap tma_out, const __grid_constant__ CUtensorMap tma_aux,
                         const __grid_constant__ GemmArgs p) {
  using Cfg = GemmCfg<BN, PAIR>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kBBytes = Cfg::kBBytes;
  constexpr int kTileM = Cfg::kTileM;
  const uint32_t pair_rank = PAIR ? ptx::cluster_ctarank() : 0u;   // 0 issues the MMAs of the pair
  const int row_off = static_cast<int>(pair_rank) * kBM;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  // Leading CTAs of a fused-collective launch first move the remote operand (activation rows in mode 1, weight rows in
  // mode 3): the operand ring is their copy ring, and when the copies are done they join the tile list (TileWalk).
  const int helpers = (!PAIR && p.coll.mode == kGatherMode) ? p.coll.helper_ctas : 0;
  if (!PAIR && static_cast<int>(blockIdx.x) < helpers) {
    if (p.coll.mode == kGatherMode) {
      constexpr int kRingPieces = Cfg::kRing / kAgPiece;   // the operand ring doubles as the copy ring
      static_assert(kRingPieces >= 2 * kAgStoresInFlight, "the copy ring needs stages for loads and for stores in flight");
      if (!ag_copy_role(p, smem, kRingPieces < kAgMaxStages ? kRingPieces : kAgMaxStages)) return;
    }
  }
  const bool joined = !PAIR && p.coll.mode == kGatherMode;   // helper CTAs take tiles too
  // a pair walks the tile list as one unit
  const int cta = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x) - (joined ? 0 : helpers);
  const int ncta = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x) - (joined ? 0 : helpers);
  const TileWalk walk{cta, ncta, joined ? helpers : 0, joined ? p.coll.helper_rounds : 0};
  uint8_t* sa = smem;
  uint8_t* sb = smem + kStages * kABytes;
  uint8_t* stage_out = smem + Cfg::kRing;
  uint8_t* stage_aux = stage_out + kBM * 128;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::kRing + Cfg::kStage);
  uint64_t* empty = full + kStages;
  uint64_t* acc_full = empty + kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* aux_bar = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    ptx::mbar_init(aux_bar, 1);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full[b], 1);
      ptx::mbar_init(&acc_empty[b], PAIR ? 8 : 4);   // pair: the epilogue warps of both CTAs arrive on rank 0's copy
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tma_a);
    ptx::tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    if (PAIR) {
      ptx::tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (PAIR) ptx::cluster_sync_all();   // the peer's barriers are initialised before anything signals them
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + kTileM - 1) / kTileM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_mn = tiles_m * tiles_n;
  const int num_tiles = tiles_mn * p.splits;
  const int num_kb_total = (p.K + kBK - 1) / kBK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ready_mblk = -1;
#ifdef TITB_GEMM_PARAM_GATHER
      int ready_n0 = -1;
#endif
      for (int rnd = walk.first_round(), tile; (tile = walk.tile(rnd)) < num_tiles && ok; ++rnd) {
        const TileCoord tc = tile_coord(p, tile, tiles_m, tiles_n, BN, kTileM, row_off);
        const int split = tc.split, m0 = tc.m0, n0 = tc.n0;
        const int nb0 = n0 + static_cast<int>(pair_rank) * Cfg::kBRows;   // first B row (output column) this CTA stages
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(num_kb_total, kb0 + p.kb_per_split);
        if (p.coll.mode == 1 && tc.mblk != ready_mblk) {
          // the rows of this m-block must have landed in the gathered buffer
          if (!wait_flag_ge<false>(p.coll.flags + tc.mblk, static_cast<uint32_t>(ag_parts_per_chunk(p.K)))) {
            *abort_flag = 1u;
            atomicExch(p.status, kStatusPeerTimeout);
            ok = false;
            break;
          }
          fence_proxy_async_all();
          ready_mblk = tc.mblk;
        }
#ifdef TITB_GEMM_PARAM_GATHER
        if (p.coll.mode == 3 && n0 != ready_n0) {
          // every 128-row chunk of the weight under this B tile must have landed in the local copy
          const int c_lo = n0 / kBM, c_hi = (min(n0 + BN, p.N) - 1) / kBM;
          for (int c = c_lo; c <= c_hi && ok; ++c) {
            if (!wait_flag_ge<false>(p.coll.flags + c, static_cast<uint32_t>(ag_parts_per_chunk(p.K)))) {
              *abort_flag = 1u;
              atomicExch(p.status, kStatusPeerTimeout);
              ok = false;
            }
          }
          if (!ok) break;
          fence_proxy_async_all();
          ready_n0 = n0;
        }
#endif
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* a_dst = sa + stage * kABytes;
          uint8_t* b_dst = sb + stage * kBBytes;
          // pair: both CTAs' bytes are counted on rank 0's barrier, which rank 0 arms for the sum
          auto load = [&](void* dst, const CUtensorMap* m, int x, int y) {
            if (PAIR) ptx::tma_load_2d_pair(dst, m, &full[stage], x, y);
            else ptx::tma_load_2d(dst, m, &full[stage], x, y);
          };
          if (!PAIR) ptx::mbar_expect_tx(&full[stage], kABytes + kBBytes);
          else if (pair_rank == 0) ptx::mbar_expect_tx(&full[stage], 2 * (kABytes + kBBytes));
          // An MN-major tile is a row of 64-column chunks (the 128-byte swizzle limits a box to 64 columns).  Over a
          // 3-D view of the matrix (64 columns, K rows, chunks) all chunks of the tile are ONE box, which lands in
          // shared memory chunk after chunk exactly as the separate boxes would: one TMA instruction per operand and
          // k-block instead of two to four (measured neutral on the weight-gradient shapes; kept for the shorter
          // producer loop).
          auto load3 = [&](void* dst, const CUtensorMap* m, int y, int z) {
            if (PAIR) ptx::tma_load_3d_pair(dst, m, &full[stage], 0, y, z);
            else ptx::tma_load_3d(dst, m, &full[stage], 0, y, z);
          };
          if (!p.a_mn) {
            load(a_dst, &tma_a, kb * kBK, m0);
          } else if (p.a_box3) {
            load3(a_dst, &tma_a, kb * kBK, m0 >> 6);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j) load(a_dst + j * (64 * kBK * 2), &tma_a, m0 + j * 64, kb * kBK);
          }
          if (!p.b_mn) {
            load(b_dst, &tma_b, kb * kBK, nb0);
          } else if (p.b_box3) {
            load3(b_dst, &tma_b, kb * kBK, nb0 >> 6);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::kBRows / 64; ++j) load(b_dst + j * (64 * kBK * 2), &tma_b, nb0 + j * 64, kb * kBK);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Give copies already issued a bounded chance to land before the CTA exits.
        for (int s = 0; s < kStages; ++s) {
          const long long t0 = clock64();
          while (!ptx::mbar_try_wait(&full[s], 0) && !ptx::mbar_try_wait(&full[s], 1) &&
                 clock64() - t0 < 2000000LL) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0 && pair_rank == 0) {
      const uint32_t idesc = ptx::make_idesc_bf16(kTileM, BN, p.a_mn, p.b_mn);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int rnd = walk.first_round(), tile; (tile = walk.tile(rnd)) < num_tiles && ok; ++rnd, ++it) {
        const int split = tile / tiles_mn;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(num_kb_total, kb0 + p.kb_per_split);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!ptx::mbar_wait(&acc_empty[buf], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * Cfg::kAccStride;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t a_base = ptx::smem_u32(sa + stage * kABytes);
          const uint32_t b_base = ptx::smem_u32(sb + stage * kBBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t adesc = ptx::make_smem_desc(a_base + k * p.a_kstep, p.a_lbo, p.a_sbo);
            const uint64_t bdesc = ptx::make_smem_desc(b_base + k * p.b_kstep, p.b_lbo, p.b_sbo);
            if (PAIR) ptx::mma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else ptx::mma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          // frees the smem stage (of both CTAs of a pair) once these MMAs retire
          if (PAIR) ptx::tc_commit_pair(&empty[stage], 3);
          else ptx::tc_commit(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          if (PAIR) ptx::tc_commit_pair(&acc_full[buf], 3);
          else ptx::tc_commit(&acc_full[buf]);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    // the accumulator buffer has been read: the MMA warp (of rank 0 in a pair) may reuse it
    auto release_acc = [&](int b) {
      if (PAIR) ptx::mbar_arrive_cluster(&acc_empty[b], 0);
      else ptx::mbar_arrive(&acc_empty[b]);
    };
    if (p.coll.mode == 2) {
      // GEMM -> reduce-scatter: the bf16 partial tile goes to slot [this rank] of the receive buffer of the rank that
      // owns its rows.  64 columns at a time are staged in shared memory (two tiles, alternating) and copied out so
      // that eight neighbouring lanes write one whole 128-byte row segment -- full NVLink write packets instead of one
      // 16-byte piece per thread and row.  One release per tile tells the owner that the partial has been written.
      const int trow = quad * 32 + lane;
      const int tid = threadIdx.x - 64;                 // 0 .. 127 among the epilogue threads
      const int crow = tid >> 3, cunit = tid & 7;       // copy-out: row within a group of 16, 16-byte unit of the row
      for (int rnd = walk.first_round(), tile; (tile = walk.tile(rnd)) < num_tiles; ++rnd, ++it) {
        const TileCoord tc = tile_coord(p, tile, tiles_m, tiles_n, BN, kTileM, row_off);
        const int m0 = tc.m0, n0 = tc.n0;
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!ptx::mbar_wait(&acc_full[buf], acc_phase, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * Cfg::kAccStride;
        const int owner = m0 / p.coll.rows_per_rank;
        const long long lrow0 = m0 - static_cast<long long>(owner) * p.coll.rows_per_rank;
        bf16* slot = static_cast<bf16*>(p.coll.peers[owner]) +
                     (static_cast<long long>(p.coll.rank) * p.coll.rows_per_rank + lrow0) * p.N;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col0 = n0 + c * 64;
          const bool last = (c == BN / 64 - 1);
          if (col0 < p.N) {
            uint32_t r0[32], r1[32];
            ptx::tmem_ld32(t_row + c * 64, r0);
            ptx::tmem_ld32(t_row + c * 64 + 32, r1);
            ptx::tmem_ld_wait();
            uint8_t* stg = (c & 1) ? stage_aux : stage_out;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const uint32_t* r = u < 4 ? r0 : r1;
              const int o = (u & 3) * 8;
              *reinterpret_cast<uint4*>(stg + trow * 128 + ((u ^ (trow & 7)) << 4)) = make_uint4(
                  pack_bf16x2(__uint_as_float(r[o]), __uint_as_float(r[o + 1])),
                  pack_bf16x2(__uint_as_float(r[o + 2]), __uint_as_float(r[o + 3])),
                  pack_bf16x2(__uint_as_float(r[o + 4]), __uint_as_float(r[o + 5])),
                  pack_bf16x2(__uint_as_float(r[o + 6]), __uint_as_float(r[o + 7])));
            }
          }
          if (last) {  // accumulator fully read: the MMA warp may reuse this TMEM buffer
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) release_acc(buf);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (col0 < p.N && col0 + cunit * 8 < p.N) {
            const uint8_t* stg = (c & 1) ? stage_aux : stage_out;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const int row = g * 16 + crow;
              if (m0 + row < p.M)
                *reinterpret_cast<uint4*>(slot + static_cast<long long>(row) * p.N + col0 + cunit * 8) =
                    *reinterpret_cast<const uint4*>(stg + row * 128 + ((cunit ^ (row & 7)) << 4));
            }
          }
        }
        // every thread's stores of this tile happen before the barrier, the barrier before the release below: one
        // system-scope release by one thread publishes the whole tile (a fence per thread cost 128 membar.sys a tile)
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tid == 0) {
          const int chunk = static_cast<int>(lrow0 / kBM);
          red_release_sys_add_u32(static_cast<uint32_t*>(p.coll.cnt_peers[owner]) + chunk, 1u);
        }
      }
      rs_reduce_phase(p, tiles_n, cta, ncta, tid);
    } else if (p.tma_store == 2) {
      // fp32 outputs (weight gradients): 32 columns at a time -> registers -> swizzled shared-memory tile -> one TMA
      // store, or one TMA reduce-add when the tile is a split-K partial or accumulates into the output.  The two
      // staging tiles alternate, so the copy of chunk c overlaps the staging of chunk c + 1.
      const int trow = quad * 32 + lane;
      const bool elected = (warp == 2 && lane == 0);
      int gchunk = 0;
      for (int rnd = walk.first_round(), tile; (tile = walk.tile(rnd)) < num_tiles; ++rnd, ++it) {
        const TileCoord tc = tile_coord(p, tile, tiles_m, tiles_n, BN, kTileM, row_off);
        const int m0 = tc.m0, n0 = tc.n0;
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!ptx::mbar_wait(&acc_full[buf], acc_phase, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * Cfg::kAccStride;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          const bool last = (c == BN / 32 - 1);
          if (col0 >= p.N) {  // whole chunk is padding
            if (last) {
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) release_acc(buf);
            }
            continue;
          }
          uint32_t r[32];
          ptx::tmem_ld32(t_row + c * 32, r);
          ptx::tmem_ld_wait();
          if (last) {  // accumulator fully read: the MMA warp may reuse this TMEM buffer
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) release_acc(buf);
          }
          if (p.alpha != nullptr) {
            const float al = *p.alpha;
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * al);
          }
          uint8_t* stg = (gchunk & 1) ? stage_aux : stage_out;
          // the copy issued two chunks ago has finished reading this staging tile
          if (elected) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
          for (int u = 0; u < 8; ++u)
            *reinterpret_cast<uint4*>(stg + trow * 128 + ((u ^ (trow & 7)) << 4)) =
                make_uint4(r[u * 4], r[u * 4 + 1], r[u * 4 + 2], r[u * 4 + 3]);
          ptx::fence_proxy_async_smem();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (elected) {
            if (p.f32_red)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                               reinterpret_cast<uint64_t>(&tma_out)),
                           "r"(ptx::smem_u32(stg)), "r"(col0), "r"(m0)
                           : "memory");
            else
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                               reinterpret_cast<uint64_t>(&tma_out)),
                           "r"(ptx::smem_u32(stg)), "r"(col0), "r"(m0)
                           : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          ++gchunk;
        }
      }
      if (elected) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all copies done before the CTA exits
    } else if (p.tma_store) {
      // bf16 outputs: 64 columns at a time -> registers -> swizzled shared-memory tile -> one TMA
      // store per tile chunk (full 128-byte lines instead of one 16-byte piece per thread and row).
      const int trow = quad * 32 + lane;
      const bool elected = (warp == 2 && lane == 0);
      // Residual / pre-activation tiles are fetched one chunk ahead by TMA into the aux staging tile.
      constexpr int kChunksPerTile = BN / 64;
      const int my_tiles = cta < num_tiles ? (num_tiles - cta + ncta - 1) / ncta : 0;
      const int total_chunks = my_tiles * kChunksPerTile;
      auto issue_aux_load = [&](int g) {  // g: running chunk index over this CTA's tiles
        const int t_local = g / kChunksPerTile;
        const TileCoord t2 = tile_coord(p, cta + t_local * ncta, tiles_m, tiles_n, BN, kTileM, row_off);
        ptx::mbar_expect_tx(aux_bar, kBM * 128);
        ptx::tma_load_2d(stage_aux, &tma_aux, aux_bar, t2.n0 + (g % kChunksPerTile) * 64, t2.m0);
      };
      int gchunk = 0;
      if (p.aux_tma_load && elected && total_chunks > 0) issue_aux_load(0);
      for (int rnd = walk.first_round(), tile; (tile = walk.tile(rnd)) < num_tiles; ++rnd, ++it) {
        const TileCoord tc = tile_coord(p, tile, tiles_m, tiles_n, BN, kTileM, row_off);
        const int m0 = tc.m0, n0 = tc.n0;
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!ptx::mbar_wait(&acc_full[buf], acc_phase, abort_flag)) break;
        ptx::tc_fence_after_sync();
        const long long row = m0 + trow;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * Cfg::kAccStride;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col0 = n0 + c * 64;
          uint4 aux_row[8];
          if (p.aux_tma_load) {
            // chunk `gchunk` of the aux operand has landed; copy this thread's row out and prefetch the next
            const bool got = ptx::mbar_wait(aux_bar, gchunk & 1, abort_flag);
            if (got) {
#pragma unroll
              for (int u = 0; u < 8; ++u)
                aux_row[u] = *reinterpret_cast<const uint4*>(stage_aux + trow * 128 + ((u ^ (trow & 7)) << 4));
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            ++gchunk;
            if (elected && gchunk < total_chunks) issue_aux_load(gchunk);
          }
          if (col0 >= p.N) {  // whole chunk is padding: nothing to read or store, but keep the barriers in step
            if (c == BN / 64 - 1) {
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) release_acc(buf);
            }
            continue;
          }
          uint32_t r0[32], r1[32];
          ptx::tmem_ld32(t_row + c * 64, r0);
          ptx::tmem_ld32(t_row + c * 64 + 32, r1);
          ptx::tmem_ld_wait();
          if (c == BN / 64 - 1) {  // accumulator fully read: the MMA warp may reuse this TMEM buffer
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) release_acc(buf);
          }
          float v[64];
#pragma unroll
          for (int j = 0; j < 32; ++j) { v[j] = __uint_as_float(r0[j]); v[32 + j] = __uint_as_float(r1[j]); }
          if (p.alpha != nullptr) {
            const float al = *p.alpha;
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] *= al;
          }
          const bool full_cols = (col0 + 64 <= p.N);
          if (p.bias != nullptr && (p.epi == TITB_EPI_BIAS || p.epi == TITB_EPI_BIAS_GELU || p.epi == TITB_EPI_BIAS_RESIDUAL)) {
            if (full_cols) {
#pragma unroll
              for (int j = 0; j < 64; j += 8) {
                const uint4 u = *reinterpret_cast<const uint4*>(p.bias + col0 + j);
                const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
                v[j] += f0.x; v[j + 1] += f0.y; v[j + 2] += f1.x; v[j + 3] += f1.y;
                v[j + 4] += f2.x; v[j + 5] += f2.y; v[j + 6] += f3.x; v[j + 7] += f3.y;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 64; ++j) if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
            }
          }
          uint32_t aux_pk[32];
          if (p.epi == TITB_EPI_BIAS_GELU) {
#pragma unroll
            for (int j = 0; j < 64; j += 2) {
              aux_pk[j >> 1] = pack_bf16x2(v[j], v[j + 1]);
              const float2 pr = unpack_bf16x2(aux_pk[j >> 1]);  // activation of the stored (rounded) pre-activation
              v[j] = gelu_fast(pr.x);
              v[j + 1] = gelu_fast(pr.y);
            }
          } else if (p.aux_tma_load) {
            // out-of-range rows / columns of the aux tile were zero-filled by the TMA load
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const float2 f0 = unpack_bf16x2(aux_row[u].x), f1 = unpack_bf16x2(aux_row[u].y), f2 = unpack_bf16x2(aux_row[u].z),
                           f3 = unpack_bf16x2(aux_row[u].w);
              const float a8[8] = {f0.x, f0.y, f1.x, f1.y, f2.x, f2.y, f3.x, f3.y};
#pragma unroll
              for (int e = 0; e < 8; ++e)
                v[u * 8 + e] = (p.epi == TITB_EPI_DGELU) ? v[u * 8 + e] * gelu_grad_fast(a8[e]) : v[u * 8 + e] + a8[e];
            }
          } else if ((p.epi == TITB_EPI_DGELU || p.epi == TITB_EPI_BIAS_RESIDUAL) && p.aux_in != nullptr && row < p.M) {
            const bf16* ai = p.aux_in + row * p.ld_aux_in + col0;
            if (full_cols) {
#pragma unroll
              for (int j = 0; j < 64; j += 8) {
                const uint4 u = *reinterpret_cast<const uint4*>(ai + j);
                const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
                const float a8[8] = {f0.x, f0.y, f1.x, f1.y, f2.x, f2.y, f3.x, f3.y};
#pragma unroll
                for (int e = 0; e < 8; ++e) v[j + e] = (p.epi == TITB_EPI_DGELU) ? v[j + e] * gelu_grad_fast(a8[e]) : v[j + e] + a8[e];
              }
            } else {
#pragma unroll
              for (int j = 0; j < 64; ++j) {
                if (col0 + j < p.N) {
                  const float a1 = __bfloat162float(ai[j]);
                  v[j] = (p.epi == TITB_EPI_DGELU) ? v[j] * gelu_grad_fast(a1) : v[j] + a1;
                }
              }
            }
          }
          // the previous chunk's TMA store must have finished reading the staging tiles
          if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint32_t off = static_cast<uint32_t>(trow * 128 + ((u ^ (trow & 7)) << 4));
            *reinterpret_cast<uint4*>(stage_out + off) =
                make_uint4(pack_bf16x2(v[u * 8], v[u * 8 + 1]), pack_bf16x2(v[u * 8 + 2], v[u * 8 + 3]),
                           pack_bf16x2(v[u * 8 + 4], v[u * 8 + 5]), pack_bf16x2(v[u * 8 + 6], v[u * 8 + 7]));
            if (p.epi == TITB_EPI_BIAS_GELU && p.aux_out != nullptr)
              *reinterpret_cast<uint4*>(stage_aux + off) =
                  make_uint4(aux_pk[u * 4], aux_pk[u * 4 + 1], aux_pk[u * 4 + 2], aux_pk[u * 4 + 3]);
          }
          ptx::fence_proxy_async_smem();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (elected) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                             reinterpret_cast<uint64_t>(&tma_out)),
                         "r"(ptx::smem_u32(stage_out)), "r"(col0), "r"(m0)
                         : "memory");
            if (p.epi == TITB_EPI_BIAS_GELU && p.aux_out != nullptr)
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                               reinterpret_cast<uint64_t>(&tma_aux)),
                           "r"(ptx::smem_u32(stage_aux)), "r"(col0), "r"(m0)
                           : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      }
      if (elected) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all stores done before the CTA exits
    } else
    for (int rnd = walk.first_round(), tile; (tile = walk.tile(rnd)) < num_tiles; ++rnd, ++it) {
      const TileCoord tc = tile_coord(p, tile, tiles_m, tiles_n, BN, kTileM, row_off);
      const int split = tc.split, m0 = tc.m0, n0 = tc.n0;
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!ptx::mbar_wait(&acc_full[buf], acc_phase, abort_flag)) break;
      ptx::tc_fence_after_sync();
      const long long row = m0 + quad * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * Cfg::kAccStride;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld32(t_row + c * 32, r);
        ptx::tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          epilogue_row32(p, v, row, col0, split);
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) release_acc(buf);
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (PAIR) ptx::cluster_sync_all();   // neither CTA leaves while the other may still signal its barriers
  if (warp == 1) {
    __syncwarp();
    if (PAIR) ptx::tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    else ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, kStatusMbarTimeout);
}

// out (+)= sum_s ws[s] ; ws is fp32 [splits, M*N] with N contiguous, out has row stride ldo.
template <typename OutT>
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, OutT* __restrict__ out, long long M, int N,
                                     long long ldo, int splits, int accumulate, const float* __restrict__ alpha) {
  const long long total = M * N;
  const float al = alpha ? *alpha : 1.f;
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < total;
       i += (long long)gridDim.x * blockDim.x * 4) {
    // N % 4 == 0 is enforced by the host, so a group of 4 never straddles a row.
    float4 acc = *reinterpret_cast<const float4*>(ws + i);
    for (int s = 1; s < splits; ++s) {
      float4 t = *reinterpret_cast<const float4*>(ws + s * total + i);
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
    acc.x *= al; acc.y *= al; acc.z *= al; acc.w *= al;
    const long long r = i / N;
    const int c = static_cast<int>(i - r * N);
    OutT* o = out + r * ldo + c;
    if (accumulate) {
      acc.x += to_f32(o[0]); acc.y += to_f32(o[1]); acc.z += to_f32(o[2]); acc.w += to_f32(o[3]);
    }
    o[0] = from_f32<OutT>(acc.x); o[1] = from_f32<OutT>(acc.y);
    o[2] = from_f32<OutT>(acc.z); o[3] = from_f32<OutT>(acc.w);
  }
}

// ------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// bf16 matrix stored [outer, inner] with `ld` elements between rows; box = box_inner x box_outer.
bool make_tmap_bf16_2d(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                       uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  // The encoder is a driver-API entry point and needs a current context.  A thread that has made
  // no runtime call yet (e.g. a fresh autograd worker thread) has none bound: bind the device's
  // primary context once per thread through the runtime.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    static int reported = 0;
    if (reported++ < 4)
      fprintf(stderr, "titb200: cuTensorMapEncodeTiled failed (CUresult %d): base=%p inner=%llu outer=%llu ld=%llu box=%ux%u\n",
              static_cast<int>(r), base, static_cast<unsigned long long>(inner), static_cast<unsigned long long>(outer),
              static_cast<unsigned long long>(ld), box_inner, box_outer);
  }
  return r == CUDA_SUCCESS;
}

// fp32 matrix stored [outer, inner] with `ld` elements between rows; box = box_inner x box_outer (128-byte rows).
bool make_tmap_f32_2d(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  static thread_local bool ctx_bound = false;   // see make_tmap_bf16_2d
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 4};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int g_no_tma_store = 0;  // set by titb_gemm_set_tma_store(0): A/B switch for the epilogue store path

// Estimated duration of a GEMM for a tile width and a split-K factor, in units of one k-block (64 deep) of a
// lightly loaded SM (about 0.4 us, measured: the same for 128-, 192- and 256-wide tiles when few CTAs run).  When
// most SMs are busy the operand traffic out of L2 sets the pace and a k-block costs more, in proportion to the
// bytes it loads ((128 + BN) x 64 x 2): about 1.7 units for a 128 x 256 tile on a full machine.  The epilogue of
// the last tile of a CTA is exposed (earlier ones overlap the next main loop); a split adds the zero fill of the
// output and the contention of the partial tiles' reduce-adds.
static double plan_cost(int M, int N, int K, int bn, int splits, int sms) {
  const long long tm = (M + kBM - 1) / kBM, tn = (N + bn - 1) / bn;
  const int kb = (K + kBK - 1) / kBK;
  const int kb_per = (kb + splits - 1) / splits;
  const int s = (kb + kb_per - 1) / kb_per;
  const long long tiles = tm * tn * s;
  const long long waves = (tiles + sms - 1) / sms;
  const double load = tiles >= sms ? 1.0 : (double)tiles / sms;
  const double c_kb = 1.0 + 0.7 * load * (128.0 + bn) / 384.0;
  double cost = waves * (double)(kb_per > 3 ? kb_per : 3) * c_kb + 3.0 * bn / 256.0;
  if (s > 1) cost += 4.0 + 0.5 * s;
  return cost;
}

static int pick_tile_n(int M, int N, int K, int splits) {
  // 128 x 256 tiles move the fewest operand bytes per FLOP; 192 and 128 win when they fill the last wave better
  // (widths such as 768 and 3072 = 6 x 128).  A narrower tile must save more than 5% to be taken.
  if (N <= 128) return 128;
  const int sms = device_sm_count();
  const double c256 = plan_cost(M, N, K, 256, splits, sms), c192 = plan_cost(M, N, K, 192, splits, sms),
               c128 = plan_cost(M, N, K, 128, splits, sms);
  int bn = 256;
  double best = c256;
  if (c192 < best * 0.95) { bn = 192; best = c192; }
  if (c128 < best * 0.95 && c128 < c256 * 0.95) { bn = 128; best = c128; }
  return bn;
}

}  // namespace titb

using namespace titb;

#ifndef TITB_GEMM_PARAM_GATHER
static int* g_status_dev[64] = {nullptr};

TITB_API int* titb_status_ptr(void) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!g_status_dev[dev]) {
    if (cudaMalloc(&g_status_dev[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(g_status_dev[dev], 0, sizeof(int));
  }
  return g_status_dev[dev];
}

TITB_API int titb_status_read(int clear, cudaStream_t stream) {
  int* p = titb_status_ptr();
  if (!p) return -1;
  int h = 0;
  if (cudaMemcpyAsync(&h, p, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
  if (clear && h != 0) cudaMemsetAsync(p, 0, sizeof(int), stream);
  return h;
}

TITB_API void titb_gemm_set_tma_store(int enabled) { g_no_tma_store = enabled ? 0 : 1; }

TITB_API int titb_gemm_pick_tile(int M, int N, int K, int splits) { return pick_tile_n(M, N, K, splits < 1 ? 1 : splits); }

TITB_API int titb_gemm_pick_splits(int M, int N, int K) {
  // Joint choice of split-K factor and tile width by estimated duration (plan_cost): the reduction is split when the
  // output has too few tiles to fill the GPU -- weight gradients: small outputs, K = the token count -- and each
  // split still runs a pipeline of at least 8 k-blocks.  (Callers use the result only where the partial tiles can
  // be summed: fp32 outputs without a fused epilogue.)
  const int sms = device_sm_count();
  const int kb = (K + kBK - 1) / kBK;
  int best_s = 1;
  double best = 1e30;
  for (int s = 1; s <= 16; ++s) {
    if (s > 1 && kb / s < 8) break;
    for (int bn : {256, 192, 128}) {
      if (bn > 128 && N <= 128) continue;
      const double c = plan_cost(M, N, K, bn, s, sms);
      if (c < best * (s > best_s ? 0.97 : 1.0)) { best = c; best_s = s; }   // a deeper split must pay for itself
    }
  }
  return best_s;
}
#endif  // !TITB_GEMM_PARAM_GATHER

static bool deterministic_reductions() {
  static const bool det = [] { const char* e = getenv("TITB200_DETERMINISTIC"); return e && e[0] == '1'; }();
  return det;
}
// 3-D view of an MN-major bf16 matrix [k rows, mn columns] (mn a multiple of 64): dims (64, k, mn / 64), so that a box of
// (64, box_k, chunks) covers `chunks` neighbouring 64-column chunks of box_k rows.
static bool make_tmap_bf16_mn3d(CUtensorMap* m, const void* base, uint64_t mn, uint64_t k, uint64_t ld, uint32_t box_k,
                                uint32_t chunks) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || (mn & 63) || chunks < 1 || chunks > 256) return false;
  static thread_local bool ctx_bound = false;   // see make_tmap_bf16_2d
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[3] = {64, k, mn / 64};
  cuuint64_t strides[2] = {ld * 2, 128};
  cuuint32_t box[3] = {64, box_k, chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool f32_tma_eligible(const TitbGemmDesc* d) {
  return d->out_fp32 && d->epilogue == TITB_EPI_NONE && (d->coll == nullptr || d->coll->mode == 0) &&
         !(reinterpret_cast<uintptr_t>(d->out) & 15) && !(d->ldo & 3) && g_no_tma_store == 0;
}

constexpr double kTflopsPerSm = 10.8;   // bf16 tensor throughput of one SM at the sustained clock (1.6 PFLOP/s / 148)

template <int BN, bool PAIR>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tout, const CUtensorMap& taux,
                       const GemmArgs& args, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, PAIR>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  const int tiles = ((args.M + Cfg::kTileM - 1) / Cfg::kTileM) * ((args.N + BN - 1) / BN) * args.splits;
  if (PAIR) {
    // clusters of two CTAs, one pair per tile in flight; the pair count is capped at half the SMs
    if (args.coll.mode) return TITB_ERR_SHAPE;
    int pairs = device_sm_count() / 2;
    if (tiles < pairs) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = Cfg::kSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_tcgen05_kernel<BN, PAIR>, ta, tb, tout, taux, args);
    return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
  }
  const int sms = device_sm_count();
  if (args.coll.mode == 1 || args.coll.mode == 3) {
    // All-gather -> GEMM (of activation rows, or of weight rows in mode 3): how many CTAs copy, and for how many rounds
    // of the tile list they are excused.  The copy has to stay ahead of the GEMM CTAs, which reach the first remote rows
    // after 1 / world of the tiles; the model below (microseconds of one CTA) errs on the side of more helpers, which
    // cost little because they join the GEMM afterwards.  A copying CTA moves about 35 GB/s of local memory (measured)
    // and less from a peer; the owner's rows of a gathered weight are already in place.
    GemmArgs a2 = args;
    const double t_tile = 2.0 * kBM * BN * args.K / (kTflopsPerSm * 1e6);
    const double shard = 2.0 * args.K * args.coll.rows_per_rank;
    const double remote = shard * (args.coll.world - 1), local = args.coll.mode == 1 ? shard : 0.0;
    const double w_copy = remote / 15e3 + local / 35e3;                  // CTA-microseconds
    const double t_total = (tiles * t_tile + w_copy) / sms;
    int H = args.coll.helper_ctas;
    if (H <= 0) {
      const double window = t_total * (args.coll.world > 1 ? 1.0 - 1.0 / args.coll.world : 1.0);
      H = static_cast<int>(1.5 * w_copy / (window > 1.0 ? window : 1.0)) + 1;
      if (H < 8) H = 8;
      if (H > 64) H = 64;                                                // the link is full long before that
    }
    if (H > sms / 2) H = sms / 2;
    int grid = tiles + H < sms ? tiles + H : sms;
    if (grid <= H) return TITB_ERR_SHAPE;
    int rounds = static_cast<int>(w_copy / H / t_tile + 0.999);
    a2.coll.helper_ctas = H;
    a2.coll.helper_rounds = rounds < 1 ? 1 : rounds;
    gemm_bf16_tcgen05_kernel<BN, PAIR><<<grid, kGemmThreads, Cfg::kSmem, stream>>>(ta, tb, tout, taux, a2);
    return static_cast<int>(cudaGetLastError());
  }
  int grid = tiles < sms ? tiles : sms;
  gemm_bf16_tcgen05_kernel<BN, PAIR><<<grid, kGemmThreads, Cfg::kSmem, stream>>>(ta, tb, tout, taux, args);
  return static_cast<int>(cudaGetLastError());
}

#ifndef TITB_GEMM_PARAM_GATHER
TITB_API int titb_gemm_split_in_place(const TitbGemmDesc* d) { return (f32_tma_eligible(d) && !deterministic_reductions()) ? 1 : 0; }
#endif

TITB_API int TITB_GEMM_ENTRY(const TitbGemmDesc* d, cudaStream_t stream) {
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return 0;
  (void)cudaGetLastError();  // do not report an error left behind by an earlier, unrelated call
  // TMA needs 16-byte aligned bases and row strides.
  if ((reinterpret_cast<uintptr_t>(d->a) & 15) || (reinterpret_cast<uintptr_t>(d->b) & 15) || (d->lda & 7) ||
      (d->ldb & 7))
    return TITB_ERR_ALIGNMENT;
  int splits = d->splits < 1 ? 1 : d->splits;
  const int num_kb = (d->K + kBK - 1) / kBK;
  if (splits > num_kb) splits = num_kb;
  // fp32 results without a fused epilogue (weight gradients) leave through shared-memory staging and TMA: a plain
  // store, or a reduce-add when the tile accumulates into the output or is one of several split-K partials -- the
  // partial tiles then meet in the output itself (added in L2), with no workspace and no second kernel.  The order
  // of those additions is not fixed for three or more partials; TITB200_DETERMINISTIC=1 keeps the fixed-order
  // workspace + reduction kernel instead.
  const bool f32_tma_ok = f32_tma_eligible(d);
  const bool red_split = f32_tma_ok && !deterministic_reductions();
  if (splits > 1 && !red_split && (d->workspace == nullptr || (d->N & 3))) splits = 1;
  // tile_n = 512 asks for CTA pairs on 256 x 256 tiles (cta_group::2); 128 / 192 / 256 are single-CTA 128 x tile_n
  int bn = d->tile_n ? d->tile_n : pick_tile_n(d->M, d->N, d->K, splits);
  // CTA pairs for long reductions over an MN-major B operand (weight gradients, and dgrads with a wide output): a pair
  // stages half of the B tile per CTA.  Measured on the GPT-2 and LLaMA-3 1B layer shapes: up to 16 % faster from 2048
  // reduction elements per split on, slower below that and on 768-wide dgrad outputs.
  if (d->tile_n == 0 && d->b_mn_major && (d->coll == nullptr || d->coll->mode == 0) && d->M >= 2 * kBM && d->N >= 256 &&
      (num_kb + splits - 1) / splits >= 32 && (d->a_mn_major || d->N >= 1024))
    bn = 512;
  bool pair = false;
  if (bn == 512) {
    pair = (d->coll == nullptr || d->coll->mode == 0) && d->M > kBM && d->N > 128;
    bn = 256;
  }

  CUtensorMap ta, tb;
  bool ok;
  // MN-major operands whose extent is a multiple of 64 are fetched as one 3-D box per k-block; the 2-D map with one
  // box per 64-column chunk covers ragged extents
  bool a_box3 = false, b_box3 = false;
  if (!d->a_mn_major) {
    ok = make_tmap_bf16_2d(&ta, d->a, d->K, d->M, d->lda, kBK, kBM);
  } else {
    a_box3 = (d->M & 63) == 0 && make_tmap_bf16_mn3d(&ta, d->a, d->M, d->K, d->lda, kBK, kBM / 64);
    ok = a_box3 || make_tmap_bf16_2d(&ta, d->a, d->M, d->K, d->lda, 64, kBK);
  }
  if (!d->b_mn_major) {
    ok = ok && make_tmap_bf16_2d(&tb, d->b, d->K, d->N, d->ldb, kBK, pair ? bn / 2 : bn);
  } else {
    b_box3 = (d->N & 63) == 0 && make_tmap_bf16_mn3d(&tb, d->b, d->N, d->K, d->ldb, kBK, (pair ? bn / 2 : bn) / 64);
    ok = ok && (b_box3 || make_tmap_bf16_2d(&tb, d->b, d->N, d->K, d->ldb, 64, kBK));
  }
  if (!ok) return TITB_ERR_TENSOR_MAP;

  GemmArgs a{};
  a.M = d->M; a.N = d->N; a.K = d->K;
  a.a_mn = d->a_mn_major ? 1 : 0;
  a.b_mn = d->b_mn_major ? 1 : 0;
  a.a_box3 = a_box3 ? 1 : 0; a.b_box3 = b_box3 ? 1 : 0;
  a.out = (splits > 1 && !red_split) ? d->workspace : d->out;
  a.ldo = d->ldo;
  a.out_fp32 = d->out_fp32; a.accumulate = d->accumulate; a.epi = d->epilogue;
  a.bias = static_cast<const bf16*>(d->bias);
  a.aux_in = static_cast<const bf16*>(d->aux_in); a.ld_aux_in = d->ld_aux_in;
  a.aux_out = static_cast<bf16*>(d->aux_out); a.ld_aux_out = d->ld_aux_out;
  a.kb_per_split = (num_kb + splits - 1) / splits;
  splits = (num_kb + a.kb_per_split - 1) / a.kb_per_split;  // no empty trailing split
  a.splits = splits;
  const int out_vec = d->out_fp32 ? 3 : 7;
  a.vec_ok = !((d->ldo & out_vec) || (reinterpret_cast<uintptr_t>(d->out) & 15) ||
               (d->bias && (reinterpret_cast<uintptr_t>(d->bias) & 15)) ||
               (d->aux_in && ((reinterpret_cast<uintptr_t>(d->aux_in) & 15) || (d->ld_aux_in & 7))) ||
               (d->aux_out && ((reinterpret_cast<uintptr_t>(d->aux_out) & 15) || (d->ld_aux_out & 7))));
  // K-major: 32 bytes per 16-wide k step inside the 128-byte row, 8-row groups 1024 bytes apart.
  // MN-major: 16 k-rows of 128 bytes per step, 64-wide chunks one TMA box (64 x kBK) apart.
  const uint32_t mn_lbo = 64 * kBK * 2, mn_sbo = 1024, mn_kstep = 16 * 128;
  a.a_lbo = a.a_mn ? mn_lbo : 16; a.a_sbo = a.a_mn ? mn_sbo : 1024; a.a_kstep = a.a_mn ? mn_kstep : 32;
  a.b_lbo = a.b_mn ? mn_lbo : 16; a.b_sbo = a.b_mn ? mn_sbo : 1024; a.b_kstep = a.b_mn ? mn_kstep : 32;
  a.alpha = static_cast<const float*>(d->alpha);
  a.status = titb_status_ptr();
  if (!a.status) return static_cast<int>(cudaErrorMemoryAllocation);
  if (d->coll != nullptr && d->coll->mode != 0) {
    const TitbGemmColl* c = d->coll;
#ifdef TITB_GEMM_PARAM_GATHER
    if (c->mode != 3) return TITB_ERR_SHAPE;   // this copy of the kernel serves the parameter gather only
    if (c->world < 1 || c->world > 16 || c->rows_per_rank % kBM || d->N != c->rows_per_rank * c->world || splits != 1 ||
        (d->K & 7) || d->b_mn_major || d->ldb != d->K || d->b != c->gathered || (bn != 128 && bn != 256))   // helper_ctas <= 0: the launcher chooses
      return TITB_ERR_SHAPE;
#else
    if (c->world < 1 || c->world > 16 || c->rows_per_rank % kBM || d->M != c->rows_per_rank * c->world || splits != 1 ||
        (d->N & 7) || (d->K & 7))   // mode 1: helper_ctas <= 0 lets the launcher choose
      return TITB_ERR_SHAPE;
#endif
    if (c->mode == 2 && (d->epilogue != TITB_EPI_NONE || d->accumulate || d->alpha)) return TITB_ERR_SHAPE;
    a.coll.mode = c->mode; a.coll.world = c->world; a.coll.rank = c->rank;
    a.coll.helper_ctas = c->helper_ctas; a.coll.rows_per_rank = c->rows_per_rank;
    for (int i = 0; i < c->world; ++i) {
      a.coll.peers[i] = reinterpret_cast<void*>(c->peer_ptrs[i]);
      a.coll.cnt_peers[i] = c->cnt_ptrs ? reinterpret_cast<void*>(c->cnt_ptrs[i]) : nullptr;
    }
    a.coll.gathered = static_cast<bf16*>(c->gathered);
    a.coll.flags = static_cast<uint32_t*>(c->flags);
    a.coll.rs_out = static_cast<bf16*>(c->rs_out);
    a.coll.rs_bias = static_cast<const bf16*>(c->rs_bias);
    a.coll.rs_residual = static_cast<const bf16*>(c->rs_residual);
    if (c->mode == 1) {
      // chunk flags start at 0 for every launch (stream-ordered, capturable)
      cudaError_t e = cudaMemsetAsync(c->flags, 0, sizeof(uint32_t) * (d->M / kBM), stream);
      if (e != cudaSuccess) return static_cast<int>(e);
    }
#ifdef TITB_GEMM_PARAM_GATHER
    if (c->mode == 3) {
      cudaError_t e = cudaMemsetAsync(c->flags, 0, sizeof(uint32_t) * (d->N / kBM), stream);
      if (e != cudaSuccess) return static_cast<int>(e);
    }
#endif
  }

  // bf16 results (and the GELU pre-activation) leave through TMA stores when their layout allows it
  CUtensorMap tout = ta, taux = ta;  // placeholders when unused
  const bool out_tma_ok = !d->out_fp32 && !d->accumulate && splits == 1 && a.coll.mode != 2 &&
                          !(reinterpret_cast<uintptr_t>(d->out) & 15) && !(d->ldo & 7) &&
                          (!d->aux_out || (!(reinterpret_cast<uintptr_t>(d->aux_out) & 15) && !(d->ld_aux_out & 7))) &&
                          (!d->aux_in || a.vec_ok) && (!d->bias || a.vec_ok) && g_no_tma_store == 0;
  if (out_tma_ok) {
    bool okm = make_tmap_bf16_2d(&tout, d->out, d->N, d->M, d->ldo, 64, kBM);
    if (okm && d->aux_out) okm = make_tmap_bf16_2d(&taux, d->aux_out, d->N, d->M, d->ld_aux_out, 64, kBM);
    a.tma_store = okm ? 1 : 0;
    if (okm && !d->aux_out && d->aux_in && (d->epilogue == TITB_EPI_DGELU || d->epilogue == TITB_EPI_BIAS_RESIDUAL) &&
        !(reinterpret_cast<uintptr_t>(d->aux_in) & 15) && !(d->ld_aux_in & 7))
      a.aux_tma_load = make_tmap_bf16_2d(&taux, d->aux_in, d->N, d->M, d->ld_aux_in, 64, kBM) ? 1 : 0;
  }
  if (f32_tma_ok && (splits == 1 || red_split)) {
    if (make_tmap_f32_2d(&tout, d->out, d->N, d->M, d->ldo, 32, kBM)) {
      a.tma_store = 2;
      a.f32_red = (splits > 1 || d->accumulate) ? 1 : 0;
      if (splits > 1 && !d->accumulate) {   // the partial tiles are added to zeros
        cudaError_t e = cudaMemset2DAsync(d->out, static_cast<size_t>(d->ldo) * 4, 0, static_cast<size_t>(d->N) * 4, d->M, stream);
        if (e != cudaSuccess) return static_cast<int>(e);
      }
    } else if (splits > 1 && red_split) {
      return TITB_ERR_TENSOR_MAP;
    }
  }
  if (bn != 128 && bn != 192 && bn != 256) return TITB_ERR_SHAPE;
  int rc = pair          ? launch_gemm<256, true>(ta, tb, tout, taux, a, stream)
           : (bn == 256) ? launch_gemm<256, false>(ta, tb, tout, taux, a, stream)
           : (bn == 192) ? launch_gemm<192, false>(ta, tb, tout, taux, a, stream)
                         : launch_gemm<128, false>(ta, tb, tout, taux, a, stream);
  if (rc != 0) return rc;
  if (a.coll.mode == 2) {
    // every partial of this call has been counted when the kernel ends; the counters start the next call at zero
    // (peers send that call's tiles only after a cross-GPU barrier that follows this memset in stream order)
    cudaError_t e = cudaMemsetAsync(a.coll.flags, 0, sizeof(uint32_t) * (a.coll.rows_per_rank / kBM), stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  if (splits > 1 && a.tma_store != 2) {
    const long long total = static_cast<long long>(d->M) * d->N;
    int blocks = static_cast<int>((total / 4 + 255) / 256);
    if (blocks > device_sm_count() * 8) blocks = device_sm_count() * 8;
    if (d->out_fp32)
      splitk_reduce_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(d->workspace),
                                                               static_cast<float*>(d->out), d->M, d->N, d->ldo,
                                                               splits, d->accumulate, static_cast<const float*>(d->alpha));
    else
      splitk_reduce_kernel<bf16><<<blocks, 256, 0, stream>>>(static_cast<const float*>(d->workspace),
                                                              static_cast<bf16*>(d->out), d->M, d->N, d->ldo, splits,
                                                              d->accumulate, static_cast<const float*>(d->alpha));
    rc = static_cast<int>(cudaGetLastError());
  }
  return rc;
}

#ifndef TITB_GEMM_PARAM_GATHER
// ------------------------------------------------------------- fp32 SIMT GEMM
// Kept for fp32 tensors on the GPU (API parity with the reference's fp32-only
// Matmul/Linear); not a hot path.  64x64 tile, 16-deep k slab, 4x4 per thread.
namespace titb {
__global__ void __launch_bounds__(256) sgemm_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                    float* __restrict__ C, int M, int N, int K, int ta, int tb,
                                                    int accumulate) {
  __shared__ float As[16][64 + 1];
  __shared__ float Bs[16][64 + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      int kk = i & 15, mm = i >> 4;
      int gm = m0 + mm, gk = k0 + kk;
      float va = 0.f, vb = 0.f;
      if (gm < M && gk < K) va = ta ? A[(long long)gk * M + gm] : A[(long long)gm * K + gk];
      int gn = n0 + mm;
      if (gn < N && gk < K) vb = tb ? B[(long long)gn * K + gk] : B[(long long)gk * N + gn];
      As[kk][mm] = va;
      Bs[kk][mm] = vb;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm < M && gn < N) {
        float* c = C + (long long)gm * N + gn;
        *c = accumulate ? *c + acc[i][j] : acc[i][j];
      }
    }
}
}  // namespace titb

TITB_API int titb_sgemm(const float* A, const float* B, float* C, int M, int N, int K, int trans_a, int trans_b,
                        int accumulate, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  titb::sgemm_kernel<<<grid, 256, 0, stream>>>(A, B, C, M, N, K, trans_a, trans_b, accumulate);
  return static_cast<int>(cudaGetLastError());
}
#endif  // !TITB_GEMM_PARAM_GATHER
