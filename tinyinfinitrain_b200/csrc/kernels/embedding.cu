// Token + position embedding, forward and backward.
//
// Counterpart of infini_train/src/kernels/cuda/embedding.cu:16-31 (one thread per
// output element) and :52-67 (one thread per token looping over C with atomicAdd).
// Here a row is moved with 128-bit accesses, the position-embedding add of
// example/gpt2/net.cc:205-209 is fused into the gather, and the position gradient
// is a deterministic sum over the batch.  The token gradient is scattered with
// fp32 reductions into the main-gradient buffer (duplicates make the order of those
// additions run-dependent).
#include "api.h"
#include "common.cuh"

namespace titb {

template <typename T>
__global__ void embedding_fwd_kernel(const long long* __restrict__ idx, const T* __restrict__ wte,
                                     const T* __restrict__ wpe, T* __restrict__ out, long long BT, int T_, int C,
                                     int pos_offset) {
  constexpr int VN = VecN<T>::n;
  const int cv = C / VN;
  const long long total = BT * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long bt = i / cv;
    const int c = (int)(i - bt * cv) * VN;
    const long long tok = idx[bt];
    Pack<T, VN> a = ld128(wte + tok * C + c);
    if (wpe != nullptr) {
      const int t = (int)(bt % T_) + pos_offset;
      Pack<T, VN> p = ld128(wpe + (long long)t * C + c);
#pragma unroll
      for (int e = 0; e < VN; ++e) a.v[e] = from_f32<T>(to_f32(a.v[e]) + to_f32(p.v[e]));
    }
    st128(out + bt * C + c, a);
  }
}

template <typename T>
__global__ void embedding_bwd_wte_kernel(const long long* __restrict__ idx, const T* __restrict__ dout,
                                         float* __restrict__ dwte, long long BT, int C, int vocab_lo, int vocab_hi) {
  constexpr int VN = VecN<T>::n;
  const int cv = C / VN;
  const long long total = BT * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long bt = i / cv;
    const int c = (int)(i - bt * cv) * VN;
    const long long tok = idx[bt];
    if (tok < vocab_lo || tok >= vocab_hi) continue;  // rows owned by another vocabulary shard
    Pack<T, VN> g = ld128(dout + bt * C + c);
    float* dst = dwte + (tok - vocab_lo) * C + c;
#pragma unroll
    for (int e = 0; e < VN; ++e) atomicAdd(dst + e, to_f32(g.v[e]));
  }
}

template <typename T>
__global__ void embedding_bwd_wpe_kernel(const T* __restrict__ dout, float* __restrict__ dwpe, int B, int T_, int C) {
  constexpr int VN = VecN<T>::n;
  const int cv = C / VN;
  const long long total = (long long)T_ * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / cv);
    const int c = (int)(i - (long long)t * cv) * VN;
    float acc[VN];
#pragma unroll
    for (int e = 0; e < VN; ++e) acc[e] = 0.f;
    for (int b = 0; b < B; ++b) {
      Pack<T, VN> g = ld128(dout + ((long long)b * T_ + t) * C + c);
#pragma unroll
      for (int e = 0; e < VN; ++e) acc[e] += to_f32(g.v[e]);
    }
    float* dst = dwpe + (long long)t * C + c;
#pragma unroll
    for (int e = 0; e < VN; ++e) dst[e] += acc[e];
  }
}

// ---- vocabulary-parallel table (rows split over the tensor-parallel ranks, tokens split by sequence) --------------
// Every token's row lives on exactly one rank, so the gather needs no reduction: the owner of the row stores it
// straight into the token-shard buffer of the rank that owns the token (peer-mapped memory), and the backward pulls
// the gradient rows it owns from the token owners.  Only the rows that are needed cross NVLink: M/world rows per rank
// instead of the M rows of the masked-gather + reduce-scatter formulation.
struct PeerRowPtrs {
  unsigned long long p[16];
};

// One warp per token.  Rank 0 also writes zero rows for ids outside [0, vocab_total), so every row of every
// destination is written exactly once per call.
template <typename T>
__global__ void __launch_bounds__(256) embedding_vp_push_kernel(const long long* __restrict__ idx, const T* __restrict__ w,
                                                                PeerRowPtrs dst, long long M, long long Ms, int C,
                                                                long long lo, long long hi, long long vocab_total,
                                                                int zero_strays) {
  constexpr int VN = VecN<T>::n;
  const int lane = threadIdx.x & 31;
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long t = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); t < M; t += nwarps) {
    const long long tok = idx[t];
    const bool mine = tok >= lo && tok < hi;
    const bool stray = zero_strays && (tok < 0 || tok >= vocab_total);
    if (!mine && !stray) continue;
    const long long r = t / Ms;
    T* d = reinterpret_cast<T*>(dst.p[r]) + (t - r * Ms) * C;
    const T* s = w + (mine ? tok - lo : 0) * C;
    for (int c = lane * VN; c < C; c += 32 * VN) {
      Pack<T, VN> a;
      if (mine) {
        a = ld128(s + c);
      } else {
#pragma unroll
        for (int e = 0; e < VN; ++e) a.v[e] = from_f32<T>(0.f);
      }
      st128(d + c, a);
    }
  }
}

// One warp per token: gradient rows of the ids this rank owns, read from the token owner's buffer and added (fp32) to
// the local table gradient.
template <typename T>
__global__ void __launch_bounds__(256) embedding_vp_pull_bwd_kernel(const long long* __restrict__ idx, PeerRowPtrs src,
                                                                    float* __restrict__ dw, long long M, long long Ms,
                                                                    int C, long long lo, long long hi) {
  constexpr int VN = VecN<T>::n;
  const int lane = threadIdx.x & 31;
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long t = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); t < M; t += nwarps) {
    const long long tok = idx[t];
    if (tok < lo || tok >= hi) continue;
    const long long r = t / Ms;
    const T* s = reinterpret_cast<const T*>(src.p[r]) + (t - r * Ms) * C;
    float* d = dw + (tok - lo) * C;
    for (int c = lane * VN; c < C; c += 32 * VN) {
      Pack<T, VN> g = ld128(s + c);
#pragma unroll
      for (int e = 0; e < VN; ++e) atomicAdd(d + c + e, to_f32(g.v[e]));
    }
  }
}

static inline int blocks_for(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = device_sm_count() * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace titb
using namespace titb;

TITB_API int titb_embedding_fwd(const long long* idx, const void* wte, const void* wpe, void* out, long long BT, int T,
                                int C, int pos_offset, int dtype, cudaStream_t st) {
  if (BT <= 0) return 0;
  const int vn = dtype == 1 ? 8 : 4;
  if (C % vn) return (int)cudaErrorInvalidValue;
  const int blocks = blocks_for(BT * (C / vn));
  if (dtype == 1) embedding_fwd_kernel<bf16><<<blocks, 256, 0, st>>>(idx, (const bf16*)wte, (const bf16*)wpe, (bf16*)out, BT, T, C, pos_offset);
  else embedding_fwd_kernel<float><<<blocks, 256, 0, st>>>(idx, (const float*)wte, (const float*)wpe, (float*)out, BT, T, C, pos_offset);
  return (int)cudaGetLastError();
}

TITB_API int titb_embedding_bwd(const long long* idx, const void* dout, float* dwte, float* dwpe, long long BT, int T,
                                int C, int vocab_lo, int vocab_hi, int dtype, cudaStream_t st) {
  if (BT <= 0) return 0;
  const int vn = dtype == 1 ? 8 : 4;
  if (C % vn) return (int)cudaErrorInvalidValue;
  if (dwte) {
    const int blocks = blocks_for(BT * (C / vn));
    if (dtype == 1) embedding_bwd_wte_kernel<bf16><<<blocks, 256, 0, st>>>(idx, (const bf16*)dout, dwte, BT, C, vocab_lo, vocab_hi);
    else embedding_bwd_wte_kernel<float><<<blocks, 256, 0, st>>>(idx, (const float*)dout, dwte, BT, C, vocab_lo, vocab_hi);
  }
  if (dwpe) {
    const int B = (int)(BT / T);
    const int blocks = blocks_for((long long)T * (C / vn));
    if (dtype == 1) embedding_bwd_wpe_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)dout, dwpe, B, T, C);
    else embedding_bwd_wpe_kernel<float><<<blocks, 256, 0, st>>>((const float*)dout, dwpe, B, T, C);
  }
  return (int)cudaGetLastError();
}

static int vp_args_ok(const unsigned long long* ptrs, int world, long long M, long long Ms, int C, int vn) {
  if (world < 1 || world > 16 || Ms <= 0 || M != Ms * world || C % vn) return 0;
  for (int r = 0; r < world; ++r)
    if (ptrs[r] == 0 || (ptrs[r] & 15)) return 0;
  return 1;
}

TITB_API int titb_embedding_vp_push(const long long* idx, const void* w, const unsigned long long* dst_ptrs, int world,
                                    long long M, long long Ms, int C, long long vocab_lo, long long vocab_hi,
                                    long long vocab_total, int zero_strays, int dtype, cudaStream_t st) {
  const int vn = dtype == 1 ? 8 : 4;
  if (!vp_args_ok(dst_ptrs, world, M, Ms, C, vn)) return (int)cudaErrorInvalidValue;
  PeerRowPtrs p{};
  for (int r = 0; r < world; ++r) p.p[r] = dst_ptrs[r];
  const int blocks = blocks_for(M * 32);
  if (dtype == 1)
    embedding_vp_push_kernel<bf16><<<blocks, 256, 0, st>>>(idx, (const bf16*)w, p, M, Ms, C, vocab_lo, vocab_hi,
                                                           vocab_total, zero_strays);
  else
    embedding_vp_push_kernel<float><<<blocks, 256, 0, st>>>(idx, (const float*)w, p, M, Ms, C, vocab_lo, vocab_hi,
                                                            vocab_total, zero_strays);
  return (int)cudaGetLastError();
}

TITB_API int titb_embedding_vp_pull_bwd(const long long* idx, const unsigned long long* src_ptrs, int world, float* dw,
                                        long long M, long long Ms, int C, long long vocab_lo, long long vocab_hi,
                                        int dtype, cudaStream_t st) {
  const int vn = dtype == 1 ? 8 : 4;
  if (!vp_args_ok(src_ptrs, world, M, Ms, C, vn) || dw == nullptr) return (int)cudaErrorInvalidValue;
  PeerRowPtrs p{};
  for (int r = 0; r < world; ++r) p.p[r] = src_ptrs[r];
  const int blocks = blocks_for(M * 32);
  if (dtype == 1)
    embedding_vp_pull_bwd_kernel<bf16><<<blocks, 256, 0, st>>>(idx, p, dw, M, Ms, C, vocab_lo, vocab_hi);
  else
    embedding_vp_pull_bwd_kernel<float><<<blocks, 256, 0, st>>>(idx, p, dw, M, Ms, C, vocab_lo, vocab_hi);
  return (int)cudaGetLastError();
}
