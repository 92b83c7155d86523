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

static inline int blocks_for(long long n) {
  long long b = (n + 255) / 256;
  return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
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
