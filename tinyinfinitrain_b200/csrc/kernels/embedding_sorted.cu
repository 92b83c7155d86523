// Deterministic token-embedding gradient: sort (token id, position) keys, then sum each run of equal ids in
// position order and add it to its row of the fp32 gradient buffer -- no atomics, so the result is bit-identical
// from run to run however often a token repeats.
//
// The reference's backward lets one thread per token atomicAdd into dW (infini_train/src/kernels/cuda/embedding.cu:52-67),
// and so does the default kernel of this library (embedding.cu); this variant trades about one sort of B*T keys for
// reproducibility.  A step has few tokens (8 x 1024 ... 4 x 4096) compared with the vocabulary, so the keys of one
// step fit in the shared memory of ONE thread block, where a bitonic network sorts them.
#include "api.h"
#include "common.cuh"

namespace titb {

constexpr int kSortThreads = 1024;
constexpr unsigned long long kKeyNone = ~0ull;   // padding and tokens of other vocabulary shards: sorted to the end

// keys[i] = (id - vocab_lo) << 32 | position for tokens of this shard; `npad` (a power of two >= n) keys are sorted
// ascending in shared memory and written to `sorted`.
__global__ void __launch_bounds__(kSortThreads) embedding_sort_kernel(const long long* __restrict__ idx, long long n, int npad,
                                                                      int vocab_lo, int vocab_hi,
                                                                      unsigned long long* __restrict__ sorted) {
  extern __shared__ unsigned long long skeys[];
  for (int i = threadIdx.x; i < npad; i += kSortThreads) {
    unsigned long long k = kKeyNone;
    if (i < n) {
      const long long tok = idx[i];
      if (tok >= vocab_lo && tok < vocab_hi)
        k = (static_cast<unsigned long long>(tok - vocab_lo) << 32) | static_cast<unsigned long long>(i);
    }
    skeys[i] = k;
  }
  __syncthreads();
  for (int k = 2; k <= npad; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < npad; i += kSortThreads) {
        const int l = i ^ j;
        if (l > i) {
          const unsigned long long a = skeys[i], b = skeys[l];
          const bool ascending = (i & k) == 0;
          if ((a > b) == ascending) { skeys[i] = b; skeys[l] = a; }
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < npad; i += kSortThreads) sorted[i] = skeys[i];
}

// One warp per sorted slot; the warp whose slot starts a run of equal ids sums the run's gradient rows (in position
// order) and adds the sum to the row of dwte.  Rows are walked in chunks of 32 lanes x VN columns.
template <typename T>
__global__ void __launch_bounds__(256) embedding_segment_reduce_kernel(const unsigned long long* __restrict__ sorted, int npad,
                                                                       const T* __restrict__ dout, float* __restrict__ dwte,
                                                                       int C) {
  constexpr int VN = VecN<T>::n;
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long s = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); s < npad; s += warps) {
    const unsigned long long key = sorted[s];
    if (key == kKeyNone) continue;
    const unsigned int row = static_cast<unsigned int>(key >> 32);
    if (s > 0 && static_cast<unsigned int>(sorted[s - 1] >> 32) == row) continue;      // not the head of its run
    // length of the run (keys are sorted, so it is contiguous)
    long long len = 1;
    while (s + len < npad && static_cast<unsigned int>(sorted[s + len] >> 32) == row && sorted[s + len] != kKeyNone) ++len;
    for (int c0 = lane * VN; c0 < C; c0 += 32 * VN) {
      // four independent partial sums (rows j, j+1, j+2, j+3 of each group of four) keep four loads in flight; they
      // are combined in a fixed order, so the result depends only on the sorted order, never on timing
      float acc[4][VN];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int e = 0; e < VN; ++e) acc[u][e] = 0.f;
      for (long long j = 0; j < len; j += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (j + u < len) {
            const long long pos = static_cast<long long>(sorted[s + j + u] & 0xffffffffull);
            Pack<T, VN> g = ld128(dout + pos * C + c0);
#pragma unroll
            for (int e = 0; e < VN; ++e) acc[u][e] += to_f32(g.v[e]);
          }
        }
      }
      float* dst = dwte + static_cast<long long>(row) * C + c0;
#pragma unroll
      for (int e = 0; e < VN; ++e) dst[e] += (acc[0][e] + acc[1][e]) + (acc[2][e] + acc[3][e]);
    }
  }
}

}  // namespace titb
using namespace titb;

// Largest token count one sort handles (keys must fit the shared memory of one block).
TITB_API int titb_embedding_sorted_max_tokens(void) { return 16384; }

TITB_API int titb_embedding_bwd_wte_sorted(const long long* idx, const void* dout, float* dwte, long long BT, int C,
                                           int vocab_lo, int vocab_hi, int dtype, unsigned long long* scratch_keys,
                                           cudaStream_t st) {
  if (BT <= 0) return 0;
  const int vn = dtype == 1 ? 8 : 4;
  if (BT > titb_embedding_sorted_max_tokens() || C % vn) return TITB_ERR_SHAPE;
  int npad = 2;
  while (npad < BT) npad <<= 1;
  const size_t smem = static_cast<size_t>(npad) * sizeof(unsigned long long);
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(embedding_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         titb_embedding_sorted_max_tokens() * (int)sizeof(unsigned long long));
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  embedding_sort_kernel<<<1, kSortThreads, smem, st>>>(idx, BT, npad, vocab_lo, vocab_hi, scratch_keys);
  const int blocks = (npad + 7) / 8;      // 8 warps per block, one warp per sorted slot
  if (dtype == 1)
    embedding_segment_reduce_kernel<bf16><<<blocks, 256, 0, st>>>(scratch_keys, npad, (const bf16*)dout, dwte, C);
  else
    embedding_segment_reduce_kernel<float><<<blocks, 256, 0, st>>>(scratch_keys, npad, (const float*)dout, dwte, C);
  return (int)cudaGetLastError();
}
