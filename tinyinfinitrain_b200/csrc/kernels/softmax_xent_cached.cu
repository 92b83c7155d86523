// Fused softmax cross entropy with the logits row held in shared memory between the two passes.
//
// The regular kernel (softmax_xent.cu) reads every row twice from global memory: once for the online max / sum and
// once to turn it into the gradient.  A GPT-2 row (50304 bf16 = 98 KB) fits in the 227 KB of shared memory of an SM,
// so this variant reads it once, keeps it on chip, and writes the gradient from there: 2 instead of 3 passes over
// the [rows, V] tensor, which is the whole cost of this memory-bound kernel.  Same arithmetic and contract as
// titb_xent_fwd_bwd (reference: infini_train/src/kernels/cuda/cross_entropy.cu:30-71, :115-163).
#include "api.h"
#include "common.cuh"

namespace titb {

constexpr int kXcThreads = 512;
constexpr long long kXcMaxRowBytes = 200 * 1024;

struct XcMaxSum { float m, s; };
__device__ __forceinline__ XcMaxSum xc_combine(XcMaxSum a, XcMaxSum b) {
  const float m = fmaxf(a.m, b.m);
  if (m == -INFINITY) return {m, 0.f};
  return {m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}

template <typename T>
__global__ void __launch_bounds__(kXcThreads) xent_cached_kernel(const T* logits, const long long* __restrict__ targets,
                                                                 float* __restrict__ losses, T* dlogits, int V, long long ld,
                                                                 float grad_scale, const float* __restrict__ upstream) {
  constexpr int VN = VecN<T>::n;
  extern __shared__ uint4 xc_smem[];
  Pack<T, VN>* srow = reinterpret_cast<Pack<T, VN>*>(xc_smem);
  __shared__ float red_m[kXcThreads / 32], red_s[kXcThreads / 32];
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  const int ldv = static_cast<int>(ld / VN);
  const long long tgt = targets[row];
  const bool valid = tgt >= 0 && tgt < V;
  const float x_tgt = valid ? to_f32(x[tgt]) : 0.f;       // read before the row can be overwritten in place

  XcMaxSum acc{-INFINITY, 0.f};
  for (int i = threadIdx.x; i < ldv; i += kXcThreads) {
    Pack<T, VN> p = ld128(x + static_cast<long long>(i) * VN);
    srow[i] = p;
    const int c0 = i * VN;
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < VN; ++e)
      if (c0 + e < V) mx = fmaxf(mx, to_f32(p.v[e]));
    if (mx > -INFINITY) {
      const float m = fmaxf(acc.m, mx);
      float s = acc.s * __expf(acc.m - m);
#pragma unroll
      for (int e = 0; e < VN; ++e)
        if (c0 + e < V) s += __expf(to_f32(p.v[e]) - m);
      acc = {m, s};
    }
  }
  // block reduction of (max, sum)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    XcMaxSum t{__shfl_xor_sync(0xffffffffu, acc.m, o), __shfl_xor_sync(0xffffffffu, acc.s, o)};
    acc = xc_combine(acc, t);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) { red_m[w] = acc.m; red_s[w] = acc.s; }
  __syncthreads();                                         // also orders the srow[] writes before pass 2
  XcMaxSum r = lane < kXcThreads / 32 ? XcMaxSum{red_m[lane], red_s[lane]} : XcMaxSum{-INFINITY, 0.f};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    XcMaxSum t{__shfl_xor_sync(0xffffffffu, r.m, o), __shfl_xor_sync(0xffffffffu, r.s, o)};
    r = xc_combine(r, t);
  }
  const float lse = r.m + logf(r.s);
  if (threadIdx.x == 0 && losses != nullptr) losses[row] = valid ? lse - x_tgt : 0.f;
  if (dlogits == nullptr) return;
  float g = grad_scale;
  if (upstream != nullptr) g *= *upstream;
  if (!valid) g = 0.f;
  T* dx = dlogits + row * ld;
  for (int i = threadIdx.x; i < ldv; i += kXcThreads) {
    const Pack<T, VN> p = srow[i];
    Pack<T, VN> o;
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      const int c = i * VN + e;
      float pr = (c < V) ? __expf(to_f32(p.v[e]) - lse) : 0.f;
      if (c == tgt) pr -= 1.f;
      o.v[e] = from_f32<T>(g * pr);
    }
    st128(dx + static_cast<long long>(i) * VN, o);
  }
}

template <typename T>
static int launch_cached(const void* logits, const long long* targets, float* losses, void* dlogits, long long rows, int V,
                         long long ld, float grad_scale, const float* upstream, cudaStream_t st) {
  const size_t smem = static_cast<size_t>(ld) * sizeof(T);
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(xent_cached_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kXcMaxRowBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  xent_cached_kernel<T><<<(unsigned)rows, kXcThreads, smem, st>>>((const T*)logits, targets, losses, (T*)dlogits, V, ld,
                                                                  grad_scale, upstream);
  return (int)cudaGetLastError();
}

}  // namespace titb
using namespace titb;

// 1 when the row-cached kernel can take this problem (16-byte aligned rows that fit in shared memory).
TITB_API int titb_xent_cached_ok(const void* logits, long long ld, int dtype) {
  const int vn = dtype == 1 ? 8 : 4;
  const long long bytes = ld * (dtype == 1 ? 2 : 4);
  return !(reinterpret_cast<uintptr_t>(logits) & 15) && (ld % vn == 0) && bytes <= kXcMaxRowBytes && bytes > 0;
}

TITB_API int titb_xent_fwd_bwd_cached(const void* logits, const long long* targets, float* losses, void* dlogits,
                                      long long rows, int V, long long ld, float grad_scale, const float* upstream,
                                      int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (!titb_xent_cached_ok(logits, ld, dtype) || (dlogits && (reinterpret_cast<uintptr_t>(dlogits) & 15)) || V > ld)
    return TITB_ERR_SHAPE;
  return dtype == 1 ? launch_cached<bf16>(logits, targets, losses, dlogits, rows, V, ld, grad_scale, upstream, st)
                    : launch_cached<float>(logits, targets, losses, dlogits, rows, V, ld, grad_scale, upstream, st);
}
