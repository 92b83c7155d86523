// Gradient-norm clipping on the device: sum of squares of a flat fp32 gradient buffer (local, or of this rank's
// shard of the cross-rank sum read over NVLink), the clip coefficient, and the in-place scaling by a coefficient
// that lives in device memory -- so a training step captured in a CUDA graph clips with the norm of that step.
//
// The reference has no gradient clipping (its optimizers are SGD and Adam only: infini_train/src/optimizer.cc).
// Every reduction here is a fixed-order two-stage sum, so the norm is reproducible run to run.
#include "api.h"
#include "common.cuh"

namespace titb {

constexpr int kClipThreads = 256;
constexpr int kClipMaxBlocks = 1024;   // partial sums per launch: partials[] must hold this many floats

__device__ __forceinline__ float4 clip_mc_ld_reduce(const float* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}

// partials[blockIdx.x] = sum over this block's grid-stride share of x[i]^2 (zero for blocks without work).
__global__ void __launch_bounds__(kClipThreads) sumsq_partial_kernel(const float* __restrict__ x, long long n,
                                                                     float* __restrict__ partials) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long nvec = n / 4, stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const float4 v = *reinterpret_cast<const float4*>(x + i * 4);
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long long i = nvec * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) acc += x[i] * x[i];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

struct RsSumsqArgs {
  const void* grads[16];   // fp32 flat gradient buffer of every rank (peer mapped)
  const float* grad_mc;    // multicast address of the gradient buffer, or null
  long long shard_off, shard_n;
  int world, rank;
};
// Same read path as the fused reduce-scatter + Adam kernel, but only the squared norm of the summed shard is kept.
__global__ void __launch_bounds__(kClipThreads) rs_sumsq_kernel(const RsSumsqArgs a, float* __restrict__ partials) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long nvec = a.shard_n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long glob = a.shard_off + i * 4;
    float4 g;
    if (a.grad_mc != nullptr) {
      g = clip_mc_ld_reduce(a.grad_mc + glob);
    } else {
      g = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int q = 0; q < a.world; ++q) {
        const int pr = (a.rank + q) % a.world;
        const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(a.grads[pr]) + glob);
        g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
      }
    }
    acc += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

// total = sum(partials[0..n)); with max_norm > 0: out[0] = norm = sqrt(total) * pre_scale,
// out[1] = min(1, max_norm / (norm + 1e-6)); with max_norm <= 0: out[0] = total (a partial result to be combined).
__global__ void __launch_bounds__(kClipThreads) clip_coef_kernel(const float* __restrict__ partials, int n, float pre_scale,
                                                                 float max_norm, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partials[i];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) {
    if (max_norm > 0.f) {
      const float norm = sqrtf(acc) * pre_scale;
      out[0] = norm;
      out[1] = fminf(1.f, max_norm / (norm + 1e-6f));
    } else {
      out[0] = acc;
    }
  }
}

__global__ void __launch_bounds__(kClipThreads) scale_by_dev_kernel(float* __restrict__ x, long long n,
                                                                    const float* __restrict__ coef) {
  const float c = coef[0];
  if (c == 1.f) return;                                   // the common case: nothing to clip, nothing to write
  const long long nvec = n / 4, stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float4 v = *reinterpret_cast<float4*>(x + i * 4);
    v.x *= c; v.y *= c; v.z *= c; v.w *= c;
    *reinterpret_cast<float4*>(x + i * 4) = v;
  }
  for (long long i = nvec * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) x[i] *= c;
}

static inline int clip_blocks(long long n) {
  long long b = (n / 4 + kClipThreads - 1) / kClipThreads;
  return (int)(b < 1 ? 1 : (b > kClipMaxBlocks ? kClipMaxBlocks : b));
}

}  // namespace titb
using namespace titb;

TITB_API int titb_clip_max_partials(void) { return kClipMaxBlocks; }

TITB_API int titb_sumsq_partials(const float* x, long long n, float* partials, int* n_partials, cudaStream_t st) {
  if (n <= 0 || (reinterpret_cast<uintptr_t>(x) & 15)) return TITB_ERR_ALIGNMENT;
  const int blocks = clip_blocks(n);
  sumsq_partial_kernel<<<blocks, kClipThreads, 0, st>>>(x, n, partials);
  *n_partials = blocks;
  return (int)cudaGetLastError();
}

TITB_API int titb_rs_sumsq_partials(const unsigned long long* grad_ptrs, const void* grad_mc, long long shard_off,
                                    long long shard_n, int world, int rank, float* partials, int* n_partials,
                                    cudaStream_t st) {
  if (world < 1 || world > 16 || shard_n <= 0 || (shard_n & 3) || (shard_off & 3)) return TITB_ERR_SHAPE;
  RsSumsqArgs a{};
  for (int i = 0; i < world; ++i) a.grads[i] = reinterpret_cast<const void*>(grad_ptrs[i]);
  a.grad_mc = static_cast<const float*>(grad_mc);
  a.shard_off = shard_off; a.shard_n = shard_n; a.world = world; a.rank = rank;
  const int blocks = clip_blocks(shard_n);
  rs_sumsq_kernel<<<blocks, kClipThreads, 0, st>>>(a, partials);
  *n_partials = blocks;
  return (int)cudaGetLastError();
}

TITB_API int titb_clip_coef(const float* partials, int n_partials, float pre_scale, float max_norm, float* out,
                            cudaStream_t st) {
  if (n_partials < 1) return TITB_ERR_SHAPE;
  clip_coef_kernel<<<1, kClipThreads, 0, st>>>(partials, n_partials, pre_scale, max_norm, out);
  return (int)cudaGetLastError();
}

TITB_API int titb_scale_by_dev(float* x, long long n, const float* coef, cudaStream_t st) {
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(x) & 15) return TITB_ERR_ALIGNMENT;
  scale_by_dev_kernel<<<clip_blocks(n), kClipThreads, 0, st>>>(x, n, coef);
  return (int)cudaGetLastError();
}
