// Column sums of a [rows, C] matrix (bias gradients) in ONE launch: every CTA folds a strip of rows into a partial
// row of fp32 sums, and the CTA that finishes last for its column strip folds the partial rows in a fixed order.
// The two-launch version in pointwise.cu spends most of its time in launch gaps and in a second kernel that has
// only C/32 CTAs; here the tail runs inside the first kernel on data that is still in L2.
//
// Deterministic: which CTA does the final fold depends on timing, but the fold always adds the same partial rows
// in the same order, and each partial row is produced by a fixed-order sum.
//
// The reference computes bias gradients with a cuBLAS GEMV against a vector of ones
// (infini_train/src/kernels/cuda/linear.cu:233-240, LinearBackward).
#include "api.h"
#include "common.cuh"

namespace titb {

constexpr int kCfThreads = 256;        // 8 warps: warp w takes rows w, w+8, ... of the CTA's row strip
constexpr int kCfMaxParts = 256;       // partial rows per column strip; scratch holds parts * C floats

// counters[strip] counts the CTAs of a column strip that have published their partial row.  The last one resets
// it to zero, so the array needs zeroing only once; launches that share it must be ordered on one stream.
template <typename T>
__global__ void __launch_bounds__(kCfThreads)
colsum_fused_kernel(const T* __restrict__ x, float* __restrict__ scratch, unsigned* __restrict__ counters,
                    float* __restrict__ out, long long rows, int C, int accumulate) {
  constexpr int VN = VecN<T>::n;
  constexpr int W = 32 * VN;           // columns per strip
  __shared__ float sm[8][W + 4];
  __shared__ unsigned ticket;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c0 = blockIdx.x * W, c = c0 + tx * VN;
  const int parts = gridDim.y;

  float acc[VN];
#pragma unroll
  for (int e = 0; e < VN; ++e) acc[e] = 0.f;
  if (c < C) {
    const long long step = (long long)parts * 8;
    long long r = (long long)blockIdx.y * 8 + ty;
    // four independent 16-byte loads in flight per thread
    for (; r + 3 * step < rows; r += 4 * step) {
      const Pack<T, VN> v0 = ld128(x + r * C + c), v1 = ld128(x + (r + step) * C + c),
                        v2 = ld128(x + (r + 2 * step) * C + c), v3 = ld128(x + (r + 3 * step) * C + c);
#pragma unroll
      for (int e = 0; e < VN; ++e) acc[e] += (to_f32(v0.v[e]) + to_f32(v1.v[e])) + (to_f32(v2.v[e]) + to_f32(v3.v[e]));
    }
    for (; r < rows; r += step) {
      const Pack<T, VN> v = ld128(x + r * C + c);
#pragma unroll
      for (int e = 0; e < VN; ++e) acc[e] += to_f32(v.v[e]);
    }
  }
#pragma unroll
  for (int e = 0; e < VN; ++e) sm[ty][tx * VN + e] = acc[e];
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += kCfThreads) {
    if (c0 + i < C) {
      float t = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) t += sm[j][i];
      scratch[(long long)blockIdx.y * C + c0 + i] = t;
    }
  }
  // publish: every thread's partial stores are made visible device-wide before one thread takes the ticket
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) ticket = atomicAdd(&counters[blockIdx.x], 1u);
  __syncthreads();
  if (ticket != (unsigned)(parts - 1)) return;
  __threadfence();                     // order the reads below after the ticket

  // last CTA of this strip: warp w folds partial rows w, w+8, ...; each lane owns four columns per pass
  for (int base = 0; base < W; base += 128) {
    const int cc = base + tx * 4;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c0 + cc < C) {
#pragma unroll 8
      for (int p = ty; p < parts; p += 8) {
        const float4 t = __ldcg(reinterpret_cast<const float4*>(scratch + (long long)p * C + c0 + cc));
        s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
      }
    }
    sm[ty][cc] = s.x; sm[ty][cc + 1] = s.y; sm[ty][cc + 2] = s.z; sm[ty][cc + 3] = s.w;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += kCfThreads) {
    if (c0 + i < C) {
      float t = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) t += sm[j][i];
      out[c0 + i] = accumulate ? out[c0 + i] + t : t;
    }
  }
  if (threadIdx.x == 0) counters[blockIdx.x] = 0u;
}

static int colsum_fused_parts(long long rows, int strips) {
  // about four CTAs per SM in total, at least 32 rows per CTA, at most kCfMaxParts partial rows
  int parts = (148 * 4 + strips - 1) / strips;
  const long long by_rows = (rows + 31) / 32;
  if (parts > by_rows) parts = (int)by_rows;
  if (parts > kCfMaxParts) parts = kCfMaxParts;
  return parts < 1 ? 1 : parts;
}

}  // namespace titb

using namespace titb;

// True when the one-launch kernel can take this problem: 16-byte rows, whole vectors per row, C a multiple of 4
// (float4 reads of the partial rows).
TITB_API int titb_colsum_fused_ok(const void* x, long long rows, int C, int dtype) {
  const int vn = dtype == 1 ? 8 : 4;
  return rows > 0 && C > 0 && (C % vn) == 0 && (C % 4) == 0 && !((uintptr_t)x & 15);
}
// Floats of scratch and unsigned counters that titb_colsum_fused needs for this shape.
TITB_API long long titb_colsum_fused_scratch(long long rows, int C, int dtype) {
  const int w = 32 * (dtype == 1 ? 8 : 4);
  return (long long)colsum_fused_parts(rows, (C + w - 1) / w) * C;
}
TITB_API int titb_colsum_fused_counters(int C, int dtype) {
  const int w = 32 * (dtype == 1 ? 8 : 4);
  return (C + w - 1) / w;
}
// counters: zero before the first use; left zero by every launch.
TITB_API int titb_colsum_fused(const void* x, float* out, long long rows, int C, int dtype, int accumulate,
                               float* scratch, unsigned* counters, cudaStream_t st) {
  if (!titb_colsum_fused_ok(x, rows, C, dtype) || !scratch || !counters) return (int)cudaErrorInvalidValue;
  const int w = 32 * (dtype == 1 ? 8 : 4);
  const int strips = (C + w - 1) / w;
  dim3 grid(strips, colsum_fused_parts(rows, strips));
  if (dtype == 1)
    colsum_fused_kernel<bf16><<<grid, kCfThreads, 0, st>>>((const bf16*)x, scratch, counters, out, rows, C, accumulate);
  else
    colsum_fused_kernel<float><<<grid, kCfThreads, 0, st>>>((const float*)x, scratch, counters, out, rows, C, accumulate);
  return (int)cudaGetLastError();
}
