// LayerNorm / RMSNorm backward in ONE launch for rows that a warp can hold (C <= 128 vectors of 16 bytes):
// dx, and the finished dweight / dbias, with no second-stage kernels.
//
// Differences from norm_bwd_kernel + partial_colsum_kernel in norm.cu:
//  * one CTA of eight warps per SM and four rows in flight per warp, i.e. four times the bytes outstanding per SM
//    (the two-launch version keeps 8 warps x 1 row per SM in flight and is latency bound); the register budget of
//    a single resident CTA holds the four rows without spilling;
//  * the dweight / dbias partial rows are folded by the CTAs themselves: the CTA that finishes last in a group of
//    four folds the group's rows, the group that finishes last folds the group rows and writes the result.
//    Which CTA does a fold depends on timing, what it adds and in which order does not: results are bit-stable;
//  * an optional `dres` operand is added to dx, so the gradient that arrives through the residual connection
//    does not need an add kernel of its own.
//
// Counterpart of infini_train/src/kernels/cuda/layernorm.cu:87-138 (LayerNormBackward: one atomicAdd per element
// per token for dweight / dbias).
#include "api.h"
#include "common.cuh"

namespace titb {

// Tells the compiler that the 16 bytes of `p` may have changed: values converted from them earlier cannot be
// reused afterwards, so between the two uses of a row only the packed form stays in registers.
template <typename P>
__device__ __forceinline__ void keep_packed(P& p) {
  static_assert(sizeof(P) == 16, "one 128-bit pack");
  uint4& u = *reinterpret_cast<uint4*>(&p);
  asm volatile("" : "+r"(u.x), "+r"(u.y), "+r"(u.z), "+r"(u.w));
}

constexpr int kNb1Threads = 256;
constexpr int kNb1Warps = kNb1Threads / 32;
constexpr int kNb1Rows = 4;                            // rows a warp keeps in flight
constexpr int kNb1GroupCtas = 4;
constexpr int kNb1Groups = 37;
constexpr int kNb1Ctas = kNb1GroupCtas * kNb1Groups;   // 148 = one per SM

// scratch: [kNb1Ctas][2C] CTA rows, then [kNb1Groups][2C] group rows (dweight in the first C floats of a row,
// dbias in the second).  counters: [0] groups finished, [1 + g] CTAs of group g finished; zero before the first
// launch, left zero by every launch.
template <typename T, int MAXV, bool RMS>
__global__ void __launch_bounds__(kNb1Threads, 1)
norm_bwd_onepass_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                        const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                        const T* dres, T* dx, float* __restrict__ dw_out,
                        float* __restrict__ db_out, float* __restrict__ scratch, unsigned* __restrict__ counters,
                        long long rows, int C, int accumulate) {
  constexpr int VN = VecN<T>::n;
  extern __shared__ float acc_smem[];   // [2C]
  __shared__ unsigned ticket;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const long long warp = blockIdx.x * (long long)kNb1Warps + wib;
  const long long nwarps = (long long)gridDim.x * kNb1Warps;
  const int nvec = C / VN;
  const float inv_c = 1.f / (float)C;

  float dwacc[MAXV][VN], dbacc[MAXV][VN];
  Pack<T, VN> wv[MAXV];
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = lane + k * 32;
#pragma unroll
    for (int e = 0; e < VN; ++e) { dwacc[k][e] = 0.f; dbacc[k][e] = 0.f; }
    if (i < nvec) wv[k] = ld128(w + i * VN);
  }

  for (long long row0 = warp; row0 < rows; row0 += kNb1Rows * nwarps) {
    Pack<T, VN> xv[kNb1Rows][MAXV], dv[kNb1Rows][MAXV];
    float mean[kNb1Rows], rstd[kNb1Rows];
    // all rows' loads are issued before the first reduction
#pragma unroll
    for (int u = 0; u < kNb1Rows; ++u) {
      const long long row = row0 + u * nwarps;
      const bool live = row < rows;
      mean[u] = (RMS || !live) ? 0.f : mean_in[row];
      rstd[u] = live ? rstd_in[row] : 0.f;
#pragma unroll
      for (int k = 0; k < MAXV; ++k) {
        const int i = lane + k * 32;
        if (live && i < nvec) {
          xv[u][k] = ld128(x + row * C + i * VN);
          dv[u][k] = ld128(dy + row * C + i * VN);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kNb1Rows; ++u) {
      const long long row = row0 + u * nwarps;
      if (row >= rows) continue;          // uniform across the warp
      float s1 = 0.f, s2 = 0.f;           // sum(dnorm), sum(dnorm * norm)
#pragma unroll
      for (int k = 0; k < MAXV; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
#pragma unroll
          for (int e = 0; e < VN; ++e) {
            const float n = (to_f32(xv[u][k].v[e]) - mean[u]) * rstd[u];
            const float g = to_f32(dv[u][k].v[e]);
            const float dn = g * to_f32(wv[k].v[e]);
            s1 += dn;
            s2 += dn * n;
            dwacc[k][e] += g * n;
            dbacc[k][e] += g;
          }
        }
      }
      s1 = warp_sum(s1);
      s2 = warp_sum(s2);
#pragma unroll
      for (int k = 0; k < MAXV; ++k) { keep_packed(xv[u][k]); keep_packed(dv[u][k]); }
      const float m1 = RMS ? 0.f : s1 * inv_c, m2 = s2 * inv_c;
#pragma unroll
      for (int k = 0; k < MAXV; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
          Pack<T, VN> ov, rv;
          if (dres != nullptr) rv = ld128(dres + row * C + i * VN);
#pragma unroll
          for (int e = 0; e < VN; ++e) {
            const float n = (to_f32(xv[u][k].v[e]) - mean[u]) * rstd[u];
            const float dn = to_f32(dv[u][k].v[e]) * to_f32(wv[k].v[e]);
            float o = (dn - m1 - n * m2) * rstd[u];
            if (dres != nullptr) o += to_f32(rv.v[e]);
            ov.v[e] = from_f32<T>(o);
          }
          st128(dx + row * C + i * VN, ov);
        }
      }
    }
  }

  // the warps of the CTA fold their sums in warp order through shared memory
  for (int g = 0; g < kNb1Warps; ++g) {
    if (wib == g) {
#pragma unroll
      for (int k = 0; k < MAXV; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
#pragma unroll
          for (int e = 0; e < VN; ++e) {
            const int c = i * VN + e;
            acc_smem[c] = (g == 0 ? 0.f : acc_smem[c]) + dwacc[k][e];
            if (!RMS) acc_smem[C + c] = (g == 0 ? 0.f : acc_smem[C + c]) + dbacc[k][e];
          }
        }
      }
    }
    __syncthreads();
  }
  const int W2 = RMS ? C : 2 * C;         // floats of a partial row that carry data
  float* my_row = scratch + (long long)blockIdx.x * 2 * C;
  for (int c = threadIdx.x; c < W2; c += kNb1Threads) my_row[c] = acc_smem[c];

  // ---- fold inside the group of four CTAs -----------------------------------------------------------------
  const int group = blockIdx.x / kNb1GroupCtas;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) ticket = atomicAdd(&counters[1 + group], 1u);
  __syncthreads();
  if (ticket != (unsigned)(kNb1GroupCtas - 1)) return;
  __threadfence();
  // Both folds read whole float4 columns with every load of a column issued before the first add: the tail is a
  // single CTA, so its time is the number of dependent round trips to L2, not bandwidth.
  float* group_rows = scratch + (long long)kNb1Ctas * 2 * C;
  {
    const float* first = scratch + (long long)group * kNb1GroupCtas * 2 * C;
    for (int c = threadIdx.x * 4; c < W2; c += kNb1Threads * 4) {
      float4 v[kNb1GroupCtas];
#pragma unroll
      for (int j = 0; j < kNb1GroupCtas; ++j) v[j] = __ldcg(reinterpret_cast<const float4*>(first + (long long)j * 2 * C + c));
      float4 t = v[0];
#pragma unroll
      for (int j = 1; j < kNb1GroupCtas; ++j) { t.x += v[j].x; t.y += v[j].y; t.z += v[j].z; t.w += v[j].w; }
      *reinterpret_cast<float4*>(group_rows + (long long)group * 2 * C + c) = t;
    }
  }
  if (threadIdx.x == 0) counters[1 + group] = 0u;

  // ---- fold across groups --------------------------------------------------------------------------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) ticket = atomicAdd(&counters[0], 1u);
  __syncthreads();
  if (ticket != (unsigned)(kNb1Groups - 1)) return;
  __threadfence();
  for (int c = threadIdx.x * 4; c < W2; c += kNb1Threads * 4) {
    float4 v[kNb1Groups];
#pragma unroll
    for (int j = 0; j < kNb1Groups; ++j) v[j] = __ldcg(reinterpret_cast<const float4*>(group_rows + (long long)j * 2 * C + c));
    float4 t = v[0];
#pragma unroll
    for (int j = 1; j < kNb1Groups; ++j) { t.x += v[j].x; t.y += v[j].y; t.z += v[j].z; t.w += v[j].w; }
    float* out = c < C ? dw_out + c : db_out + (c - C);   // C is a multiple of 4: the four columns share a side
    if (accumulate) { t.x += out[0]; t.y += out[1]; t.z += out[2]; t.w += out[3]; }
    out[0] = t.x; out[1] = t.y; out[2] = t.z; out[3] = t.w;
  }
  if (threadIdx.x == 0) counters[0] = 0u;
}

template <typename T, bool RMS>
static int norm_bwd_onepass_launch(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                   const void* dres, void* dx, float* dw, float* db, float* scratch,
                                   unsigned* counters, long long rows, int C, int accumulate, cudaStream_t st) {
  constexpr int VN = VecN<T>::n;
  const int maxv = (C / VN + 31) / 32;
  const size_t sm = 2 * (size_t)C * sizeof(float);
#define TITB_NB1(MV)                                                                                              \
  norm_bwd_onepass_kernel<T, MV, RMS><<<kNb1Ctas, kNb1Threads, sm, st>>>(                                        \
      (const T*)dy, (const T*)x, (const T*)w, mean, rstd, (const T*)dres, (T*)dx, dw, db, scratch, counters, rows, \
      C, accumulate)
  switch (maxv) {
    case 1: TITB_NB1(1); break;
    case 2: TITB_NB1(2); break;
    case 3: TITB_NB1(3); break;
    case 4: TITB_NB1(4); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef TITB_NB1
  return (int)cudaGetLastError();
}

}  // namespace titb

using namespace titb;

// True when the one-launch backward can take this problem.
TITB_API int titb_norm_bwd_onepass_ok(long long rows, int C, int dtype, const void* dy, const void* x, const void* w,
                                      const void* dres, const void* dx) {
  const int vn = dtype == 1 ? 8 : 4;
  if (rows <= 0 || C <= 0 || (C % vn) != 0 || C / vn > 128) return 0;
  const uintptr_t bits = (uintptr_t)dy | (uintptr_t)x | (uintptr_t)w | (uintptr_t)dres | (uintptr_t)dx;
  return (bits & 15) == 0;
}
// Floats of scratch and unsigned counter words the launch needs.
TITB_API long long titb_norm_bwd_onepass_scratch(int C) { return (long long)(kNb1Ctas + kNb1Groups) * 2 * C; }
TITB_API int titb_norm_bwd_onepass_counters() { return 1 + kNb1Groups; }

// rms != 0: RMSNorm (mean and db are ignored).  dres may be null.  counters: zero before the first launch; every
// launch leaves them zero; launches that share them must be ordered on one stream.
TITB_API int titb_norm_bwd_onepass(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                   const void* dres, void* dx, float* dw, float* db, float* scratch,
                                   unsigned* counters, long long rows, int C, int dtype, int rms, int accumulate_wgrad,
                                   cudaStream_t st) {
  if (!titb_norm_bwd_onepass_ok(rows, C, dtype, dy, x, w, dres, dx) || !scratch || !counters || !dw ||
      (!rms && (!db || !mean)))
    return (int)cudaErrorInvalidValue;
  if (dtype == 1)
    return rms ? norm_bwd_onepass_launch<bf16, true>(dy, x, w, mean, rstd, dres, dx, dw, db, scratch, counters, rows, C,
                                                     accumulate_wgrad, st)
               : norm_bwd_onepass_launch<bf16, false>(dy, x, w, mean, rstd, dres, dx, dw, db, scratch, counters, rows,
                                                      C, accumulate_wgrad, st);
  return rms ? norm_bwd_onepass_launch<float, true>(dy, x, w, mean, rstd, dres, dx, dw, db, scratch, counters, rows, C,
                                                    accumulate_wgrad, st)
             : norm_bwd_onepass_launch<float, false>(dy, x, w, mean, rstd, dres, dx, dw, db, scratch, counters, rows,
                                                     C, accumulate_wgrad, st);
}
