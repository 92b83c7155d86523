// LayerNorm and RMSNorm, forward and backward, for bf16 and fp32 rows.
//
// Counterpart of infini_train/src/kernels/cuda/layernorm.cu:9-55 (forward) and
// :87-138 (backward).  Differences that matter on B200:
//  * a row is read once with 128-bit loads and kept in registers (the reference
//    makes two passes and uses E[x^2]-mean^2; here the variance is the two-pass
//    form computed from registers),
//  * one warp owns a row when it fits (no block barrier); wide rows use a CTA,
//  * dweight/dbias are reduced deterministically in two stages through a scratch
//    buffer instead of one atomicAdd per element per token (reference :135-136).
#include "api.h"
#include "common.cuh"

namespace titb {

// Sum two values over the G threads that share a row.
template <int G>
__device__ __forceinline__ void group_sum2(float& a, float& b, float* red) {
  a = warp_sum(a);
  b = warp_sum(b);
  if constexpr (G > 32) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    constexpr int NW = G / 32;
    __syncthreads();
    if (lane == 0) { red[w] = a; red[NW + w] = b; }
    __syncthreads();
    float ra = (lane < NW) ? red[lane] : 0.f;
    float rb = (lane < NW) ? red[NW + lane] : 0.f;
    a = warp_sum(ra);
    b = warp_sum(rb);
  }
}

// G = 32: one warp per row, several rows per CTA.  G > 32: the CTA (G threads) owns a row.
template <typename T, int MAXV, int G, bool RMS>
__global__ void norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                long long rows, int C, float eps) {
  constexpr int VN = VecN<T>::n;
  __shared__ float red[2 * (G > 32 ? G / 32 : 1)];
  const int tig = (G == 32) ? (threadIdx.x & 31) : threadIdx.x;  // thread in group
  const long long row = (G == 32) ? (blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5)) : blockIdx.x;
  if (G == 32 && row >= rows) return;
  const int nvec = C / VN;
  const T* xr = x + row * C;
  Pack<T, VN> xv[MAXV];
  float s = 0.f, s2 = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = tig + k * G;
    if (i < nvec) {
      xv[k] = ld128(xr + i * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) s += to_f32(xv[k].v[e]);
    }
  }
  float dummy = 0.f;
  group_sum2<G>(s, dummy, red);
  const float mean = RMS ? 0.f : s / C;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = tig + k * G;
    if (i < nvec) {
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        float d = to_f32(xv[k].v[e]) - mean;
        s2 += d * d;
      }
    }
  }
  dummy = 0.f;
  group_sum2<G>(s2, dummy, red);
  const float rstd = rsqrtf(s2 / C + eps);
  if (tig == 0) {
    if (!RMS && mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  T* yr = y + row * C;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = tig + k * G;
    if (i < nvec) {
      Pack<T, VN> wv = ld128(w + i * VN), ov;
      Pack<T, VN> bv;
      if (!RMS) bv = ld128(b + i * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        float n = (to_f32(xv[k].v[e]) - mean) * rstd;
        float o = n * to_f32(wv.v[e]);
        if (!RMS) o += to_f32(bv.v[e]);
        ov.v[e] = from_f32<T>(o);
      }
      st128(yr + i * VN, ov);
    }
  }
}

// Backward.  Every group walks rows with a grid stride and keeps dw/db partial sums
// for the columns it owns in registers; the partials go to scratch[2][nparts][C].
template <typename T, int MAXV, int G, bool RMS>
__global__ void norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                const T* __restrict__ dres, const float* __restrict__ mean_in,
                                const float* __restrict__ rstd_in, T* __restrict__ dx, float* __restrict__ scratch,
                                long long rows, int C, int nparts) {
  constexpr int VN = VecN<T>::n;
  __shared__ float red[2 * (G > 32 ? G / 32 : 1)];
  const int tig = (G == 32) ? (threadIdx.x & 31) : threadIdx.x;
  const int groups_per_block = (G == 32) ? (blockDim.x >> 5) : 1;
  const int gib = (G == 32) ? (threadIdx.x >> 5) : 0;  // group in block
  const long long group = blockIdx.x * (long long)groups_per_block + gib;
  const long long ngroups = gridDim.x * (long long)groups_per_block;
  const int nvec = C / VN;

  float dwacc[MAXV][VN], dbacc[MAXV][VN];
  Pack<T, VN> wv[MAXV];
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = tig + k * G;
#pragma unroll
    for (int e = 0; e < VN; ++e) { dwacc[k][e] = 0.f; dbacc[k][e] = 0.f; }
    if (i < nvec) wv[k] = ld128(w + i * VN);
  }

  for (long long row = group; row < rows; row += ngroups) {
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    const T* xr = x + row * C;
    const T* dyr = dy + row * C;
    Pack<T, VN> xv[MAXV], dv[MAXV];
    float s1 = 0.f, s2 = 0.f;  // sum(dnorm), sum(dnorm * norm)
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = tig + k * G;
      if (i < nvec) {
        xv[k] = ld128(xr + i * VN);
        dv[k] = ld128(dyr + i * VN);
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          float n = (to_f32(xv[k].v[e]) - mean) * rstd;
          float g = to_f32(dv[k].v[e]);
          float dn = g * to_f32(wv[k].v[e]);
          s1 += dn;
          s2 += dn * n;
          dwacc[k][e] += g * n;
          dbacc[k][e] += g;
        }
      }
    }
    group_sum2<G>(s1, s2, red);
    const float m1 = RMS ? 0.f : s1 / C, m2 = s2 / C;
    T* dxr = dx + row * C;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = tig + k * G;
      if (i < nvec) {
        Pack<T, VN> ov, rv;
        if (dres != nullptr) rv = ld128(dres + row * C + i * VN);
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          float n = (to_f32(xv[k].v[e]) - mean) * rstd;
          float dn = to_f32(dv[k].v[e]) * to_f32(wv[k].v[e]);
          float o = (dn - m1 - n * m2) * rstd;
          if (dres != nullptr) o += to_f32(rv.v[e]);
          ov.v[e] = from_f32<T>(o);
        }
        st128(dxr + i * VN, ov);
      }
    }
  }

  // Stage 1 of the dw/db reduction: the groups of a CTA fold their sums in a fixed
  // order through shared memory, then the CTA writes one partial row.
  extern __shared__ float acc_smem[];  // [2][C] when G == 32
  float* dwp = scratch + (long long)blockIdx.x * C;
  float* dbp = scratch + ((long long)nparts + blockIdx.x) * C;
  if constexpr (G == 32) {
    for (int g = 0; g < groups_per_block; ++g) {
      if (gib == g) {
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
          const int i = tig + k * G;
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
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      dwp[c] = acc_smem[c];
      if (!RMS) dbp[c] = acc_smem[C + c];
    }
  } else {
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = tig + k * G;
      if (i < nvec) {
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          dwp[i * VN + e] = dwacc[k][e];
          if (!RMS) dbp[i * VN + e] = dbacc[k][e];
        }
      }
    }
  }
}

template <typename P>
__device__ __forceinline__ void opaque128(P& p) {
  static_assert(sizeof(P) == 16, "128-bit pack expected");
  uint32_t* u = reinterpret_cast<uint32_t*>(&p);
  asm volatile("" : "+r"(u[0]), "+r"(u[1]), "+r"(u[2]), "+r"(u[3]));
}

// Four independent warp sums with interleaved shuffles (one exposed shuffle latency instead of four).
__device__ __forceinline__ void warp_sum4(float& a, float& b, float& c, float& d) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ta = __shfl_xor_sync(0xffffffffu, a, o), tb = __shfl_xor_sync(0xffffffffu, b, o);
    const float tc = __shfl_xor_sync(0xffffffffu, c, o), td = __shfl_xor_sync(0xffffffffu, d, o);
    a += ta; b += tb; c += tc; d += td;
  }
}

// Backward for rows that fit one warp (C <= 32 * NV * VN): 8 warps per CTA, 2 CTAs per SM, every warp keeps
// two rows in flight (all loads of both rows are issued before the first use), which puts about 100 KB of
// loads in flight per SM.  `dres` (optional) is a gradient that arrives through a residual connection around
// the norm: it is added to dx here instead of by a separate kernel.  The dweight / dbias partial sums of a warp
// live in its private slice of shared memory (registers are needed for the two rows), laid out so that every
// access is a conflict-free float4 per lane; at the end they are folded over the CTA's warps in warp order and
// leave as one partial row per CTA: scratch[0][cta][C] (dweight), scratch[1][cta][C] (dbias).
template <typename T, int NV, bool RMS>
__global__ void __launch_bounds__(256, 2)
norm_bwd_rows2_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                      const T* __restrict__ dres, const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                      T* __restrict__ dx, float* __restrict__ scratch, long long rows, int C, int nparts) {
  constexpr int VN = VecN<T>::n;
  constexpr int Q = VN / 4;                       // float4 groups per 128-bit vector
  constexpr int kPerWarp = NV * Q * 32 * 4;       // floats of one gradient held by one warp
  constexpr int kGrads = RMS ? 1 : 2;
  extern __shared__ float4 acc4[];                // [8 warps][kGrads][NV][Q][32 lanes] float4
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long gw = blockIdx.x * 8LL + warp, nw = gridDim.x * 8LL;
  const int nvec = C / VN;
  const float invC = 1.f / C;
  float4* my_dw = acc4 + (warp * kGrads) * (kPerWarp / 4);
  float4* my_db = my_dw + kPerWarp / 4;

  Pack<T, VN> wv[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = lane + k * 32;
    if (i < nvec) wv[k] = ld128(w + i * VN);
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      my_dw[(k * Q + q) * 32 + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (!RMS) my_db[(k * Q + q) * 32 + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }

  for (long long r0 = gw; r0 < rows; r0 += 2 * nw) {
    const long long r1 = r0 + nw;
    const bool has1 = r1 < rows;
    Pack<T, VN> xa[NV], da[NV], xb[NV], db_[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = lane + k * 32;
      if (i < nvec) {
        xa[k] = ld128(x + r0 * C + i * VN);
        da[k] = ld128(dy + r0 * C + i * VN);
        if (has1) {
          xb[k] = ld128(x + r1 * C + i * VN);
          db_[k] = ld128(dy + r1 * C + i * VN);
        }
      }
    }
    const float mean0 = RMS ? 0.f : mean_in[r0], rstd0 = rstd_in[r0];
    const float mean1 = (RMS || !has1) ? 0.f : mean_in[r1], rstd1 = has1 ? rstd_in[r1] : 0.f;
    float s1a = 0.f, s2a = 0.f, s1b = 0.f, s2b = 0.f;  // sum(dnorm), sum(dnorm * norm) of the two rows
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = lane + k * 32;
      if (i < nvec) {
#pragma unroll
        for (int q = 0; q < Q; ++q) {
          float gw4[4], gb4[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int e = q * 4 + j;
            const float wf = to_f32(wv[k].v[e]);
            const float n0 = (to_f32(xa[k].v[e]) - mean0) * rstd0;
            const float g0 = to_f32(da[k].v[e]);
            s1a += g0 * wf;
            s2a += g0 * wf * n0;
            gw4[j] = g0 * n0;
            gb4[j] = g0;
            if (has1) {
              const float n1 = (to_f32(xb[k].v[e]) - mean1) * rstd1;
              const float g1 = to_f32(db_[k].v[e]);
              s1b += g1 * wf;
              s2b += g1 * wf * n1;
              gw4[j] += g1 * n1;
              gb4[j] += g1;
            }
          }
          float4 a = my_dw[(k * Q + q) * 32 + lane];
          a.x += gw4[0]; a.y += gw4[1]; a.z += gw4[2]; a.w += gw4[3];
          my_dw[(k * Q + q) * 32 + lane] = a;
          if (!RMS) {
            float4 b = my_db[(k * Q + q) * 32 + lane];
            b.x += gb4[0]; b.y += gb4[1]; b.z += gb4[2]; b.w += gb4[3];
            my_db[(k * Q + q) * 32 + lane] = b;
          }
        }
      }
    }
    warp_sum4(s1a, s2a, s1b, s2b);
    // The packed rows pass through an opaque no-op: the compiler then unpacks them again below instead of keeping
    // every converted element of both rows alive across the reduction (which spilled).
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      opaque128(xa[k]); opaque128(da[k]); opaque128(xb[k]); opaque128(db_[k]);
    }
    const float m1a = RMS ? 0.f : s1a * invC, m2a = s2a * invC;
    const float m1b = RMS ? 0.f : s1b * invC, m2b = s2b * invC;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = lane + k * 32;
      if (i < nvec) {
        Pack<T, VN> oa, ob, ra, rb;
        if (dres != nullptr) {
          ra = ld128(dres + r0 * C + i * VN);
          if (has1) rb = ld128(dres + r1 * C + i * VN);
        }
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          const float wf = to_f32(wv[k].v[e]);
          const float n0 = (to_f32(xa[k].v[e]) - mean0) * rstd0;
          float o0 = (to_f32(da[k].v[e]) * wf - m1a - n0 * m2a) * rstd0;
          if (dres != nullptr) o0 += to_f32(ra.v[e]);
          oa.v[e] = from_f32<T>(o0);
          if (has1) {
            const float n1 = (to_f32(xb[k].v[e]) - mean1) * rstd1;
            float o1 = (to_f32(db_[k].v[e]) * wf - m1b - n1 * m2b) * rstd1;
            if (dres != nullptr) o1 += to_f32(rb.v[e]);
            ob.v[e] = from_f32<T>(o1);
          }
        }
        st128(dx + r0 * C + i * VN, oa);
        if (has1) st128(dx + r1 * C + i * VN, ob);
      }
    }
  }

  // fold the 8 warps' sums in warp order; one partial row per CTA.  Column c = vec * VN + q * 4 + j lives at
  // float index ((k * Q + q) * 32 + lane) * 4 + j of a warp's slice, with vec = lane + 32 k.
  __syncthreads();
  const float* accf = reinterpret_cast<const float*>(acc4);
  float* dwp = scratch + (long long)blockIdx.x * C;
  float* dbp = scratch + ((long long)nparts + blockIdx.x) * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const int vec = c / VN, e = c - vec * VN;
    const int k = vec >> 5, ln = vec & 31, q = e >> 2, j = e & 3;
    const int idx = ((k * Q + q) * 32 + ln) * 4 + j;
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      tw += accf[(g * kGrads) * kPerWarp + idx];
      if (!RMS) tb += accf[(g * kGrads + 1) * kPerWarp + idx];
    }
    dwp[c] = tw;
    if (!RMS) dbp[c] = tb;
  }
}

// Stage 2: out[c] (+)= sum_p scratch[p][c] in a fixed order.  The partial rows are a megabyte at most, so the pass is
// pure latency: 32 columns per CTA and kFoldTy threads per column, each summing every kFoldTy-th partial row with four
// independent accumulators (four loads in flight), then one fixed-order fold through shared memory.
constexpr int kFoldTy = 32;
__device__ __forceinline__ void fold_partial_rows(const float* __restrict__ src, float* __restrict__ out, int used, int C,
                                                  int accumulate) {
  __shared__ float sm[kFoldTy][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < C) {
    int p = ty;
    for (; p + 3 * kFoldTy < used; p += 4 * kFoldTy) {
      s0 += src[(long long)p * C + c];
      s1 += src[(long long)(p + kFoldTy) * C + c];
      s2 += src[(long long)(p + 2 * kFoldTy) * C + c];
      s3 += src[(long long)(p + 3 * kFoldTy) * C + c];
    }
    for (; p < used; p += kFoldTy) s0 += src[(long long)p * C + c];
  }
  sm[ty][tx] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (ty == 0 && c < C) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < kFoldTy; ++j) t += sm[j][tx];
    out[c] = accumulate ? out[c] + t : t;
  }
}

// Both gradients in one launch: blockIdx.y = 0 folds the dweight partial rows, 1 the dbias rows.
__global__ void __launch_bounds__(32 * kFoldTy)
partial_colsum2_kernel(const float* __restrict__ scratch, float* __restrict__ dw, float* __restrict__ db, int used,
                       int nparts, int C, int accumulate) {
  fold_partial_rows(scratch + (long long)blockIdx.y * nparts * C, blockIdx.y == 0 ? dw : db, used, C, accumulate);
}

// Scalar fallbacks (any C): CTA per row, re-reading the row from L1/L2.
template <typename T, bool RMS>
__global__ void norm_fwd_generic(const T* x, const T* w, const T* b, T* y, float* mean_out, float* rstd_out,
                                 long long rows, int C, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * C;
  float s = 0.f;
  if (!RMS) for (int i = threadIdx.x; i < C; i += blockDim.x) s += to_f32(xr[i]);
  const float mean = RMS ? 0.f : block_sum(s, red) / C;
  float s2 = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) { float d = to_f32(xr[i]) - mean; s2 += d * d; }
  const float rstd = rsqrtf(block_sum(s2, red) / C + eps);
  if (threadIdx.x == 0) {
    if (!RMS && mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float o = (to_f32(xr[i]) - mean) * rstd * to_f32(w[i]);
    if (!RMS) o += to_f32(b[i]);
    y[row * C + i] = from_f32<T>(o);
  }
}
template <typename T, bool RMS>
__global__ void norm_bwd_dx_generic(const T* dy, const T* x, const T* w, const T* dres, const float* mean_in,
                                    const float* rstd_in, T* dx, long long rows, int C) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const float mean = RMS ? 0.f : mean_in[row], rstd = rstd_in[row];
  float s1 = 0.f, s2 = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float n = (to_f32(x[row * C + i]) - mean) * rstd;
    float dn = to_f32(dy[row * C + i]) * to_f32(w[i]);
    s1 += dn; s2 += dn * n;
  }
  s1 = block_sum(s1, red);
  s2 = block_sum(s2, red);
  const float m1 = RMS ? 0.f : s1 / C, m2 = s2 / C;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float n = (to_f32(x[row * C + i]) - mean) * rstd;
    float dn = to_f32(dy[row * C + i]) * to_f32(w[i]);
    float o = (dn - m1 - n * m2) * rstd;
    if (dres != nullptr) o += to_f32(dres[row * C + i]);
    dx[row * C + i] = from_f32<T>(o);
  }
}
template <typename T, bool RMS>
__global__ void norm_bwd_dw_generic(const T* dy, const T* x, const float* mean_in, const float* rstd_in, float* dw,
                                    float* db, long long rows, int C, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float sw = 0.f, sb = 0.f;
  for (long long r = 0; r < rows; ++r) {
    float g = to_f32(dy[r * C + c]);
    float n = (to_f32(x[r * C + c]) - (RMS ? 0.f : mean_in[r])) * rstd_in[r];
    sw += g * n; sb += g;
  }
  dw[c] = accumulate ? dw[c] + sw : sw;
  if (!RMS && db) db[c] = accumulate ? db[c] + sb : sb;
}

// Sizes of the caller-provided scratch, fixed so that callers (and the allocation-free entry point) can size it without
// a device query; grids are derived from the SM count of the device and clamped to these.
constexpr int kNormBwdBlocks = 296;  // most CTAs the warp-per-row backward kernels launch
constexpr int kNormBwdParts = 592;   // partial rows per gradient in the scratch buffer

struct NormPlan {
  int G;      // 32 or 256; 0 = generic fallback
  int maxv;   // register vectors per thread
};
template <typename T>
static NormPlan plan_norm(int C) {
  constexpr int VN = VecN<T>::n;
  NormPlan p{0, 0};
  if (C % VN != 0) return p;
  const int nvec = C / VN;
  if (nvec <= 32 * 4) { p.G = 32; p.maxv = 4; }
  else if (nvec <= 32 * 8) { p.G = 32; p.maxv = 8; }
  else if (nvec <= 256 * 2) { p.G = 256; p.maxv = 2; }
  else if (nvec <= 256 * 8) { p.G = 256; p.maxv = 8; }
  return p;
}

template <typename T, bool RMS>
static int norm_fwd_launch(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                           long long rows, int C, float eps, cudaStream_t st) {
  if (rows <= 0) return 0;
  const T* X = static_cast<const T*>(x); const T* W = static_cast<const T*>(w); const T* Bv = static_cast<const T*>(b);
  T* Y = static_cast<T*>(y);
  NormPlan p = plan_norm<T>(C);
  const bool aligned = !((uintptr_t)x & 15) && !((uintptr_t)y & 15) && !((uintptr_t)w & 15) && !((uintptr_t)b & 15);
  if (p.G == 32 && aligned) {
    const int blocks = (int)((rows + 3) / 4);
    if (p.maxv == 4) norm_fwd_kernel<T, 4, 32, RMS><<<blocks, 128, 0, st>>>(X, W, Bv, Y, mean, rstd, rows, C, eps);
    else norm_fwd_kernel<T, 8, 32, RMS><<<blocks, 128, 0, st>>>(X, W, Bv, Y, mean, rstd, rows, C, eps);
  } else if (p.G == 256 && aligned) {
    if (p.maxv == 2) norm_fwd_kernel<T, 2, 256, RMS><<<(unsigned)rows, 256, 0, st>>>(X, W, Bv, Y, mean, rstd, rows, C, eps);
    else norm_fwd_kernel<T, 8, 256, RMS><<<(unsigned)rows, 256, 0, st>>>(X, W, Bv, Y, mean, rstd, rows, C, eps);
  } else {
    norm_fwd_generic<T, RMS><<<(unsigned)rows, 256, 0, st>>>(X, W, Bv, Y, mean, rstd, rows, C, eps);
  }
  return (int)cudaGetLastError();
}


template <typename T, bool RMS>
static int norm_bwd_launch(const void* dy, const void* x, const void* w, const void* dres, const float* mean,
                           const float* rstd, void* dx, float* dw, float* db, float* scratch, long long rows, int C,
                           int accumulate, cudaStream_t st) {
  if (rows <= 0) return 0;
  constexpr int VN = VecN<T>::n;
  const T* DY = static_cast<const T*>(dy); const T* X = static_cast<const T*>(x); const T* W = static_cast<const T*>(w);
  const T* R = static_cast<const T*>(dres);
  T* DX = static_cast<T*>(dx);
  NormPlan p = plan_norm<T>(C);
  const bool aligned = !((uintptr_t)x & 15) && !((uintptr_t)dy & 15) && !((uintptr_t)w & 15) && !((uintptr_t)dx & 15) &&
                       !((uintptr_t)dres & 15);
  if (p.G != 0 && aligned && scratch != nullptr) {
    const int nparts = kNormBwdParts;  // scratch is [2][kNormBwdParts][C]; the first `used` rows are written
    int used;
    if (p.G == 32) {
      used = 2 * device_sm_count();
      if (used > kNormBwdBlocks) used = kNormBwdBlocks;
      const int nv = (C / VN + 31) / 32;  // 128-bit vectors per lane
      auto launch = [&](auto kern, int NVc) {
        // per warp and gradient: NVc vectors * VN floats * 32 lanes
        const size_t sm = 8 * (size_t)(RMS ? 1 : 2) * NVc * VN * 32 * sizeof(float);
        if (sm > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        kern<<<used, 256, sm, st>>>(DY, X, W, R, mean, rstd, DX, scratch, rows, C, nparts);
      };
      if (nv <= 3) launch(norm_bwd_rows2_kernel<T, 3, RMS>, 3);
      else if (nv <= 4) launch(norm_bwd_rows2_kernel<T, 4, RMS>, 4);
      else {  // up to 8 vectors per lane: one row at a time per warp, sums in registers
        used = kNormBwdBlocks;
        norm_bwd_kernel<T, 8, 32, RMS><<<used, 128, 2 * (size_t)C * sizeof(float), st>>>(DY, X, W, R, mean, rstd, DX, scratch, rows, C, nparts);
      }
    } else {
      used = kNormBwdParts;
      if (p.maxv == 2) norm_bwd_kernel<T, 2, 256, RMS><<<used, 256, 0, st>>>(DY, X, W, R, mean, rstd, DX, scratch, rows, C, nparts);
      else norm_bwd_kernel<T, 8, 256, RMS><<<used, 256, 0, st>>>(DY, X, W, R, mean, rstd, DX, scratch, rows, C, nparts);
    }
    partial_colsum2_kernel<<<dim3((C + 31) / 32, (!RMS && db) ? 2 : 1), 32 * kFoldTy, 0, st>>>(scratch, dw, db, used, nparts, C, accumulate);
  } else {
    norm_bwd_dx_generic<T, RMS><<<(unsigned)rows, 256, 0, st>>>(DY, X, W, R, mean, rstd, DX, rows, C);
    norm_bwd_dw_generic<T, RMS><<<(C + 127) / 128, 128, 0, st>>>(DY, X, mean, rstd, dw, db, rows, C, accumulate);
  }
  return (int)cudaGetLastError();
}

}  // namespace titb

using namespace titb;

TITB_API int titb_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                                long long rows, int C, float eps, int dtype, cudaStream_t stream) {
  return dtype == 1 ? norm_fwd_launch<bf16, false>(x, w, b, y, mean, rstd, rows, C, eps, stream)
                    : norm_fwd_launch<float, false>(x, w, b, y, mean, rstd, rows, C, eps, stream);
}
TITB_API int titb_layernorm_bwd_blocks(long long) { return kNormBwdParts; }
TITB_API int titb_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                void* dx, float* dw, float* db, float* scratch, long long rows, int C, int dtype,
                                int accumulate_wgrad, const void* dres, cudaStream_t stream) {
  return dtype == 1
             ? norm_bwd_launch<bf16, false>(dy, x, w, dres, mean, rstd, dx, dw, db, scratch, rows, C, accumulate_wgrad, stream)
             : norm_bwd_launch<float, false>(dy, x, w, dres, mean, rstd, dx, dw, db, scratch, rows, C, accumulate_wgrad, stream);
}
TITB_API int titb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int C, float eps,
                              int dtype, cudaStream_t stream) {
  return dtype == 1 ? norm_fwd_launch<bf16, true>(x, w, w, y, nullptr, rstd, rows, C, eps, stream)
                    : norm_fwd_launch<float, true>(x, w, w, y, nullptr, rstd, rows, C, eps, stream);
}
TITB_API int titb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                              float* scratch, long long rows, int C, int dtype, int accumulate_wgrad, const void* dres,
                              cudaStream_t stream) {
  return dtype == 1
             ? norm_bwd_launch<bf16, true>(dy, x, w, dres, nullptr, rstd, dx, dw, nullptr, scratch, rows, C, accumulate_wgrad, stream)
             : norm_bwd_launch<float, true>(dy, x, w, dres, nullptr, rstd, dx, dw, nullptr, scratch, rows, C, accumulate_wgrad, stream);
}
