// Element-wise, broadcast, cast, fill, transpose and column-sum kernels.
//
// Counterparts of the reference's infini_train/src/kernels/cuda/elementwise.cu
// (unary :14-21/:141-150, binary with broadcast :23-48/:152-171), sigmoid.cu,
// fill.cu, transform.cu (tril/triu :9-54, transpose :138-165) and the
// ReduceColumns kernel of linear.cu:130-146.  Here every kernel moves 128 bits
// per thread per access, takes bf16 or fp32, and keeps broadcast metadata in
// kernel parameters (the reference allocates and copies it per call).
#include "api.h"
#include "common.cuh"

namespace titb {

constexpr int kEwThreads = 256;

static inline int ew_blocks(long long nvec) {
  long long b = (nvec + kEwThreads - 1) / kEwThreads;
  const long long cap = 148LL * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

// Applies f to every element; vector body + scalar tail.
template <typename T, typename F>
__global__ void map1_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, int vec, F f) {
  constexpr int VN = VecN<T>::n;
  const long long nvec = vec ? n / VN : 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<T, VN> a = ld128(x + i * VN), o;
#pragma unroll
    for (int e = 0; e < VN; ++e) o.v[e] = from_f32<T>(f(to_f32(a.v[e])));
    st128(y + i * VN, o);
  }
  for (long long i = nvec * VN + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = from_f32<T>(f(to_f32(x[i])));
}
template <typename T, typename F>
__global__ void map2_kernel(const T* __restrict__ a_, const T* __restrict__ b_, T* __restrict__ y, long long n, int vec,
                            F f) {
  constexpr int VN = VecN<T>::n;
  const long long nvec = vec ? n / VN : 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<T, VN> a = ld128(a_ + i * VN), b = ld128(b_ + i * VN), o;
#pragma unroll
    for (int e = 0; e < VN; ++e) o.v[e] = from_f32<T>(f(to_f32(a.v[e]), to_f32(b.v[e])));
    st128(y + i * VN, o);
  }
  for (long long i = nvec * VN + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = from_f32<T>(f(to_f32(a_[i]), to_f32(b_[i])));
}

template <typename T, typename F>
static int map1(const void* x, void* y, long long n, cudaStream_t st, F f) {
  if (n <= 0) return 0;
  const int al = !((uintptr_t)x & 15) && !((uintptr_t)y & 15);
  map1_kernel<T, F><<<ew_blocks(al ? n / VecN<T>::n + 1 : n), kEwThreads, 0, st>>>((const T*)x, (T*)y, n, al, f);
  return (int)cudaGetLastError();
}
template <typename T, typename F>
static int map2(const void* a, const void* b, void* y, long long n, cudaStream_t st, F f) {
  if (n <= 0) return 0;
  const int al = !((uintptr_t)a & 15) && !((uintptr_t)b & 15) && !((uintptr_t)y & 15);
  map2_kernel<T, F><<<ew_blocks(al ? n / VecN<T>::n + 1 : n), kEwThreads, 0, st>>>((const T*)a, (const T*)b, (T*)y, n, al,
                                                                                  f);
  return (int)cudaGetLastError();
}

#define DISPATCH_DT(dtype, CALL_F32, CALL_BF16) ((dtype) == 1 ? (CALL_BF16) : (CALL_F32))

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// SwiGLU over a fused [rows, 2F] projection.
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int F) {
  constexpr int VN = VecN<T>::n;
  const int fv = F / VN;
  const long long total = rows * fv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / fv;
    const int c = (int)(i - r * fv) * VN;
    Pack<T, VN> g = ld128(x + r * 2 * F + c), u = ld128(x + r * 2 * F + F + c), o;
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      float gf = to_f32(g.v[e]);
      o.v[e] = from_f32<T>(gf * sigmoidf_(gf) * to_f32(u.v[e]));
    }
    st128(y + r * F + c, o);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx, long long rows,
                                  int F) {
  constexpr int VN = VecN<T>::n;
  const int fv = F / VN;
  const long long total = rows * fv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / fv;
    const int c = (int)(i - r * fv) * VN;
    Pack<T, VN> g = ld128(x + r * 2 * F + c), u = ld128(x + r * 2 * F + F + c), d = ld128(dy + r * F + c), og, ou;
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      float gf = to_f32(g.v[e]), uf = to_f32(u.v[e]), df = to_f32(d.v[e]);
      float s = sigmoidf_(gf);
      float silu = gf * s;
      og.v[e] = from_f32<T>(df * uf * (s + silu * (1.f - s)));
      ou.v[e] = from_f32<T>(df * silu);
    }
    st128(dx + r * 2 * F + c, og);
    st128(dx + r * 2 * F + F + c, ou);
  }
}

// Rotary embedding on [B, T, H, hd]: pairs (i, i + hd/2), angle (t + offset) * theta^(-2i/hd).
template <typename T>
__global__ void rope_kernel(const T* x, T* y, long long BT, int T_, int H, int hd, long long stride_t,
                            int pos_offset, float log2_theta, int inverse) {
  constexpr int VN = VecN<T>::n;
  const int half = hd / 2;
  const int hv = half / VN;
  const long long total = BT * H * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % hv);
    const long long bth = i / hv;
    const long long bt = bth / H;
    const int t = (int)(bt % T_) + pos_offset;
    const int hh = (int)(bth - bt * H);
    const T* xp = x + bt * stride_t + hh * hd + v * VN;
    T* yp = y + bt * stride_t + hh * hd + v * VN;
    Pack<T, VN> a = ld128(xp), b = ld128(xp + half), oa, ob;
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      const int idx = v * VN + e;
      const float inv_freq = exp2f(-log2_theta * (2.f * idx / hd));
      float s, c;
      sincosf(t * inv_freq, &s, &c);
      if (inverse) s = -s;
      const float af = to_f32(a.v[e]), bf = to_f32(b.v[e]);
      oa.v[e] = from_f32<T>(af * c - bf * s);
      ob.v[e] = from_f32<T>(bf * c + af * s);
    }
    st128(yp, oa);
    st128(yp + half, ob);
  }
}

template <typename TS, typename TD>
__global__ void cast_kernel(const TS* __restrict__ x, TD* __restrict__ y, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 3 < n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) y[i + e] = from_f32<TD>(to_f32(x[i + e]));
    } else {
      for (long long j = i; j < n; ++j) y[j] = from_f32<TD>(to_f32(x[j]));
    }
  }
}

template <typename T>
__global__ void fill_kernel(T* __restrict__ y, long long n, float value) {
  const T v = from_f32<T>(value);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = v;
}

// y = a (op) broadcast(b), generic N-d broadcast; metadata by value.
template <typename T>
__global__ void binary_bcast_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y,
                                    long long n, TitbBroadcast bc) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    long long rem = i, bo = 0;
#pragma unroll 1
    for (int d = bc.ndim - 1; d >= 0; --d) {
      const long long q = rem / bc.a_dims[d];
      bo += (rem - q * bc.a_dims[d]) * bc.b_strides[d];
      rem = q;
    }
    const float af = to_f32(a[i]), bf = to_f32(b[bo]);
    float r;
    switch (op) {
      case TITB_ADD: r = af + bf; break;
      case TITB_SUB: r = af - bf; break;
      case TITB_MUL: r = af * bf; break;
      default: r = af / bf; break;
    }
    y[i] = from_f32<T>(r);
  }
}

// Tiled transpose of the last two dims: in [batch, R, C] -> out [batch, C, R].
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ x, T* __restrict__ y, int R, int C) {
  __shared__ T tile[32][33];
  const long long base = (long long)blockIdx.z * R * C;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < R && c < C) tile[j][threadIdx.x] = x[base + (long long)r * C + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < R && c < C) y[base + (long long)c * R + r] = tile[threadIdx.x][j];
  }
}

template <typename T>
__global__ void tri_kernel(const T* __restrict__ x, T* __restrict__ y, int R, int C, int diagonal, int upper) {
  const long long n = (long long)R * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / C), c = (int)(i % C);
    const bool keep = upper ? (r - c + diagonal <= 0) : (r - c + diagonal >= 0);
    y[i] = keep ? x[i] : from_f32<T>(0.f);
  }
}

// Column sums of a [rows, C] matrix in two deterministic stages (bias gradients).
constexpr int kColsumParts = 296;  // partial rows in the caller-provided scratch; the grid is sized from the SM count and clamped to it
// Stage 1: a warp reads whole row segments (coalesced), four rows in flight, and keeps the sums of its NV * VN
// columns per lane in registers; the 8 warps of a CTA fold their sums in warp order through shared memory and the
// CTA writes one partial row.  blockIdx.y selects a strip of 32 * NV * VN columns.
template <typename T, int NV>
__global__ void __launch_bounds__(256, 2) colsum_rows_kernel(const T* __restrict__ x, float* __restrict__ scratch,
                                                          long long rows, int C) {
  constexpr int VN = VecN<T>::n;
  constexpr int kStrip = 32 * NV * VN;
  __shared__ float sm[kStrip];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.y * kStrip;
  const long long gw = blockIdx.x * 8LL + warp, nw = gridDim.x * 8LL;
  float acc[NV][VN];
#pragma unroll
  for (int k = 0; k < NV; ++k)
#pragma unroll
    for (int e = 0; e < VN; ++e) acc[k][e] = 0.f;
  // one pointer per lane walks down the rows (row stride of this warp: nw rows); which of the NV vectors of a row lie
  // inside the matrix is the same for every row
  const long long step = nw * static_cast<long long>(C);
  const T* px = x + gw * static_cast<long long>(C) + c0 + lane * VN;
  bool in[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) in[k] = c0 + (lane + k * 32) * VN < C;
  for (long long r = gw; r < rows; r += 4 * nw, px += 4 * step) {
    Pack<T, VN> v[4][NV];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const bool row_ok = r + q * nw < rows;
#pragma unroll
      for (int k = 0; k < NV; ++k)
        if (row_ok && in[k]) v[q][k] = ld128(px + q * step + k * 32 * VN);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const bool row_ok = r + q * nw < rows;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        if (row_ok && in[k]) {
#pragma unroll
          for (int e = 0; e < VN; ++e) acc[k][e] += to_f32(v[q][k].v[e]);
        }
      }
    }
  }
  for (int g = 0; g < 8; ++g) {
    if (warp == g) {
#pragma unroll
      for (int k = 0; k < NV; ++k)
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          const int i = (lane + k * 32) * VN + e;
          sm[i] = (g == 0 ? 0.f : sm[i]) + acc[k][e];
        }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < kStrip; i += blockDim.x)
    if (c0 + i < C) scratch[(long long)blockIdx.x * C + c0 + i] = sm[i];
}
// Stage 2: out[c] (+)= sum over the partial rows, fixed order.  A megabyte at most, so pure latency: 32 columns per CTA,
// kFoldTy threads per column, four independent accumulators per thread (four loads in flight), one shared-memory fold.
constexpr int kFoldTy = 32;
__global__ void __launch_bounds__(32 * kFoldTy)
colsum_stage2(const float* __restrict__ scratch, float* __restrict__ out, int nparts, int C, int accumulate) {
  __shared__ float sm[kFoldTy][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < C) {
    int p = ty;
    for (; p + 3 * kFoldTy < nparts; p += 4 * kFoldTy) {
      s0 += scratch[(long long)p * C + c];
      s1 += scratch[(long long)(p + kFoldTy) * C + c];
      s2 += scratch[(long long)(p + 2 * kFoldTy) * C + c];
      s3 += scratch[(long long)(p + 3 * kFoldTy) * C + c];
    }
    for (; p < nparts; p += kFoldTy) s0 += scratch[(long long)p * C + c];
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
template <typename T>
__global__ void colsum_generic(const T* __restrict__ x, float* __restrict__ out, long long rows, int C, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (long long r = 0; r < rows; ++r) s += to_f32(x[r * C + c]);
  out[c] = accumulate ? out[c] + s : s;
}

}  // namespace titb

using namespace titb;

TITB_API int titb_gelu_fwd(const void* x, void* y, long long n, int dtype, cudaStream_t st) {
  auto f = [] __device__(float v) { return gelu_tanh(v); };
  return DISPATCH_DT(dtype, (map1<float>(x, y, n, st, f)), (map1<bf16>(x, y, n, st, f)));
}
TITB_API int titb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, int dtype, cudaStream_t st) {
  auto f = [] __device__(float g, float v) { return g * gelu_tanh_grad(v); };
  return DISPATCH_DT(dtype, (map2<float>(dy, x, dx, n, st, f)), (map2<bf16>(dy, x, dx, n, st, f)));
}

TITB_API int titb_swiglu_fwd(const void* x, void* y, long long rows, int F, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  const int vn = dtype == 1 ? 8 : 4;
  if (F % vn) return (int)cudaErrorInvalidValue;
  const int blocks = ew_blocks(rows * (F / vn));
  if (dtype == 1) swiglu_fwd_kernel<bf16><<<blocks, kEwThreads, 0, st>>>((const bf16*)x, (bf16*)y, rows, F);
  else swiglu_fwd_kernel<float><<<blocks, kEwThreads, 0, st>>>((const float*)x, (float*)y, rows, F);
  return (int)cudaGetLastError();
}
TITB_API int titb_swiglu_bwd(const void* dy, const void* x, void* dx, long long rows, int F, int dtype,
                             cudaStream_t st) {
  if (rows <= 0) return 0;
  const int vn = dtype == 1 ? 8 : 4;
  if (F % vn) return (int)cudaErrorInvalidValue;
  const int blocks = ew_blocks(rows * (F / vn));
  if (dtype == 1) swiglu_bwd_kernel<bf16><<<blocks, kEwThreads, 0, st>>>((const bf16*)dy, (const bf16*)x, (bf16*)dx, rows, F);
  else swiglu_bwd_kernel<float><<<blocks, kEwThreads, 0, st>>>((const float*)dy, (const float*)x, (float*)dx, rows, F);
  return (int)cudaGetLastError();
}

TITB_API int titb_rope(const void* x, void* y, int B, int T, int H, int hd, int pos_offset, float theta, int inverse,
                       int dtype, cudaStream_t st) {
  return titb_rope_strided(x, y, B, T, H, hd, (long long)H * hd, pos_offset, theta, inverse, dtype, st);
}

TITB_API int titb_rope_strided(const void* x, void* y, int B, int T, int H, int hd, long long stride_t, int pos_offset,
                               float theta, int inverse, int dtype, cudaStream_t st) {
  const long long BT = (long long)B * T;
  if (BT <= 0) return 0;
  const int vn = dtype == 1 ? 8 : 4;
  if ((hd / 2) % vn) return (int)cudaErrorInvalidValue;
  const int blocks = ew_blocks(BT * H * (hd / 2 / vn));
  const float l2 = log2f(theta);
  if (dtype == 1) rope_kernel<bf16><<<blocks, kEwThreads, 0, st>>>((const bf16*)x, (bf16*)y, BT, T, H, hd, stride_t, pos_offset, l2, inverse);
  else rope_kernel<float><<<blocks, kEwThreads, 0, st>>>((const float*)x, (float*)y, BT, T, H, hd, stride_t, pos_offset, l2, inverse);
  return (int)cudaGetLastError();
}

template <typename T>
static int unary_fwd_t(int op, const void* x, void* y, long long n, float s, cudaStream_t st) {
  switch (op) {
    case TITB_NEG: return map1<T>(x, y, n, st, [] __device__(float v) { return -v; });
    case TITB_RECIPROCAL: return map1<T>(x, y, n, st, [] __device__(float v) { return 1.f / v; });
    case TITB_SIN: return map1<T>(x, y, n, st, [] __device__(float v) { return sinf(v); });
    case TITB_COS: return map1<T>(x, y, n, st, [] __device__(float v) { return cosf(v); });
    case TITB_TANH: return map1<T>(x, y, n, st, [] __device__(float v) { return tanhf(v); });
    case TITB_POW_SCALAR_EXP: return map1<T>(x, y, n, st, [s] __device__(float v) { return powf(v, s); });
    case TITB_POW_SCALAR_BASE: return map1<T>(x, y, n, st, [s] __device__(float v) { return powf(s, v); });
    case TITB_RSQRT: return map1<T>(x, y, n, st, [] __device__(float v) { return 1.f / sqrtf(v); });
    case TITB_EQUALS_SCALAR: return map1<T>(x, y, n, st, [s] __device__(float v) { return v == s ? 1.f : 0.f; });
    case TITB_ADD_SCALAR: return map1<T>(x, y, n, st, [s] __device__(float v) { return v + s; });
    case TITB_MUL_SCALAR: return map1<T>(x, y, n, st, [s] __device__(float v) { return v * s; });
    case TITB_SIGMOID: return map1<T>(x, y, n, st, [] __device__(float v) { return 1.f / (1.f + expf(-v)); });
    case TITB_COPY: return map1<T>(x, y, n, st, [] __device__(float v) { return v; });
  }
  return (int)cudaErrorInvalidValue;
}
TITB_API int titb_unary_fwd(int op, const void* x, void* y, long long n, float s, int dtype, cudaStream_t st) {
  return DISPATCH_DT(dtype, (unary_fwd_t<float>(op, x, y, n, s, st)), (unary_fwd_t<bf16>(op, x, y, n, s, st)));
}

template <typename T>
static int unary_bwd_t(int op, const void* dy, const void* sv, void* dx, long long n, float s, cudaStream_t st) {
  switch (op) {
    case TITB_NEG: return map2<T>(dy, sv, dx, n, st, [] __device__(float g, float) { return -g; });
    case TITB_RECIPROCAL: return map2<T>(dy, sv, dx, n, st, [] __device__(float g, float x) { return -g / (x * x); });
    case TITB_SIN: return map2<T>(dy, sv, dx, n, st, [] __device__(float g, float x) { return g * cosf(x); });
    case TITB_COS: return map2<T>(dy, sv, dx, n, st, [] __device__(float g, float x) { return -g * sinf(x); });
    case TITB_TANH: return map2<T>(dy, sv, dx, n, st, [] __device__(float g, float y) { return g * (1.f - y * y); });
    case TITB_POW_SCALAR_EXP:
      return map2<T>(dy, sv, dx, n, st, [s] __device__(float g, float x) { return g * s * powf(x, s - 1.f); });
    case TITB_POW_SCALAR_BASE:
      return map2<T>(dy, sv, dx, n, st, [s] __device__(float g, float x) { return g * logf(s) * powf(s, x); });
    case TITB_RSQRT: return map2<T>(dy, sv, dx, n, st, [] __device__(float g, float x) { return g * (-0.5f / (x * sqrtf(x))); });
    case TITB_ADD_SCALAR: return map2<T>(dy, sv, dx, n, st, [] __device__(float g, float) { return g; });
    case TITB_MUL_SCALAR: return map2<T>(dy, sv, dx, n, st, [s] __device__(float g, float) { return g * s; });
    case TITB_SIGMOID: return map2<T>(dy, sv, dx, n, st, [] __device__(float g, float y) { return g * y * (1.f - y); });
    case TITB_COPY: return map2<T>(dy, sv, dx, n, st, [] __device__(float g, float) { return g; });
  }
  return (int)cudaErrorInvalidValue;
}
TITB_API int titb_unary_bwd(int op, const void* dy, const void* saved, void* dx, long long n, float s, int dtype,
                            cudaStream_t st) {
  return DISPATCH_DT(dtype, (unary_bwd_t<float>(op, dy, saved, dx, n, s, st)),
                     (unary_bwd_t<bf16>(op, dy, saved, dx, n, s, st)));
}

TITB_API int titb_binary_fwd(int op, const void* a, const void* b, void* y, long long n, TitbBroadcast bc, int dtype,
                             cudaStream_t st) {
  if (n <= 0) return 0;
  const int blocks = ew_blocks(n);
  if (dtype == 1) binary_bcast_kernel<bf16><<<blocks, kEwThreads, 0, st>>>(op, (const bf16*)a, (const bf16*)b, (bf16*)y, n, bc);
  else binary_bcast_kernel<float><<<blocks, kEwThreads, 0, st>>>(op, (const float*)a, (const float*)b, (float*)y, n, bc);
  return (int)cudaGetLastError();
}

TITB_API int titb_cast(const void* x, void* y, long long n, int sd, int dd, cudaStream_t st) {
  if (n <= 0) return 0;
  const int blocks = ew_blocks(n / 4 + 1);
  if (sd == 0 && dd == 1) cast_kernel<float, bf16><<<blocks, kEwThreads, 0, st>>>((const float*)x, (bf16*)y, n);
  else if (sd == 1 && dd == 0) cast_kernel<bf16, float><<<blocks, kEwThreads, 0, st>>>((const bf16*)x, (float*)y, n);
  else if (sd == 0 && dd == 0) cast_kernel<float, float><<<blocks, kEwThreads, 0, st>>>((const float*)x, (float*)y, n);
  else cast_kernel<bf16, bf16><<<blocks, kEwThreads, 0, st>>>((const bf16*)x, (bf16*)y, n);
  return (int)cudaGetLastError();
}

TITB_API int titb_fill(void* y, long long n, float value, int dtype, cudaStream_t st) {
  if (n <= 0) return 0;
  if (dtype == 1) fill_kernel<bf16><<<ew_blocks(n), kEwThreads, 0, st>>>((bf16*)y, n, value);
  else fill_kernel<float><<<ew_blocks(n), kEwThreads, 0, st>>>((float*)y, n, value);
  return (int)cudaGetLastError();
}

TITB_API int titb_transpose(const void* x, void* y, long long batch, int R, int C, int dtype, cudaStream_t st) {
  if (batch <= 0 || R <= 0 || C <= 0) return 0;
  dim3 grid((C + 31) / 32, (R + 31) / 32, (unsigned)batch), block(32, 8);
  if (dtype == 1) transpose_kernel<bf16><<<grid, block, 0, st>>>((const bf16*)x, (bf16*)y, R, C);
  else transpose_kernel<float><<<grid, block, 0, st>>>((const float*)x, (float*)y, R, C);
  return (int)cudaGetLastError();
}

TITB_API int titb_tri(const void* x, void* y, int R, int C, int diagonal, int upper, int dtype, cudaStream_t st) {
  const long long n = (long long)R * C;
  if (n <= 0) return 0;
  if (dtype == 1) tri_kernel<bf16><<<ew_blocks(n), kEwThreads, 0, st>>>((const bf16*)x, (bf16*)y, R, C, diagonal, upper);
  else tri_kernel<float><<<ew_blocks(n), kEwThreads, 0, st>>>((const float*)x, (float*)y, R, C, diagonal, upper);
  return (int)cudaGetLastError();
}

TITB_API int titb_colsum_blocks(long long) { return kColsumParts; }
TITB_API int titb_colsum(const void* x, float* out, long long rows, int C, int dtype, int accumulate, float* scratch,
                         cudaStream_t st) {
  if (C <= 0) return 0;
  const int vn = dtype == 1 ? 8 : 4;
  if (scratch && (C % vn) == 0 && !((uintptr_t)x & 15) && rows > 0) {
    // strips of 32 * NV vectors; NV = 3 fits widths that are multiples of 768 (bf16) exactly, NV = 4 otherwise
    const int nvec = C / vn;
    const int nv = (nvec % 96 == 0 || nvec <= 96) ? 3 : 4;
    const int strips = (nvec + 32 * nv - 1) / (32 * nv);
    int parts = (2 * device_sm_count() + strips - 1) / strips;
    if (parts > kColsumParts) parts = kColsumParts;
    if (parts > (rows + 7) / 8) parts = (int)((rows + 7) / 8);
    dim3 grid(parts, strips);
    if (dtype == 1) {
      if (nv == 3) colsum_rows_kernel<bf16, 3><<<grid, 256, 0, st>>>((const bf16*)x, scratch, rows, C);
      else colsum_rows_kernel<bf16, 4><<<grid, 256, 0, st>>>((const bf16*)x, scratch, rows, C);
    } else {
      if (nv == 3) colsum_rows_kernel<float, 3><<<grid, 256, 0, st>>>((const float*)x, scratch, rows, C);
      else colsum_rows_kernel<float, 4><<<grid, 256, 0, st>>>((const float*)x, scratch, rows, C);
    }
    colsum_stage2<<<(C + 31) / 32, 32 * kFoldTy, 0, st>>>(scratch, out, parts, C, accumulate);
  } else {
    if (dtype == 1) colsum_generic<bf16><<<(C + 127) / 128, 128, 0, st>>>((const bf16*)x, out, rows, C, accumulate);
    else colsum_generic<float><<<(C + 127) / 128, 128, 0, st>>>((const float*)x, out, rows, C, accumulate);
  }
  return (int)cudaGetLastError();
}
