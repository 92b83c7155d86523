// Reductions along one axis, N-d strided gather/scatter (slice, split, stack, repeat-interleave,
// general permute), masked fill and outer product.
//
// Counterparts of the reference's infini_train/src/kernels/cuda/reduction.cu (Mean/Sum/Max/Min
// forward and backward), transform.cu (Mask :56-93, RepeatInterleave :167-end), slice.cu,
// split.cu, stack.cu and outer.cu.  The reference launches one kernel per op with its shape
// metadata copied to device memory on every call; here one gather kernel and one scatter kernel
// serve every view-like op with the (at most 6-d) shape and strides passed as kernel parameters,
// and the reductions pick a warp-per-row or a column-strip schedule from the inner extent.
#include <cfloat>

#include "api.h"
#include "common.cuh"

namespace titb {

constexpr int kTfThreads = 256;

static inline int tf_blocks(long long n, int per_block = kTfThreads) {
  long long b = (n + per_block - 1) / per_block;
  const long long cap = 148LL * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

// ---------------------------------------------------------------------------------- reductions
// x viewed as [outer, n, inner]; y [outer, inner].  op: 0 sum, 1 mean, 2 max, 3 min.
struct RedOp {
  int op;
  __device__ float init() const { return op == 2 ? -FLT_MAX : (op == 3 ? FLT_MAX : 0.f); }
  __device__ bool better(float cand, float cur) const { return op == 2 ? cand > cur : cand < cur; }
};

// inner == 1: one warp per output element, lanes stride over n.
template <typename T>
__global__ void reduce_rows_kernel(const T* __restrict__ x, T* __restrict__ y, long long* __restrict__ idx,
                                   long long outer, long long n, RedOp r) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long o = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); o < outer; o += warps) {
    const T* row = x + o * n;
    float acc = r.init();
    long long best = 0;
    if (r.op < 2) {
      for (long long i = lane; i < n; i += 32) acc += to_f32(row[i]);
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
      if (r.op == 1) acc /= (float)n;
    } else {
      for (long long i = lane; i < n; i += 32) {
        const float v = to_f32(row[i]);
        if (r.better(v, acc)) { acc = v; best = i; }
      }
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, acc, s);
        const long long oi = __shfl_xor_sync(0xffffffffu, best, s);
        // ties go to the lowest index, like a sequential scan
        if (r.better(ov, acc) || (ov == acc && oi < best)) { acc = ov; best = oi; }
      }
    }
    if (lane == 0) {
      y[o] = from_f32<T>(acc);
      if (idx != nullptr) idx[o] = best;
    }
  }
}

// inner > 1: one thread per (outer, inner) output, walking n with stride inner (coalesced over inner).
template <typename T>
__global__ void reduce_strided_kernel(const T* __restrict__ x, T* __restrict__ y, long long* __restrict__ idx,
                                      long long outer, long long n, long long inner, RedOp r) {
  const long long total = outer * inner;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += stride) {
    const long long o = t / inner, in = t % inner;
    const T* p = x + o * n * inner + in;
    float acc = r.init();
    long long best = 0;
    if (r.op < 2) {
      for (long long i = 0; i < n; ++i) acc += to_f32(p[i * inner]);
      if (r.op == 1) acc /= (float)n;
    } else {
      for (long long i = 0; i < n; ++i) {
        const float v = to_f32(p[i * inner]);
        if (r.better(v, acc)) { acc = v; best = i; }
      }
    }
    y[t] = from_f32<T>(acc);
    if (idx != nullptr) idx[t] = best;
  }
}

// Backward: dx[o, i, in] = g[o, in] * scale (sum / mean) or g[o, in] * (i == idx[o, in]) (max / min).
template <typename T>
__global__ void reduce_bwd_kernel(const T* __restrict__ g, const long long* __restrict__ idx, T* __restrict__ dx,
                                  long long outer, long long n, long long inner, float scale) {
  const long long total = outer * n * inner;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += stride) {
    const long long in = t % inner, i = (t / inner) % n, o = t / (inner * n);
    const float gv = to_f32(g[o * inner + in]);
    float v;
    if (idx == nullptr) v = gv * scale;
    else v = (idx[o * inner + in] == i) ? gv : 0.f;
    dx[t] = from_f32<T>(v);
  }
}

// ------------------------------------------------------------------- N-d strided gather / scatter
struct View6 {
  long long size[6];    // extents of the contiguous side (row-major)
  long long stride[6];  // element strides of the strided side (0 repeats, negative not used)
  long long offset;     // element offset of the strided side
  int nd;
};

template <typename T>
__device__ __forceinline__ long long strided_index(const View6& v, long long t) {
  long long off = v.offset;
#pragma unroll
  for (int d = 5; d >= 0; --d) {
    if (d < v.nd) {
      const long long q = t / v.size[d];
      off += (t - q * v.size[d]) * v.stride[d];
      t = q;
    }
  }
  return off;
}

// out (contiguous, n elements) <- in (strided)
template <typename T>
__global__ void gather_kernel(const T* __restrict__ in, T* __restrict__ out, long long n, const View6 v) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < n; t += stride)
    out[t] = in[strided_index<T>(v, t)];
}
// out (strided) <- or += in (contiguous).  Accumulation is for views that repeat elements
// (stride 0, the backward of repeat-interleave): it uses atomics; plain stores otherwise.
template <typename T>
__global__ void scatter_kernel(const T* __restrict__ in, T* __restrict__ out, long long n, const View6 v,
                               int accumulate) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < n; t += stride) {
    const long long o = strided_index<T>(v, t);
    if (accumulate) atomicAdd(out + o, in[t]);
    else out[o] = in[t];
  }
}

// ------------------------------------------------------------------------------ mask / outer
// y = mask ? value : x, the mask repeating by modulo over the flattened input (mask_n elements)
__device__ __forceinline__ float mask_value(float m) { return m; }
__device__ __forceinline__ float mask_value(bf16 m) { return __bfloat162float(m); }
__device__ __forceinline__ float mask_value(unsigned char m) { return static_cast<float>(m); }

template <typename T, typename M>
__global__ void mask_fill_kernel(const T* __restrict__ x, const M* __restrict__ mask, T* __restrict__ y, long long n,
                                 long long mask_n, float value, int flags) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const T fill = from_f32<T>(value);
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < n; t += stride) {
    const float mv = mask_value(mask[t % mask_n]);
    const bool m = (flags & 2) ? (mv == 1.f) : (mv != 0.f);
    // forward: masked positions take `value`; backward (flag bit 0): masked positions pass no gradient
    y[t] = m ? ((flags & 1) ? from_f32<T>(0.f) : fill) : x[t];
  }
}

template <typename T>
__global__ void outer_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, long long M,
                             long long N) {
  const long long total = M * N;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += stride)
    y[t] = from_f32<T>(to_f32(a[t / N]) * to_f32(b[t % N]));
}
// da[i] = sum_j g[i, j] b[j]  (warp per row)
template <typename T>
__global__ void outer_bwd_a_kernel(const T* __restrict__ g, const T* __restrict__ b, T* __restrict__ da, long long M,
                                   long long N) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long i = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); i < M; i += warps) {
    float acc = 0.f;
    for (long long j = lane; j < N; j += 32) acc += to_f32(g[i * N + j]) * to_f32(b[j]);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) da[i] = from_f32<T>(acc);
  }
}
// db[j] = sum_i g[i, j] a[i]  (thread per column, coalesced over j)
template <typename T>
__global__ void outer_bwd_b_kernel(const T* __restrict__ g, const T* __restrict__ a, T* __restrict__ db, long long M,
                                   long long N) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x; j < N; j += stride) {
    float acc = 0.f;
    for (long long i = 0; i < M; ++i) acc += to_f32(g[i * N + j]) * to_f32(a[i]);
    db[j] = from_f32<T>(acc);
  }
}

template <typename T>
static int reduce_impl(const void* x, void* y, long long* idx, long long outer, long long n, long long inner, int op,
                       cudaStream_t st) {
  RedOp r{op};
  if (inner == 1)
    reduce_rows_kernel<T><<<tf_blocks(outer, kTfThreads / 32), kTfThreads, 0, st>>>((const T*)x, (T*)y, idx, outer, n, r);
  else
    reduce_strided_kernel<T><<<tf_blocks(outer * inner), kTfThreads, 0, st>>>((const T*)x, (T*)y, idx, outer, n, inner, r);
  return (int)cudaGetLastError();
}

static bool fill_view(View6* v, int nd, const long long* size, const long long* stride, long long offset,
                      long long* total) {
  if (nd < 0 || nd > 6) return false;
  v->nd = nd;
  v->offset = offset;
  long long n = 1;
  for (int d = 0; d < 6; ++d) {
    v->size[d] = d < nd ? size[d] : 1;
    v->stride[d] = d < nd ? stride[d] : 0;
    if (d < nd && size[d] < 0) return false;
    n *= v->size[d];
  }
  *total = n;
  return true;
}

}  // namespace titb

using namespace titb;

TITB_API int titb_reduce(const void* x, void* y, long long* idx, long long outer, long long n, long long inner, int op,
                         int dtype, cudaStream_t stream) {
  if (outer <= 0 || inner <= 0) return 0;
  if (n <= 0 || op < 0 || op > 3) return TITB_ERR_SHAPE;
  return dtype == 1 ? reduce_impl<bf16>(x, y, idx, outer, n, inner, op, stream)
                            : reduce_impl<float>(x, y, idx, outer, n, inner, op, stream);
}

TITB_API int titb_reduce_bwd(const void* g, const long long* idx, void* dx, long long outer, long long n,
                             long long inner, float scale, int dtype, cudaStream_t stream) {
  const long long total = outer * n * inner;
  if (total <= 0) return 0;
  if (dtype == 1)
    reduce_bwd_kernel<bf16><<<tf_blocks(total), kTfThreads, 0, stream>>>((const bf16*)g, idx, (bf16*)dx, outer, n, inner, scale);
  else
    reduce_bwd_kernel<float><<<tf_blocks(total), kTfThreads, 0, stream>>>((const float*)g, idx, (float*)dx, outer, n, inner, scale);
  return (int)cudaGetLastError();
}

TITB_API int titb_gather_nd(const void* in, void* out, int nd, const long long* size, const long long* in_stride,
                            long long in_offset, int elem_bytes, cudaStream_t stream) {
  View6 v;
  long long n;
  if (!fill_view(&v, nd, size, in_stride, in_offset, &n)) return TITB_ERR_SHAPE;
  if (n == 0) return 0;
  if (elem_bytes == 2)
    gather_kernel<unsigned short><<<tf_blocks(n), kTfThreads, 0, stream>>>((const unsigned short*)in, (unsigned short*)out, n, v);
  else if (elem_bytes == 4)
    gather_kernel<unsigned int><<<tf_blocks(n), kTfThreads, 0, stream>>>((const unsigned int*)in, (unsigned int*)out, n, v);
  else if (elem_bytes == 8)
    gather_kernel<unsigned long long><<<tf_blocks(n), kTfThreads, 0, stream>>>((const unsigned long long*)in, (unsigned long long*)out, n, v);
  else return TITB_ERR_SHAPE;
  return (int)cudaGetLastError();
}

TITB_API int titb_scatter_nd(const void* in, void* out, int nd, const long long* size, const long long* out_stride,
                             long long out_offset, int dtype, int accumulate, cudaStream_t stream) {
  View6 v;
  long long n;
  if (!fill_view(&v, nd, size, out_stride, out_offset, &n)) return TITB_ERR_SHAPE;
  if (n == 0) return 0;
  if (dtype == 1)
    scatter_kernel<bf16><<<tf_blocks(n), kTfThreads, 0, stream>>>((const bf16*)in, (bf16*)out, n, v, accumulate);
  else
    scatter_kernel<float><<<tf_blocks(n), kTfThreads, 0, stream>>>((const float*)in, (float*)out, n, v, accumulate);
  return (int)cudaGetLastError();
}

TITB_API int titb_mask_fill(const void* x, const void* mask, void* y, long long n, long long mask_n, float value,
                            int backward, int dtype, int mask_dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (mask_n <= 0) return TITB_ERR_SHAPE;
  const int blocks = tf_blocks(n);
#define TITB_MASK_CASE(T, M) \
  mask_fill_kernel<T, M><<<blocks, kTfThreads, 0, stream>>>((const T*)x, (const M*)mask, (T*)y, n, mask_n, value, backward)
  if (dtype == 1) {
    if (mask_dtype == 1) TITB_MASK_CASE(bf16, bf16);
    else if (mask_dtype == 0) TITB_MASK_CASE(bf16, float);
    else TITB_MASK_CASE(bf16, unsigned char);
  } else {
    if (mask_dtype == 1) TITB_MASK_CASE(float, bf16);
    else if (mask_dtype == 0) TITB_MASK_CASE(float, float);
    else TITB_MASK_CASE(float, unsigned char);
  }
#undef TITB_MASK_CASE
  return (int)cudaGetLastError();
}

TITB_API int titb_outer(const void* a, const void* b, void* y, long long M, long long N, int dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (dtype == 1) outer_kernel<bf16><<<tf_blocks(M * N), kTfThreads, 0, stream>>>((const bf16*)a, (const bf16*)b, (bf16*)y, M, N);
  else outer_kernel<float><<<tf_blocks(M * N), kTfThreads, 0, stream>>>((const float*)a, (const float*)b, (float*)y, M, N);
  return (int)cudaGetLastError();
}

TITB_API int titb_outer_bwd(const void* g, const void* a, const void* b, void* da, void* db, long long M, long long N,
                            int dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (dtype == 1) {
    outer_bwd_a_kernel<bf16><<<tf_blocks(M, kTfThreads / 32), kTfThreads, 0, stream>>>((const bf16*)g, (const bf16*)b, (bf16*)da, M, N);
    outer_bwd_b_kernel<bf16><<<tf_blocks(N), kTfThreads, 0, stream>>>((const bf16*)g, (const bf16*)a, (bf16*)db, M, N);
  } else {
    outer_bwd_a_kernel<float><<<tf_blocks(M, kTfThreads / 32), kTfThreads, 0, stream>>>((const float*)g, (const float*)b, (float*)da, M, N);
    outer_bwd_b_kernel<float><<<tf_blocks(N), kTfThreads, 0, stream>>>((const float*)g, (const float*)a, (float*)db, M, N);
  }
  return (int)cudaGetLastError();
}
