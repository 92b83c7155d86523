// Row softmax (any axis) and the fused softmax-cross-entropy loss + gradient.
//
// Counterparts of infini_train/src/kernels/cuda/softmax.cu:25-72,122-152 and
// cross_entropy.cu:30-71 (forward, 3 passes, then a device sync and a host-side
// mean at :103-112) and :115-163 (backward, which ignores the upstream gradient).
// Here the loss kernel makes one online-softmax pass over the row with 128-bit
// loads, the mean is a device kernel, the gradient honours an upstream scalar,
// can be written over the logits in place, index math is 64-bit and padded
// vocabulary columns get a zero gradient.
#include "api.h"
#include "common.cuh"

namespace titb {

struct MaxSum { float m, s; };
__device__ __forceinline__ MaxSum ms_combine(MaxSum a, MaxSum b) {
  const float m = fmaxf(a.m, b.m);
  if (m == -INFINITY) return {m, 0.f};
  return {m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}
__device__ __forceinline__ MaxSum ms_warp(MaxSum v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum t{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = ms_combine(v, t);
  }
  return v;
}
__device__ __forceinline__ MaxSum ms_block(MaxSum v, float* red) {  // red: >= 64 floats
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = ms_warp(v);
  __syncthreads();
  if (lane == 0) { red[w] = v.m; red[32 + w] = v.s; }
  __syncthreads();
  MaxSum r = (lane < nw) ? MaxSum{red[lane], red[32 + lane]} : MaxSum{-INFINITY, 0.f};
  return ms_warp(r);
}

// One CTA per row.  losses[row] = logsumexp - logit[target]; optional gradient
// dlogits = (grad_scale * upstream) * (softmax - onehot) for columns < V and 0 for padding.
template <typename T>
__global__ void __launch_bounds__(512)
xent_kernel(const T* logits, const long long* __restrict__ targets, float* __restrict__ losses,
            T* dlogits, int V, long long ld, float grad_scale, const float* __restrict__ upstream, int vec_ok) {
  constexpr int VN = VecN<T>::n;
  __shared__ float red[64];
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  const int nvec = vec_ok ? V / VN : 0;
  // The target logit is read before any thread can overwrite the row (in-place gradient).
  const long long tgt = targets[row];
  const float x_tgt = (tgt >= 0 && tgt < V) ? to_f32(x[tgt]) : 0.f;
  MaxSum acc{-INFINITY, 0.f};
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    Pack<T, VN> p = ld128(x + i * VN);
    float mx = to_f32(p.v[0]);
#pragma unroll
    for (int e = 1; e < VN; ++e) mx = fmaxf(mx, to_f32(p.v[e]));
    const float m = fmaxf(acc.m, mx);
    float s = acc.s * __expf(acc.m - m);
#pragma unroll
    for (int e = 0; e < VN; ++e) s += __expf(to_f32(p.v[e]) - m);
    acc = {m, s};
  }
  for (int i = nvec * VN + threadIdx.x; i < V; i += blockDim.x) acc = ms_combine(acc, MaxSum{to_f32(x[i]), 1.f});
  acc = ms_block(acc, red);
  const float lse = acc.m + logf(acc.s);
  if (threadIdx.x == 0 && losses != nullptr) {
    const bool valid = tgt >= 0 && tgt < V;
    losses[row] = valid ? lse - x_tgt : 0.f;
  }
  if (dlogits == nullptr) return;
  float g = grad_scale;
  if (upstream != nullptr) g *= *upstream;
  if (tgt < 0 || tgt >= V) g = 0.f;  // ignored row
  T* dx = dlogits + row * ld;
  const int ldv = vec_ok ? (int)(ld / VN) : 0;
  for (int i = threadIdx.x; i < ldv; i += blockDim.x) {
    Pack<T, VN> p = ld128(x + i * VN), o;
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      const int c = i * VN + e;
      float pr = (c < V) ? __expf(to_f32(p.v[e]) - lse) : 0.f;
      if (c == tgt) pr -= 1.f;
      o.v[e] = from_f32<T>(g * pr);
    }
    st128(dx + i * VN, o);
  }
  for (long long c = (long long)ldv * VN + threadIdx.x; c < ld; c += blockDim.x) {
    float pr = (c < V) ? __expf(to_f32(x[c]) - lse) : 0.f;
    if (c == tgt) pr -= 1.f;
    dx[c] = from_f32<T>(g * pr);
  }
}

// ---- vocabulary-parallel cross entropy -------------------------------------------------------------------
// The vocabulary is split over the ranks of a tensor-parallel group: this rank's logits [rows, ld] hold global
// columns [vocab_lo, vocab_lo + V_valid) (anything beyond is padding).  Pass 1 reduces each row of the slice to
// (max, sum exp(x - max), logit of the target if it falls in the slice) and stores the triple at slot `rank` of
// a [world, rows, 3] table on every destination pointer (peer stores into symmetric memory, or one local
// table that the host all-gathers).  Pass 2 reads the complete table, forms the global log-sum-exp and writes
// loss rows and, in place, grad_scale * (softmax - onehot) for the slice.  The full [rows, V] logits never
// exist on one GPU.
struct VpDst {
  float* p[16];
  int n;
};

template <typename T>
__global__ void __launch_bounds__(512)
xent_vp_stats_kernel(const T* __restrict__ logits, const long long* __restrict__ targets, const VpDst dst, int rank,
                     long long rows, int V_valid, long long ld, long long vocab_lo, int vec_ok) {
  constexpr int VN = VecN<T>::n;
  __shared__ float red[64];
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  const int nvec = vec_ok ? V_valid / VN : 0;
  MaxSum acc{-INFINITY, 0.f};
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    Pack<T, VN> p = ld128(x + i * VN);
    float mx = to_f32(p.v[0]);
#pragma unroll
    for (int e = 1; e < VN; ++e) mx = fmaxf(mx, to_f32(p.v[e]));
    const float m = fmaxf(acc.m, mx);
    float s = acc.s * __expf(acc.m - m);
#pragma unroll
    for (int e = 0; e < VN; ++e) s += __expf(to_f32(p.v[e]) - m);
    acc = {m, s};
  }
  for (int i = nvec * VN + threadIdx.x; i < V_valid; i += blockDim.x) acc = ms_combine(acc, MaxSum{to_f32(x[i]), 1.f});
  acc = ms_block(acc, red);
  if (threadIdx.x == 0) {
    const long long t = targets[row] - vocab_lo;
    const float x_tgt = (t >= 0 && t < V_valid) ? to_f32(x[t]) : 0.f;
    const long long slot = (static_cast<long long>(rank) * rows + row) * 3;
    for (int d = 0; d < dst.n; ++d) {
      float* o = dst.p[d] + slot;
      o[0] = acc.m; o[1] = acc.s; o[2] = x_tgt;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(512)
xent_vp_grad_kernel(T* logits, const long long* __restrict__ targets, const float* __restrict__ stats, int world,
                    float* __restrict__ losses, long long rows, int V_valid, long long ld, long long vocab_lo,
                    long long vocab_size, float grad_scale, int vec_ok) {
  constexpr int VN = VecN<T>::n;
  const long long row = blockIdx.x;
  // every thread folds the (at most 16) per-rank triples itself: cheaper than a block broadcast
  MaxSum g{-INFINITY, 0.f};
  float x_tgt = 0.f;
  for (int r = 0; r < world; ++r) {
    const float* s = stats + (static_cast<long long>(r) * rows + row) * 3;
    g = ms_combine(g, MaxSum{s[0], s[1]});
    x_tgt += s[2];
  }
  const float lse = g.m + logf(g.s);
  const long long tgt = targets[row];
  const bool valid = tgt >= 0 && tgt < vocab_size;
  if (threadIdx.x == 0 && losses != nullptr) losses[row] = valid ? lse - x_tgt : 0.f;
  const float gs = valid ? grad_scale : 0.f;
  const long long t_local = tgt - vocab_lo;
  T* x = logits + row * ld;
  const int ldv = vec_ok ? (int)(ld / VN) : 0;
  for (int i = threadIdx.x; i < ldv; i += blockDim.x) {
    Pack<T, VN> p = ld128(x + i * VN), o;
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      const int c = i * VN + e;
      float pr = (c < V_valid) ? __expf(to_f32(p.v[e]) - lse) : 0.f;
      if (c == t_local) pr -= 1.f;
      o.v[e] = from_f32<T>(gs * pr);
    }
    st128(x + i * VN, o);
  }
  for (long long c = (long long)ldv * VN + threadIdx.x; c < ld; c += blockDim.x) {
    float pr = (c < V_valid) ? __expf(to_f32(x[c]) - lse) : 0.f;
    if (c == t_local) pr -= 1.f;
    x[c] = from_f32<T>(gs * pr);
  }
}

// out[0] = scale * sum(x), fixed summation order.
__global__ void mean_kernel(const float* __restrict__ x, float* __restrict__ out, long long n, float scale) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = s * scale;
}

// Softmax over `axis` of an (outer, axis, inner) view.  One warp per (outer, inner) line.
template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long outer, int axis,
                                   long long inner) {
  const long long line = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (line >= outer * inner) return;
  const int lane = threadIdx.x & 31;
  const long long o = line / inner, in = line - o * inner;
  const T* xp = x + o * axis * inner + in;
  T* yp = y + o * axis * inner + in;
  float mx = -INFINITY;
  for (int i = lane; i < axis; i += 32) mx = fmaxf(mx, to_f32(xp[(long long)i * inner]));
  mx = warp_max(mx);
  float s = 0.f;
  for (int i = lane; i < axis; i += 32) s += expf(to_f32(xp[(long long)i * inner]) - mx);
  s = warp_sum(s);
  const float inv = 1.f / s;
  for (int i = lane; i < axis; i += 32)
    yp[(long long)i * inner] = from_f32<T>(expf(to_f32(xp[(long long)i * inner]) - mx) * inv);
}
template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx,
                                   long long outer, int axis, long long inner) {
  const long long line = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (line >= outer * inner) return;
  const int lane = threadIdx.x & 31;
  const long long o = line / inner, in = line - o * inner;
  const long long base = o * axis * inner + in;
  float dot = 0.f;
  for (int i = lane; i < axis; i += 32) dot += to_f32(dy[base + (long long)i * inner]) * to_f32(y[base + (long long)i * inner]);
  dot = warp_sum(dot);
  for (int i = lane; i < axis; i += 32) {
    const long long k = base + (long long)i * inner;
    dx[k] = from_f32<T>(to_f32(y[k]) * (to_f32(dy[k]) - dot));
  }
}

}  // namespace titb
using namespace titb;

TITB_API int titb_xent_fwd_bwd(const void* logits, const long long* targets, float* losses, void* dlogits,
                               long long rows, int V, long long ld, float grad_scale, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  const int vn = dtype == 1 ? 8 : 4;
  const int vec_ok = !((uintptr_t)logits & 15) && !((uintptr_t)dlogits & 15) && (ld % vn == 0);
  const int threads = V >= 8192 ? 512 : 128;
  if (dtype == 1)
    xent_kernel<bf16><<<(unsigned)rows, threads, 0, st>>>((const bf16*)logits, targets, losses, (bf16*)dlogits, V, ld, grad_scale, nullptr, vec_ok);
  else
    xent_kernel<float><<<(unsigned)rows, threads, 0, st>>>((const float*)logits, targets, losses, (float*)dlogits, V, ld, grad_scale, nullptr, vec_ok);
  return (int)cudaGetLastError();
}

// Backward-only form: recomputes the row statistics and scales by a device-side upstream scalar.
TITB_API int titb_xent_bwd(const void* logits, const long long* targets, void* dlogits, const float* upstream,
                           long long rows, int V, long long ld, float grad_scale, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  const int vn = dtype == 1 ? 8 : 4;
  const int vec_ok = !((uintptr_t)logits & 15) && !((uintptr_t)dlogits & 15) && (ld % vn == 0);
  const int threads = V >= 8192 ? 512 : 128;
  if (dtype == 1)
    xent_kernel<bf16><<<(unsigned)rows, threads, 0, st>>>((const bf16*)logits, targets, nullptr, (bf16*)dlogits, V, ld, grad_scale, upstream, vec_ok);
  else
    xent_kernel<float><<<(unsigned)rows, threads, 0, st>>>((const float*)logits, targets, nullptr, (float*)dlogits, V, ld, grad_scale, upstream, vec_ok);
  return (int)cudaGetLastError();
}

TITB_API int titb_mean(const float* x, float* out, long long n, float scale, cudaStream_t st) {
  mean_kernel<<<1, 1024, 0, st>>>(x, out, n, scale);
  return (int)cudaGetLastError();
}

TITB_API int titb_softmax_fwd(const void* x, void* y, long long outer, int axis, long long inner, int dtype,
                              cudaStream_t st) {
  const long long lines = outer * inner;
  if (lines <= 0 || axis <= 0) return 0;
  const unsigned blocks = (unsigned)((lines + 3) / 4);
  if (dtype == 1) softmax_fwd_kernel<bf16><<<blocks, 128, 0, st>>>((const bf16*)x, (bf16*)y, outer, axis, inner);
  else softmax_fwd_kernel<float><<<blocks, 128, 0, st>>>((const float*)x, (float*)y, outer, axis, inner);
  return (int)cudaGetLastError();
}
TITB_API int titb_softmax_bwd(const void* dy, const void* y, void* dx, long long outer, int axis, long long inner,
                              int dtype, cudaStream_t st) {
  const long long lines = outer * inner;
  if (lines <= 0 || axis <= 0) return 0;
  const unsigned blocks = (unsigned)((lines + 3) / 4);
  if (dtype == 1) softmax_bwd_kernel<bf16><<<blocks, 128, 0, st>>>((const bf16*)dy, (const bf16*)y, (bf16*)dx, outer, axis, inner);
  else softmax_bwd_kernel<float><<<blocks, 128, 0, st>>>((const float*)dy, (const float*)y, (float*)dx, outer, axis, inner);
  return (int)cudaGetLastError();
}

static inline int vp_valid_cols(long long V_local, long long vocab_lo, long long vocab_size) {
  long long v = vocab_size - vocab_lo;
  if (v > V_local) v = V_local;
  return (int)(v < 0 ? 0 : v);
}

TITB_API int titb_xent_vp_stats(const void* logits, const long long* targets, const unsigned long long* dst_ptrs,
                                int n_dst, int rank, long long rows, long long V_local, long long ld,
                                long long vocab_lo, long long vocab_size, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (n_dst < 1 || n_dst > 16 || V_local > ld) return TITB_ERR_SHAPE;
  VpDst dst{};
  dst.n = n_dst;
  for (int i = 0; i < n_dst; ++i) dst.p[i] = reinterpret_cast<float*>(dst_ptrs[i]);
  const int Vv = vp_valid_cols(V_local, vocab_lo, vocab_size);
  const int vn = dtype == 1 ? 8 : 4;
  const int vec_ok = !((uintptr_t)logits & 15) && (ld % vn == 0);
  const int threads = Vv >= 8192 ? 512 : 256;
  if (dtype == 1)
    xent_vp_stats_kernel<bf16><<<(unsigned)rows, threads, 0, st>>>((const bf16*)logits, targets, dst, rank, rows, Vv, ld, vocab_lo, vec_ok);
  else
    xent_vp_stats_kernel<float><<<(unsigned)rows, threads, 0, st>>>((const float*)logits, targets, dst, rank, rows, Vv, ld, vocab_lo, vec_ok);
  return (int)cudaGetLastError();
}

TITB_API int titb_xent_vp_grad(void* logits, const long long* targets, const float* stats, int world, float* losses,
                               long long rows, long long V_local, long long ld, long long vocab_lo,
                               long long vocab_size, float grad_scale, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (world < 1 || world > 16 || V_local > ld) return TITB_ERR_SHAPE;
  const int Vv = vp_valid_cols(V_local, vocab_lo, vocab_size);
  const int vn = dtype == 1 ? 8 : 4;
  const int vec_ok = !((uintptr_t)logits & 15) && (ld % vn == 0);
  const int threads = ld >= 8192 ? 512 : 256;
  if (dtype == 1)
    xent_vp_grad_kernel<bf16><<<(unsigned)rows, threads, 0, st>>>((bf16*)logits, targets, stats, world, losses, rows, Vv, ld, vocab_lo, vocab_size, grad_scale, vec_ok);
  else
    xent_vp_grad_kernel<float><<<(unsigned)rows, threads, 0, st>>>((float*)logits, targets, stats, world, losses, rows, Vv, ld, vocab_lo, vocab_size, grad_scale, vec_ok);
  return (int)cudaGetLastError();
}
