// NVLink / NVSwitch communication kernels over peer-mapped (symmetric) memory.
//
// The reference has no communication layer at all (single device enforced in
// infini_train/src/device.cc:11-17).  These kernels are the data-parallel side of
// this framework:
//
//  * barrier_kernel: cross-GPU barrier on per-rank signal pads, release/acquire at
//    system scope, monotonically increasing epoch kept in device memory so the same
//    launch can be replayed from a CUDA graph.  The wait is bounded; on timeout the
//    kernel records kStatusPeerTimeout and returns.
//  * rs_adam_ag_kernel: ZeRO-1 step in ONE kernel.  Each rank owns a contiguous shard
//    of the flat parameter space.  For its shard it (1) reduces the fp32 gradients of
//    all ranks -- plain peer loads over NVLink, or one multimem.ld_reduce that lets
//    the NVSwitch do the sum -- (2) applies the scale and the Adam/AdamW update to
//    its fp32 master weights and moments in registers, and (3) writes the rounded
//    bf16 parameters into every rank's parameter buffer (peer stores or one
//    multimem.st broadcast).  Reduce-scatter, optimizer and all-gather never
//    round-trip through HBM as separate passes.
//  * allreduce_small_kernel: sum/max of a few floats across ranks (loss, timings).
#include "api.h"
#include "common.cuh"

namespace titb {

constexpr int kMaxRanks = 16;

struct PeerPtrs {
  void* p[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st_b32x4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

// One CTA.  Thread p signals rank p and then waits for rank p's signal.
// pads.p[r] is rank r's pad: an array of uint32 slots, slot [channel * kMaxRanks + src].
__global__ void barrier_kernel(PeerPtrs pads, int rank, int world, int channel, uint32_t* epoch, int* status,
                               long long budget_cycles) {
  __shared__ uint32_t e_sh;
  if (threadIdx.x == 0) {
    __threadfence_system();  // everything this GPU wrote before the barrier is visible to peers first
    e_sh = *epoch + 1;
    *epoch = e_sh;
  }
  __syncthreads();
  const uint32_t e = e_sh;
  const int p = threadIdx.x;
  if (p < world) {
    uint32_t* remote = static_cast<uint32_t*>(pads.p[p]) + channel * kMaxRanks + rank;
    st_release_sys(remote, e);
    const uint32_t* mine = static_cast<const uint32_t*>(pads.p[rank]) + channel * kMaxRanks + p;
    const long long t0 = clock64();
    bool ok = true;
    while (static_cast<int32_t>(ld_acquire_sys(mine) - e) < 0) {
      __nanosleep(64);
      if (clock64() - t0 > budget_cycles) { ok = false; break; }
    }
    if (!ok) atomicExch(status, kStatusPeerTimeout);
  }
  __syncthreads();
  if (threadIdx.x == 0) __threadfence_system();
}

struct RsAdamArgs {
  PeerPtrs grads;        // fp32 flat gradient buffer of every rank (peer mapped)
  PeerPtrs params;       // bf16 flat parameter buffer of every rank (peer mapped)
  const float* grad_mc;  // multicast address of the gradient buffer (or null)
  void* param_mc;        // multicast address of the parameter buffer (or null)
  float* master;         // local fp32 shard state, length shard_n
  float* m;
  float* v;
  long long shard_off;   // first element of this rank's shard in the flat space
  long long shard_n;     // elements per shard (multiple of 8)
  int world, rank;
  float lr, b1, b2, eps, wd, bc1, bc2, gscale;
  const float* dev_state;  // optional {t, bc1, bc2, lr}
};

// One 8-element group of the shard: reduced gradient in `g`, Adam on the fp32 state, bf16 result to every rank.
__device__ __forceinline__ void rs_adam_update8(const RsAdamArgs& a, long long loc, long long glob, const float (&g)[8], float lr,
                                                float bc1, float bc2) {
  float4 m0 = *reinterpret_cast<const float4*>(a.m + loc), m1 = *reinterpret_cast<const float4*>(a.m + loc + 4);
  float4 v0 = *reinterpret_cast<const float4*>(a.v + loc), v1 = *reinterpret_cast<const float4*>(a.v + loc + 4);
  float4 w0 = *reinterpret_cast<const float4*>(a.master + loc), w1 = *reinterpret_cast<const float4*>(a.master + loc + 4);
  float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
  float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float ge = g[e] * a.gscale;
    mm[e] = a.b1 * mm[e] + (1.f - a.b1) * ge;
    vv[e] = a.b2 * vv[e] + (1.f - a.b2) * ge * ge;
    ww[e] -= lr * ((mm[e] / bc1) / (sqrtf(vv[e] / bc2) + a.eps) + a.wd * ww[e]);
  }
  *reinterpret_cast<float4*>(a.m + loc) = make_float4(mm[0], mm[1], mm[2], mm[3]);
  *reinterpret_cast<float4*>(a.m + loc + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
  *reinterpret_cast<float4*>(a.v + loc) = make_float4(vv[0], vv[1], vv[2], vv[3]);
  *reinterpret_cast<float4*>(a.v + loc + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
  *reinterpret_cast<float4*>(a.master + loc) = make_float4(ww[0], ww[1], ww[2], ww[3]);
  *reinterpret_cast<float4*>(a.master + loc + 4) = make_float4(ww[4], ww[5], ww[6], ww[7]);
  const uint4 packed = make_uint4(pack_bf16x2(ww[0], ww[1]), pack_bf16x2(ww[2], ww[3]), pack_bf16x2(ww[4], ww[5]),
                                  pack_bf16x2(ww[6], ww[7]));
  if (a.param_mc != nullptr) {
    multimem_st_b32x4(static_cast<bf16*>(a.param_mc) + glob, packed);
  } else {
    for (int q = 0; q < a.world; ++q) {
      const int pr = (a.rank + q) % a.world;
      *reinterpret_cast<uint4*>(static_cast<bf16*>(a.params.p[pr]) + glob) = packed;
    }
  }
}

// Every thread handles kGroups 8-element groups per trip and issues all of their remote gradient loads before it
// uses the first: a load that crosses NVLink (or is reduced in the switch) takes microseconds, and the link is only
// busy when megabytes are outstanding.
__global__ void __launch_bounds__(256) rs_adam_ag_kernel(const RsAdamArgs a) {
  float lr = a.lr, bc1 = a.bc1, bc2 = a.bc2;
  if (a.dev_state != nullptr) { bc1 = a.dev_state[1]; bc2 = a.dev_state[2]; lr = a.dev_state[3]; }
  constexpr int kGroups = 4;
  const long long nvec = a.shard_n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += kGroups * stride) {
    float g[kGroups][8];
    if (a.grad_mc != nullptr) {
#pragma unroll
      for (int u = 0; u < kGroups; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) {
          const long long glob = a.shard_off + i * 8;
          const float4 g0 = multimem_ld_reduce_f32x4(a.grad_mc + glob);
          const float4 g1 = multimem_ld_reduce_f32x4(a.grad_mc + glob + 4);
          g[u][0] = g0.x; g[u][1] = g0.y; g[u][2] = g0.z; g[u][3] = g0.w;
          g[u][4] = g1.x; g[u][5] = g1.y; g[u][6] = g1.z; g[u][7] = g1.w;
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < kGroups; ++u)
#pragma unroll
        for (int e = 0; e < 8; ++e) g[u][e] = 0.f;
      // start at this rank and wrap, so the ranks do not all read the same peer at once
      for (int q = 0; q < a.world; ++q) {
        const int pr = (a.rank + q) % a.world;
        float4 t0[kGroups], t1[kGroups];
#pragma unroll
        for (int u = 0; u < kGroups; ++u) {
          const long long i = i0 + u * stride;
          if (i < nvec) {
            const float* src = static_cast<const float*>(a.grads.p[pr]) + a.shard_off + i * 8;
            t0[u] = *reinterpret_cast<const float4*>(src);
            t1[u] = *reinterpret_cast<const float4*>(src + 4);
          } else {
            t0[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            t1[u] = t0[u];
          }
        }
#pragma unroll
        for (int u = 0; u < kGroups; ++u) {
          g[u][0] += t0[u].x; g[u][1] += t0[u].y; g[u][2] += t0[u].z; g[u][3] += t0[u].w;
          g[u][4] += t1[u].x; g[u][5] += t1[u].y; g[u][6] += t1[u].z; g[u][7] += t1[u].w;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kGroups; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) rs_adam_update8(a, i * 8, a.shard_off + i * 8, g[u], lr, bc1, bc2);
    }
  }
}

// out[i] = reduce over ranks of bufs.p[r][i] for a handful of floats (op 0 = sum, 1 = max).
__global__ void allreduce_small_kernel(PeerPtrs bufs, float* out, int n, int world, int op) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = op == 1 ? -INFINITY : 0.f;
  for (int r = 0; r < world; ++r) {
    const float x = static_cast<const float*>(bufs.p[r])[i];
    acc = op == 1 ? fmaxf(acc, x) : acc + x;
  }
  out[i] = acc;
}

}  // namespace titb
using namespace titb;

static PeerPtrs to_peers(const unsigned long long* ptrs, int world) {
  PeerPtrs pp{};
  for (int i = 0; i < world && i < kMaxRanks; ++i) pp.p[i] = reinterpret_cast<void*>(ptrs[i]);
  return pp;
}

TITB_API int titb_comm_barrier(const unsigned long long* pad_ptrs, int rank, int world, int channel,
                               unsigned int* epoch, double timeout_s, cudaStream_t st) {
  (void)cudaGetLastError();
  if (world > kMaxRanks || channel < 0 || channel >= 8) return TITB_ERR_SHAPE;
  int* status = titb_status_ptr();
  if (!status) return (int)cudaErrorMemoryAllocation;
  const long long budget = (long long)(timeout_s * 1.9e9);
  barrier_kernel<<<1, 32, 0, st>>>(to_peers(pad_ptrs, world), rank, world, channel, epoch, status, budget);
  return (int)cudaGetLastError();
}

TITB_API int titb_rs_adam_ag(const TitbRsAdamDesc* d, cudaStream_t st) {
  (void)cudaGetLastError();
  if (d->world > kMaxRanks || (d->shard_n & 7)) return TITB_ERR_SHAPE;
  RsAdamArgs a{};
  a.grads = to_peers(d->grad_ptrs, d->world);
  a.params = to_peers(d->param_ptrs, d->world);
  a.grad_mc = static_cast<const float*>(d->grad_mc);
  a.param_mc = d->param_mc;
  a.master = d->master; a.m = d->m; a.v = d->v;
  a.shard_off = d->shard_off; a.shard_n = d->shard_n;
  a.world = d->world; a.rank = d->rank;
  a.lr = d->lr; a.b1 = d->beta1; a.b2 = d->beta2; a.eps = d->eps; a.wd = d->weight_decay;
  a.bc1 = d->bc1; a.bc2 = d->bc2; a.gscale = d->grad_scale; a.dev_state = d->dev_state;
  long long nvec = d->shard_n / 8;
  int blocks = (int)((nvec + 255) / 256);
  const int cap = d->max_blocks > 0 ? d->max_blocks : device_sm_count() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  rs_adam_ag_kernel<<<blocks, 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}

TITB_API int titb_allreduce_small(const unsigned long long* buf_ptrs, float* out, int n, int world, int op,
                                  cudaStream_t st) {
  (void)cudaGetLastError();
  if (world > kMaxRanks) return TITB_ERR_SHAPE;
  allreduce_small_kernel<<<(n + 127) / 128, 128, 0, st>>>(to_peers(buf_ptrs, world), out, n, world, op);
  return (int)cudaGetLastError();
}
