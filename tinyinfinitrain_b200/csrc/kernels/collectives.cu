// Standalone collectives over a symmetric buffer: in-place all-reduce (sum) and all-gather, for tensors that are
// not produced or consumed by one of the fused kernels (replicated-parameter gradients under tensor parallelism,
// plain data parallelism without ZeRO, parameter broadcasts).
//
//  * all-reduce, two-shot: rank r owns the slice [r n/W, (r+1) n/W) of the buffer.  It reads that slice of every
//    rank's copy -- one multimem.ld_reduce per 16 bytes when the buffer has a multicast mapping (the NVSwitch adds),
//    otherwise a rotated loop of peer loads -- scales the sum and writes it into every rank's copy (multimem.st or
//    peer stores).  In place is safe: slice r is read by rank r only.
//  * all-gather: rank r writes its own slice of its local copy into every rank's copy.
//  * signal / wait: a point-to-point flag with a bounded wait (producer / consumer hand-offs between two ranks).
//
// The two collective kernels wait for nothing: the caller brackets them with the device barrier (all inputs
// written before, all outputs landed after), exactly as the ZeRO-1 step does.  The reference has no collectives
// (infini_train/src/device.cc:11-17 enforces a single device).
#include "api.h"
#include "common.cuh"

namespace titb {

constexpr int kCollMaxRanks = 16;
struct CollPtrs {
  void* p[kCollMaxRanks];
};

__device__ __forceinline__ float4 coll_mc_ld_reduce_f32(const void* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
// eight bf16 values, summed across the ranks with fp32 accumulation inside the switch
__device__ __forceinline__ uint4 coll_mc_ld_reduce_bf16(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
__device__ __forceinline__ void coll_mc_st(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

struct AllReduceArgs {
  CollPtrs bufs;          // every rank's copy as mapped on this GPU
  void* mc;               // multicast address of the buffer, or null
  long long slice_off;    // this rank's slice, in 16-byte units from the start of the buffer
  long long slice_vecs;   // 16-byte units in the slice
  int world, rank;
  float scale;            // applied to the sum (1 / world for a mean)
};

template <bool BF16>
__global__ void __launch_bounds__(256) allreduce_twoshot_kernel(const AllReduceArgs a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.slice_vecs; i += stride) {
    const long long at = (a.slice_off + i) * 16;   // byte offset
    float f[8];
    if (a.mc != nullptr) {
      if (BF16) {
        const uint4 u = coll_mc_ld_reduce_bf16(static_cast<const char*>(a.mc) + at);
        const float2 p0 = unpack_bf16x2(u.x), p1 = unpack_bf16x2(u.y), p2 = unpack_bf16x2(u.z), p3 = unpack_bf16x2(u.w);
        f[0] = p0.x; f[1] = p0.y; f[2] = p1.x; f[3] = p1.y; f[4] = p2.x; f[5] = p2.y; f[6] = p3.x; f[7] = p3.y;
      } else {
        const float4 v = coll_mc_ld_reduce_f32(static_cast<const char*>(a.mc) + at);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
      // fixed order starting at rank 0: every rank computes the same bits for a given slice owner, and a re-run
      // of the same step gives the same sum
      for (int q = 0; q < a.world; ++q) {
        const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const char*>(a.bufs.p[q]) + at);
        if (BF16) {
          const float2 p0 = unpack_bf16x2(u.x), p1 = unpack_bf16x2(u.y), p2 = unpack_bf16x2(u.z), p3 = unpack_bf16x2(u.w);
          f[0] += p0.x; f[1] += p0.y; f[2] += p1.x; f[3] += p1.y; f[4] += p2.x; f[5] += p2.y; f[6] += p3.x; f[7] += p3.y;
        } else {
          f[0] += __uint_as_float(u.x); f[1] += __uint_as_float(u.y); f[2] += __uint_as_float(u.z); f[3] += __uint_as_float(u.w);
        }
      }
    }
    uint4 o;
    if (BF16) {
      o.x = pack_bf16x2(f[0] * a.scale, f[1] * a.scale); o.y = pack_bf16x2(f[2] * a.scale, f[3] * a.scale);
      o.z = pack_bf16x2(f[4] * a.scale, f[5] * a.scale); o.w = pack_bf16x2(f[6] * a.scale, f[7] * a.scale);
    } else {
      o.x = __float_as_uint(f[0] * a.scale); o.y = __float_as_uint(f[1] * a.scale);
      o.z = __float_as_uint(f[2] * a.scale); o.w = __float_as_uint(f[3] * a.scale);
    }
    if (a.mc != nullptr) {
      coll_mc_st(static_cast<char*>(a.mc) + at, o);
    } else {
      for (int q = 0; q < a.world; ++q) {
        const int pr = (a.rank + q) % a.world;     // rotated: the ranks do not all write to the same peer at once
        *reinterpret_cast<uint4*>(static_cast<char*>(a.bufs.p[pr]) + at) = o;
      }
    }
  }
}

struct AllGatherArgs {
  CollPtrs bufs;
  void* mc;
  long long slice_off, slice_vecs;   // this rank's slice in 16-byte units
  int world, rank;
};

__global__ void __launch_bounds__(256) allgather_kernel(const AllGatherArgs a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const char* mine = static_cast<const char*>(a.bufs.p[a.rank]);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.slice_vecs; i += stride) {
    const long long at = (a.slice_off + i) * 16;
    const uint4 v = *reinterpret_cast<const uint4*>(mine + at);
    if (a.mc != nullptr) {
      coll_mc_st(static_cast<char*>(a.mc) + at, v);   // also rewrites the local copy with the same bytes
    } else {
      for (int q = 1; q < a.world; ++q) {
        const int pr = (a.rank + q) % a.world;
        *reinterpret_cast<uint4*>(static_cast<char*>(a.bufs.p[pr]) + at) = v;
      }
    }
  }
}

// Point-to-point flag: the producer publishes `value` in a 32-bit word of the consumer's memory after everything it
// wrote before; the consumer waits until the word has reached `value` (values only grow, compared as a signed
// difference so that they may wrap).  The wait is bounded: when the budget runs out the kernel records
// kStatusPeerTimeout and returns, and the stream carries on.
__global__ void signal_kernel(uint32_t* remote_word, uint32_t value) {
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote_word), "r"(value) : "memory");
}
__global__ void wait_kernel(const uint32_t* local_word, uint32_t value, long long budget_cycles, int* status) {
  const long long t0 = clock64();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local_word) : "memory");
    if (static_cast<int32_t>(v - value) >= 0) break;
    __nanosleep(64);
    if (clock64() - t0 > budget_cycles) {
      atomicExch(status, kStatusPeerTimeout);
      break;
    }
  }
  __threadfence_system();
}

static int coll_blocks(long long vecs, int max_blocks) {
  long long b = (vecs + 255) / 256;
  const int cap = max_blocks > 0 ? max_blocks : device_sm_count() * 2;
  if (b > cap) b = cap;
  return b < 1 ? 1 : (int)b;
}

}  // namespace titb

using namespace titb;

// In-place sum (times `scale`) over the ranks of `nbytes` bytes at byte offset `byte_off` of a symmetric buffer.
// dtype: 0 fp32, 1 bf16.  byte_off and nbytes / world must be multiples of 16.  The caller runs the device barrier
// before (every rank's input is in its copy) and after (every slice has been written everywhere).
TITB_API int titb_symm_allreduce(const unsigned long long* buf_ptrs, unsigned long long mc_ptr, long long byte_off,
                                 long long nbytes, int dtype, int world, int rank, float scale, int max_blocks,
                                 cudaStream_t st) {
  (void)cudaGetLastError();
  if (world < 1 || world > kCollMaxRanks || rank < 0 || rank >= world) return TITB_ERR_SHAPE;
  if (nbytes <= 0) return 0;
  if ((byte_off & 15) || (nbytes % (16LL * world)) != 0) return TITB_ERR_SHAPE;
  AllReduceArgs a{};
  for (int i = 0; i < world; ++i) a.bufs.p[i] = reinterpret_cast<void*>(buf_ptrs[i]);
  a.mc = reinterpret_cast<void*>(mc_ptr);
  a.slice_vecs = nbytes / 16 / world;
  a.slice_off = byte_off / 16 + a.slice_vecs * rank;
  a.world = world; a.rank = rank; a.scale = scale;
  const int blocks = coll_blocks(a.slice_vecs, max_blocks);
  if (dtype == 1) allreduce_twoshot_kernel<true><<<blocks, 256, 0, st>>>(a);
  else allreduce_twoshot_kernel<false><<<blocks, 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}

// All-gather in place: rank r's slice (bytes [byte_off + r nbytes/world, ...) of its own copy) is written into
// every rank's copy.  Same alignment rules and barrier contract as the all-reduce.
TITB_API int titb_symm_allgather(const unsigned long long* buf_ptrs, unsigned long long mc_ptr, long long byte_off,
                                 long long nbytes, int world, int rank, int max_blocks, cudaStream_t st) {
  (void)cudaGetLastError();
  if (world < 1 || world > kCollMaxRanks || rank < 0 || rank >= world) return TITB_ERR_SHAPE;
  if (nbytes <= 0) return 0;
  if ((byte_off & 15) || (nbytes % (16LL * world)) != 0) return TITB_ERR_SHAPE;
  AllGatherArgs a{};
  for (int i = 0; i < world; ++i) a.bufs.p[i] = reinterpret_cast<void*>(buf_ptrs[i]);
  a.mc = reinterpret_cast<void*>(mc_ptr);
  a.slice_vecs = nbytes / 16 / world;
  a.slice_off = byte_off / 16 + a.slice_vecs * rank;
  a.world = world; a.rank = rank;
  allgather_kernel<<<coll_blocks(a.slice_vecs, max_blocks), 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}

// Producer side of a flag: after all earlier work of the stream, store `value` (release, system scope) into the
// 32-bit word at `remote_word` (an address in a peer's symmetric memory as mapped on this GPU, or local memory).
TITB_API int titb_symm_signal(unsigned long long remote_word, unsigned int value, cudaStream_t st) {
  (void)cudaGetLastError();
  if (!remote_word || (remote_word & 3)) return TITB_ERR_SHAPE;
  signal_kernel<<<1, 1, 0, st>>>(reinterpret_cast<uint32_t*>(remote_word), value);
  return (int)cudaGetLastError();
}
// Consumer side: the stream waits until the word at `local_word` has reached `value`, at most `timeout_s` seconds;
// on expiry the library status word is set to the peer-timeout code and the stream continues.
TITB_API int titb_symm_wait(unsigned long long local_word, unsigned int value, double timeout_s, cudaStream_t st) {
  (void)cudaGetLastError();
  if (!local_word || (local_word & 3)) return TITB_ERR_SHAPE;
  int* status = titb_status_ptr();
  if (!status) return (int)cudaErrorMemoryAllocation;
  wait_kernel<<<1, 1, 0, st>>>(reinterpret_cast<const uint32_t*>(local_word), value, (long long)(timeout_s * 1.9e9), status);
  return (int)cudaGetLastError();
}
