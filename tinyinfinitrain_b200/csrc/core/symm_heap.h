// Symmetric-memory heap: every rank of a node-local group allocates the same number of bytes of device memory
// with the CUDA virtual-memory-management API, exports its allocation as a POSIX file descriptor, passes the
// descriptor to every peer over a unix-domain socket (SCM_RIGHTS), imports the peers' descriptors and maps all of
// them into its own address space.  After that, kernels on any GPU can load from and store to any rank's copy
// through plain pointers (NVLink peer access).  Where the driver supports it, one multicast object is bound over
// the same physical memory so that kernels can use `multimem.ld_reduce` / `multimem.st` through NVSwitch.
//
// The reference has no counterpart: its TensorBuffer (infini_train/include/tensor.h:51-66, src/tensor.cc:58-96)
// is a private cudaMallocAsync allocation and the project has no communication layer at all.
//
// The driver is reached through a table of function pointers (DriverApi).  Production code fills it from the
// CUDA driver with cudaGetDriverEntryPoint; tests install a stand-in that backs "device memory" with memfd
// host memory, which exercises the export / descriptor passing / import / map protocol between real processes
// on a machine without a GPU.
#pragma once

#include <cuda.h>

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace titb::symm {

struct DriverApi {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                         unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  // multicast entry points may be null (driver without NVLS support, or the stand-in): the heap then has no
  // multicast address and kernels take their peer-pointer branch
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                               unsigned long long);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
};

// Entry points of the installed CUDA driver; `ok` is false (and `error` says why) when one of the mandatory ones
// cannot be resolved, e.g. on a machine without a driver.
struct DriverLookup {
  DriverApi api{};
  bool ok = false;
  std::string error;
};
DriverLookup load_cuda_driver();
// Stand-in driver over memfd + mmap (host memory).  Handles are file descriptors; no multicast.
DriverApi host_memory_driver();

struct Allocation {
  size_t bytes = 0;                 // rounded up to the allocation (and multicast) granularity
  std::vector<uint64_t> ptrs;       // ptrs[r]: rank r's copy as mapped in this process (ptrs[rank] is the local copy)
  uint64_t mc_ptr = 0;              // multicast mapping, 0 when unavailable
};

class Heap {
 public:
  // `key` must be the same string on every rank of the group and unique per group and job (it names the
  // abstract unix sockets).  `device` is the CUDA device ordinal of this rank.
  Heap(int rank, int world, int device, std::string key, DriverApi api, bool want_multicast);
  ~Heap();
  Heap(const Heap&) = delete;
  Heap& operator=(const Heap&) = delete;

  // Opens this rank's listening socket.  Every rank must have returned from listen() before any rank calls
  // exchange() (the caller separates the two with a barrier of its process group).
  void listen();
  // Collective, phase 1: allocate, export, pass descriptors, import and map the peers' allocations; create /
  // import the multicast object and add this device to it.  Returns the allocation id.
  int exchange(size_t bytes);
  // True when this rank holds the multicast object and has added its device.  The caller combines the answers of
  // all ranks (a MIN all-reduce, which is also the barrier phase 2 needs) and passes the result to finish().
  bool multicast_ready(int id) const;
  // Collective, phase 2, after a barrier that follows phase 1 on every rank (all devices must have been added
  // to the multicast object before memory is bound): bind this rank's memory and map the multicast address.
  // A failure here leaves mc_ptr == 0; the caller agrees on the outcome once more and calls drop_multicast()
  // everywhere if any rank failed, so that all ranks take the same branch in the kernels.
  const Allocation& finish(int id, bool use_multicast = true);
  void drop_multicast(int id);
  const Allocation& get(int id) const;
  void release(int id);

  int rank() const { return rank_; }
  int world() const { return world_; }
  double socket_timeout_s = 60.0;   // bound on every accept / connect wait; expiry throws, nothing spins forever

 private:
  struct Entry;
  void send_fd(int peer, int fd, int alloc_id, int kind);
  void recv_fds(int expected, int alloc_id, std::vector<int>* mem_fds, int* mc_fd);
  std::string socket_name(int r) const;

  int rank_, world_, device_;
  std::string key_;
  DriverApi api_;
  bool want_mc_;
  int listen_fd_ = -1;
  std::vector<std::unique_ptr<Entry>> entries_;
  // descriptors that arrived for an allocation id that this rank has not reached yet
  struct Pending { int src, alloc_id, kind, fd; };
  std::vector<Pending> pending_;
};

}  // namespace titb::symm
