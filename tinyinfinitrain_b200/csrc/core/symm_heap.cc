#include "core/symm_heap.h"

#include <cuda_runtime_api.h>
#include <fcntl.h>
#include <poll.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace titb::symm {

namespace {

constexpr int32_t kMagic = 0x53594d48;  // "SYMH"
enum Kind : int32_t { kMemHandle = 0, kMulticastHandle = 1, kNoMulticast = 2 };
struct Header { int32_t magic, src, alloc_id, kind; };

[[noreturn]] void fail(const std::string& what) { throw std::runtime_error("symmetric heap: " + what); }
void check(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) fail(std::string(what) + " failed with CUresult " + std::to_string(static_cast<int>(r)));
}
size_t round_up(size_t v, size_t g) { return (v + g - 1) / g * g; }
double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// CUDA driver
DriverLookup load_cuda_driver() {
  DriverLookup out;
  auto get = [&](const char* name, bool mandatory) -> void* {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      f = nullptr;
    (void)cudaGetLastError();
    if (f == nullptr && mandatory && out.error.empty()) out.error = std::string("driver entry point ") + name + " not found";
    return f;
  };
  DriverApi& a = out.api;
  a.MemCreate = reinterpret_cast<decltype(a.MemCreate)>(get("cuMemCreate", true));
  a.MemRelease = reinterpret_cast<decltype(a.MemRelease)>(get("cuMemRelease", true));
  a.MemGetAllocationGranularity =
      reinterpret_cast<decltype(a.MemGetAllocationGranularity)>(get("cuMemGetAllocationGranularity", true));
  a.MemExportToShareableHandle =
      reinterpret_cast<decltype(a.MemExportToShareableHandle)>(get("cuMemExportToShareableHandle", true));
  a.MemImportFromShareableHandle =
      reinterpret_cast<decltype(a.MemImportFromShareableHandle)>(get("cuMemImportFromShareableHandle", true));
  a.MemAddressReserve = reinterpret_cast<decltype(a.MemAddressReserve)>(get("cuMemAddressReserve", true));
  a.MemAddressFree = reinterpret_cast<decltype(a.MemAddressFree)>(get("cuMemAddressFree", true));
  a.MemMap = reinterpret_cast<decltype(a.MemMap)>(get("cuMemMap", true));
  a.MemUnmap = reinterpret_cast<decltype(a.MemUnmap)>(get("cuMemUnmap", true));
  a.MemSetAccess = reinterpret_cast<decltype(a.MemSetAccess)>(get("cuMemSetAccess", true));
  a.MulticastCreate = reinterpret_cast<decltype(a.MulticastCreate)>(get("cuMulticastCreate", false));
  a.MulticastAddDevice = reinterpret_cast<decltype(a.MulticastAddDevice)>(get("cuMulticastAddDevice", false));
  a.MulticastBindMem = reinterpret_cast<decltype(a.MulticastBindMem)>(get("cuMulticastBindMem", false));
  a.MulticastGetGranularity =
      reinterpret_cast<decltype(a.MulticastGetGranularity)>(get("cuMulticastGetGranularity", false));
  out.ok = out.error.empty();
  return out;
}

// ---------------------------------------------------------------------------------------------------------------
// Stand-in driver: "device memory" is a memfd, a generic allocation handle is its descriptor, address
// reservations are PROT_NONE anonymous mappings that MemMap overlays with MAP_FIXED.
namespace hostdrv {
constexpr size_t kGranularity = 65536;
CUresult MemCreate(CUmemGenericAllocationHandle* h, size_t size, const CUmemAllocationProp*, unsigned long long) {
  const int fd = memfd_create("titb-symm", 0);
  if (fd < 0) return CUDA_ERROR_OUT_OF_MEMORY;
  if (ftruncate(fd, static_cast<off_t>(size)) != 0) { close(fd); return CUDA_ERROR_OUT_OF_MEMORY; }
  *h = static_cast<CUmemGenericAllocationHandle>(fd);
  return CUDA_SUCCESS;
}
CUresult MemRelease(CUmemGenericAllocationHandle h) { return close(static_cast<int>(h)) == 0 ? CUDA_SUCCESS : CUDA_ERROR_INVALID_VALUE; }
CUresult MemGetAllocationGranularity(size_t* g, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) {
  *g = kGranularity;
  return CUDA_SUCCESS;
}
CUresult MemExport(void* out, CUmemGenericAllocationHandle h, CUmemAllocationHandleType, unsigned long long) {
  const int fd = dup(static_cast<int>(h));
  if (fd < 0) return CUDA_ERROR_INVALID_VALUE;
  *static_cast<int*>(out) = fd;
  return CUDA_SUCCESS;
}
CUresult MemImport(CUmemGenericAllocationHandle* h, void* os_handle, CUmemAllocationHandleType) {
  const int fd = dup(static_cast<int>(reinterpret_cast<intptr_t>(os_handle)));
  if (fd < 0) return CUDA_ERROR_INVALID_VALUE;
  *h = static_cast<CUmemGenericAllocationHandle>(fd);
  return CUDA_SUCCESS;
}
CUresult MemAddressReserve(CUdeviceptr* p, size_t size, size_t, CUdeviceptr, unsigned long long) {
  void* a = mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (a == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
  *p = reinterpret_cast<CUdeviceptr>(a);
  return CUDA_SUCCESS;
}
CUresult MemAddressFree(CUdeviceptr p, size_t size) {
  return munmap(reinterpret_cast<void*>(p), size) == 0 ? CUDA_SUCCESS : CUDA_ERROR_INVALID_VALUE;
}
CUresult MemMap(CUdeviceptr p, size_t size, size_t offset, CUmemGenericAllocationHandle h, unsigned long long) {
  void* a = mmap(reinterpret_cast<void*>(p), size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, static_cast<int>(h),
                 static_cast<off_t>(offset));
  return a == MAP_FAILED ? CUDA_ERROR_INVALID_VALUE : CUDA_SUCCESS;
}
CUresult MemUnmap(CUdeviceptr p, size_t size) {
  void* a = mmap(reinterpret_cast<void*>(p), size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_FIXED, -1, 0);
  return a == MAP_FAILED ? CUDA_ERROR_INVALID_VALUE : CUDA_SUCCESS;
}
CUresult MemSetAccess(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) { return CUDA_SUCCESS; }
}  // namespace hostdrv

DriverApi host_memory_driver() {
  DriverApi a{};
  a.MemCreate = hostdrv::MemCreate;
  a.MemRelease = hostdrv::MemRelease;
  a.MemGetAllocationGranularity = hostdrv::MemGetAllocationGranularity;
  a.MemExportToShareableHandle = hostdrv::MemExport;
  a.MemImportFromShareableHandle = hostdrv::MemImport;
  a.MemAddressReserve = hostdrv::MemAddressReserve;
  a.MemAddressFree = hostdrv::MemAddressFree;
  a.MemMap = hostdrv::MemMap;
  a.MemUnmap = hostdrv::MemUnmap;
  a.MemSetAccess = hostdrv::MemSetAccess;
  return a;  // multicast entry points stay null
}

// ---------------------------------------------------------------------------------------------------------------
struct Heap::Entry {
  size_t bytes = 0;
  std::vector<CUmemGenericAllocationHandle> handles;  // [world]; handles[rank] is the local allocation
  std::vector<CUdeviceptr> va;                         // [world]
  CUmemGenericAllocationHandle mc_handle = 0;
  bool has_mc_handle = false, device_added = false, finished = false, released = false;
  CUdeviceptr mc_va = 0;
  Allocation pub;
};

Heap::Heap(int rank, int world, int device, std::string key, DriverApi api, bool want_multicast)
    : rank_(rank), world_(world), device_(device), key_(std::move(key)), api_(api),
      want_mc_(want_multicast && api.MulticastCreate && api.MulticastAddDevice && api.MulticastBindMem &&
               api.MulticastGetGranularity && world > 1) {
  if (rank < 0 || rank >= world || world < 1 || world > 64) fail("bad rank / world");
  if (socket_name(world - 1).size() > 100) fail("key too long for a unix socket name");
}

Heap::~Heap() {
  for (size_t i = 0; i < entries_.size(); ++i) {
    try { release(static_cast<int>(i)); } catch (...) {}
  }
  for (auto& p : pending_) if (p.fd >= 0) close(p.fd);
  if (listen_fd_ >= 0) close(listen_fd_);
}

std::string Heap::socket_name(int r) const { return "titb-symm-" + key_ + "-" + std::to_string(r); }

static socklen_t abstract_addr(const std::string& name, sockaddr_un* addr) {
  std::memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  // abstract namespace: sun_path[0] == 0, no file system entry, gone when the last descriptor closes
  std::memcpy(addr->sun_path + 1, name.data(), name.size());
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

void Heap::listen() {
  if (listen_fd_ >= 0) return;
  const int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) fail(std::string("socket: ") + std::strerror(errno));
  sockaddr_un addr;
  const socklen_t len = abstract_addr(socket_name(rank_), &addr);
  if (bind(fd, reinterpret_cast<sockaddr*>(&addr), len) != 0) {
    const std::string e = std::strerror(errno);
    close(fd);
    fail("bind " + socket_name(rank_) + ": " + e);
  }
  if (::listen(fd, 256) != 0) {
    const std::string e = std::strerror(errno);
    close(fd);
    fail("listen: " + e);
  }
  listen_fd_ = fd;
}

void Heap::send_fd(int peer, int fd, int alloc_id, int kind) {
  const double deadline = now_s() + socket_timeout_s;
  int s = -1;
  sockaddr_un addr;
  const socklen_t len = abstract_addr(socket_name(peer), &addr);
  for (;;) {
    s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (s < 0) fail(std::string("socket: ") + std::strerror(errno));
    if (connect(s, reinterpret_cast<sockaddr*>(&addr), len) == 0) break;
    const int e = errno;
    close(s);
    if ((e != ECONNREFUSED && e != ENOENT && e != EAGAIN) || now_s() > deadline)
      fail("connect to rank " + std::to_string(peer) + ": " + std::strerror(e));
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
  Header h{kMagic, rank_, alloc_id, kind};
  iovec iov{&h, sizeof(h)};
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  if (fd >= 0) {
    std::memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  const ssize_t n = sendmsg(s, &msg, MSG_NOSIGNAL);
  const int e = errno;
  close(s);
  if (n != static_cast<ssize_t>(sizeof(h))) fail("sendmsg to rank " + std::to_string(peer) + ": " + std::strerror(e));
}

void Heap::recv_fds(int expected, int alloc_id, std::vector<int>* mem_fds, int* mc_fd) {
  int got = 0;
  auto take = [&](const Pending& p) {
    if (p.kind == kMemHandle) {
      if (p.src < 0 || p.src >= world_ || (*mem_fds)[p.src] >= 0) fail("duplicate or invalid memory handle message");
      (*mem_fds)[p.src] = p.fd;
    } else if (p.kind == kMulticastHandle) {
      *mc_fd = p.fd;
    }  // kNoMulticast carries no descriptor
    ++got;
  };
  for (size_t i = 0; i < pending_.size();) {
    if (pending_[i].alloc_id == alloc_id) { take(pending_[i]); pending_.erase(pending_.begin() + i); }
    else ++i;
  }
  const double deadline = now_s() + socket_timeout_s;
  while (got < expected) {
    const double left = deadline - now_s();
    if (left <= 0) fail("timed out waiting for " + std::to_string(expected - got) + " descriptor message(s)");
    pollfd pfd{listen_fd_, POLLIN, 0};
    const int pr = poll(&pfd, 1, static_cast<int>(left * 1000) + 1);
    if (pr < 0 && errno == EINTR) continue;
    if (pr < 0) fail(std::string("poll: ") + std::strerror(errno));
    if (pr == 0) continue;
    const int c = accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
    if (c < 0) { if (errno == EINTR || errno == EAGAIN) continue; fail(std::string("accept: ") + std::strerror(errno)); }
    timeval tv{static_cast<time_t>(socket_timeout_s), 0};
    setsockopt(c, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    Header h{};
    iovec iov{&h, sizeof(h)};
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    std::memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    const ssize_t n = recvmsg(c, &msg, MSG_CMSG_CLOEXEC | MSG_WAITALL);
    close(c);
    if (n != static_cast<ssize_t>(sizeof(h)) || h.magic != kMagic) fail("malformed descriptor message");
    int fd = -1;
    for (cmsghdr* cm = CMSG_FIRSTHDR(&msg); cm != nullptr; cm = CMSG_NXTHDR(&msg, cm))
      if (cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS) std::memcpy(&fd, CMSG_DATA(cm), sizeof(int));
    if (h.kind != kNoMulticast && fd < 0) fail("descriptor message without a descriptor");
    Pending p{h.src, h.alloc_id, h.kind, fd};
    if (h.alloc_id == alloc_id) take(p);
    else pending_.push_back(p);  // a peer that is already one allocation ahead
  }
}

int Heap::exchange(size_t bytes) {
  if (bytes == 0) fail("zero-byte allocation");
  if (world_ > 1 && listen_fd_ < 0) fail("listen() has not been called");
  const int id = static_cast<int>(entries_.size());
  entries_.push_back(std::make_unique<Entry>());
  Entry& e = *entries_.back();
  e.handles.assign(world_, 0);
  e.va.assign(world_, 0);

  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  check(api_.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  CUmulticastObjectProp mp{};
  bool mc = want_mc_;
  if (mc) {
    mp.numDevices = static_cast<unsigned>(world_);
    mp.size = round_up(bytes, gran);
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (api_.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > 0) {
      if (mg > gran) gran = mg;  // both are powers of two
    } else {
      mc = false;
    }
  }
  e.bytes = round_up(bytes, gran);
  mp.size = e.bytes;

  check(api_.MemCreate(&e.handles[rank_], e.bytes, &prop, 0), "cuMemCreate");
  if (world_ > 1) {
    int fd = -1;
    check(api_.MemExportToShareableHandle(&fd, e.handles[rank_], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
          "cuMemExportToShareableHandle");
    for (int p = 0; p < world_; ++p)
      if (p != rank_) send_fd(p, fd, id, kMemHandle);
    close(fd);
    // rank 0 owns the multicast object and tells every peer whether there is one
    if (want_mc_ && rank_ == 0) {
      int mfd = -1;
      if (mc && api_.MulticastCreate(&e.mc_handle, &mp) == CUDA_SUCCESS) {
        e.has_mc_handle = true;
        if (api_.MemExportToShareableHandle(&mfd, e.mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS)
          mfd = -1;
      }
      for (int p = 1; p < world_; ++p) send_fd(p, mfd, id, mfd >= 0 ? kMulticastHandle : kNoMulticast);
      if (mfd >= 0) close(mfd);
      else if (e.has_mc_handle) { api_.MemRelease(e.mc_handle); e.has_mc_handle = false; }
    }
    std::vector<int> fds(world_, -1);
    int mc_fd = -1;
    recv_fds(world_ - 1 + ((want_mc_ && rank_ != 0) ? 1 : 0), id, &fds, &mc_fd);
    for (int p = 0; p < world_; ++p) {
      if (p == rank_) continue;
      const CUresult r = api_.MemImportFromShareableHandle(&e.handles[p], reinterpret_cast<void*>(static_cast<intptr_t>(fds[p])),
                                                           CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      close(fds[p]);
      check(r, "cuMemImportFromShareableHandle");
    }
    if (mc_fd >= 0) {
      if (mc && api_.MemImportFromShareableHandle(&e.mc_handle, reinterpret_cast<void*>(static_cast<intptr_t>(mc_fd)),
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS)
        e.has_mc_handle = true;
      close(mc_fd);
    }
  }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int p = 0; p < world_; ++p) {
    check(api_.MemAddressReserve(&e.va[p], e.bytes, gran, 0, 0), "cuMemAddressReserve");
    check(api_.MemMap(e.va[p], e.bytes, 0, e.handles[p], 0), "cuMemMap");
    check(api_.MemSetAccess(e.va[p], e.bytes, &acc, 1), "cuMemSetAccess");
  }
  if (e.has_mc_handle) e.device_added = api_.MulticastAddDevice(e.mc_handle, static_cast<CUdevice>(device_)) == CUDA_SUCCESS;
  e.pub.bytes = e.bytes;
  e.pub.ptrs.assign(e.va.begin(), e.va.end());
  return id;
}

const Allocation& Heap::finish(int id, bool use_multicast) {
  if (id < 0 || id >= static_cast<int>(entries_.size()) || entries_[id]->released) fail("bad allocation id");
  Entry& e = *entries_[id];
  if (e.finished) return e.pub;
  e.finished = true;
  if (!use_multicast || !e.has_mc_handle || !e.device_added) return e.pub;
  if (api_.MulticastBindMem(e.mc_handle, 0, e.handles[rank_], 0, e.bytes, 0) != CUDA_SUCCESS) return e.pub;
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUdeviceptr va = 0;
  if (api_.MemAddressReserve(&va, e.bytes, 0, 0, 0) != CUDA_SUCCESS) return e.pub;
  if (api_.MemMap(va, e.bytes, 0, e.mc_handle, 0) != CUDA_SUCCESS || api_.MemSetAccess(va, e.bytes, &acc, 1) != CUDA_SUCCESS) {
    api_.MemAddressFree(va, e.bytes);
    return e.pub;
  }
  e.mc_va = va;
  e.pub.mc_ptr = va;
  return e.pub;
}

bool Heap::multicast_ready(int id) const {
  if (id < 0 || id >= static_cast<int>(entries_.size())) fail("bad allocation id");
  return entries_[id]->has_mc_handle && entries_[id]->device_added;
}

void Heap::drop_multicast(int id) {
  if (id < 0 || id >= static_cast<int>(entries_.size())) fail("bad allocation id");
  Entry& e = *entries_[id];
  if (e.mc_va) {
    api_.MemUnmap(e.mc_va, e.bytes);
    api_.MemAddressFree(e.mc_va, e.bytes);
    e.mc_va = 0;
  }
  e.pub.mc_ptr = 0;
}

const Allocation& Heap::get(int id) const {
  if (id < 0 || id >= static_cast<int>(entries_.size()) || entries_[id]->released) fail("bad allocation id");
  return entries_[id]->pub;
}

void Heap::release(int id) {
  if (id < 0 || id >= static_cast<int>(entries_.size())) fail("bad allocation id");
  Entry& e = *entries_[id];
  if (e.released) return;
  e.released = true;
  drop_multicast(id);
  if (e.has_mc_handle) api_.MemRelease(e.mc_handle);
  for (int p = 0; p < world_; ++p) {
    if (e.va[p]) {
      api_.MemUnmap(e.va[p], e.bytes);
      api_.MemAddressFree(e.va[p], e.bytes);
    }
    if (e.handles[p]) api_.MemRelease(e.handles[p]);
  }
  e.pub = Allocation{};
}

}  // namespace titb::symm
