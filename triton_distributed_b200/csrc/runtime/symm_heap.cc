// Symmetric heap: one CUDA VMM allocation per rank, mapped by every rank of the node into one
// virtual-address window (slot k = rank k's memory), optionally bound to an NVLS multicast object.
//
// Role in the reference: the NVSHMEM symmetric heap reached through nvshmem4py
// (python/triton_dist/utils.py:107-150: init by unique id over the torch process group,
// nvshmem.core.tensor / get_peer_tensor / free_tensor) and nvshmemx_mc_ptr for multimem kernels.
// Here the heap is built directly from cuMemCreate + POSIX file-descriptor handles that the ranks
// pass to each other over abstract unix datagram sockets (SCM_RIGHTS), with a cudaMalloc + CUDA IPC
// mode for machines where file-descriptor export is refused (that mode has no multicast).
//
// The Python side (runtime/heap.py) drives the collective parts: who exports, who imports, and the
// process-group barriers between "all devices added" and "bind".
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace b200 {

struct Heap {
  int device = 0;
  int rank = 0;
  int world = 1;
  bool vmm = true;
  uint64_t bytes = 0;  // per-rank heap size (rounded to granularity)
  // VMM mode
  CUdeviceptr va_base = 0;  // window of world * bytes
  CUmemGenericAllocationHandle handles[kMaxRanks] = {};
  bool mapped[kMaxRanks] = {};
  // IPC mode
  void* ipc_ptrs[kMaxRanks] = {};
  // multicast
  bool mc_bound = false;
  bool mc_added = false;
  CUmemGenericAllocationHandle mc_handle = 0;
  CUdeviceptr mc_va = 0;
  // status block (pinned host memory, device-visible)
  uint32_t* status_host = nullptr;
  uint32_t* status_dev = nullptr;
  uint64_t timeout_ns = 5000000000ull;
  // allocator (offset -> size)
  std::mutex mu;
  std::map<uint64_t, uint64_t> free_list;
  std::map<uint64_t, uint64_t> live;
};

static uint64_t round_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

static CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

static int set_rw_access(const DriverApi* d, CUdeviceptr va, uint64_t bytes, int device) {
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  B200_CHECK_CU(d->cuMemSetAccess(va, bytes, &acc, 1));
  return kOk;
}

static int multicast_supported(const DriverApi* d, int device) {
  CUdevice dev;
  if (d->cuDeviceGet(&dev, device) != CUDA_SUCCESS) return 0;
  int v = 0;
  if (d->cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
  return v;
}

static int alloc_status_block(Heap* h) {
  B200_CHECK_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&h->status_host), 64, cudaHostAllocMapped));
  memset(h->status_host, 0, 64);
  B200_CHECK_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&h->status_dev), h->status_host, 0));
  return kOk;
}

}  // namespace b200

using namespace b200;

// ------------------------------------------------------------------------------------------------
// creation
// ------------------------------------------------------------------------------------------------
B200_API int b200_heap_create(int device, int rank, int world, uint64_t bytes, int want_multicast, void** out) {
  B200_REQUIRE(world >= 1 && world <= kMaxRanks, "world size %d not in [1, %d]", world, kMaxRanks);
  B200_REQUIRE(rank >= 0 && rank < world, "rank %d out of range", rank);
  const DriverApi* d = driver();
  if (!d) return kErrDriverUnavailable;
  B200_CHECK_CUDA(cudaSetDevice(device));
  B200_CHECK_CUDA(cudaFree(nullptr));

  CUmemAllocationProp prop = alloc_prop(device);
  size_t gran = 0;
  B200_CHECK_CU(d->cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  if (want_multicast && world > 1 && multicast_supported(d, device)) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = world;
    mp.size = round_up(bytes, gran);
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d->cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran)
      gran = mg;
  }
  Heap* h = new Heap();
  h->device = device;
  h->rank = rank;
  h->world = world;
  h->vmm = true;
  h->bytes = round_up(bytes, gran);
  CUresult r = d->cuMemCreate(&h->handles[rank], h->bytes, &prop, 0);
  if (r != CUDA_SUCCESS) {
    delete h;
    return set_error(kErrUnsupported, "cuMemCreate(%llu bytes, POSIX fd handle) failed: CUresult %d",
                     static_cast<unsigned long long>(bytes), static_cast<int>(r));
  }
  r = d->cuMemAddressReserve(&h->va_base, h->bytes * world, gran, 0, 0);
  if (r != CUDA_SUCCESS) {
    d->cuMemRelease(h->handles[rank]);
    delete h;
    return set_error(static_cast<int>(r), "cuMemAddressReserve failed: CUresult %d", static_cast<int>(r));
  }
  CUdeviceptr mine = h->va_base + h->bytes * rank;
  B200_CHECK_CU(d->cuMemMap(mine, h->bytes, 0, h->handles[rank], 0));
  int rc = set_rw_access(d, mine, h->bytes, device);
  if (rc != kOk) return rc;
  h->mapped[rank] = true;
  B200_CHECK_CUDA(cudaMemset(reinterpret_cast<void*>(mine), 0, h->bytes));
  rc = alloc_status_block(h);
  if (rc != kOk) return rc;
  h->free_list[0] = h->bytes;
  *out = h;
  return kOk;
}

// cudaMalloc + CUDA IPC mode: no uniform stride, no multicast; peers are reached through the base table.
B200_API int b200_heap_create_ipc(int device, int rank, int world, uint64_t bytes, void** out) {
  B200_REQUIRE(world >= 1 && world <= kMaxRanks, "world size %d not in [1, %d]", world, kMaxRanks);
  B200_CHECK_CUDA(cudaSetDevice(device));
  Heap* h = new Heap();
  h->device = device;
  h->rank = rank;
  h->world = world;
  h->vmm = false;
  h->bytes = round_up(bytes, 2u << 20);
  cudaError_t e = cudaMalloc(&h->ipc_ptrs[rank], h->bytes);
  if (e != cudaSuccess) {
    delete h;
    return set_error(static_cast<int>(e), "cudaMalloc(%llu) failed: %s", static_cast<unsigned long long>(bytes),
                     cudaGetErrorString(e));
  }
  B200_CHECK_CUDA(cudaMemset(h->ipc_ptrs[rank], 0, h->bytes));
  int rc = alloc_status_block(h);
  if (rc != kOk) return rc;
  h->free_list[0] = h->bytes;
  *out = h;
  return kOk;
}

B200_API int b200_heap_is_vmm(void* heap) { return static_cast<Heap*>(heap)->vmm ? 1 : 0; }
B200_API uint64_t b200_heap_bytes(void* heap) { return static_cast<Heap*>(heap)->bytes; }

// ------------------------------------------------------------------------------------------------
// peer exchange
// ------------------------------------------------------------------------------------------------
B200_API int b200_heap_export_fd(void* heap, int* fd) {
  Heap* h = static_cast<Heap*>(heap);
  const DriverApi* d = driver();
  if (!d) return kErrDriverUnavailable;
  B200_REQUIRE(h->vmm, "heap is in IPC mode");
  int out = -1;
  B200_CHECK_CU(d->cuMemExportToShareableHandle(&out, h->handles[h->rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd = out;
  return kOk;
}

// Takes ownership of `fd` (closed after import).
B200_API int b200_heap_import_fd(void* heap, int peer, int fd) {
  Heap* h = static_cast<Heap*>(heap);
  const DriverApi* d = driver();
  if (!d) return kErrDriverUnavailable;
  B200_REQUIRE(h->vmm, "heap is in IPC mode");
  B200_REQUIRE(peer >= 0 && peer < h->world && peer != h->rank, "bad peer %d", peer);
  B200_CHECK_CUDA(cudaSetDevice(h->device));
  CUresult r = d->cuMemImportFromShareableHandle(&h->handles[peer], reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  if (r != CUDA_SUCCESS) return set_error(static_cast<int>(r), "cuMemImportFromShareableHandle: CUresult %d", (int)r);
  CUdeviceptr va = h->va_base + h->bytes * peer;
  B200_CHECK_CU(d->cuMemMap(va, h->bytes, 0, h->handles[peer], 0));
  int rc = set_rw_access(d, va, h->bytes, h->device);
  if (rc != kOk) return rc;
  h->mapped[peer] = true;
  return kOk;
}

B200_API int b200_heap_export_ipc(void* heap, void* handle64) {
  Heap* h = static_cast<Heap*>(heap);
  B200_REQUIRE(!h->vmm, "heap is in VMM mode");
  cudaIpcMemHandle_t ipc;
  B200_CHECK_CUDA(cudaIpcGetMemHandle(&ipc, h->ipc_ptrs[h->rank]));
  static_assert(sizeof(ipc) == 64, "cudaIpcMemHandle_t is 64 bytes");
  memcpy(handle64, &ipc, 64);
  return kOk;
}

B200_API int b200_heap_import_ipc(void* heap, int peer, const void* handle64) {
  Heap* h = static_cast<Heap*>(heap);
  B200_REQUIRE(!h->vmm, "heap is in VMM mode");
  B200_REQUIRE(peer >= 0 && peer < h->world && peer != h->rank, "bad peer %d", peer);
  B200_CHECK_CUDA(cudaSetDevice(h->device));
  cudaIpcMemHandle_t ipc;
  memcpy(&ipc, handle64, 64);
  B200_CHECK_CUDA(cudaIpcOpenMemHandle(&h->ipc_ptrs[peer], ipc, cudaIpcMemLazyEnablePeerAccess));
  return kOk;
}

// ------------------------------------------------------------------------------------------------
// NVLS multicast
// ------------------------------------------------------------------------------------------------
B200_API int b200_heap_multicast_supported(void* heap) {
  Heap* h = static_cast<Heap*>(heap);
  const DriverApi* d = driver();
  if (!d || !h->vmm || h->world < 2) return 0;
  return multicast_supported(d, h->device);
}

// Rank 0: create the multicast object and export it.
B200_API int b200_heap_mc_create(void* heap, int* fd) {
  Heap* h = static_cast<Heap*>(heap);
  const DriverApi* d = driver();
  if (!d) return kErrDriverUnavailable;
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = h->world;
  mp.size = h->bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUresult r = d->cuMulticastCreate(&h->mc_handle, &mp);
  if (r != CUDA_SUCCESS) return set_error(kErrUnsupported, "cuMulticastCreate failed: CUresult %d", (int)r);
  int out = -1;
  B200_CHECK_CU(d->cuMemExportToShareableHandle(&out, h->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd = out;
  return kOk;
}

B200_API int b200_heap_mc_import(void* heap, int fd) {
  Heap* h = static_cast<Heap*>(heap);
  const DriverApi* d = driver();
  if (!d) return kErrDriverUnavailable;
  CUresult r = d->cuMemImportFromShareableHandle(&h->mc_handle, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  if (r != CUDA_SUCCESS) return set_error(kErrUnsupported, "import of multicast handle failed: CUresult %d", (int)r);
  return kOk;
}

B200_API int b200_heap_mc_add_device(void* heap) {
  Heap* h = static_cast<Heap*>(heap);
  const DriverApi* d = driver();
  if (!d) return kErrDriverUnavailable;
  CUdevice dev;
  B200_CHECK_CU(d->cuDeviceGet(&dev, h->device));
  CUresult r = d->cuMulticastAddDevice(h->mc_handle, dev);
  if (r != CUDA_SUCCESS) return set_error(kErrUnsupported, "cuMulticastAddDevice failed: CUresult %d", (int)r);
  h->mc_added = true;
  return kOk;
}

// Every rank, after ALL ranks returned from b200_heap_mc_add_device.
B200_API int b200_heap_mc_bind(void* heap) {
  Heap* h = static_cast<Heap*>(heap);
  const DriverApi* d = driver();
  if (!d) return kErrDriverUnavailable;
  B200_CHECK_CUDA(cudaSetDevice(h->device));
  CUresult r = d->cuMulticastBindMem(h->mc_handle, 0, h->handles[h->rank], 0, h->bytes, 0);
  if (r != CUDA_SUCCESS) return set_error(kErrUnsupported, "cuMulticastBindMem failed: CUresult %d", (int)r);
  h->mc_bound = true;
  size_t gran = 2u << 20;
  B200_CHECK_CU(d->cuMemAddressReserve(&h->mc_va, h->bytes, gran, 0, 0));
  B200_CHECK_CU(d->cuMemMap(h->mc_va, h->bytes, 0, h->mc_handle, 0));
  return set_rw_access(d, h->mc_va, h->bytes, h->device);
}

// Drop the multicast mapping (used when a peer failed to bind, and by destroy).
B200_API int b200_heap_mc_release(void* heap) {
  Heap* h = static_cast<Heap*>(heap);
  const DriverApi* d = driver();
  if (!d) return kErrDriverUnavailable;
  if (h->mc_va) {
    d->cuMemUnmap(h->mc_va, h->bytes);
    d->cuMemAddressFree(h->mc_va, h->bytes);
    h->mc_va = 0;
  }
  if (h->mc_bound) {
    CUdevice dev;
    if (d->cuDeviceGet(&dev, h->device) == CUDA_SUCCESS) d->cuMulticastUnbind(h->mc_handle, dev, 0, h->bytes);
    h->mc_bound = false;
  }
  if (h->mc_handle) {
    d->cuMemRelease(h->mc_handle);
    h->mc_handle = 0;
  }
  return kOk;
}

// ------------------------------------------------------------------------------------------------
// queries
// ------------------------------------------------------------------------------------------------
B200_API uint64_t b200_heap_base(void* heap, int peer) {
  Heap* h = static_cast<Heap*>(heap);
  if (peer < 0 || peer >= h->world) return 0;
  if (h->vmm) return h->mapped[peer] ? static_cast<uint64_t>(h->va_base + h->bytes * peer) : 0;
  return reinterpret_cast<uint64_t>(h->ipc_ptrs[peer]);
}
B200_API uint64_t b200_heap_mc_base(void* heap) { return static_cast<uint64_t>(static_cast<Heap*>(heap)->mc_va); }

B200_API int b200_heap_set_timeout_ms(void* heap, uint64_t ms) {
  static_cast<Heap*>(heap)->timeout_ns = ms * 1000000ull;
  return kOk;
}

// Fill the by-value kernel argument. `out` points to sizeof(SymmCtx) bytes.
B200_API int b200_heap_get_ctx(void* heap, void* out) {
  Heap* h = static_cast<Heap*>(heap);
  SymmCtx c;
  memset(&c, 0, sizeof(c));
  c.rank = h->rank;
  c.world = h->world;
  for (int k = 0; k < h->world; ++k) {
    c.heap_base[k] = b200_heap_base(heap, k);
    B200_REQUIRE(c.heap_base[k] != 0, "peer %d is not mapped yet", k);
  }
  c.mc_base = static_cast<uint64_t>(h->mc_va);
  c.heap_bytes = h->bytes;
  c.status = h->status_dev;
  c.timeout_ns = h->timeout_ns;
  memcpy(out, &c, sizeof(c));
  return kOk;
}
B200_API int b200_symm_ctx_size() { return static_cast<int>(sizeof(SymmCtx)); }

// Copy the 16-word status block; word 0 is a StatusCode.
B200_API int b200_heap_status(void* heap, uint32_t* out16) {
  Heap* h = static_cast<Heap*>(heap);
  for (int i = 0; i < 16; ++i) out16[i] = reinterpret_cast<volatile uint32_t*>(h->status_host)[i];
  return kOk;
}
B200_API int b200_heap_status_clear(void* heap) {
  Heap* h = static_cast<Heap*>(heap);
  for (int i = 0; i < 16; ++i) reinterpret_cast<volatile uint32_t*>(h->status_host)[i] = 0;
  return kOk;
}

// ------------------------------------------------------------------------------------------------
// allocator: first fit over [0, bytes). Every rank issues the same sequence of calls, so offsets
// agree across ranks without communication.
// ------------------------------------------------------------------------------------------------
B200_API int b200_heap_alloc(void* heap, uint64_t bytes, uint64_t align, uint64_t* offset) {
  Heap* h = static_cast<Heap*>(heap);
  if (align < 256) align = 256;
  B200_REQUIRE((align & (align - 1)) == 0, "alignment %llu is not a power of two", (unsigned long long)align);
  bytes = round_up(bytes == 0 ? 1 : bytes, 256);
  std::lock_guard<std::mutex> g(h->mu);
  for (auto it = h->free_list.begin(); it != h->free_list.end(); ++it) {
    uint64_t start = round_up(it->first, align);
    uint64_t end = it->first + it->second;
    if (start + bytes <= end) {
      uint64_t fo = it->first, fs = it->second;
      h->free_list.erase(it);
      if (start > fo) h->free_list[fo] = start - fo;
      if (start + bytes < fo + fs) h->free_list[start + bytes] = fo + fs - (start + bytes);
      h->live[start] = bytes;
      *offset = start;
      return kOk;
    }
  }
  return set_error(kErrOutOfHeap, "symmetric heap exhausted: %llu bytes requested, heap is %llu bytes",
                   (unsigned long long)bytes, (unsigned long long)h->bytes);
}

B200_API int b200_heap_free(void* heap, uint64_t offset) {
  Heap* h = static_cast<Heap*>(heap);
  std::lock_guard<std::mutex> g(h->mu);
  auto it = h->live.find(offset);
  B200_REQUIRE(it != h->live.end(), "offset %llu is not a live allocation", (unsigned long long)offset);
  uint64_t size = it->second;
  h->live.erase(it);
  auto ins = h->free_list.emplace(offset, size).first;
  auto next = std::next(ins);
  if (next != h->free_list.end() && ins->first + ins->second == next->first) {
    ins->second += next->second;
    h->free_list.erase(next);
  }
  if (ins != h->free_list.begin()) {
    auto prev = std::prev(ins);
    if (prev->first + prev->second == ins->first) {
      prev->second += ins->second;
      h->free_list.erase(ins);
    }
  }
  return kOk;
}

B200_API uint64_t b200_heap_live_bytes(void* heap) {
  Heap* h = static_cast<Heap*>(heap);
  std::lock_guard<std::mutex> g(h->mu);
  uint64_t s = 0;
  for (auto& kv : h->live) s += kv.second;
  return s;
}

// ------------------------------------------------------------------------------------------------
// destruction. The caller synchronises the device and runs a process-group barrier first, so no
// peer still has kernels reading this rank's memory.
// ------------------------------------------------------------------------------------------------
B200_API int b200_heap_destroy(void* heap) {
  Heap* h = static_cast<Heap*>(heap);
  if (!h) return kOk;
  cudaSetDevice(h->device);
  cudaDeviceSynchronize();
  const DriverApi* d = driver();
  if (h->vmm && d) {
    b200_heap_mc_release(heap);
    for (int k = 0; k < h->world; ++k) {
      if (h->mapped[k]) d->cuMemUnmap(h->va_base + h->bytes * k, h->bytes);
      if (h->handles[k]) d->cuMemRelease(h->handles[k]);
    }
    if (h->va_base) d->cuMemAddressFree(h->va_base, h->bytes * h->world);
  } else if (!h->vmm) {
    for (int k = 0; k < h->world; ++k) {
      if (k == h->rank) continue;
      if (h->ipc_ptrs[k]) cudaIpcCloseMemHandle(h->ipc_ptrs[k]);
    }
    if (h->ipc_ptrs[h->rank]) cudaFree(h->ipc_ptrs[h->rank]);
  }
  if (h->status_host) cudaFreeHost(h->status_host);
  delete h;
  return kOk;
}

// ------------------------------------------------------------------------------------------------
// file-descriptor passing over abstract unix datagram sockets
// ------------------------------------------------------------------------------------------------
static socklen_t abstract_addr(sockaddr_un* sa, const char* name) {
  memset(sa, 0, sizeof(*sa));
  sa->sun_family = AF_UNIX;
  size_t n = strlen(name);
  if (n > sizeof(sa->sun_path) - 2) n = sizeof(sa->sun_path) - 2;
  memcpy(sa->sun_path + 1, name, n);  // leading NUL = abstract namespace (no file to clean up)
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

B200_API int b200_fd_socket_open(const char* name, int* sock_out) {
  int s = socket(AF_UNIX, SOCK_DGRAM, 0);
  if (s < 0) return set_error(kErrSocket, "socket(AF_UNIX): %s", strerror(errno));
  sockaddr_un sa;
  socklen_t len = abstract_addr(&sa, name);
  if (bind(s, reinterpret_cast<sockaddr*>(&sa), len) != 0) {
    int e = errno;
    close(s);
    return set_error(kErrSocket, "bind(@%s): %s", name, strerror(e));
  }
  *sock_out = s;
  return kOk;
}
B200_API int b200_fd_socket_close(int sock) {
  close(sock);
  return kOk;
}

// Send `fd` with a 2 x int32 payload {tag, aux}.
B200_API int b200_fd_send(int sock, const char* dst_name, int fd, int tag, int aux) {
  sockaddr_un sa;
  socklen_t len = abstract_addr(&sa, dst_name);
  int payload[2] = {tag, aux};
  iovec iov = {payload, sizeof(payload)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_name = &sa;
  msg.msg_namelen = len;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  for (int attempt = 0; attempt < 200; ++attempt) {
    if (sendmsg(sock, &msg, 0) >= 0) return kOk;
    if (errno == ECONNREFUSED || errno == ENOENT || errno == EAGAIN) {  // peer not bound yet
      usleep(10000);
      continue;
    }
    break;
  }
  return set_error(kErrSocket, "sendmsg(@%s): %s", dst_name, strerror(errno));
}

B200_API int b200_fd_recv(int sock, int timeout_ms, int* fd_out, int* tag_out, int* aux_out) {
  pollfd p = {sock, POLLIN, 0};
  int pr = poll(&p, 1, timeout_ms);
  if (pr == 0) return set_error(kErrTimeout, "no file descriptor arrived within %d ms", timeout_ms);
  if (pr < 0) return set_error(kErrSocket, "poll: %s", strerror(errno));
  int payload[2] = {0, 0};
  iovec iov = {payload, sizeof(payload)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  if (recvmsg(sock, &msg, 0) < 0) return set_error(kErrSocket, "recvmsg: %s", strerror(errno));
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS)
    return set_error(kErrSocket, "message carried no file descriptor");
  memcpy(fd_out, CMSG_DATA(c), sizeof(int));
  *tag_out = payload[0];
  *aux_out = payload[1];
  return kOk;
}
