// Symmetric heap over the CUDA virtual-memory-management API.
//
// Each rank owns one physical allocation (cuMemCreate, exportable as a POSIX
// file descriptor).  Every process reserves ONE virtual window of
// world_size * stride bytes and maps rank r's allocation at window + r * stride,
// so device code reaches a peer's copy of an object by adding
// (peer - self) * stride to its own pointer: no table of bases is needed.  When
// all devices support NVLS multicast, the heaps are additionally bound to one
// multicast object whose mapping (`mc_base`) aliases every rank's heap at once.
//
// Two process models, same layout:
//   * single process: this process creates and maps every rank's allocation
//     (reference: SymmetricHeap.create_all, tileccl/memory/symmetric_heap.py:238-343);
//   * one process per rank: allocation handles are exported as file descriptors
//     and passed to the peers over Unix sockets (reference: CUDA IPC handles over
//     torch.distributed, tileccl/memory/symmetric_heap.py:749-828).
//
// Allocation inside the heap is a 256-byte aligned bump pointer that is never
// rewound except by an explicit reset, as in the reference's TorchBumpAllocator
// (tileccl/memory/allocators.py:477-607).  Symmetric allocation is collective by
// construction: every rank must allocate the same sizes in the same order.
#include <cuda_runtime.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include "../api.h"
#include "bootstrap.h"
#include "errors.h"

namespace tileccl {
namespace {

constexpr uint64_t kAlign = 256;

enum HeapMode { kLocalOnly = 0, kSingleProcess = 1, kMultiProcess = 2 };
enum Transport { kNone = 0, kVmmSingleProcess = 1, kVmmFd = 2, kVmmFabric = 3 };

// State shared by all rank handles of one window (one per process).
struct Window {
  CUdeviceptr base = 0;
  size_t stride = 0;
  int world_size = 0;
  size_t granularity = 0;
  std::vector<CUmemGenericAllocationHandle> mem;  // per rank (imported for peers)
  std::vector<bool> mapped;
  std::vector<int> devices;                       // per rank, -1 = not on this process
  CUdeviceptr mc_base = 0;
  CUmemGenericAllocationHandle mc_handle = 0;
  bool mc_created = false, mc_mapped = false;
  std::vector<bool> mc_bound;
  int mode = kLocalOnly;
  int transport = kNone;

  ~Window() { teardown(); }

  void teardown() {
    const DriverApi& d = driver();
    if (!d.ok) return;
    if (mc_mapped) {
      d.cuMemUnmap(mc_base, stride);
      mc_mapped = false;
    }
    if (mc_base) {
      d.cuMemAddressFree(mc_base, stride);
      mc_base = 0;
    }
    if (mc_created) {
      for (size_t r = 0; r < mc_bound.size(); ++r) {
        if (mc_bound[r] && d.cuMulticastUnbind && devices[r] >= 0) {
          CUdevice dev;
          if (d.cuDeviceGet(&dev, devices[r]) == CUDA_SUCCESS)
            d.cuMulticastUnbind(mc_handle, dev, 0, stride);
        }
      }
      d.cuMemRelease(mc_handle);
      mc_created = false;
    }
    for (size_t r = 0; r < mem.size(); ++r) {
      if (mapped[r]) {
        d.cuMemUnmap(base + r * stride, stride);
        mapped[r] = false;
      }
      if (mem[r]) {
        d.cuMemRelease(mem[r]);
        mem[r] = 0;
      }
    }
    if (base) {
      d.cuMemAddressFree(base, stride * world_size);
      base = 0;
    }
  }
};

struct Heap {
  std::shared_ptr<Window> win;
  int rank = 0;
  int device = 0;
  uint64_t requested = 0;
  uint64_t bump = 0;
  std::mutex mu;
};

int make_props(int device, CUmemAllocationProp* prop) {
  std::memset(prop, 0, sizeof(*prop));
  prop->type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop->location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop->location.id = device;
  prop->requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return kOk;
}

int ensure_context(int device) {
  TCCL_CHECK_CUDA(cudaSetDevice(device));
  TCCL_CHECK_CUDA(cudaFree(nullptr));  // forces primary-context creation
  return kOk;
}

bool all_support_multicast(const std::vector<int>& devices) {
  const DriverApi& d = driver();
  if (!d.cuMulticastCreate || !d.cuMulticastAddDevice || !d.cuMulticastBindMem ||
      !d.cuMulticastGetGranularity)
    return false;
  for (int ord : devices) {
    CUdevice dev;
    int a = 0;
    if (d.cuDeviceGet(&dev, ord) != CUDA_SUCCESS) return false;
    if (d.cuDeviceGetAttribute(&a, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS ||
        !a)
      return false;
  }
  return true;
}

int set_access(CUdeviceptr ptr, size_t size, const std::vector<int>& devices) {
  const DriverApi& d = driver();
  std::vector<int> uniq(devices);
  std::sort(uniq.begin(), uniq.end());
  uniq.erase(std::unique(uniq.begin(), uniq.end()), uniq.end());
  std::vector<CUmemAccessDesc> acc;
  for (int ord : uniq) {
    if (ord < 0) continue;
    CUmemAccessDesc a;
    std::memset(&a, 0, sizeof(a));
    a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    a.location.id = ord;
    a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    acc.push_back(a);
  }
  TCCL_CHECK_CU(d.cuMemSetAccess(ptr, size, acc.data(), acc.size()));
  return kOk;
}

int compute_stride(uint64_t size, const std::vector<int>& devices, bool want_mc, size_t* gran_out,
                   size_t* stride_out) {
  const DriverApi& d = driver();
  size_t gran = 0;
  for (int ord : devices) {
    CUmemAllocationProp prop;
    make_props(ord, &prop);
    size_t g = 0;
    TCCL_CHECK_CU(d.cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    gran = std::max(gran, g);
  }
  if (want_mc) {
    CUmulticastObjectProp mp;
    std::memset(&mp, 0, sizeof(mp));
    mp.numDevices = static_cast<unsigned>(devices.size());
    mp.size = size;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t g = 0;
    if (d.cuMulticastGetGranularity(&g, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS)
      gran = std::max(gran, g);
  }
  if (gran == 0) gran = 2u << 20;
  *gran_out = gran;
  *stride_out = ((size + gran - 1) / gran) * gran;
  return kOk;
}

}  // namespace
}  // namespace tileccl

using namespace tileccl;

extern "C" int tccl_heap_create_local(int32_t world_size, uint64_t size, const int32_t* devices,
                                      int32_t want_nvls, void** handles_out) {
  TCCL_REQUIRE_DRIVER();
  TCCL_CHECK_ARG(world_size >= 1 && world_size <= TCCL_MAX_RANKS, "world_size must be 1..8");
  TCCL_CHECK_ARG(size > 0, "heap size must be positive");
  TCCL_CHECK_ARG(devices != nullptr && handles_out != nullptr, "null argument");
  const DriverApi& d = driver();
  int prev_dev = 0;
  TCCL_CHECK_CUDA(cudaGetDevice(&prev_dev));

  auto win = std::make_shared<Window>();
  win->world_size = world_size;
  win->devices.assign(devices, devices + world_size);
  win->mem.assign(world_size, 0);
  win->mapped.assign(world_size, false);
  win->mc_bound.assign(world_size, false);
  win->mode = world_size == 1 ? kLocalOnly : kSingleProcess;
  win->transport = world_size == 1 ? kNone : kVmmSingleProcess;

  for (int r = 0; r < world_size; ++r) {
    int rc = ensure_context(devices[r]);
    if (rc) return rc;
  }
  // One multicast binding per device: only possible when every rank has its own GPU.
  std::vector<int> uniq(win->devices);
  std::sort(uniq.begin(), uniq.end());
  const bool distinct = std::unique(uniq.begin(), uniq.end()) == uniq.end();
  const bool use_mc = want_nvls && world_size > 1 && distinct && all_support_multicast(win->devices);

  int rc = compute_stride(size, win->devices, use_mc, &win->granularity, &win->stride);
  if (rc) return rc;
  TCCL_CHECK_CU(d.cuMemAddressReserve(&win->base, win->stride * world_size, win->granularity, 0, 0));
  for (int r = 0; r < world_size; ++r) {
    TCCL_CHECK_CUDA(cudaSetDevice(devices[r]));
    CUmemAllocationProp prop;
    make_props(devices[r], &prop);
    TCCL_CHECK_CU(d.cuMemCreate(&win->mem[r], win->stride, &prop, 0));
    TCCL_CHECK_CU(d.cuMemMap(win->base + r * win->stride, win->stride, 0, win->mem[r], 0));
    win->mapped[r] = true;
  }
  rc = set_access(win->base, win->stride * world_size, win->devices);
  if (rc) return rc;

  if (use_mc) {
    CUmulticastObjectProp mp;
    std::memset(&mp, 0, sizeof(mp));
    mp.numDevices = static_cast<unsigned>(world_size);
    mp.size = win->stride;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    if (d.cuMulticastCreate(&win->mc_handle, &mp) == CUDA_SUCCESS) {
      win->mc_created = true;
      bool ok = true;
      for (int r = 0; r < world_size && ok; ++r) {
        CUdevice dev;
        ok = d.cuDeviceGet(&dev, devices[r]) == CUDA_SUCCESS &&
             d.cuMulticastAddDevice(win->mc_handle, dev) == CUDA_SUCCESS;
      }
      for (int r = 0; r < world_size && ok; ++r) {
        ok = d.cuMulticastBindMem(win->mc_handle, 0, win->mem[r], 0, win->stride, 0) == CUDA_SUCCESS;
        win->mc_bound[r] = ok;
      }
      if (ok) ok = d.cuMemAddressReserve(&win->mc_base, win->stride, win->granularity, 0, 0) ==
                   CUDA_SUCCESS;
      if (ok) {
        ok = d.cuMemMap(win->mc_base, win->stride, 0, win->mc_handle, 0) == CUDA_SUCCESS;
        win->mc_mapped = ok;
      }
      if (ok) ok = set_access(win->mc_base, win->stride, win->devices) == kOk;
      if (!ok) {
        // NVLS is an optimisation: fall back to plain peer mappings.
        if (win->mc_mapped) { d.cuMemUnmap(win->mc_base, win->stride); win->mc_mapped = false; }
        if (win->mc_base) { d.cuMemAddressFree(win->mc_base, win->stride); win->mc_base = 0; }
      }
    }
  }
  for (int r = 0; r < world_size; ++r) {
    // Fresh heap memory is all zeroes (see the multi-process path for why that matters).
    TCCL_CHECK_CUDA(cudaSetDevice(devices[r]));
    TCCL_CHECK_CUDA(cudaMemset(reinterpret_cast<void*>(win->base + r * win->stride), 0, win->stride));
    TCCL_CHECK_CUDA(cudaDeviceSynchronize());
  }
  for (int r = 0; r < world_size; ++r) {
    Heap* h = new Heap();
    h->win = win;
    h->rank = r;
    h->device = devices[r];
    h->requested = size;
    handles_out[r] = h;
  }
  TCCL_CHECK_CUDA(cudaSetDevice(prev_dev));
  return kOk;
}

extern "C" int tccl_heap_create_multiprocess(int32_t rank, int32_t world_size, uint64_t size,
                                             int32_t device, const char* job_id, int32_t want_nvls,
                                             int32_t timeout_ms, void** handle_out) {
  TCCL_REQUIRE_DRIVER();
  TCCL_CHECK_ARG(world_size >= 1 && world_size <= TCCL_MAX_RANKS, "world_size must be 1..8");
  TCCL_CHECK_ARG(rank >= 0 && rank < world_size, "rank out of range");
  TCCL_CHECK_ARG(size > 0 && job_id != nullptr && handle_out != nullptr, "bad argument");
  const DriverApi& d = driver();
  int rc = ensure_context(device);
  if (rc) return rc;

  Bootstrap boot(rank, world_size, job_id, timeout_ms > 0 ? timeout_ms : 60000);
  if (!boot.open()) return fail(kErrSystem, "bootstrap: " + boot.error());

  auto win = std::make_shared<Window>();
  win->world_size = world_size;
  win->devices.assign(world_size, -1);
  win->devices[rank] = device;
  win->mem.assign(world_size, 0);
  win->mapped.assign(world_size, false);
  win->mc_bound.assign(world_size, false);
  win->mode = world_size == 1 ? kLocalOnly : kMultiProcess;
  win->transport = world_size == 1 ? kNone : kVmmFd;

  // Agree on NVLS: every rank must be able to, and want to.
  std::vector<int> my_dev{device};
  uint64_t can_mc = (want_nvls && world_size > 1 && all_support_multicast(my_dev)) ? 1 : 0;
  std::vector<uint64_t> votes;
  if (!boot.all_gather(1, can_mc, -1, &votes, nullptr))
    return fail(kErrSystem, "bootstrap (capability vote): " + boot.error());
  bool use_mc = true;
  for (uint64_t v : votes) use_mc = use_mc && v != 0;

  // Same stride everywhere: take the largest granularity any rank reports.
  size_t gran = 0, stride = 0;
  rc = compute_stride(size, my_dev, false, &gran, &stride);
  if (rc) return rc;
  if (use_mc) {
    CUmulticastObjectProp mp;
    std::memset(&mp, 0, sizeof(mp));
    mp.numDevices = static_cast<unsigned>(world_size);
    mp.size = size;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t g = 0;
    if (d.cuMulticastGetGranularity(&g, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS)
      gran = std::max(gran, g);
  }
  std::vector<uint64_t> grans;
  if (!boot.all_gather(2, gran, -1, &grans, nullptr))
    return fail(kErrSystem, "bootstrap (granularity): " + boot.error());
  for (uint64_t g : grans) gran = std::max<size_t>(gran, g);
  stride = ((size + gran - 1) / gran) * gran;
  win->granularity = gran;
  win->stride = stride;

  TCCL_CHECK_CU(d.cuMemAddressReserve(&win->base, stride * world_size, gran, 0, 0));
  CUmemAllocationProp prop;
  make_props(device, &prop);
  TCCL_CHECK_CU(d.cuMemCreate(&win->mem[rank], stride, &prop, 0));
  TCCL_CHECK_CU(d.cuMemMap(win->base + rank * stride, stride, 0, win->mem[rank], 0));
  win->mapped[rank] = true;

  if (world_size > 1) {
    int my_fd = -1;
    TCCL_CHECK_CU(d.cuMemExportToShareableHandle(&my_fd, win->mem[rank],
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    std::vector<int> fds;
    std::vector<uint64_t> strides;
    bool ok = boot.all_gather(3, stride, my_fd, &strides, &fds);
    close(my_fd);
    if (!ok) return fail(kErrSystem, "bootstrap (handle exchange): " + boot.error());
    for (int r = 0; r < world_size; ++r) {
      if (r == rank) continue;
      if (strides[r] != stride) {
        for (int f : fds) if (f >= 0 && f != my_fd) close(f);
        return fail(kErrInvalid, "rank " + std::to_string(r) + " created a heap of a different size");
      }
      CUresult cr = d.cuMemImportFromShareableHandle(
          &win->mem[r], reinterpret_cast<void*>(static_cast<intptr_t>(fds[r])),
          CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      close(fds[r]);
      if (cr != CUDA_SUCCESS)
        return fail(kErrCuda, "cuMemImportFromShareableHandle(rank " + std::to_string(r) + "): " +
                                  driver_error_string(cr));
      TCCL_CHECK_CU(d.cuMemMap(win->base + r * stride, stride, 0, win->mem[r], 0));
      win->mapped[r] = true;
    }
  }
  rc = set_access(win->base, stride * world_size, my_dev);
  if (rc) return rc;

  if (use_mc) {
    // Rank 0 creates the multicast object; everyone adds its device, then
    // (after a barrier: all devices must be added first) binds its memory.
    bool ok = true;
    int mc_fd = -1;
    if (rank == 0) {
      CUmulticastObjectProp mp;
      std::memset(&mp, 0, sizeof(mp));
      mp.numDevices = static_cast<unsigned>(world_size);
      mp.size = stride;
      mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      ok = d.cuMulticastCreate(&win->mc_handle, &mp) == CUDA_SUCCESS;
      if (ok) {
        win->mc_created = true;
        ok = d.cuMemExportToShareableHandle(&mc_fd, win->mc_handle,
                                            CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) ==
             CUDA_SUCCESS;
      }
    }
    uint64_t created = ok ? 1 : 0;
    if (!boot.broadcast(4, 0, &created, &mc_fd))
      return fail(kErrSystem, "bootstrap (multicast handle): " + boot.error());
    ok = created != 0;
    if (ok && rank != 0) {
      ok = d.cuMemImportFromShareableHandle(&win->mc_handle,
                                            reinterpret_cast<void*>(static_cast<intptr_t>(mc_fd)),
                                            CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS;
      win->mc_created = ok;
    }
    if (mc_fd >= 0) close(mc_fd);
    CUdevice dev;
    if (ok) ok = d.cuDeviceGet(&dev, device) == CUDA_SUCCESS &&
                 d.cuMulticastAddDevice(win->mc_handle, dev) == CUDA_SUCCESS;
    std::vector<uint64_t> oks;
    if (!boot.all_gather(5, ok ? 1 : 0, -1, &oks, nullptr))
      return fail(kErrSystem, "bootstrap (multicast add): " + boot.error());
    for (uint64_t v : oks) ok = ok && v != 0;
    if (ok) {
      ok = d.cuMulticastBindMem(win->mc_handle, 0, win->mem[rank], 0, stride, 0) == CUDA_SUCCESS;
      win->mc_bound[rank] = ok;
      if (ok) ok = d.cuMemAddressReserve(&win->mc_base, stride, gran, 0, 0) == CUDA_SUCCESS;
      if (ok) {
        ok = d.cuMemMap(win->mc_base, stride, 0, win->mc_handle, 0) == CUDA_SUCCESS;
        win->mc_mapped = ok;
      }
      if (ok) ok = set_access(win->mc_base, stride, my_dev) == kOk;
    }
    if (!boot.all_gather(6, ok ? 1 : 0, -1, &oks, nullptr))
      return fail(kErrSystem, "bootstrap (multicast bind): " + boot.error());
    bool all_ok = true;
    for (uint64_t v : oks) all_ok = all_ok && v != 0;
    if (!all_ok) {
      // Some rank could not bind: nobody uses the multicast alias.
      if (win->mc_mapped) { d.cuMemUnmap(win->mc_base, stride); win->mc_mapped = false; }
      if (win->mc_base) { d.cuMemAddressFree(win->mc_base, stride); win->mc_base = 0; }
    }
  }
  // The heap starts out zeroed, and is zeroed BEFORE any peer can reach it: flags and
  // counters carved out of fresh heap memory need no further initialisation (a memset
  // issued later by the owner could wipe a signal that a faster peer has already sent).
  TCCL_CHECK_CUDA(cudaMemset(reinterpret_cast<void*>(win->base + rank * stride), 0, stride));
  TCCL_CHECK_CUDA(cudaDeviceSynchronize());
  if (world_size > 1 && !boot.barrier(7))
    return fail(kErrSystem, "bootstrap (final barrier): " + boot.error());

  Heap* h = new Heap();
  h->win = win;
  h->rank = rank;
  h->device = device;
  h->requested = size;
  *handle_out = h;
  return kOk;
}

extern "C" int tccl_heap_info(void* handle, TcclHeapInfo* out) {
  TCCL_CHECK_ARG(handle != nullptr && out != nullptr, "null argument");
  Heap* h = static_cast<Heap*>(handle);
  out->window_base = h->win->base;
  out->stride = h->win->stride;
  out->mc_base = h->win->mc_mapped ? h->win->mc_base : 0;
  out->requested_size = h->requested;
  out->granularity = h->win->granularity;
  out->rank = h->rank;
  out->world_size = h->win->world_size;
  out->device = h->device;
  out->mode = h->win->mode;
  out->transport = h->win->transport;
  out->nvls_bound = h->win->mc_mapped ? 1 : 0;
  return kOk;
}

extern "C" int tccl_heap_destroy(void* handle) {
  if (handle == nullptr) return kOk;
  Heap* h = static_cast<Heap*>(handle);
  // The window is torn down when its last rank handle goes away.
  delete h;
  return kOk;
}

extern "C" int tccl_heap_alloc(void* handle, uint64_t bytes, uint64_t* offset_out) {
  TCCL_CHECK_ARG(handle != nullptr && offset_out != nullptr, "null argument");
  Heap* h = static_cast<Heap*>(handle);
  std::lock_guard<std::mutex> lock(h->mu);
  uint64_t start = (h->bump + kAlign - 1) / kAlign * kAlign;
  uint64_t need = bytes == 0 ? kAlign : bytes;
  if (start + need > h->requested) {
    return fail(kErrInvalid, "symmetric heap exhausted: requested " + std::to_string(bytes) +
                                 " bytes, " + std::to_string(h->requested - std::min<uint64_t>(start, h->requested)) +
                                 " free of " + std::to_string(h->requested));
  }
  h->bump = start + need;
  *offset_out = start;
  return kOk;
}

extern "C" int tccl_heap_reset(void* handle) {
  TCCL_CHECK_ARG(handle != nullptr, "null argument");
  Heap* h = static_cast<Heap*>(handle);
  std::lock_guard<std::mutex> lock(h->mu);
  h->bump = 0;
  return kOk;
}

extern "C" int tccl_heap_bytes_allocated(void* handle, uint64_t* out) {
  TCCL_CHECK_ARG(handle != nullptr && out != nullptr, "null argument");
  Heap* h = static_cast<Heap*>(handle);
  std::lock_guard<std::mutex> lock(h->mu);
  *out = h->bump;
  return kOk;
}

// Host-only entry point used by the tests of the rendezvous layer: all-gathers
// one (payload, fd) per rank.  fds_out[rank] is the caller's own descriptor.
extern "C" int tccl_bootstrap_allgather(int32_t rank, int32_t world_size, const char* job_id,
                                        int32_t timeout_ms, uint64_t payload, int32_t fd,
                                        uint64_t* payloads_out, int32_t* fds_out) {
  TCCL_CHECK_ARG(job_id != nullptr && payloads_out != nullptr && fds_out != nullptr, "null argument");
  TCCL_CHECK_ARG(rank >= 0 && rank < world_size, "rank out of range");
  Bootstrap boot(rank, world_size, job_id, timeout_ms);
  if (!boot.open()) return fail(kErrSystem, "bootstrap: " + boot.error());
  std::vector<uint64_t> payloads;
  std::vector<int> fds;
  if (!boot.all_gather(1, payload, fd, &payloads, &fds))
    return fail(kErrTimeout, "bootstrap: " + boot.error());
  // Keep the listening socket alive until every rank has everything.
  if (!boot.barrier(2)) return fail(kErrTimeout, "bootstrap: " + boot.error());
  for (int r = 0; r < world_size; ++r) {
    payloads_out[r] = payloads[r];
    fds_out[r] = fds[r];
  }
  return kOk;
}
