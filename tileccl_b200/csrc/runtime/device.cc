// Device and topology query.  Replaces the reference's ctypes wrappers around
// libcudart plus its `nvidia-smi topo -m` parsing (tileccl/backends/cuda.py:79-187,
// 326-372) with direct runtime/driver attribute queries, including the three
// capabilities the symmetric heap depends on: VMM, POSIX-fd / fabric handle
// export, and NVLS multicast.
#include <cuda_runtime.h>

#include <cstring>

#include "../api.h"
#include "errors.h"

using namespace tileccl;

extern "C" int tccl_device_count(int32_t* count) {
  TCCL_CHECK_ARG(count != nullptr, "null argument");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;  // no driver / no device is a valid answer, not an error
  }
  *count = n;
  return kOk;
}

extern "C" int tccl_device_props(int32_t ordinal, TcclDeviceProps* out) {
  TCCL_CHECK_ARG(out != nullptr, "null argument");
  std::memset(out, 0, sizeof(*out));
  cudaDeviceProp prop;
  TCCL_CHECK_CUDA(cudaGetDeviceProperties(&prop, ordinal));
  std::strncpy(out->name, prop.name, sizeof(out->name) - 1);
  out->ordinal = ordinal;
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->sm_count = prop.multiProcessorCount;
  out->warp_size = prop.warpSize;
  out->max_smem_per_block_optin = static_cast<int32_t>(prop.sharedMemPerBlockOptin);
  out->l2_bytes = prop.l2CacheSize;
  out->mem_bus_bits = prop.memoryBusWidth;
  out->total_mem = static_cast<int64_t>(prop.totalGlobalMem);
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, ordinal) == cudaSuccess) out->clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, ordinal) == cudaSuccess)
    out->mem_clock_khz = v;
  (void)cudaGetLastError();

  const DriverApi& d = driver();
  if (d.ok) {
    CUdevice dev;
    if (d.cuDeviceGet(&dev, ordinal) == CUDA_SUCCESS) {
      int a = 0;
      if (d.cuDeviceGetAttribute(&a, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED,
                                 dev) == CUDA_SUCCESS)
        out->vmm_supported = a;
      if (d.cuDeviceGetAttribute(&a, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED,
                                 dev) == CUDA_SUCCESS)
        out->posix_fd_handles = a;
      if (d.cuDeviceGetAttribute(&a, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_FABRIC_SUPPORTED, dev) ==
          CUDA_SUCCESS)
        out->fabric_handles = a;
      if (d.cuDeviceGetAttribute(&a, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS)
        out->multicast_supported = a;
    }
  }
  return kOk;
}

extern "C" int tccl_peer_matrix(int32_t n, int32_t* access, int32_t* native_atomics) {
  TCCL_CHECK_ARG(n >= 0 && access != nullptr, "bad argument");
  for (int i = 0; i < n; ++i) {
    for (int j = 0; j < n; ++j) {
      int can = (i == j) ? 1 : 0, atom = (i == j) ? 1 : 0;
      if (i != j) {
        TCCL_CHECK_CUDA(cudaDeviceCanAccessPeer(&can, i, j));
        if (can && native_atomics) {
          if (cudaDeviceGetP2PAttribute(&atom, cudaDevP2PAttrNativeAtomicSupported, i, j) !=
              cudaSuccess) {
            (void)cudaGetLastError();
            atom = 0;
          }
        }
      }
      access[i * n + j] = can;
      if (native_atomics) native_atomics[i * n + j] = atom;
    }
  }
  return kOk;
}
