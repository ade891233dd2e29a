#include "driver_api.h"

#include <cuda_runtime.h>

#include <mutex>

namespace tileccl {

namespace {

template <typename Fn>
bool resolve(const char* name, Fn*& out, std::string& err) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) {
    (void)cudaGetLastError();
    if (err.empty()) {
      err = std::string("driver entry point '") + name + "' unavailable";
      if (e != cudaSuccess) err += std::string(": ") + cudaGetErrorString(e);
    }
    out = nullptr;
    return false;
  }
  out = reinterpret_cast<Fn*>(fn);
  return true;
}

DriverApi load() {
  DriverApi d;
  bool ok = true;
#define TILECCL_RESOLVE(NAME) ok = resolve(#NAME, d.NAME, d.error) && ok
  TILECCL_RESOLVE(cuInit);
  TILECCL_RESOLVE(cuGetErrorString);
  TILECCL_RESOLVE(cuDeviceGet);
  TILECCL_RESOLVE(cuDeviceGetCount);
  TILECCL_RESOLVE(cuDeviceGetName);
  TILECCL_RESOLVE(cuDeviceTotalMem);
  TILECCL_RESOLVE(cuDeviceGetAttribute);
  TILECCL_RESOLVE(cuDeviceCanAccessPeer);
  TILECCL_RESOLVE(cuDeviceGetP2PAttribute);
  TILECCL_RESOLVE(cuCtxGetCurrent);
  TILECCL_RESOLVE(cuCtxSetCurrent);
  TILECCL_RESOLVE(cuDevicePrimaryCtxRetain);
  TILECCL_RESOLVE(cuMemGetAllocationGranularity);
  TILECCL_RESOLVE(cuMemCreate);
  TILECCL_RESOLVE(cuMemRelease);
  TILECCL_RESOLVE(cuMemAddressReserve);
  TILECCL_RESOLVE(cuMemAddressFree);
  TILECCL_RESOLVE(cuMemMap);
  TILECCL_RESOLVE(cuMemUnmap);
  TILECCL_RESOLVE(cuMemSetAccess);
  TILECCL_RESOLVE(cuMemExportToShareableHandle);
  TILECCL_RESOLVE(cuMemImportFromShareableHandle);
  TILECCL_RESOLVE(cuTensorMapEncodeTiled);
  // Multicast entry points exist from CUDA 12.1 drivers on; their absence only
  // disables NVLS, so it is not an error.
  std::string ignored;
  resolve("cuMulticastCreate", d.cuMulticastCreate, ignored);
  resolve("cuMulticastAddDevice", d.cuMulticastAddDevice, ignored);
  resolve("cuMulticastBindMem", d.cuMulticastBindMem, ignored);
  resolve("cuMulticastUnbind", d.cuMulticastUnbind, ignored);
  resolve("cuMulticastGetGranularity", d.cuMulticastGetGranularity, ignored);
#undef TILECCL_RESOLVE
  d.ok = ok;
  return d;
}

}  // namespace

const DriverApi& driver() {
  static DriverApi api = load();
  return api;
}

std::string driver_error_string(CUresult r) {
  const DriverApi& d = driver();
  const char* s = nullptr;
  if (d.cuGetErrorString && d.cuGetErrorString(r, &s) == CUDA_SUCCESS && s)
    return std::string(s) + " (CUresult " + std::to_string(static_cast<int>(r)) + ")";
  return "CUresult " + std::to_string(static_cast<int>(r));
}

}  // namespace tileccl
