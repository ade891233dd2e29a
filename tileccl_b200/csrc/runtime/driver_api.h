// Lazily resolved CUDA driver entry points.  The library never links against
// libcuda: it has to import on a machine without a GPU driver (planning, CPU
// emulation and the test suite run there), so every driver call goes through
// this table, filled on first use through cudaGetDriverEntryPoint.
#pragma once
#include <cuda.h>

#include <string>

namespace tileccl {

struct DriverApi {
  bool ok = false;
  std::string error;

  CUresult (*cuInit)(unsigned) = nullptr;
  CUresult (*cuGetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*cuDeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*cuDeviceGetCount)(int*) = nullptr;
  CUresult (*cuDeviceGetName)(char*, int, CUdevice) = nullptr;
  CUresult (*cuDeviceTotalMem)(size_t*, CUdevice) = nullptr;
  CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*cuDeviceCanAccessPeer)(int*, CUdevice, CUdevice) = nullptr;
  CUresult (*cuDeviceGetP2PAttribute)(int*, CUdevice_P2PAttribute, CUdevice, CUdevice) = nullptr;
  CUresult (*cuCtxGetCurrent)(CUcontext*) = nullptr;
  CUresult (*cuCtxSetCurrent)(CUcontext) = nullptr;
  CUresult (*cuDevicePrimaryCtxRetain)(CUcontext*, CUdevice) = nullptr;
  CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                            CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                          unsigned long long) = nullptr;
  CUresult (*cuMemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr,
                                  unsigned long long) = nullptr;
  CUresult (*cuMemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                       unsigned long long) = nullptr;
  CUresult (*cuMemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*cuMemExportToShareableHandle)(void*, CUmemGenericAllocationHandle,
                                           CUmemAllocationHandleType,
                                           unsigned long long) = nullptr;
  CUresult (*cuMemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*,
                                             CUmemAllocationHandleType) = nullptr;
  CUresult (*cuMulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) =
      nullptr;
  CUresult (*cuMulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*cuMulticastBindMem)(CUmemGenericAllocationHandle, size_t,
                                 CUmemGenericAllocationHandle, size_t, size_t,
                                 unsigned long long) = nullptr;
  CUresult (*cuMulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*cuMulticastGetGranularity)(size_t*, const CUmulticastObjectProp*,
                                        CUmulticastGranularity_flags) = nullptr;
  CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                     const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                     const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
};

// Returns the process-wide table; `ok` is false (with `error` set) when no
// driver is present.
const DriverApi& driver();

// "CUDA_ERROR_xxx: text" for a driver status.
std::string driver_error_string(CUresult r);

}  // namespace tileccl
