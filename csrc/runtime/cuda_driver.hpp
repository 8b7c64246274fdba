// Lazily resolved CUDA driver API (dlopen of libcuda.so.1), so that the runtime library loads and
// its CPU backend works on a machine without a GPU or driver. Replaces the reference's ctypes
// bindings (iris/host/platform/hip.py:14-846, iris/drivers/fabric/nvidia.py:156-262).
#pragma once
#include <cuda.h>
#include <string>

namespace iris_rt {

struct DriverApi {
  bool ok = false;
  std::string error;
#define IRIS_DRV(name) decltype(&::name) name = nullptr;
  IRIS_DRV(cuInit)
  IRIS_DRV(cuDriverGetVersion)
  IRIS_DRV(cuDeviceGetCount)
  IRIS_DRV(cuDeviceGet)
  IRIS_DRV(cuDeviceGetAttribute)
  IRIS_DRV(cuDeviceGetName)
  IRIS_DRV(cuDeviceCanAccessPeer)
  IRIS_DRV(cuDeviceGetP2PAttribute)
  IRIS_DRV(cuCtxGetCurrent)
  IRIS_DRV(cuCtxSetCurrent)
  IRIS_DRV(cuCtxGetDevice)
  IRIS_DRV(cuCtxSynchronize)
  IRIS_DRV(cuDevicePrimaryCtxRetain)
  IRIS_DRV(cuGetErrorString)
  IRIS_DRV(cuMemGetAddressRange_v2)
  IRIS_DRV(cuMemAlloc_v2)
  IRIS_DRV(cuMemFree_v2)
  IRIS_DRV(cuMemsetD8_v2)
  IRIS_DRV(cuIpcGetMemHandle)
  IRIS_DRV(cuIpcOpenMemHandle_v2)
  IRIS_DRV(cuIpcCloseMemHandle)
  IRIS_DRV(cuMemCreate)
  IRIS_DRV(cuMemRelease)
  IRIS_DRV(cuMemAddressReserve)
  IRIS_DRV(cuMemAddressFree)
  IRIS_DRV(cuMemMap)
  IRIS_DRV(cuMemUnmap)
  IRIS_DRV(cuMemSetAccess)
  IRIS_DRV(cuMemExportToShareableHandle)
  IRIS_DRV(cuMemImportFromShareableHandle)
  IRIS_DRV(cuMemGetAllocationGranularity)
  IRIS_DRV(cuMemRetainAllocationHandle)
  IRIS_DRV(cuMulticastCreate)
  IRIS_DRV(cuMulticastAddDevice)
  IRIS_DRV(cuMulticastBindMem)
  IRIS_DRV(cuMulticastUnbind)
  IRIS_DRV(cuMulticastGetGranularity)
#undef IRIS_DRV
};

// Returns the table; `ok` is false (with `error` set) when libcuda or a symbol is missing.
// Tests may install a fake table with set_driver_for_testing.
const DriverApi& driver();
void set_driver_for_testing(const DriverApi* fake);
std::string cu_error(CUresult r);
// Make the primary context of `device` current on this thread if none is.
CUresult ensure_context(int device);

}  // namespace iris_rt
