#include "cuda_driver.hpp"

#include <dlfcn.h>
#include <mutex>
#include <string.h>

namespace iris_rt {

namespace {
DriverApi g_api;
const DriverApi* g_fake = nullptr;
std::once_flag g_once;

void load() {
  void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) {
    g_api.error = "libcuda.so.1 not found (no NVIDIA driver on this machine)";
    return;
  }
  bool all = true;
  std::string missing;
#define IRIS_SYM(name)                                             \
  g_api.name = (decltype(g_api.name))dlsym(h, #name);              \
  if (!g_api.name) { all = false; missing += std::string(#name) + " "; }
  IRIS_SYM(cuInit)
  IRIS_SYM(cuDriverGetVersion)
  IRIS_SYM(cuDeviceGetCount)
  IRIS_SYM(cuDeviceGet)
  IRIS_SYM(cuDeviceGetAttribute)
  IRIS_SYM(cuDeviceGetName)
  IRIS_SYM(cuDeviceCanAccessPeer)
  IRIS_SYM(cuDeviceGetP2PAttribute)
  IRIS_SYM(cuCtxGetCurrent)
  IRIS_SYM(cuCtxSetCurrent)
  IRIS_SYM(cuCtxGetDevice)
  IRIS_SYM(cuCtxSynchronize)
  IRIS_SYM(cuDevicePrimaryCtxRetain)
  IRIS_SYM(cuGetErrorString)
  IRIS_SYM(cuMemGetAddressRange_v2)
  IRIS_SYM(cuMemAlloc_v2)
  IRIS_SYM(cuMemFree_v2)
  IRIS_SYM(cuMemsetD8_v2)
  IRIS_SYM(cuIpcGetMemHandle)
  IRIS_SYM(cuIpcOpenMemHandle_v2)
  IRIS_SYM(cuIpcCloseMemHandle)
  IRIS_SYM(cuMemCreate)
  IRIS_SYM(cuMemRelease)
  IRIS_SYM(cuMemAddressReserve)
  IRIS_SYM(cuMemAddressFree)
  IRIS_SYM(cuMemMap)
  IRIS_SYM(cuMemUnmap)
  IRIS_SYM(cuMemSetAccess)
  IRIS_SYM(cuMemExportToShareableHandle)
  IRIS_SYM(cuMemImportFromShareableHandle)
  IRIS_SYM(cuMemGetAllocationGranularity)
  IRIS_SYM(cuMemRetainAllocationHandle)
  IRIS_SYM(cuMulticastCreate)
  IRIS_SYM(cuMulticastAddDevice)
  IRIS_SYM(cuMulticastBindMem)
  IRIS_SYM(cuMulticastUnbind)
  IRIS_SYM(cuMulticastGetGranularity)
#undef IRIS_SYM
  if (!all) {
    g_api.error = "libcuda is missing symbols: " + missing;
    return;
  }
  CUresult r = g_api.cuInit(0);
  if (r != CUDA_SUCCESS) {
    g_api.error = "cuInit failed with code " + std::to_string((int)r);
    return;
  }
  g_api.ok = true;
}
}  // namespace

const DriverApi& driver() {
  if (g_fake) return *g_fake;
  std::call_once(g_once, load);
  return g_api;
}

void set_driver_for_testing(const DriverApi* fake) { g_fake = fake; }

std::string cu_error(CUresult r) {
  const DriverApi& d = driver();
  const char* s = nullptr;
  if (d.cuGetErrorString && d.cuGetErrorString(r, &s) == CUDA_SUCCESS && s) return std::string(s) + " (" + std::to_string((int)r) + ")";
  return "CUDA error " + std::to_string((int)r);
}

CUresult ensure_context(int device) {
  const DriverApi& d = driver();
  if (!d.ok) return CUDA_ERROR_NOT_INITIALIZED;
  CUcontext cur = nullptr;
  d.cuCtxGetCurrent(&cur);
  if (cur) {
    CUdevice dev;
    if (d.cuCtxGetDevice(&dev) == CUDA_SUCCESS && (int)dev == device) return CUDA_SUCCESS;
  }
  CUdevice dev;
  CUresult r = d.cuDeviceGet(&dev, device);
  if (r != CUDA_SUCCESS) return r;
  CUcontext ctx;
  r = d.cuDevicePrimaryCtxRetain(&ctx, dev);
  if (r != CUDA_SUCCESS) return r;
  return d.cuCtxSetCurrent(ctx);
}

}  // namespace iris_rt
