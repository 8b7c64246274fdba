// Driver-level memory primitives exported one by one, for `iris_b200.hip` (the names of the reference's
// ctypes layer, iris/host/platform/hip.py:326-846: hip_malloc / hip_free, get_allocation_granularity,
// mem_create, mem_address_reserve, mem_map, mem_set_access, mem_export_to_shareable_handle, ...).
// The symmetric heap does not go through these (it owns its sequence of calls in symmetric_heap.cpp);
// they exist so that user code and tests can build their own mappings the way the reference's users do.
// Every function returns 0 or the negated CUresult, -1000 when no driver is loaded.
#include <stdint.h>
#include <string.h>

#include "cuda_driver.hpp"

using namespace iris_rt;

namespace {
constexpr int kNoDriver = -1000;

int rc(CUresult r) { return r == CUDA_SUCCESS ? 0 : -(int)r; }

void fill_prop(CUmemAllocationProp& prop, int device, int fabric) {
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = fabric ? CU_MEM_HANDLE_TYPE_FABRIC : CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
}
}  // namespace

extern "C" {

int iris_rt_driver_version(int* version) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  return rc(d.cuDriverGetVersion(version));
}

int iris_rt_error_string(int code, char* out, int len) {
  std::string s = cu_error((CUresult)code);
  if (out && len > 0) {
    strncpy(out, s.c_str(), (size_t)len - 1);
    out[len - 1] = 0;
  }
  return 0;
}

// ---- plain device allocations
int iris_rt_malloc(int device, uint64_t size, uint64_t* ptr) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  CUresult r = ensure_context(device);
  if (r != CUDA_SUCCESS) return rc(r);
  CUdeviceptr p = 0;
  r = d.cuMemAlloc_v2(&p, size);
  *ptr = (uint64_t)p;
  return rc(r);
}

int iris_rt_free(uint64_t ptr) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  return rc(d.cuMemFree_v2((CUdeviceptr)ptr));
}

// ---- virtual memory management
int iris_rt_mem_granularity(int device, int fabric, int recommended, uint64_t* gran) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  CUmemAllocationProp prop;
  fill_prop(prop, device, fabric);
  size_t g = 0;
  CUresult r = d.cuMemGetAllocationGranularity(&g, &prop, recommended ? CU_MEM_ALLOC_GRANULARITY_RECOMMENDED : CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  *gran = g;
  return rc(r);
}

int iris_rt_mem_create(uint64_t size, int device, int fabric, uint64_t* handle) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  CUresult r = ensure_context(device);
  if (r != CUDA_SUCCESS) return rc(r);
  CUmemAllocationProp prop;
  fill_prop(prop, device, fabric);
  CUmemGenericAllocationHandle h = 0;
  r = d.cuMemCreate(&h, size, &prop, 0);
  *handle = (uint64_t)h;
  return rc(r);
}

int iris_rt_mem_release(uint64_t handle) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  return rc(d.cuMemRelease((CUmemGenericAllocationHandle)handle));
}

int iris_rt_mem_address_reserve(uint64_t size, uint64_t alignment, uint64_t hint, uint64_t* ptr) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  CUdeviceptr p = 0;
  CUresult r = d.cuMemAddressReserve(&p, size, alignment, (CUdeviceptr)hint, 0);
  *ptr = (uint64_t)p;
  return rc(r);
}

int iris_rt_mem_address_free(uint64_t ptr, uint64_t size) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  return rc(d.cuMemAddressFree((CUdeviceptr)ptr, size));
}

int iris_rt_mem_map(uint64_t ptr, uint64_t size, uint64_t offset, uint64_t handle) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  return rc(d.cuMemMap((CUdeviceptr)ptr, size, offset, (CUmemGenericAllocationHandle)handle, 0));
}

int iris_rt_mem_unmap(uint64_t ptr, uint64_t size) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  return rc(d.cuMemUnmap((CUdeviceptr)ptr, size));
}

// Read-write access for `count` devices listed in `devices`.
int iris_rt_mem_set_access(uint64_t ptr, uint64_t size, const int* devices, int count) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  if (count < 1 || count > 64) return -(int)CUDA_ERROR_INVALID_VALUE;
  CUmemAccessDesc acc[64];
  memset(acc, 0, sizeof(acc));
  for (int i = 0; i < count; ++i) {
    acc[i].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc[i].location.id = devices[i];
    acc[i].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  }
  return rc(d.cuMemSetAccess((CUdeviceptr)ptr, size, acc, (size_t)count));
}

// POSIX file descriptor of an allocation handle (the counterpart of a DMA-BUF export), and back.
int iris_rt_mem_export_fd(uint64_t handle, int* fd) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  int out = -1;
  CUresult r = d.cuMemExportToShareableHandle(&out, (CUmemGenericAllocationHandle)handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  *fd = out;
  return rc(r);
}

int iris_rt_mem_import_fd(int fd, uint64_t* handle) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  CUmemGenericAllocationHandle h = 0;
  CUresult r = d.cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  *handle = (uint64_t)h;
  return rc(r);
}

// The allocation handle that backs a mapped address (retained: release it when done).
int iris_rt_mem_retain_handle(uint64_t ptr, uint64_t* handle) {
  const DriverApi& d = driver();
  if (!d.ok) return kNoDriver;
  CUmemGenericAllocationHandle h = 0;
  CUresult r = d.cuMemRetainAllocationHandle(&h, (void*)(uintptr_t)ptr);
  *handle = (uint64_t)h;
  return rc(r);
}

}  // extern "C"
