// A stand-in for the CUDA driver's memory API on host memory, for tests on machines without a GPU.
// Allocation handles are memfd files, address reservations are PROT_NONE mappings, cuMemMap maps the
// file over the reserved range, exported handles are duplicated descriptors: enough for the virtual
// memory primitives (reserve / create / map / set access / export / import / unmap / release) to
// behave as on a device, including two mappings of one allocation showing the same bytes.
// `iris_rt_install_fake_driver(n)` switches the runtime to it with `n` devices, `(0)` switches back.
// Nothing here touches a GPU. (The reference tests its driver layer against a Python fake,
// tests/unittests/test_drivers.py:1-198.)
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <unistd.h>

#include <map>
#include <mutex>

#include "cuda_driver.hpp"

#ifndef MFD_CLOEXEC
#define MFD_CLOEXEC 0x0001U
#endif
extern "C" int memfd_create(const char* name, unsigned int flags);

using namespace iris_rt;

namespace {

constexpr size_t kGranularity = 2u << 20;

struct Alloc { int fd; size_t size; };
struct Range { size_t size; };
struct Mapping { size_t size; uint64_t handle; };

std::mutex g_mu;
int g_devices = 0;
int g_current = -1;
uint64_t g_next = 1;
std::map<uint64_t, Alloc> g_allocs;       // handle -> backing file
std::map<uint64_t, Range> g_ranges;       // reserved base -> size
std::map<uint64_t, Mapping> g_maps;       // mapped address -> mapping
std::map<uint64_t, size_t> g_plain;       // cuMemAlloc'd blocks
int g_fail_after = 0;                     // > 0: the g_fail_after-th memory call from now fails (fault injection on the host)

// True when this call is the one that was asked to fail.
bool injected_failure() {
  std::lock_guard<std::mutex> l(g_mu);
  if (g_fail_after <= 0) return false;
  return --g_fail_after == 0;
}

CUresult f_init(unsigned) { return CUDA_SUCCESS; }
CUresult f_version(int* v) { *v = 12090; return CUDA_SUCCESS; }
CUresult f_count(int* n) { *n = g_devices; return CUDA_SUCCESS; }
CUresult f_get(CUdevice* d, int ordinal) {
  if (ordinal < 0 || ordinal >= g_devices) return CUDA_ERROR_INVALID_DEVICE;
  *d = ordinal;
  return CUDA_SUCCESS;
}
CUresult f_attr(int* v, CUdevice_attribute a, CUdevice) {
  switch (a) {
    case CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT: *v = 148; break;
    case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR: *v = 10; break;
    case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR: *v = 0; break;
    case CU_DEVICE_ATTRIBUTE_CLOCK_RATE: *v = 1965000; break;
    default: *v = 0;
  }
  return CUDA_SUCCESS;
}
CUresult f_name(char* out, int len, CUdevice) {
  strncpy(out, "fake device (host memory)", (size_t)len - 1);
  out[len - 1] = 0;
  return CUDA_SUCCESS;
}
CUresult f_peer(int* can, CUdevice a, CUdevice b) { *can = (a != b); return CUDA_SUCCESS; }
CUresult f_p2p_attr(int* v, CUdevice_P2PAttribute, CUdevice, CUdevice) { *v = 1; return CUDA_SUCCESS; }
CUresult f_ctx_get(CUcontext* c) { *c = g_current >= 0 ? (CUcontext)(uintptr_t)(g_current + 1) : nullptr; return CUDA_SUCCESS; }
CUresult f_ctx_set(CUcontext c) { g_current = c ? (int)(uintptr_t)c - 1 : -1; return CUDA_SUCCESS; }
CUresult f_ctx_dev(CUdevice* d) {
  if (g_current < 0) return CUDA_ERROR_INVALID_CONTEXT;
  *d = g_current;
  return CUDA_SUCCESS;
}
CUresult f_sync() { return CUDA_SUCCESS; }
CUresult f_retain(CUcontext* c, CUdevice d) { *c = (CUcontext)(uintptr_t)(d + 1); return CUDA_SUCCESS; }
CUresult f_errstr(CUresult r, const char** s) {
  *s = r == CUDA_SUCCESS ? "no error" : r == CUDA_ERROR_INVALID_VALUE ? "invalid argument" : r == CUDA_ERROR_OUT_OF_MEMORY ? "out of memory" : "fake driver error";
  return CUDA_SUCCESS;
}

CUresult f_granularity(size_t* g, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) { *g = kGranularity; return CUDA_SUCCESS; }

CUresult f_create(CUmemGenericAllocationHandle* h, size_t size, const CUmemAllocationProp* prop, unsigned long long) {
  if (injected_failure()) return CUDA_ERROR_OUT_OF_MEMORY;
  if (size == 0 || size % kGranularity) return CUDA_ERROR_INVALID_VALUE;
  if (prop->location.id < 0 || prop->location.id >= g_devices) return CUDA_ERROR_INVALID_DEVICE;
  int fd = memfd_create("iris-fake-vmm", MFD_CLOEXEC);
  if (fd < 0) return CUDA_ERROR_OUT_OF_MEMORY;
  if (ftruncate(fd, (off_t)size) != 0) { close(fd); return CUDA_ERROR_OUT_OF_MEMORY; }
  std::lock_guard<std::mutex> l(g_mu);
  *h = g_next++;
  g_allocs[*h] = Alloc{fd, size};
  return CUDA_SUCCESS;
}
CUresult f_release(CUmemGenericAllocationHandle h) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_allocs.find(h);
  if (it == g_allocs.end()) return CUDA_ERROR_INVALID_VALUE;
  close(it->second.fd);          // existing mappings keep the pages alive, as on the device
  g_allocs.erase(it);
  return CUDA_SUCCESS;
}
CUresult f_reserve(CUdeviceptr* p, size_t size, size_t, CUdeviceptr, unsigned long long) {
  if (injected_failure()) return CUDA_ERROR_OUT_OF_MEMORY;
  if (size == 0 || size % kGranularity) return CUDA_ERROR_INVALID_VALUE;
  void* a = mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  if (a == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
  std::lock_guard<std::mutex> l(g_mu);
  g_ranges[(uint64_t)a] = Range{size};
  *p = (CUdeviceptr)a;
  return CUDA_SUCCESS;
}
CUresult f_addr_free(CUdeviceptr p, size_t size) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_ranges.find((uint64_t)p);
  if (it == g_ranges.end() || it->second.size != size) return CUDA_ERROR_INVALID_VALUE;
  for (auto& m : g_maps)
    if (m.first >= (uint64_t)p && m.first < (uint64_t)p + size) return CUDA_ERROR_INVALID_VALUE;   // still mapped
  munmap((void*)p, size);
  g_ranges.erase(it);
  return CUDA_SUCCESS;
}
bool inside_reservation(uint64_t p, size_t size) {
  for (auto& r : g_ranges)
    if (p >= r.first && p + size <= r.first + r.second.size) return true;
  return false;
}
CUresult f_map(CUdeviceptr p, size_t size, size_t offset, CUmemGenericAllocationHandle h, unsigned long long) {
  if (injected_failure()) return CUDA_ERROR_OUT_OF_MEMORY;
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_allocs.find(h);
  if (it == g_allocs.end() || offset != 0 || size != it->second.size || !inside_reservation((uint64_t)p, size)) return CUDA_ERROR_INVALID_VALUE;
  if (g_maps.count((uint64_t)p)) return CUDA_ERROR_INVALID_VALUE;
  void* a = mmap((void*)p, size, PROT_NONE, MAP_SHARED | MAP_FIXED, it->second.fd, 0);   // no access until cuMemSetAccess
  if (a == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
  g_maps[(uint64_t)p] = Mapping{size, h};
  return CUDA_SUCCESS;
}
CUresult f_unmap(CUdeviceptr p, size_t size) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_maps.find((uint64_t)p);
  if (it == g_maps.end() || it->second.size != size) return CUDA_ERROR_INVALID_VALUE;
  mmap((void*)p, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);   // back to a bare reservation
  g_maps.erase(it);
  return CUDA_SUCCESS;
}
CUresult f_access(CUdeviceptr p, size_t size, const CUmemAccessDesc* desc, size_t count) {
  if (injected_failure()) return CUDA_ERROR_OUT_OF_MEMORY;
  std::lock_guard<std::mutex> l(g_mu);
  if (count == 0) return CUDA_ERROR_INVALID_VALUE;
  for (size_t i = 0; i < count; ++i)
    if (desc[i].location.id < 0 || desc[i].location.id >= g_devices) return CUDA_ERROR_INVALID_DEVICE;
  // the range must consist of whole mappings
  uint64_t at = (uint64_t)p;
  while (at < (uint64_t)p + size) {
    auto it = g_maps.find(at);
    if (it == g_maps.end()) return CUDA_ERROR_INVALID_VALUE;
    at += it->second.size;
  }
  return mprotect((void*)p, size, PROT_READ | PROT_WRITE) == 0 ? CUDA_SUCCESS : CUDA_ERROR_INVALID_VALUE;
}
// A fabric handle of the stand-in: 64 bytes holding a tag and the allocation's number. It can only be
// imported by the process that exported it, which is all a single-process driver test needs.
constexpr char kFabricTag[8] = {'i', 'r', 'i', 's', 'f', 'a', 'b', 0};

CUresult f_export(void* out, CUmemGenericAllocationHandle h, CUmemAllocationHandleType type, unsigned long long) {
  if (injected_failure()) return CUDA_ERROR_OUT_OF_MEMORY;
  if (type == CU_MEM_HANDLE_TYPE_FABRIC) {
    std::lock_guard<std::mutex> l(g_mu);
    if (!g_allocs.count(h)) return CUDA_ERROR_INVALID_VALUE;
    memset(out, 0, 64);
    memcpy(out, kFabricTag, 8);
    memcpy((char*)out + 8, &h, sizeof(h));
    return CUDA_SUCCESS;
  }
  if (type != CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) return CUDA_ERROR_NOT_SUPPORTED;
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_allocs.find(h);
  if (it == g_allocs.end()) return CUDA_ERROR_INVALID_VALUE;
  int fd = dup(it->second.fd);
  if (fd < 0) return CUDA_ERROR_OUT_OF_MEMORY;
  *(int*)out = fd;
  return CUDA_SUCCESS;
}
CUresult f_import(CUmemGenericAllocationHandle* h, void* os_handle, CUmemAllocationHandleType type) {
  if (injected_failure()) return CUDA_ERROR_OUT_OF_MEMORY;
  if (type == CU_MEM_HANDLE_TYPE_FABRIC) {
    if (memcmp(os_handle, kFabricTag, 8) != 0) return CUDA_ERROR_INVALID_VALUE;
    CUmemGenericAllocationHandle src = 0;
    memcpy(&src, (const char*)os_handle + 8, sizeof(src));
    std::lock_guard<std::mutex> l(g_mu);
    auto it = g_allocs.find(src);
    if (it == g_allocs.end()) return CUDA_ERROR_INVALID_VALUE;
    int fd = dup(it->second.fd);
    if (fd < 0) return CUDA_ERROR_OUT_OF_MEMORY;
    *h = g_next++;
    g_allocs[*h] = Alloc{fd, it->second.size};
    return CUDA_SUCCESS;
  }
  if (type != CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) return CUDA_ERROR_NOT_SUPPORTED;
  int fd = dup((int)(uintptr_t)os_handle);
  if (fd < 0) return CUDA_ERROR_INVALID_VALUE;
  off_t size = lseek(fd, 0, SEEK_END);
  if (size <= 0) { close(fd); return CUDA_ERROR_INVALID_VALUE; }
  std::lock_guard<std::mutex> l(g_mu);
  *h = g_next++;
  g_allocs[*h] = Alloc{fd, (size_t)size};
  return CUDA_SUCCESS;
}
CUresult f_retain_handle(CUmemGenericAllocationHandle* h, void* addr) {
  std::lock_guard<std::mutex> l(g_mu);
  for (auto& m : g_maps)
    if ((uint64_t)addr >= m.first && (uint64_t)addr < m.first + m.second.size) {
      auto it = g_allocs.find(m.second.handle);
      if (it == g_allocs.end()) return CUDA_ERROR_INVALID_VALUE;
      int fd = dup(it->second.fd);
      *h = g_next++;
      g_allocs[*h] = Alloc{fd, it->second.size};
      return CUDA_SUCCESS;
    }
  return CUDA_ERROR_INVALID_VALUE;
}
CUresult f_range(CUdeviceptr* base, size_t* size, CUdeviceptr p) {
  std::lock_guard<std::mutex> l(g_mu);
  for (auto& m : g_maps)
    if ((uint64_t)p >= m.first && (uint64_t)p < m.first + m.second.size) { *base = m.first; *size = m.second.size; return CUDA_SUCCESS; }
  for (auto& b : g_plain)
    if ((uint64_t)p >= b.first && (uint64_t)p < b.first + b.second) { *base = b.first; *size = b.second; return CUDA_SUCCESS; }
  return CUDA_ERROR_INVALID_VALUE;
}
CUresult f_alloc(CUdeviceptr* p, size_t size) {
  void* a = mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (a == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
  std::lock_guard<std::mutex> l(g_mu);
  g_plain[(uint64_t)a] = size;
  *p = (CUdeviceptr)a;
  return CUDA_SUCCESS;
}
CUresult f_free(CUdeviceptr p) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_plain.find((uint64_t)p);
  if (it == g_plain.end()) return CUDA_ERROR_INVALID_VALUE;
  munmap((void*)p, it->second);
  g_plain.erase(it);
  return CUDA_SUCCESS;
}
CUresult f_memset(CUdeviceptr p, unsigned char v, size_t n) { memset((void*)p, v, n); return CUDA_SUCCESS; }
CUresult f_ipc_get(CUipcMemHandle*, CUdeviceptr) { return CUDA_ERROR_NOT_SUPPORTED; }
CUresult f_ipc_open(CUdeviceptr*, CUipcMemHandle, unsigned) { return CUDA_ERROR_NOT_SUPPORTED; }
CUresult f_ipc_close(CUdeviceptr) { return CUDA_ERROR_NOT_SUPPORTED; }
CUresult f_mc_create(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) { return CUDA_ERROR_NOT_SUPPORTED; }
CUresult f_mc_add(CUmemGenericAllocationHandle, CUdevice) { return CUDA_ERROR_NOT_SUPPORTED; }
CUresult f_mc_bind(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) { return CUDA_ERROR_NOT_SUPPORTED; }
CUresult f_mc_unbind(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) { return CUDA_ERROR_NOT_SUPPORTED; }
CUresult f_mc_gran(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) { return CUDA_ERROR_NOT_SUPPORTED; }

DriverApi g_fake_api;

}  // namespace

// Fault injection for tests: the k-th memory call from now (create, reserve, map, set access, export,
// import) returns CUDA_ERROR_OUT_OF_MEMORY; 0 disarms.
extern "C" void iris_rt_fake_fail_after(int k) {
  std::lock_guard<std::mutex> l(g_mu);
  g_fail_after = k;
}

// Allocations, address reservations and mappings currently alive in the stand-in (leak checks).
extern "C" int iris_rt_fake_live_objects() {
  std::lock_guard<std::mutex> l(g_mu);
  return (int)(g_allocs.size() + g_ranges.size() + g_maps.size() + g_plain.size());
}

extern "C" int iris_rt_install_fake_driver(int devices) {
  if (devices <= 0) {
    set_driver_for_testing(nullptr);
    return 0;
  }
  g_devices = devices;
  DriverApi& a = g_fake_api;
  a.ok = true;
  a.error.clear();
  a.cuInit = f_init;
  a.cuDriverGetVersion = f_version;
  a.cuDeviceGetCount = f_count;
  a.cuDeviceGet = f_get;
  a.cuDeviceGetAttribute = f_attr;
  a.cuDeviceGetName = f_name;
  a.cuDeviceCanAccessPeer = f_peer;
  a.cuDeviceGetP2PAttribute = f_p2p_attr;
  a.cuCtxGetCurrent = f_ctx_get;
  a.cuCtxSetCurrent = f_ctx_set;
  a.cuCtxGetDevice = f_ctx_dev;
  a.cuCtxSynchronize = f_sync;
  a.cuDevicePrimaryCtxRetain = f_retain;
  a.cuGetErrorString = f_errstr;
  a.cuMemGetAddressRange_v2 = f_range;
  a.cuMemAlloc_v2 = f_alloc;
  a.cuMemFree_v2 = f_free;
  a.cuMemsetD8_v2 = f_memset;
  a.cuIpcGetMemHandle = f_ipc_get;
  a.cuIpcOpenMemHandle_v2 = f_ipc_open;
  a.cuIpcCloseMemHandle = f_ipc_close;
  a.cuMemCreate = f_create;
  a.cuMemRelease = f_release;
  a.cuMemAddressReserve = f_reserve;
  a.cuMemAddressFree = f_addr_free;
  a.cuMemMap = f_map;
  a.cuMemUnmap = f_unmap;
  a.cuMemSetAccess = f_access;
  a.cuMemExportToShareableHandle = f_export;
  a.cuMemImportFromShareableHandle = f_import;
  a.cuMemGetAllocationGranularity = f_granularity;
  a.cuMemRetainAllocationHandle = f_retain_handle;
  a.cuMulticastCreate = f_mc_create;
  a.cuMulticastAddDevice = f_mc_add;
  a.cuMulticastBindMem = f_mc_bind;
  a.cuMulticastUnbind = f_mc_unbind;
  a.cuMulticastGetGranularity = f_mc_gran;
  set_driver_for_testing(&a);
  return devices;
}
