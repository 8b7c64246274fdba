// Symmetric heap: one region per rank, allocated once, exported once and mapped once into every
// peer of the NVLink domain; allocation is a bump pointer, so offsets are symmetric by
// construction and no per-allocation collective is needed (the reference re-runs its peer
// exchange after every allocation, iris/host/memory/symmetric_heap.py:95-130,174-322).
//
// Backends:
//   kVmm   cuMemCreate + cuMemMap, shared as a POSIX file descriptor (SCM_RIGHTS, fd_mesh.cpp) or a
//          fabric handle; can also be bound to an NVLS multicast object (cuMulticast*), which gives
//          the heap a second "multicast" mapping used by multimem instructions.
//   kIpc   cuMemAlloc + cuIpcGetMemHandle / cuIpcOpenMemHandle (fallback, no NVLS).
//   kCpu   memfd + mmap(MAP_SHARED): peers are other processes on the host; used for tests and for
//          fault injection without a GPU.
// Reference counterparts: allocators/torch_allocator.py:25-245, allocators/vmem_allocator.py:37-344,
// iris/drivers/fabric/nvidia.py:265-454.
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <unistd.h>

#include <mutex>
#include <string>
#include <vector>

#include "cuda_driver.hpp"

#ifndef MFD_CLOEXEC
#define MFD_CLOEXEC 0x0001U
#endif
extern "C" int memfd_create(const char*, unsigned int);

namespace iris_rt {

enum HeapKind { kVmm = 0, kIpc = 1, kCpu = 2 };

struct Heap {
  int kind = kCpu;
  int device = 0, rank = 0, world = 1;
  uint64_t size = 0;          // usable bytes
  uint64_t mapped_size = 0;   // rounded to the mapping granularity
  uint64_t base = 0;          // own mapping
  uint64_t offset = 0;        // bump pointer
  std::vector<uint64_t> peer_base;
  std::vector<int> peer_kind;  // how a peer mapping must be undone: 0 none, 1 vmm, 2 ipc, 3 mmap
  std::vector<CUmemGenericAllocationHandle> peer_handle;
  CUmemGenericAllocationHandle handle = 0;
  bool fabric = false;
  int cpu_fd = -1;
  // multicast
  CUmemGenericAllocationHandle mc_handle = 0;
  uint64_t mc_base = 0;
  uint64_t mc_size = 0;
  bool mc_bound = false;
  // Growable VMM heaps (the reference's VMemAllocator, allocators/vmem_allocator.py:55-212): `reserve` bytes of
  // address space are reserved for the own mapping and for every peer's window; the first segment is the
  // heap created up front, later segments (on-demand growth, or an external allocation mapped in without a
  // copy) are mapped behind it at the same offset on every rank.
  struct Segment {
    uint64_t offset = 0, size = 0;
    CUmemGenericAllocationHandle handle = 0;
    bool external = false;     // a retained handle of somebody else's allocation: released, never freed twice
  };
  uint64_t reserve = 0;        // 0: not growable (address space = mapped_size)
  uint64_t first_size = 0;     // mapped size of the segment created with the heap
  std::vector<Segment> segs;                               // own segments after the first
  std::vector<std::vector<Segment>> peer_segs;             // per peer: its later segments mapped here
  std::mutex mu;
  std::string error;
};

static void set_err(char* err, int errlen, const std::string& s) {
  if (err && errlen > 0) {
    snprintf(err, errlen, "%s", s.c_str());
  }
}

static uint64_t round_up(uint64_t x, uint64_t g) { return (x + g - 1) / g * g; }

static bool vmm_prop(int device, bool fabric, CUmemAllocationProp& prop, uint64_t& gran, std::string& e) {
  const DriverApi& d = driver();
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = fabric ? CU_MEM_HANDLE_TYPE_FABRIC : CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t g = 0;
  CUresult r = d.cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) { e = "cuMemGetAllocationGranularity: " + cu_error(r); return false; }
  gran = g;
  return true;
}

// Reserve `reserve` (>= size) bytes of address space and map `h` at its start.
static bool vmm_map(int device, CUmemGenericAllocationHandle h, uint64_t size, uint64_t& va, std::string& e, uint64_t reserve = 0) {
  const DriverApi& d = driver();
  CUdeviceptr p = 0;
  if (reserve < size) reserve = size;
  CUresult r = d.cuMemAddressReserve(&p, reserve, 0, 0, 0);
  if (r != CUDA_SUCCESS) { e = "cuMemAddressReserve: " + cu_error(r); return false; }
  r = d.cuMemMap(p, size, 0, h, 0);
  if (r != CUDA_SUCCESS) { d.cuMemAddressFree(p, reserve); e = "cuMemMap: " + cu_error(r); return false; }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.cuMemSetAccess(p, size, &acc, 1);
  if (r != CUDA_SUCCESS) {
    d.cuMemUnmap(p, size);
    d.cuMemAddressFree(p, reserve);
    e = "cuMemSetAccess: " + cu_error(r);
    return false;
  }
  va = (uint64_t)p;
  return true;
}
// Map `h` at a fixed address inside an existing reservation.
static bool vmm_map_at(int device, CUmemGenericAllocationHandle h, uint64_t va, uint64_t size, std::string& e) {
  const DriverApi& d = driver();
  CUresult r = d.cuMemMap((CUdeviceptr)va, size, 0, h, 0);
  if (r != CUDA_SUCCESS) { e = "cuMemMap: " + cu_error(r); return false; }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.cuMemSetAccess((CUdeviceptr)va, size, &acc, 1);
  if (r != CUDA_SUCCESS) { d.cuMemUnmap((CUdeviceptr)va, size); e = "cuMemSetAccess: " + cu_error(r); return false; }
  return true;
}

}  // namespace iris_rt

using namespace iris_rt;

extern "C" {

// ---------------------------------------------------------------------------------- driver info
int iris_rt_cuda_ok(char* err, int errlen) {
  const DriverApi& d = driver();
  if (!d.ok) set_err(err, errlen, d.error);
  return d.ok ? 1 : 0;
}
int iris_rt_device_count() {
  const DriverApi& d = driver();
  if (!d.ok) return 0;
  int n = 0;
  return d.cuDeviceGetCount(&n) == CUDA_SUCCESS ? n : 0;
}
int iris_rt_device_attribute(int device, int attr) {
  const DriverApi& d = driver();
  if (!d.ok) return -1;
  int v = -1;
  CUdevice dev;
  if (d.cuDeviceGet(&dev, device) != CUDA_SUCCESS) return -1;
  if (d.cuDeviceGetAttribute(&v, (CUdevice_attribute)attr, dev) != CUDA_SUCCESS) return -1;
  return v;
}
int iris_rt_device_name(int device, char* out, int len) {
  const DriverApi& d = driver();
  if (!d.ok) return -1;
  CUdevice dev;
  if (d.cuDeviceGet(&dev, device) != CUDA_SUCCESS) return -1;
  return d.cuDeviceGetName(out, len, dev) == CUDA_SUCCESS ? 0 : -1;
}
int iris_rt_set_device(int device) { return ensure_context(device) == CUDA_SUCCESS ? 0 : -1; }
int iris_rt_current_device() {
  const DriverApi& d = driver();
  if (!d.ok) return -1;
  CUdevice dev;
  return d.cuCtxGetDevice(&dev) == CUDA_SUCCESS ? (int)dev : -1;
}
int iris_rt_can_access_peer(int dev, int peer) {
  const DriverApi& d = driver();
  if (!d.ok) return 0;
  int v = 0;
  CUdevice a, b;
  if (d.cuDeviceGet(&a, dev) != CUDA_SUCCESS || d.cuDeviceGet(&b, peer) != CUDA_SUCCESS) return 0;
  return d.cuDeviceCanAccessPeer(&v, a, b) == CUDA_SUCCESS ? v : 0;
}
int iris_rt_p2p_attribute(int attr, int dev, int peer) {
  const DriverApi& d = driver();
  if (!d.ok) return -1;
  int v = 0;
  CUdevice a, b;
  if (d.cuDeviceGet(&a, dev) != CUDA_SUCCESS || d.cuDeviceGet(&b, peer) != CUDA_SUCCESS) return -1;
  return d.cuDeviceGetP2PAttribute(&v, (CUdevice_P2PAttribute)attr, a, b) == CUDA_SUCCESS ? v : -1;
}
// Base and size of the allocation that contains `ptr` (reference hip.py get_address_range).
int iris_rt_address_range(uint64_t ptr, uint64_t* base, uint64_t* size) {
  const DriverApi& d = driver();
  if (!d.ok) return -1;
  CUdeviceptr b = 0;
  size_t s = 0;
  if (d.cuMemGetAddressRange_v2(&b, &s, (CUdeviceptr)ptr) != CUDA_SUCCESS) return -1;
  *base = (uint64_t)b;
  *size = (uint64_t)s;
  return 0;
}
int iris_rt_ipc_get_handle(uint64_t ptr, uint8_t* out64) {
  const DriverApi& d = driver();
  if (!d.ok) return -1;
  CUipcMemHandle h;
  if (d.cuIpcGetMemHandle(&h, (CUdeviceptr)ptr) != CUDA_SUCCESS) return -1;
  memcpy(out64, &h, 64);
  return 0;
}
int iris_rt_ipc_open_handle(const uint8_t* in64, uint64_t* ptr) {
  const DriverApi& d = driver();
  if (!d.ok) return -1;
  CUipcMemHandle h;
  memcpy(&h, in64, 64);
  CUdeviceptr p = 0;
  CUresult r = d.cuIpcOpenMemHandle_v2(&p, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS);
  if (r != CUDA_SUCCESS) return -(int)r;
  *ptr = (uint64_t)p;
  return 0;
}
int iris_rt_ipc_close_handle(uint64_t ptr) {
  const DriverApi& d = driver();
  if (!d.ok) return -1;
  return d.cuIpcCloseMemHandle((CUdeviceptr)ptr) == CUDA_SUCCESS ? 0 : -1;
}

// ---------------------------------------------------------------------------------- heap
static uint64_t g_next_reserve = 0;
// The next VMM heap created by this process reserves `bytes` of address space per mapping, so that it
// can grow (iris_heap_grow) or take in external allocations (iris_heap_import_external) up to that size.
void iris_heap_set_next_reserve(uint64_t bytes) { g_next_reserve = bytes; }

void* iris_heap_create(uint64_t size, int device, int rank, int world, int kind, int fabric, char* err, int errlen) {
  Heap* h = new Heap();
  h->peer_segs.assign(world, {});
  if (kind == kVmm && g_next_reserve > size) h->reserve = g_next_reserve;
  g_next_reserve = 0;
  h->kind = kind;
  h->device = device;
  h->rank = rank;
  h->world = world;
  h->size = size;
  h->fabric = fabric != 0;
  h->peer_base.assign(world, 0);
  h->peer_kind.assign(world, 0);
  h->peer_handle.assign(world, 0);
  std::string e;
  if (kind == kCpu) {
    long page = sysconf(_SC_PAGESIZE);
    h->mapped_size = round_up(size, (uint64_t)page);
    int fd = memfd_create("iris_b200_heap", MFD_CLOEXEC);
    if (fd < 0 || ftruncate(fd, (off_t)h->mapped_size) != 0) {
      set_err(err, errlen, std::string("memfd_create/ftruncate: ") + strerror(errno));
      if (fd >= 0) close(fd);
      delete h;
      return nullptr;
    }
    void* p = mmap(nullptr, h->mapped_size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    if (p == MAP_FAILED) {
      set_err(err, errlen, std::string("mmap: ") + strerror(errno));
      close(fd);
      delete h;
      return nullptr;
    }
    h->cpu_fd = fd;
    h->base = (uint64_t)p;
  } else {
    const DriverApi& d = driver();
    if (!d.ok) { set_err(err, errlen, d.error); delete h; return nullptr; }
    CUresult r = ensure_context(device);
    if (r != CUDA_SUCCESS) { set_err(err, errlen, "no CUDA context: " + cu_error(r)); delete h; return nullptr; }
    if (kind == kVmm) {
      CUmemAllocationProp prop;
      uint64_t gran = 0;
      if (!vmm_prop(device, h->fabric, prop, gran, e)) { set_err(err, errlen, e); delete h; return nullptr; }
      h->mapped_size = round_up(size, gran);
      // a heap that may later be bound to an NVLS multicast object must also be a multiple of
      // the multicast granularity (hundreds of MB where the driver recommends so); a growable heap is never
      // bound to one and keeps its small first segment
      if (world > 1 && !h->fabric && !h->reserve) {
        CUmulticastObjectProp mp;
        memset(&mp, 0, sizeof(mp));
        mp.numDevices = world;
        mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        mp.size = h->mapped_size;
        size_t mg = 0;
        if (d.cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > 0)
          h->mapped_size = round_up(h->mapped_size, mg);
      }
      r = d.cuMemCreate(&h->handle, h->mapped_size, &prop, 0);
      if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMemCreate: " + cu_error(r)); delete h; return nullptr; }
      if (h->reserve) h->reserve = round_up(h->reserve, gran) < h->mapped_size ? h->mapped_size : round_up(h->reserve, gran);
      h->first_size = h->mapped_size;
      if (h->reserve) h->size = h->mapped_size;        // a growable heap allocates from everything that is mapped
      if (!vmm_map(device, h->handle, h->mapped_size, h->base, e, h->reserve)) {
        d.cuMemRelease(h->handle);
        set_err(err, errlen, e);
        delete h;
        return nullptr;
      }
    } else {
      CUdeviceptr p = 0;
      h->mapped_size = round_up(size, 2ull << 20);
      r = d.cuMemAlloc_v2(&p, h->mapped_size);
      if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMemAlloc: " + cu_error(r)); delete h; return nullptr; }
      h->base = (uint64_t)p;
    }
    d.cuMemsetD8_v2((CUdeviceptr)h->base, 0, h->mapped_size);
    d.cuCtxSynchronize();
  }
  h->peer_base[rank] = h->base;
  return h;
}

uint64_t iris_heap_base(void* hp) { return ((Heap*)hp)->base; }
uint64_t iris_heap_size(void* hp) { return ((Heap*)hp)->size; }
uint64_t iris_heap_mapped_size(void* hp) { return ((Heap*)hp)->mapped_size; }
uint64_t iris_heap_offset(void* hp) { return ((Heap*)hp)->offset; }
void iris_heap_set_offset(void* hp, uint64_t off) { ((Heap*)hp)->offset = off; }
uint64_t iris_heap_peer_base(void* hp, int r) { return ((Heap*)hp)->peer_base[r]; }
uint64_t iris_heap_mc_base(void* hp) { return ((Heap*)hp)->mc_base; }
int iris_heap_kind(void* hp) { return ((Heap*)hp)->kind; }

// Bump allocation. Returns the byte offset, or -1 when the heap is exhausted.
int64_t iris_heap_alloc(void* hp, uint64_t bytes, uint64_t align) {
  Heap* h = (Heap*)hp;
  std::lock_guard<std::mutex> g(h->mu);
  if (align == 0) align = 1;
  uint64_t start = round_up(h->offset, align);
  uint64_t need = bytes == 0 ? align : bytes;
  if (start + need > h->size) return -1;
  h->offset = start + need;
  return (int64_t)start;
}

// Export: returns an fd (vmm posix / cpu), or fills a 64-byte blob (ipc / fabric).
int iris_heap_export_fd(void* hp, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  if (h->kind == kCpu) return dup(h->cpu_fd);
  if (h->kind != kVmm || h->fabric) { set_err(err, errlen, "heap has no fd export"); return -1; }
  int fd = -1;
  CUresult r = driver().cuMemExportToShareableHandle(&fd, h->handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMemExportToShareableHandle: " + cu_error(r)); return -1; }
  return fd;
}
int iris_heap_export_blob(void* hp, uint8_t* out64, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  const DriverApi& d = driver();
  if (h->kind == kIpc) {
    CUipcMemHandle ih;
    CUresult r = d.cuIpcGetMemHandle(&ih, (CUdeviceptr)h->base);
    if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuIpcGetMemHandle: " + cu_error(r)); return -1; }
    memcpy(out64, &ih, 64);
    return 0;
  }
  if (h->kind == kVmm && h->fabric) {
    CUmemFabricHandle fh;
    CUresult r = d.cuMemExportToShareableHandle(&fh, h->handle, CU_MEM_HANDLE_TYPE_FABRIC, 0);
    if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMemExportToShareableHandle(fabric): " + cu_error(r)); return -1; }
    memcpy(out64, &fh, 64);
    return 0;
  }
  set_err(err, errlen, "heap has no blob export");
  return -1;
}
int iris_heap_import_fd(void* hp, int peer, int fd, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  std::string e;
  if (h->kind == kCpu) {
    void* p = mmap(nullptr, h->mapped_size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    if (p == MAP_FAILED) { set_err(err, errlen, std::string("mmap(peer): ") + strerror(errno)); return -1; }
    h->peer_base[peer] = (uint64_t)p;
    h->peer_kind[peer] = 3;
    return 0;
  }
  const DriverApi& d = driver();
  ensure_context(h->device);
  CUmemGenericAllocationHandle ph = 0;
  CUresult r = d.cuMemImportFromShareableHandle(&ph, (void*)(intptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMemImportFromShareableHandle: " + cu_error(r)); return -1; }
  uint64_t va = 0;
  const uint64_t first = h->first_size ? h->first_size : h->mapped_size;
  if (!vmm_map(h->device, ph, first, va, e, h->reserve)) { d.cuMemRelease(ph); set_err(err, errlen, e); return -1; }
  h->peer_base[peer] = va;
  h->peer_kind[peer] = 1;
  h->peer_handle[peer] = ph;
  return 0;
}

// ---------------------------------------------------------------------------------- growth and external memory
// All of these are collective by convention (every rank grows by the same amount at the same point of its
// allocation sequence, as with every allocation on a symmetric heap); the exchange of the new segment's
// descriptor is driven from Python over the fd mesh.
static int add_own_segment(Heap* h, CUmemGenericAllocationHandle handle, uint64_t size, bool external, std::string& e) {
  if (h->mapped_size + size > h->reserve) { e = "the heap's reserved address space is exhausted"; return -1; }
  if (!vmm_map_at(h->device, handle, h->base + h->mapped_size, size, e)) return -1;
  Heap::Segment sgm;
  sgm.offset = h->mapped_size; sgm.size = size; sgm.handle = handle; sgm.external = external;
  h->segs.push_back(sgm);
  h->mapped_size += size;
  h->size = h->mapped_size;
  return (int)h->segs.size() - 1;
}
// Map `bytes` more (rounded up to the allocation granularity) behind the heap. Returns the segment index or -1.
int iris_heap_grow(void* hp, uint64_t bytes, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  std::lock_guard<std::mutex> g(h->mu);
  std::string e;
  if (h->kind != kVmm || !h->reserve) { set_err(err, errlen, "this heap was not created growable"); return -1; }
  const DriverApi& d = driver();
  ensure_context(h->device);
  CUmemAllocationProp prop;
  uint64_t gran = 0;
  if (!vmm_prop(h->device, h->fabric, prop, gran, e)) { set_err(err, errlen, e); return -1; }
  const uint64_t size = round_up(bytes, gran);
  CUmemGenericAllocationHandle handle = 0;
  CUresult r = d.cuMemCreate(&handle, size, &prop, 0);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMemCreate: " + cu_error(r)); return -1; }
  const int idx = add_own_segment(h, handle, size, false, e);
  if (idx < 0) { d.cuMemRelease(handle); set_err(err, errlen, e); return -1; }
  d.cuMemsetD8_v2((CUdeviceptr)(h->base + h->segs[idx].offset), 0, size);
  d.cuCtxSynchronize();
  return idx;
}
// Map the allocation that contains `ptr` (memory created with cuMemCreate by someone else, e.g. a framework's
// expandable segments) behind the heap WITHOUT copying it: the same physical memory then has a second address
// inside the heap, at which peers can reach it. *inner = offset of `ptr` inside the new segment.
int iris_heap_import_external(void* hp, uint64_t ptr, uint64_t* inner, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  std::lock_guard<std::mutex> g(h->mu);
  std::string e;
  if (h->kind != kVmm || !h->reserve) { set_err(err, errlen, "this heap was not created growable"); return -1; }
  const DriverApi& d = driver();
  ensure_context(h->device);
  CUmemGenericAllocationHandle handle = 0;
  CUresult r = d.cuMemRetainAllocationHandle(&handle, (void*)(uintptr_t)ptr);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMemRetainAllocationHandle (memory not created with cuMemCreate?): " + cu_error(r)); return -1; }
  CUdeviceptr abase = 0;
  size_t asize = 0;
  r = d.cuMemGetAddressRange_v2(&abase, &asize, (CUdeviceptr)ptr);
  if (r != CUDA_SUCCESS) { d.cuMemRelease(handle); set_err(err, errlen, "cuMemGetAddressRange: " + cu_error(r)); return -1; }
  const int idx = add_own_segment(h, handle, (uint64_t)asize, true, e);
  if (idx < 0) { d.cuMemRelease(handle); set_err(err, errlen, e); return -1; }
  if (inner) *inner = ptr - (uint64_t)abase;
  return idx;
}
int iris_heap_num_segments(void* hp) { return (int)((Heap*)hp)->segs.size(); }
uint64_t iris_heap_segment_offset(void* hp, int seg) { return ((Heap*)hp)->segs[seg].offset; }
uint64_t iris_heap_segment_size(void* hp, int seg) { return ((Heap*)hp)->segs[seg].size; }
uint64_t iris_heap_reserved(void* hp) { return ((Heap*)hp)->reserve; }
int iris_heap_segment_export_fd(void* hp, int seg, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  int fd = -1;
  CUresult r = driver().cuMemExportToShareableHandle(&fd, h->segs[seg].handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMemExportToShareableHandle(segment): " + cu_error(r)); return -1; }
  return fd;
}
// Map a peer's segment (received as a file descriptor) at the same offset of that peer's window.
int iris_heap_segment_import_fd(void* hp, int peer, int fd, uint64_t offset, uint64_t size, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  std::string e;
  if (h->kind != kVmm || !h->reserve || h->peer_kind[peer] != 1) { set_err(err, errlen, "no growable window for this peer"); return -1; }
  if (offset + size > h->reserve) { set_err(err, errlen, "segment beyond the reserved window"); return -1; }
  const DriverApi& d = driver();
  ensure_context(h->device);
  CUmemGenericAllocationHandle ph = 0;
  CUresult r = d.cuMemImportFromShareableHandle(&ph, (void*)(intptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMemImportFromShareableHandle(segment): " + cu_error(r)); return -1; }
  if (!vmm_map_at(h->device, ph, h->peer_base[peer] + offset, size, e)) { d.cuMemRelease(ph); set_err(err, errlen, e); return -1; }
  Heap::Segment sgm;
  sgm.offset = offset; sgm.size = size; sgm.handle = ph;
  h->peer_segs[peer].push_back(sgm);
  return 0;
}
int iris_heap_import_blob(void* hp, int peer, const uint8_t* in64, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  const DriverApi& d = driver();
  ensure_context(h->device);
  std::string e;
  if (h->kind == kIpc) {
    CUipcMemHandle ih;
    memcpy(&ih, in64, 64);
    CUdeviceptr p = 0;
    CUresult r = d.cuIpcOpenMemHandle_v2(&p, ih, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS);
    if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuIpcOpenMemHandle: " + cu_error(r)); return -1; }
    h->peer_base[peer] = (uint64_t)p;
    h->peer_kind[peer] = 2;
    return 0;
  }
  if (h->kind == kVmm && h->fabric) {
    CUmemFabricHandle fh;
    memcpy(&fh, in64, 64);
    CUmemGenericAllocationHandle ph = 0;
    CUresult r = d.cuMemImportFromShareableHandle(&ph, &fh, CU_MEM_HANDLE_TYPE_FABRIC);
    if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMemImportFromShareableHandle(fabric): " + cu_error(r)); return -1; }
    uint64_t va = 0;
    if (!vmm_map(h->device, ph, h->mapped_size, va, e)) { d.cuMemRelease(ph); set_err(err, errlen, e); return -1; }
    h->peer_base[peer] = va;
    h->peer_kind[peer] = 1;
    h->peer_handle[peer] = ph;
    return 0;
  }
  set_err(err, errlen, "heap has no blob import");
  return -1;
}

// ---------------------------------------------------------------------------------- multicast (NVLS)
// Protocol (driven from Python): rank 0 calls mc_create -> fd, sends it to every peer; every rank
// calls mc_attach(fd) [imports when not the creator, then cuMulticastAddDevice]; host barrier;
// every rank calls mc_bind [cuMulticastBindMem + map]; host barrier.
int iris_heap_mc_supported(int device) {
  const DriverApi& d = driver();
  if (!d.ok) return 0;
  int v = 0;
  CUdevice dev;
  if (d.cuDeviceGet(&dev, device) != CUDA_SUCCESS) return 0;
  if (d.cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
  return v;
}
int iris_heap_mc_create(void* hp, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  const DriverApi& d = driver();
  if (h->kind != kVmm) { set_err(err, errlen, "multicast needs the VMM heap"); return -1; }
  CUmulticastObjectProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.numDevices = h->world;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  prop.size = h->mapped_size;
  CUresult r = d.cuMulticastGetGranularity(&gran, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMulticastGetGranularity: " + cu_error(r)); return -1; }
  if (h->mapped_size % gran) { set_err(err, errlen, "heap size is not a multiple of the multicast granularity"); return -1; }
  h->mc_size = h->mapped_size;
  r = d.cuMulticastCreate(&h->mc_handle, &prop);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMulticastCreate: " + cu_error(r)); return -1; }
  int fd = -1;
  r = d.cuMemExportToShareableHandle(&fd, h->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "export multicast handle: " + cu_error(r)); return -1; }
  return fd;
}
uint64_t iris_heap_mc_granularity(void* hp) {
  Heap* h = (Heap*)hp;
  const DriverApi& d = driver();
  if (!d.ok) return 0;
  CUmulticastObjectProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.numDevices = h->world;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  prop.size = h->mapped_size;
  size_t gran = 0;
  if (d.cuMulticastGetGranularity(&gran, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return 0;
  return gran;
}
int iris_heap_mc_attach(void* hp, int fd, int is_creator, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  const DriverApi& d = driver();
  ensure_context(h->device);
  CUresult r;
  if (!is_creator) {
    r = d.cuMemImportFromShareableHandle(&h->mc_handle, (void*)(intptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    if (r != CUDA_SUCCESS) { set_err(err, errlen, "import multicast handle: " + cu_error(r)); return -1; }
    h->mc_size = h->mapped_size;
  }
  CUdevice dev;
  d.cuDeviceGet(&dev, h->device);
  r = d.cuMulticastAddDevice(h->mc_handle, dev);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMulticastAddDevice: " + cu_error(r)); return -1; }
  return 0;
}
int iris_heap_mc_bind(void* hp, char* err, int errlen) {
  Heap* h = (Heap*)hp;
  const DriverApi& d = driver();
  ensure_context(h->device);
  CUresult r = d.cuMulticastBindMem(h->mc_handle, 0, h->handle, 0, h->mc_size, 0);
  if (r != CUDA_SUCCESS) { set_err(err, errlen, "cuMulticastBindMem: " + cu_error(r)); return -1; }
  h->mc_bound = true;
  std::string e;
  uint64_t va = 0;
  if (!vmm_map(h->device, h->mc_handle, h->mc_size, va, e)) { set_err(err, errlen, "map multicast: " + e); return -1; }
  h->mc_base = va;
  return 0;
}

// Undo every mapping. All steps are attempted even when one fails (same policy as the
// reference's fabric cleanup, iris/drivers/fabric/nvidia.py:115-124); returns the failure count.
int iris_heap_destroy(void* hp) {
  Heap* h = (Heap*)hp;
  int failures = 0;
  if (h->kind == kCpu) {
    for (int r = 0; r < h->world; ++r)
      if (r != h->rank && h->peer_kind[r] == 3 && munmap((void*)h->peer_base[r], h->mapped_size) != 0) ++failures;
    if (h->base && munmap((void*)h->base, h->mapped_size) != 0) ++failures;
    if (h->cpu_fd >= 0) close(h->cpu_fd);
    delete h;
    return failures;
  }
  const DriverApi& d = driver();
  if (!d.ok) { delete h; return 1; }
  ensure_context(h->device);
  d.cuCtxSynchronize();
  if (h->mc_base) {
    if (d.cuMemUnmap((CUdeviceptr)h->mc_base, h->mc_size) != CUDA_SUCCESS) ++failures;
    if (d.cuMemAddressFree((CUdeviceptr)h->mc_base, h->mc_size) != CUDA_SUCCESS) ++failures;
  }
  if (h->mc_bound) {
    CUdevice dev;
    d.cuDeviceGet(&dev, h->device);
    if (d.cuMulticastUnbind(h->mc_handle, dev, 0, h->mc_size) != CUDA_SUCCESS) ++failures;
  }
  if (h->mc_handle && d.cuMemRelease(h->mc_handle) != CUDA_SUCCESS) ++failures;
  const uint64_t first = h->first_size ? h->first_size : h->mapped_size;      // size of the segment created with the heap
  const uint64_t window = h->reserve ? h->reserve : first;                    // address space per mapping
  for (int r = 0; r < h->world; ++r) {
    if (r == h->rank) continue;
    if (h->peer_kind[r] == 1) {
      for (auto& sg : h->peer_segs[r]) {
        if (d.cuMemUnmap((CUdeviceptr)(h->peer_base[r] + sg.offset), sg.size) != CUDA_SUCCESS) ++failures;
        if (d.cuMemRelease(sg.handle) != CUDA_SUCCESS) ++failures;
      }
      if (d.cuMemUnmap((CUdeviceptr)h->peer_base[r], first) != CUDA_SUCCESS) ++failures;
      if (d.cuMemAddressFree((CUdeviceptr)h->peer_base[r], window) != CUDA_SUCCESS) ++failures;
      if (d.cuMemRelease(h->peer_handle[r]) != CUDA_SUCCESS) ++failures;
    } else if (h->peer_kind[r] == 2) {
      if (d.cuIpcCloseMemHandle((CUdeviceptr)h->peer_base[r]) != CUDA_SUCCESS) ++failures;
    }
  }
  if (h->kind == kVmm) {
    for (auto& sg : h->segs) {
      if (d.cuMemUnmap((CUdeviceptr)(h->base + sg.offset), sg.size) != CUDA_SUCCESS) ++failures;
      if (d.cuMemRelease(sg.handle) != CUDA_SUCCESS) ++failures;
    }
    if (d.cuMemUnmap((CUdeviceptr)h->base, first) != CUDA_SUCCESS) ++failures;
    if (d.cuMemAddressFree((CUdeviceptr)h->base, window) != CUDA_SUCCESS) ++failures;
    if (d.cuMemRelease(h->handle) != CUDA_SUCCESS) ++failures;
  } else {
    if (d.cuMemFree_v2((CUdeviceptr)h->base) != CUDA_SUCCESS) ++failures;
  }
  delete h;
  return failures;
}

}  // extern "C"
