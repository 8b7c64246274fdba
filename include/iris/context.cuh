// Device-side view of a symmetric heap: the per-rank base addresses (as mapped in THIS process)
// and the address translation every RMA op is built on.
//
// Reference semantics (iris/mem/triton/context.py:17-27):
//     remote_ptr = heap_bases[to_rank] + (local_ptr - heap_bases[from_rank])
// Here the table travels by value as a kernel parameter (constant bank, one add per translation)
// instead of being re-read from global memory on every op.
#pragma once
#include "common.cuh"

namespace iris {

struct TraceBuffers {
  int32_t enabled;
  int32_t max_events;
  int32_t* counter;
  int32_t* op_index_counter;
  int32_t* event_id;
  int32_t* pid;
  int32_t* pid_m;
  int32_t* pid_n;
  int32_t* cur_rank;
  int32_t* target_rank;
  int32_t* xcc_id;
  int32_t* cu_id;
  int64_t* timestamp;
  int64_t* address;
  int64_t* duration_cycles;
  int32_t* op_index;
  int32_t* payload_size;
};

struct DeviceContext {
  int32_t rank;          // this rank (position inside the heap's rank table)
  int32_t world;         // number of ranks sharing the heap
  uint64_t heap_size;    // bytes per rank
  uint64_t mc_base;      // NVLS multicast mapping of the heap in this process (0 = none)
  int32_t* status;       // status word, nonzero after a bounded wait ran out (see Status)
  uint64_t timeout_ns;   // limit of every cross-rank wait
  TraceBuffers trace;
  uint64_t bases[kMaxRanks];

  // Build from the int64 context tensor (layout in common.cuh). `ctx` may be device or host memory.
  IRIS_HD static DeviceContext initialize(const int64_t* ctx, bool tracing = false) {
    DeviceContext c;
    c.rank = (int32_t)ctx[0];
    c.world = (int32_t)ctx[1];
    c.heap_size = ~0ull;
    c.mc_base = 0;
    c.status = nullptr;
    c.timeout_ns = 10000000000ull;
    for (int i = 0; i < c.world && i < kMaxRanks; ++i) c.bases[i] = (uint64_t)ctx[2 + i];
    const int64_t* t = ctx + 2 + c.world;
    c.trace.enabled = tracing ? (int32_t)t[0] : 0;
    c.trace.max_events = (int32_t)t[1];
    c.trace.counter = (int32_t*)t[2];
    c.trace.op_index_counter = (int32_t*)t[3];
    c.trace.event_id = (int32_t*)t[4];
    c.trace.pid = (int32_t*)t[5];
    c.trace.pid_m = (int32_t*)t[6];
    c.trace.pid_n = (int32_t*)t[7];
    c.trace.cur_rank = (int32_t*)t[8];
    c.trace.target_rank = (int32_t*)t[9];
    c.trace.xcc_id = (int32_t*)t[10];
    c.trace.cu_id = (int32_t*)t[11];
    c.trace.timestamp = (int64_t*)t[12];
    c.trace.address = (int64_t*)t[13];
    c.trace.duration_cycles = (int64_t*)t[14];
    c.trace.op_index = (int32_t*)t[15];
    c.trace.payload_size = (int32_t*)t[16];
    return c;
  }

  // Translate a pointer into rank `from`'s heap to the same offset in rank `to`'s heap.
  template <class T>
  IRIS_HD T* translate(T* p, int from, int to) const {
    return (T*)(bases[to] + ((uint64_t)p - bases[from]));
  }
  // Pointer into my own heap -> same object on `to`.
  template <class T>
  IRIS_HD T* remote(T* p, int to) const {
    return (T*)(bases[to] + ((uint64_t)p - bases[rank]));
  }
  // Pointer into my own heap -> its address in the NVLS multicast window (stores reach all ranks).
  template <class T>
  IRIS_HD T* mc(T* p) const {
    return (T*)(mc_base + ((uint64_t)p - bases[rank]));
  }
  IRIS_HD bool in_heap(const void* p, int r) const {
    uint64_t a = (uint64_t)p;
    return a >= bases[r] && a - bases[r] < heap_size;
  }
  // Record the first failure; later ones keep the first code.
  IRIS_D void fail(int code) const {
#if defined(__CUDACC__)
    if (status) atomicCAS(status, 0, code);
#else
    if (status) {
      int32_t z = 0;
      __atomic_compare_exchange_n(status, &z, (int32_t)code, false, __ATOMIC_RELAXED, __ATOMIC_RELAXED);
    }
#endif
  }
};

// Functional form of the translation used by the free-function API.
template <class T>
IRIS_HD T* translate(T* p, int from_rank, int to_rank, const uint64_t* heap_bases) {
  return (T*)(heap_bases[to_rank] + ((uint64_t)p - heap_bases[from_rank]));
}

}  // namespace iris
