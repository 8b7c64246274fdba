// Common definitions of the iris_b200 device library (sm_100a) and of its host-side twin.
//
// Every header under include/iris compiles in two modes:
//   * nvcc, device code for sm_100a: the real thing, PTX loads/stores/atomics over NVLink.
//   * a plain C++17 host compiler (IRIS_HOST_ONLY): the same functions on top of __atomic
//     builtins, used by the CPU backend whose "peers" are shared-memory mappings.
#pragma once
#include <stdint.h>
#include <stddef.h>

#if defined(__CUDACC__)
#define IRIS_HD __host__ __device__ __forceinline__
#define IRIS_D __device__ __forceinline__
#else
#define IRIS_HOST_ONLY 1
#define IRIS_HD inline
#define IRIS_D inline
#endif

namespace iris {

// Upper bound on the number of ranks in one symmetric heap. One NVLink domain of B200s is 8 GPUs
// (72 with NVL72 racks); the context struct travels as a kernel parameter, so keep it small.
constexpr int kMaxRanks = 72;

// Status codes written by kernels into the context's status word. 0 means success. Kernels never
// trap: a wait that runs out records a code and the kernel drains and returns.
enum Status : int {
  kOk = 0,
  kTimeoutBarrier = 1,     // cross-rank barrier wait ran out
  kTimeoutFlag = 2,        // wait on a producer flag ran out
  kTimeoutPipeline = 3,    // mbarrier wait inside a GEMM pipeline ran out
  kBadTranslate = 4,       // debug build: pointer outside the heap or rank out of range
  kTimeoutLock = 5,        // spin-lock acquisition ran out
};

// Memory-order and scope tags (mirror the strings of the reference API:
// sem in {relaxed, acquire, release, acq_rel}, scope in {cta, gpu, sys}).
enum class Sem : int { relaxed = 0, acquire = 1, release = 2, acq_rel = 3 };
enum class Scope : int { cta = 0, gpu = 1, sys = 2 };
// Cache operators of loads/stores ("" / .ca / .cg / .cs / .cv / .wb / .wt).
enum class CacheOp : int { none = 0, ca = 1, cg = 2, cs = 3, cv = 4, wb = 5, wt = 6 };

// Layout of the int64 device-context tensor handed out by Iris.get_device_context():
//   [cur_rank, num_ranks, heap_base_0 .. heap_base_{W-1}, trace_enabled, max_events,
//    trace_counter_ptr, op_index_counter_ptr, 13 trace buffer pointers]
// (same order as the reference, iris/host/iris.py:922-958, so tensors are interchangeable).
constexpr int kCtxHeaderWords = 2;
constexpr int kTraceWords = 17;

}  // namespace iris
