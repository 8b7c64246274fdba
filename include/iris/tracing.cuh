// Device-side event tracing into the structure-of-arrays buffers owned by the host Tracing
// manager. Same event ids and fields as the reference (iris/mem/triton/tracing.py:19-186,
// iris/host/tracing/events.py:18-99); timestamps are %globaltimer nanoseconds, cu_id is %smid,
// xcc_id is 0. With Enabled = false every call compiles to nothing.
#pragma once
#include "common.cuh"
#include "context.cuh"

namespace iris {

enum TraceEventId : int {
  kEvLoad = 0, kEvStore = 1, kEvGet = 2, kEvPut = 3, kEvCopy = 4, kEvAtomicAdd = 5, kEvAtomicSub = 6,
  kEvAtomicCas = 7, kEvAtomicXchg = 8, kEvAtomicXor = 9, kEvAtomicAnd = 10, kEvAtomicOr = 11,
  kEvAtomicMin = 12, kEvAtomicMax = 13,
};

#if defined(__CUDACC__)
template <bool Enabled>
struct Tracing {
  const TraceBuffers* tb;
  int rank;
  IRIS_D explicit Tracing(const DeviceContext& ctx) : tb(&ctx.trace), rank(ctx.rank) {}

  // Returns a handle (event slot) to pass to record_event_end, or -1 when nothing was recorded.
  IRIS_D int record_event_start(int event_id, int target_rank, const void* address, int pid_m, int pid_n,
                                int payload_bytes) const {
    if constexpr (!Enabled) return -1;
    if (!tb->enabled) return -1;
    const int idx = atomicAdd(tb->counter, 1);
    const int op = atomicAdd(tb->op_index_counter, 1);
    if (idx >= tb->max_events) return -1;
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    uint32_t sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    tb->event_id[idx] = event_id;
    tb->pid[idx] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    tb->pid_m[idx] = pid_m;
    tb->pid_n[idx] = pid_n;
    tb->cur_rank[idx] = rank;
    tb->target_rank[idx] = target_rank;
    tb->xcc_id[idx] = 0;
    tb->cu_id[idx] = (int)sm;
    tb->timestamp[idx] = (int64_t)t;
    tb->address[idx] = (int64_t)address;
    tb->duration_cycles[idx] = 0;
    tb->op_index[idx] = op;
    tb->payload_size[idx] = payload_bytes;
    return idx;
  }
  IRIS_D void record_event_end(int handle) const {
    if constexpr (!Enabled) return;
    if (handle < 0) return;
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    tb->duration_cycles[handle] = (int64_t)t;  // end timestamp, as in the reference
  }
};
#endif

}  // namespace iris
