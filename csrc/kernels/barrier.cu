// Device-side barrier across ranks and the bounded-wait probe.
//
// iris_device_barrier: one CTA; thread 0 adds 1 to its slot in every peer's SyncBlock (release,
// system scope), then polls its own block until every peer's slot reached the round it is in
// (acquire). The round counter lives in device memory, so the launch takes no host-side epoch and
// can be captured in a CUDA graph and replayed (reference: iris/host/distributed/helpers.py:
// 324-417, which traps after 1e9 spins; here a wait that runs out sets the status word).
#include <cuda_runtime.h>
#include <string.h>

#include "iris/host_api.h"
#include "iris/iris.cuh"

using namespace iris;

namespace {

__global__ void device_barrier_kernel(const __grid_constant__ DeviceContext ctx, SyncBlock* sb) {
  const int32_t e = read_epoch(sb);      // one warp: lane r signals and polls rank r
  __threadfence_system();
  barrier_signal_warp(ctx, sb);
  barrier_wait_warp(ctx, sb, e + 1);
  __syncwarp();
  if (threadIdx.x == 0) {
    sb->epoch = e + 1;
    __threadfence_system();
  }
}

// Waits until *flag >= target or timeout_ns elapsed; writes 0 (seen) or 1 (timed out) to *result.
__global__ void wait_flag_kernel(const int32_t* flag, int32_t target, unsigned long long timeout_ns, int32_t* result) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *result = wait_flag_ge_limit(flag, target, timeout_ns) ? 0 : 1;
}

__global__ void set_flag_kernel(const __grid_constant__ DeviceContext ctx, int32_t* flag_heap, int32_t value, int to_rank) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    fence_sys();
    st_release_sys(ctx.remote(flag_heap, to_rank), value);
  }
}

}  // namespace

extern "C" {

int iris_device_barrier(const IrisCtx* ctx, void* sync_block, void* stream) {
  DeviceContext c;
  memcpy(&c, ctx, sizeof(c));
  device_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c, (SyncBlock*)sync_block);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

int iris_wait_flag(const int32_t* flag, int32_t target, unsigned long long timeout_ns, int32_t* result, void* stream) {
  wait_flag_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flag, target, timeout_ns, result);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

int iris_set_flag(const IrisCtx* ctx, int32_t* flag_heap, int32_t value, int to_rank, void* stream) {
  DeviceContext c;
  memcpy(&c, ctx, sizeof(c));
  set_flag_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c, flag_heap, value, to_rank);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // extern "C"
