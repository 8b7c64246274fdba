// Flags, bounded waits and the cross-rank barrier used inside kernels.
//
// Conventions (same as the reference's locks/flags, iris/ops/matmul_all_reduce.py:129-136):
// int32 words on the symmetric heap, producers publish with release semantics at system scope,
// consumers poll with acquire loads. Unlike the reference's device barrier, which asserts after
// 1e9 spins (iris/host/distributed/helpers.py:342), every wait here has a time limit, records a
// Status in the context and returns false, so a missing peer never hangs or traps the GPU.
#pragma once
#include "common.cuh"
#include "context.cuh"
#include "rma.cuh"

namespace iris {

#if defined(__CUDACC__)
IRIS_D int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
IRIS_D int32_t ld_relaxed_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
IRIS_D int32_t ld_acquire_gpu(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
IRIS_D void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
IRIS_D void st_release_gpu(int32_t* p, int32_t v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
IRIS_D void st_relaxed_sys(int32_t* p, int32_t v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
IRIS_D void red_release_sys_add(int32_t* p, int32_t v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
IRIS_D void red_release_gpu_add(int32_t* p, int32_t v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
IRIS_D void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
IRIS_D void fence_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
IRIS_D uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
IRIS_D void backoff(unsigned ns) { __nanosleep(ns); }
#else
inline int32_t ld_acquire_sys(const int32_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline int32_t ld_relaxed_sys(const int32_t* p) { return __atomic_load_n(p, __ATOMIC_RELAXED); }
inline int32_t ld_acquire_gpu(const int32_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline void st_release_sys(int32_t* p, int32_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
inline void st_release_gpu(int32_t* p, int32_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
inline void st_relaxed_sys(int32_t* p, int32_t v) { __atomic_store_n(p, v, __ATOMIC_RELAXED); }
inline void red_release_sys_add(int32_t* p, int32_t v) { __atomic_fetch_add(p, v, __ATOMIC_RELEASE); }
inline void red_release_gpu_add(int32_t* p, int32_t v) { __atomic_fetch_add(p, v, __ATOMIC_RELEASE); }
inline void fence_sys() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
inline void fence_gpu() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
uint64_t now_ns();  // defined by the CPU backend (steady clock)
void backoff(unsigned ns);
#endif

// Poll `*p` (acquire, system scope) until it is >= `target`. False after ctx.timeout_ns.
IRIS_D bool wait_flag_ge(const DeviceContext& ctx, const int32_t* p, int32_t target, int fail_code = kTimeoutFlag) {
  for (int i = 0; i < 32; ++i)
    if (ld_acquire_sys(p) - target >= 0) return true;
  const uint64_t t0 = now_ns();
  unsigned n = 0;
  while (true) {
    if (ld_acquire_sys(p) - target >= 0) return true;
    if ((++n & 63u) == 0) {
      if (now_ns() - t0 > ctx.timeout_ns) {
        ctx.fail(fail_code);
        return false;
      }
      backoff(64);
    }
  }
}
// Same with an explicit limit (used by tests with a flag that nothing sets).
IRIS_D bool wait_flag_ge_limit(const int32_t* p, int32_t target, uint64_t timeout_ns) {
  const uint64_t t0 = now_ns();
  unsigned n = 0;
  while (true) {
    if (ld_acquire_sys(p) - target >= 0) return true;
    if ((++n & 15u) == 0 && now_ns() - t0 > timeout_ns) return false;
  }
}

// Per-op synchronisation block on the symmetric heap (same offset on every rank).
//   epoch        number of barrier rounds completed by kernels using this block
//   done         CTAs of the running kernel that finished their work
//   slots[r]     rounds signalled by rank r into this rank
struct SyncBlock {
  int32_t epoch;
  int32_t done;
  int32_t aux[6];
  int32_t slots[kMaxRanks];
};

// Tell every peer that this rank reached round `round` (one thread calls this).
IRIS_D void barrier_signal(const DeviceContext& ctx, SyncBlock* sb) {
  for (int i = 1; i < ctx.world; ++i) {
    int r = ctx.rank + i;
    if (r >= ctx.world) r -= ctx.world;
    red_release_sys_add(&ctx.remote(sb, r)->slots[ctx.rank], 1);
  }
}
// Wait until every peer signalled round `target` into my block (one thread calls this).
IRIS_D bool barrier_wait(const DeviceContext& ctx, SyncBlock* sb, int32_t target) {
  bool ok = true;
  for (int r = 0; r < ctx.world; ++r) {
    if (r == ctx.rank) continue;
    ok = wait_flag_ge(ctx, &sb->slots[r], target, kTimeoutBarrier) && ok;
    if (!ok) break;
  }
  return ok;
}

#if defined(__CUDACC__)
// Warp-parallel forms: lane r talks to rank r, so the W-1 remote atomics (and their release
// fences) and the W-1 polls overlap instead of running one after the other. All 32 lanes call.
IRIS_D void barrier_signal_warp(const DeviceContext& ctx, SyncBlock* sb) {
  const int lane = threadIdx.x & 31;
  for (int r = lane; r < ctx.world; r += 32)
    if (r != ctx.rank) red_release_sys_add(&ctx.remote(sb, r)->slots[ctx.rank], 1);
}
IRIS_D bool barrier_wait_warp(const DeviceContext& ctx, SyncBlock* sb, int32_t target) {
  const int lane = threadIdx.x & 31;
  bool ok = true;
  for (int r = lane; r < ctx.world; r += 32)
    if (r != ctx.rank) ok = wait_flag_ge(ctx, &sb->slots[r], target, kTimeoutBarrier) && ok;
  return __all_sync(0xffffffffu, ok);
}

// Kernel epilogue: every CTA calls this (all threads, blockDim.x >= 32) after its last remote
// access. The CTA that arrives last runs one cross-rank round (signal, then wait for all peers),
// so that when the kernel completes every peer's stores into this rank have been published.
// `rounds_before` is the number of rounds this kernel already ran on the block (0 or 1), `epoch0`
// the epoch read at entry.
IRIS_D void grid_exit_barrier(const DeviceContext& ctx, SyncBlock* sb, int32_t epoch0, int rounds_before) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int total = gridDim.x * gridDim.y * gridDim.z;
    s_last = atomicAdd(&sb->done, 1) == total - 1 ? 1 : 0;
  }
  __syncthreads();
  if (s_last && threadIdx.x < 32) {
    __threadfence_system();
    if (ctx.world > 1) {
      barrier_signal_warp(ctx, sb);
      barrier_wait_warp(ctx, sb, epoch0 + rounds_before + 1);
    }
    if (threadIdx.x == 0) {
      sb->done = 0;
      sb->epoch = epoch0 + rounds_before + 1;
      __threadfence_system();
    }
  }
}
// Kernel prologue round: CTA 0 signals, every CTA that touches peer memory afterwards waits
// until all peers entered (their inputs are final and their previous use of buffers is over).
IRIS_D bool grid_entry_barrier(const DeviceContext& ctx, SyncBlock* sb, int32_t epoch0) {
  __shared__ int s_ok;
  if (threadIdx.x < 32) {
    bool ok = true;
    if (ctx.world > 1) {
      if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        __threadfence_system();
        barrier_signal_warp(ctx, sb);
      }
      ok = barrier_wait_warp(ctx, sb, epoch0 + 1);
    }
    if (threadIdx.x == 0) s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  return s_ok != 0;
}
IRIS_D int32_t read_epoch(SyncBlock* sb) { return *(volatile int32_t*)&sb->epoch; }
#endif

}  // namespace iris
