// Umbrella header of the device library. A user kernel includes this, takes an iris::DeviceContext
// (by value, as a kernel parameter, or built from the int64 context tensor with
// DeviceContext::initialize) and calls the RMA functions:
//
//   __global__ void k(iris::DeviceContext ctx, float* buf, int n) {
//     iris::Ctx c(ctx);
//     int i = blockIdx.x * blockDim.x + threadIdx.x;
//     c.store(buf + i, 1.0f, /*to_rank=*/1, i < n);
//   }
//
// Ctx is the object-oriented form of the API (reference: iris/mem/triton/context.py:213-685):
// the same operations as rma.cuh with the caller's rank implied.
#pragma once
#include "common.cuh"
#include "context.cuh"
#include "rma.cuh"
#include "sync.cuh"
#include "types.cuh"
#include "tracing.cuh"
#if defined(__CUDACC__)
#include "multimem.cuh"
#include "ptx.cuh"
#include "tile_collectives.cuh"
#endif

namespace iris {

// Device intrinsics of the reference (iris/mem/utils.py:25-92).
#if defined(__CUDACC__)
IRIS_D uint64_t read_realtime() { return now_ns(); }       // nanoseconds (%globaltimer)
IRIS_D uint32_t get_cu_id() { uint32_t r; asm volatile("mov.u32 %0, %%smid;" : "=r"(r)); return r; }
IRIS_D uint32_t get_xcc_id() { return 0; }
#endif

struct Ctx {
  DeviceContext c;
  IRIS_HD explicit Ctx(const DeviceContext& ctx) : c(ctx) {}
  IRIS_HD int rank() const { return c.rank; }
  IRIS_HD int world() const { return c.world; }
  IRIS_HD const uint64_t* bases() const { return c.bases; }

  // Debug builds (-DIRIS_DEBUG): an access whose pointer lies outside this rank's heap, or whose
  // target rank does not exist, is skipped and recorded as kBadTranslate in the status word (read
  // on the host with ctx.check()). Nothing traps. Without the macro the test is the constant true.
#if defined(IRIS_DEBUG)
  IRIS_D bool ok(const void* p, int r) const {
    if (r >= 0 && r < c.world && c.in_heap(p, c.rank)) return true;
    c.fail(kBadTranslate);
    return false;
  }
#else
  IRIS_D bool ok(const void*, int) const { return true; }
#endif

  template <class T, CacheOp C = CacheOp::none, bool V = false>
  IRIS_D T load(const T* p, int from_rank, bool pred = true, T other = T()) const {
    return iris::load<T, C, V>(p, c.rank, from_rank, c.bases, pred && ok(p, from_rank), other);
  }
  template <class T, CacheOp C = CacheOp::none>
  IRIS_D void store(T* p, T v, int to_rank, bool pred = true) const {
    iris::store<T, C>(p, v, c.rank, to_rank, c.bases, pred && ok(p, to_rank));
  }
  template <class T>
  IRIS_D void get(const T* from_ptr, T* to_ptr, int from_rank, bool pred = true) const {
    iris::get(from_ptr, to_ptr, from_rank, c.rank, c.bases, pred && ok(from_ptr, from_rank));
  }
  template <class T>
  IRIS_D void put(const T* from_ptr, T* to_ptr, int to_rank, bool pred = true) const {
    iris::put(from_ptr, to_ptr, c.rank, to_rank, c.bases, pred && ok(to_ptr, to_rank));
  }
  template <class T>
  IRIS_D void copy(const T* src, T* dst, int from_rank, int to_rank, bool pred = true) const {
    iris::copy(src, dst, from_rank, to_rank, c.rank, c.bases, pred && ok(src, from_rank) && ok(dst, to_rank));
  }
#define IRIS_CTX_ATOMIC(NAME)                                                       \
  template <Sem S = Sem::acq_rel, Scope P = Scope::gpu, class T>                     \
  IRIS_D T NAME(T* p, T v, int to_rank, bool pred = true) const {                    \
    return iris::NAME<S, P>(p, v, c.rank, to_rank, c.bases, pred && ok(p, to_rank)); \
  }
  IRIS_CTX_ATOMIC(atomic_add)
  IRIS_CTX_ATOMIC(atomic_sub)
  IRIS_CTX_ATOMIC(atomic_and)
  IRIS_CTX_ATOMIC(atomic_or)
  IRIS_CTX_ATOMIC(atomic_xor)
  IRIS_CTX_ATOMIC(atomic_min)
  IRIS_CTX_ATOMIC(atomic_max)
  IRIS_CTX_ATOMIC(atomic_xchg)
#undef IRIS_CTX_ATOMIC
  template <Sem S = Sem::acq_rel, Scope P = Scope::gpu, class T>
  IRIS_D T atomic_cas(T* p, T cmp, T v, int to_rank) const {
    if (!ok(p, to_rank)) return cmp;     // debug builds only: the swap is not attempted
    return iris::atomic_cas<S, P>(p, cmp, v, c.rank, to_rank, c.bases);
  }
};

}  // namespace iris
