// CPU backend: the device header library (include/iris/*.cuh) compiled for the host, driven over
// ranges of elements. "Peers" are other processes whose memfd heaps are mapped into this one, so
// translate() + an ordinary access reaches them exactly as a peer mapping does on the GPU. The
// reference has no CPU path for its RMA ops (its tests all need real GPUs); this
// backend lets the host layer, the RMA semantics and failure handling be tested under gloo.
#include <stdint.h>
#include <string.h>
#include <time.h>

#include <chrono>
#include <thread>
#include <type_traits>

#include "iris/context.cuh"
#include "iris/rma.cuh"
#include "iris/sync.cuh"

namespace iris {
uint64_t now_ns() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
void backoff(unsigned ns) {
  if (ns >= 1000) std::this_thread::sleep_for(std::chrono::nanoseconds(ns));
  else std::this_thread::yield();
}
}  // namespace iris

using namespace iris;

namespace {

enum Op { kLoad = 0, kStore, kCopy, kGet, kPut, kAdd, kSub, kAnd, kOr, kXor, kMin, kMax, kXchg, kCas };

struct Args {
  int op, sem;
  uint64_t a, b, result;   // a: first pointer argument, b: second pointer / value array (0 = scalar)
  double fval;
  int64_t ival, icmp;
  uint64_t n;
  int from_rank, to_rank, cur_rank;
  const uint64_t* bases;
};

template <class T> T scalar_of(const Args& x) {
  if constexpr (std::is_floating_point<T>::value) return (T)x.fval;
  else return (T)x.ival;
}

template <class T> T scalar_cmp(const Args& x) {
  if constexpr (std::is_floating_point<T>::value) return (T)x.fval;
  else return (T)x.icmp;
}

template <class T, Sem S>
int run_atomic(const Args& x) {
  T* p = (T*)x.a;
  const T* vals = (const T*)x.b;
  T* res = (T*)x.result;
  const T sv = scalar_of<T>(x);
  for (uint64_t i = 0; i < x.n; ++i) {
    const T v = vals ? vals[i] : sv;
    T old;
    switch (x.op) {
      case kAdd: old = atomic_add<S, Scope::sys>(p + i, v, x.from_rank, x.to_rank, x.bases); break;
      case kSub: old = atomic_sub<S, Scope::sys>(p + i, v, x.from_rank, x.to_rank, x.bases); break;
      case kMin: old = atomic_min<S, Scope::sys>(p + i, v, x.from_rank, x.to_rank, x.bases); break;
      case kMax: old = atomic_max<S, Scope::sys>(p + i, v, x.from_rank, x.to_rank, x.bases); break;
      case kXchg: old = atomic_xchg<S, Scope::sys>(p + i, v, x.from_rank, x.to_rank, x.bases); break;
      case kCas: old = atomic_cas<S, Scope::sys>(p + i, (T)scalar_cmp<T>(x), v, x.from_rank, x.to_rank, x.bases); break;
      default:
        if constexpr (std::is_integral<T>::value) {
          if (x.op == kAnd) old = atomic_and<S, Scope::sys>(p + i, v, x.from_rank, x.to_rank, x.bases);
          else if (x.op == kOr) old = atomic_or<S, Scope::sys>(p + i, v, x.from_rank, x.to_rank, x.bases);
          else if (x.op == kXor) old = atomic_xor<S, Scope::sys>(p + i, v, x.from_rank, x.to_rank, x.bases);
          else return -3;
        } else {
          return -3;
        }
    }
    if (res) res[i] = old;
  }
  return 0;
}

template <class T>
int run(const Args& x) {
  switch (x.op) {
    case kLoad: {
      const T* p = (const T*)x.a;
      T* res = (T*)x.result;
      for (uint64_t i = 0; i < x.n; ++i) res[i] = load(p + i, x.to_rank, x.from_rank, x.bases);
      return 0;
    }
    case kStore: {
      T* p = (T*)x.a;
      const T* vals = (const T*)x.b;
      T sv;
      if constexpr (sizeof(T) == 2 && !std::is_integral<T>::value) sv = T();
      else sv = scalar_of<T>(x);
      for (uint64_t i = 0; i < x.n; ++i) store(p + i, vals ? vals[i] : sv, x.from_rank, x.to_rank, x.bases);
      return 0;
    }
    case kCopy:
      for (uint64_t i = 0; i < x.n; ++i) copy((const T*)x.a + i, (T*)x.b + i, x.from_rank, x.to_rank, x.cur_rank, x.bases);
      return 0;
    case kGet:
      for (uint64_t i = 0; i < x.n; ++i) get((const T*)x.a + i, (T*)x.b + i, x.from_rank, x.to_rank, x.bases);
      return 0;
    case kPut:
      for (uint64_t i = 0; i < x.n; ++i) put((const T*)x.a + i, (T*)x.b + i, x.from_rank, x.to_rank, x.bases);
      return 0;
    default:
      break;
  }
  if constexpr (sizeof(T) < 4) {
    return -3;  // sub-word atomics are not part of the CPU backend
  } else {
    switch (x.sem) {
      case 0: return run_atomic<T, Sem::relaxed>(x);
      case 1: return run_atomic<T, Sem::acquire>(x);
      case 2: return run_atomic<T, Sem::release>(x);
      default: return run_atomic<T, Sem::acq_rel>(x);
    }
  }
}

}  // namespace

extern "C" {

// dtype codes as in include/iris/host_api.h (0 f16, 1 bf16, 2 f32, 3 i32, 4 i8, 5 f8, 6 i64, 7 f64, 8 u8, 9 i16)
int iris_cpu_rma(int op, int dtype, int sem, uint64_t a, uint64_t b, uint64_t result, double fval, int64_t ival,
                 int64_t icmp, uint64_t n, int from_rank, int to_rank, int cur_rank, const uint64_t* bases) {
  Args x{op, sem, a, b, result, fval, ival, icmp, n, from_rank, to_rank, cur_rank, bases};
  switch (dtype) {
    case 0: case 1: case 9: return run<uint16_t>(x);
    case 2: return run<float>(x);
    case 3: return run<int32_t>(x);
    case 4: case 5: case 8: return run<uint8_t>(x);
    case 6: return run<int64_t>(x);
    case 7: return run<double>(x);
    default: return -2;
  }
}

// Bounded wait on an int32 flag (acquire): 0 when *p >= target, 1 after timeout_ns.
int iris_cpu_wait_flag(uint64_t p, int32_t target, uint64_t timeout_ns) {
  return wait_flag_ge_limit((const int32_t*)p, target, timeout_ns) ? 0 : 1;
}

// Device-style barrier on a SyncBlock of the CPU heap: signal every peer, wait for all of them.
// Returns 0, or 1 when a peer did not arrive within timeout_ns (the status word is set as well).
int iris_cpu_barrier(int rank, int world, const uint64_t* bases, uint64_t sync_block, uint64_t timeout_ns, uint64_t status) {
  DeviceContext ctx;
  memset(&ctx, 0, sizeof(ctx));
  ctx.rank = rank;
  ctx.world = world;
  ctx.timeout_ns = timeout_ns;
  ctx.status = (int32_t*)status;
  for (int i = 0; i < world; ++i) ctx.bases[i] = bases[i];
  SyncBlock* sb = (SyncBlock*)sync_block;
  const int32_t target = sb->epoch + 1;
  fence_sys();
  barrier_signal(ctx, sb);
  bool ok = barrier_wait(ctx, sb, target);
  sb->epoch = target;
  return ok ? 0 : 1;
}

}  // extern "C"
