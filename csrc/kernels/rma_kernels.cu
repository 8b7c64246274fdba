// Host-launchable elementwise forms of every device RMA op. They serve three purposes: the
// Python-level `ctx.rma.*` calls (one-sided operations on tensors without writing a kernel), the
// unit tests of the header library (each op x semantics x scope x cache operator, reference
// tests/unittests/test_{load,store,get,put,copy,atomic_*}_triton.py), and the message-passing
// example. One kernel per op family; the semantic/scope/cache variants are template instances
// selected by a switch on the host-provided codes.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <string.h>

#include "iris/host_api.h"
#include "iris/iris.cuh"

using namespace iris;

namespace {

enum Op { kLoad = 0, kStore, kCopy, kGet, kPut, kAdd, kSub, kAnd, kOr, kXor, kMin, kMax, kXchg, kCas };

struct RmaArgs {
  DeviceContext ctx;
  int op, sem, scope, cache_ld, cache_st, vol, oo;
  void* a;
  void* b;
  void* result;
  double fval;
  long long ival, icmp;
  unsigned long long n;
  int from_rank, to_rank;
};

template <class T> __device__ T scalar_of(const RmaArgs& x) {
  if constexpr (sizeof(T) == 2) return detail::bit_cast<T>((uint16_t)x.ival);
  else if constexpr (std::is_floating_point<T>::value) return (T)x.fval;
  else return (T)x.ival;
}
template <class T> __device__ T cmp_of(const RmaArgs& x) {
  if constexpr (std::is_floating_point<T>::value) return (T)x.fval;
  else return (T)x.icmp;
}

template <class T, CacheOp C, bool V>
__device__ void do_load(const RmaArgs& x, size_t i) {
  const T* p = (const T*)x.a + i;
  Tracing<true> tr(x.ctx);
  int h = tr.record_event_start(kEvLoad, x.from_rank, p, 0, 0, sizeof(T));
  T v = x.oo ? Ctx(x.ctx).load<T, C, V>(p, x.from_rank) : load<T, C, V>(p, x.ctx.rank, x.from_rank, x.ctx.bases);
  tr.record_event_end(h);
  ((T*)x.result)[i] = v;
}
template <class T, CacheOp C>
__device__ void do_store(const RmaArgs& x, size_t i) {
  T* p = (T*)x.a + i;
  const T v = x.b ? ((const T*)x.b)[i] : scalar_of<T>(x);
  Tracing<true> tr(x.ctx);
  int h = tr.record_event_start(kEvStore, x.to_rank, p, 0, 0, sizeof(T));
  if (x.oo) Ctx(x.ctx).store<T, C>(p, v, x.to_rank);
  else store<T, C>(p, v, x.ctx.rank, x.to_rank, x.ctx.bases);
  tr.record_event_end(h);
}

template <class T>
__global__ void rma_move_kernel(const __grid_constant__ RmaArgs x) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < x.n; i += stride) {
    switch (x.op) {
      case kLoad:
        if (x.vol) do_load<T, CacheOp::none, true>(x, i);
        else switch (x.cache_ld) {
          case 1: do_load<T, CacheOp::ca, false>(x, i); break;
          case 2: do_load<T, CacheOp::cg, false>(x, i); break;
          case 3: do_load<T, CacheOp::cs, false>(x, i); break;
          case 4: do_load<T, CacheOp::cv, false>(x, i); break;
          default: do_load<T, CacheOp::none, false>(x, i);
        }
        break;
      case kStore:
        switch (x.cache_st) {
          case 5: do_store<T, CacheOp::wb>(x, i); break;
          case 2: do_store<T, CacheOp::cg>(x, i); break;
          case 3: do_store<T, CacheOp::cs>(x, i); break;
          case 6: do_store<T, CacheOp::wt>(x, i); break;
          default: do_store<T, CacheOp::none>(x, i);
        }
        break;
      case kCopy:
        if (x.oo) Ctx(x.ctx).copy((const T*)x.a + i, (T*)x.b + i, x.from_rank, x.to_rank);
        else copy((const T*)x.a + i, (T*)x.b + i, x.from_rank, x.to_rank, x.ctx.rank, x.ctx.bases);
        break;
      case kGet:
        if (x.oo) Ctx(x.ctx).get((const T*)x.a + i, (T*)x.b + i, x.from_rank);
        else get((const T*)x.a + i, (T*)x.b + i, x.from_rank, x.ctx.rank, x.ctx.bases);
        break;
      case kPut:
        if (x.oo) Ctx(x.ctx).put((const T*)x.a + i, (T*)x.b + i, x.to_rank);
        else put((const T*)x.a + i, (T*)x.b + i, x.ctx.rank, x.to_rank, x.ctx.bases);
        break;
      default: break;
    }
  }
}

template <class T, Sem S, Scope P>
__device__ void do_atomic(const RmaArgs& x, size_t i) {
  T* p = (T*)x.a + i;
  const T v = x.b ? ((const T*)x.b)[i] : scalar_of<T>(x);
  const int from = x.ctx.rank, to = x.to_rank;
  const uint64_t* bases = x.ctx.bases;
  T old = T();
  Tracing<true> tr(x.ctx);
  int h = tr.record_event_start(kEvAtomicAdd + (x.op - kAdd), to, p, 0, 0, sizeof(T));
  if constexpr (std::is_same<T, float>::value || std::is_same<T, double>::value) {
    switch (x.op) {
      case kAdd: old = atomic_add<S, P>(p, v, from, to, bases); break;
      case kSub: old = atomic_sub<S, P>(p, v, from, to, bases); break;
      case kXchg: old = atomic_xchg<S, P>(p, v, from, to, bases); break;
      case kCas: old = atomic_cas<S, P>(p, cmp_of<T>(x), v, from, to, bases); break;
      default: break;
    }
  } else {
    switch (x.op) {
      case kAdd: old = atomic_add<S, P>(p, v, from, to, bases); break;
      case kSub: old = atomic_sub<S, P>(p, v, from, to, bases); break;
      case kMin: old = atomic_min<S, P>(p, v, from, to, bases); break;
      case kMax: old = atomic_max<S, P>(p, v, from, to, bases); break;
      case kXchg: old = atomic_xchg<S, P>(p, v, from, to, bases); break;
      case kCas: old = atomic_cas<S, P>(p, cmp_of<T>(x), v, from, to, bases); break;
      default:
        if constexpr (std::is_unsigned<T>::value) {
          if (x.op == kAnd) old = atomic_and<S, P>(p, v, from, to, bases);
          else if (x.op == kOr) old = atomic_or<S, P>(p, v, from, to, bases);
          else if (x.op == kXor) old = atomic_xor<S, P>(p, v, from, to, bases);
        }
    }
  }
  tr.record_event_end(h);
  if (x.result) ((T*)x.result)[i] = old;
}

template <class T, Sem S>
__device__ void atomic_scope(const RmaArgs& x, size_t i) {
  switch (x.scope) {
    case 0: do_atomic<T, S, Scope::cta>(x, i); break;
    case 1: do_atomic<T, S, Scope::gpu>(x, i); break;
    default: do_atomic<T, S, Scope::sys>(x, i);
  }
}

template <class T>
__global__ void rma_atomic_kernel(const __grid_constant__ RmaArgs x) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < x.n; i += stride) {
    switch (x.sem) {
      case 0: atomic_scope<T, Sem::relaxed>(x, i); break;
      case 1: atomic_scope<T, Sem::acquire>(x, i); break;
      case 2: atomic_scope<T, Sem::release>(x, i); break;
      default: atomic_scope<T, Sem::acq_rel>(x, i);
    }
  }
}

// 16-bit float atomic add (the only 16-bit atomic the hardware has besides CAS).
template <bool kBf16>
__global__ void rma_atomic_add16_kernel(const __grid_constant__ RmaArgs x) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < x.n; i += stride) {
    uint16_t* p = translate((uint16_t*)x.a + i, x.ctx.rank, x.to_rank, x.ctx.bases);
    const uint16_t v = x.b ? ((const uint16_t*)x.b)[i] : (uint16_t)x.ival;
    uint16_t old;
    if (x.scope == 2) old = kBf16 ? detail::atom_add_bf16<Sem::relaxed, Scope::sys>(p, v) : detail::atom_add_f16<Sem::relaxed, Scope::sys>(p, v);
    else old = kBf16 ? detail::atom_add_bf16<Sem::relaxed, Scope::gpu>(p, v) : detail::atom_add_f16<Sem::relaxed, Scope::gpu>(p, v);
    if (x.result) ((uint16_t*)x.result)[i] = old;
  }
}

// Producer/consumer message passing in one kernel pair (reference examples/06_message_passing):
// the producer rank puts `n` elements into the consumer's buffer block by block and raises one
// flag per block (release, system scope); the consumer waits for each flag (acquire, bounded) and
// copies the block out.
__global__ void msg_producer_kernel(const __grid_constant__ DeviceContext ctx, const float* src, float* dst_heap,
                                    int32_t* flags_heap, unsigned long long n, int block_elems, int consumer) {
  for (size_t blk = blockIdx.x; blk * block_elems < n; blk += gridDim.x) {
    const size_t lo = blk * block_elems;
    const size_t cnt = min((unsigned long long)block_elems, n - lo);
    put_block(ctx, src + lo, dst_heap + lo, cnt, consumer, threadIdx.x, blockDim.x);
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_sys();
      st_release_sys(ctx.remote(flags_heap + blk, consumer), 1);
    }
  }
}
__global__ void msg_consumer_kernel(const __grid_constant__ DeviceContext ctx, const float* buf_heap, float* out,
                                    int32_t* flags_heap, unsigned long long n, int block_elems) {
  __shared__ int s_ok;
  for (size_t blk = blockIdx.x; blk * block_elems < n; blk += gridDim.x) {
    if (threadIdx.x == 0) s_ok = wait_flag_ge(ctx, flags_heap + blk, 1) ? 1 : 0;
    __syncthreads();
    const bool ok = s_ok != 0;
    __syncthreads();
    if (!ok) return;
    const size_t lo = blk * block_elems;
    const size_t cnt = min((unsigned long long)block_elems, n - lo);
    for (size_t i = threadIdx.x; i < cnt; i += blockDim.x) out[lo + i] = buf_heap[lo + i];
    __syncthreads();
    if (threadIdx.x == 0) flags_heap[blk] = 0;
  }
}

template <class T>
int launch_move(const RmaArgs& x, cudaStream_t s) {
  const int threads = 256;
  const int blocks = (int)((x.n + threads - 1) / threads < 1184 ? (x.n + threads - 1) / threads : 1184);
  rma_move_kernel<T><<<blocks > 0 ? blocks : 1, threads, 0, s>>>(x);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
template <class T>
int launch_atomic(const RmaArgs& x, cudaStream_t s) {
  const int threads = 256;
  const int blocks = (int)((x.n + threads - 1) / threads < 1184 ? (x.n + threads - 1) / threads : 1184);
  rma_atomic_kernel<T><<<blocks > 0 ? blocks : 1, threads, 0, s>>>(x);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace

extern "C" {

// Elementwise RMA over n elements. op codes: 0 load, 1 store, 2 copy, 3 get, 4 put, 5 add, 6 sub,
// 7 and, 8 or, 9 xor, 10 min, 11 max, 12 xchg, 13 cas. dtype codes: IrisDType plus 7 f64, 8 u8,
// 9 i16, 10 u32, 11 u64. `a`/`b`/`result` are device pointers (b may be null: scalar operand).
int iris_rma_launch(const IrisCtx* ctx, int op, int dtype, int sem, int scope, int cache_ld, int cache_st, int vol,
                    int oo, void* a, void* b, void* result, double fval, long long ival, long long icmp,
                    unsigned long long n, int from_rank, int to_rank, void* stream) {
  RmaArgs x;
  memcpy(&x.ctx, ctx, sizeof(DeviceContext));
  x.op = op; x.sem = sem; x.scope = scope; x.cache_ld = cache_ld; x.cache_st = cache_st; x.vol = vol; x.oo = oo;
  x.a = a; x.b = b; x.result = result; x.fval = fval; x.ival = ival; x.icmp = icmp; x.n = n;
  x.from_rank = from_rank; x.to_rank = to_rank;
  cudaStream_t s = (cudaStream_t)stream;
  if (n == 0) return 0;
  if (op <= kPut) {
    switch (dtype) {
      case IRIS_F16: case IRIS_BF16: case 9: return launch_move<uint16_t>(x, s);
      case IRIS_F32: return launch_move<float>(x, s);
      case IRIS_I32: case 10: return launch_move<int32_t>(x, s);
      case IRIS_I8: case IRIS_F8E4M3: case 8: return launch_move<uint8_t>(x, s);
      case IRIS_I64: case 11: return launch_move<int64_t>(x, s);
      case 7: return launch_move<double>(x, s);
      default: return -2;
    }
  }
  if ((dtype == IRIS_F16 || dtype == IRIS_BF16) && op == kAdd) {
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 1184 ? (n + threads - 1) / threads : 1184);
    if (dtype == IRIS_BF16) rma_atomic_add16_kernel<true><<<blocks, threads, 0, s>>>(x);
    else rma_atomic_add16_kernel<false><<<blocks, threads, 0, s>>>(x);
    return cudaGetLastError() == cudaSuccess ? 0 : -21;
  }
  switch (dtype) {
    case IRIS_F32: return launch_atomic<float>(x, s);
    case IRIS_I32: return launch_atomic<int32_t>(x, s);
    case 10: return launch_atomic<uint32_t>(x, s);
    case IRIS_I64: return launch_atomic<int64_t>(x, s);
    case 11: return launch_atomic<uint64_t>(x, s);
    case 7: return launch_atomic<double>(x, s);
    default: return -2;
  }
}

int iris_msg_producer(const IrisCtx* ctx, const float* src, float* dst_heap, int32_t* flags_heap, unsigned long long n,
                      int block_elems, int consumer, void* stream) {
  DeviceContext c;
  memcpy(&c, ctx, sizeof(c));
  const int blocks = (int)((n + block_elems - 1) / block_elems);
  msg_producer_kernel<<<blocks < 148 ? blocks : 148, 256, 0, (cudaStream_t)stream>>>(c, src, dst_heap, flags_heap, n,
                                                                                  block_elems, consumer);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
int iris_msg_consumer(const IrisCtx* ctx, const float* buf_heap, float* out, int32_t* flags_heap, unsigned long long n,
                      int block_elems, void* stream) {
  DeviceContext c;
  memcpy(&c, ctx, sizeof(c));
  const int blocks = (int)((n + block_elems - 1) / block_elems);
  msg_consumer_kernel<<<blocks < 148 ? blocks : 148, 256, 0, (cudaStream_t)stream>>>(c, buf_heap, out, flags_heap, n,
                                                                                  block_elems);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // extern "C"
