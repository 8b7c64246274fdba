// Tile-level collectives for use INSIDE user kernels: one CTA moves or reduces one BLOCK_M x
// BLOCK_N tile of a row-major matrix that lives at the same heap offset on every rank.
// Same set and same ownership rules as the methods of the reference's DeviceContext
// (iris/mem/triton/context.py:687-997):
//   all_reduce_atomic     add my tile into every rank's destination (destination pre-zeroed)
//   all_reduce_spinlock   per-(tile, destination) lock, read-modify-write under the lock
//   all_reduce_one_shot   wait for every rank's "tile ready" lock, pull all W copies, sum, store
//   all_reduce_two_shot   owner (tile_id % W) pulls and sums, then stores the result to all ranks
//   all_gather            store my tile into every rank's destination at my rank's row/col block
//   gather                pull one rank's tile into local memory
//   all_to_all            exchange column chunks of a tile row block
//   reduce_scatter        owner of contiguous tile blocks (last rank takes the remainder) pulls+sums
// All threads of the CTA call the function. Waits are bounded (ctx.timeout_ns) and return false
// after recording a status; accumulation is fp32.
#pragma once
#include "common.cuh"
#include "context.cuh"
#include "rma.cuh"
#include "sync.cuh"
#include "types.cuh"
#if defined(__CUDACC__)
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace iris {
namespace tile {

template <class T> IRIS_D float to_f32(T v) { return (float)v; }
template <> IRIS_D float to_f32<__half>(__half v) { return __half2float(v); }
template <> IRIS_D float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <class T> IRIS_D T from_f32(float v) { return (T)v; }
template <> IRIS_D __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> IRIS_D __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <class T> IRIS_D void red_add(T* p, float v);
template <> IRIS_D void red_add<float>(float* p, float v) { asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory"); }
template <> IRIS_D void red_add<__half>(__half* p, float v) {
  __half h = __float2half_rn(v);
  asm volatile("red.relaxed.sys.global.add.noftz.f16 [%0], %1;" ::"l"(p), "h"(*(uint16_t*)&h) : "memory");
}
template <> IRIS_D void red_add<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  __nv_bfloat16 h = __float2bfloat16_rn(v);
  asm volatile("red.relaxed.sys.global.add.noftz.bf16 [%0], %1;" ::"l"(p), "h"(*(uint16_t*)&h) : "memory");
}

// Iterate the in-bounds elements of a tile with the CTA's threads.
template <class T, class F>
IRIS_D void for_each(const TensorView<T>& v, const TileView& t, F f) {
  const int rows = min(t.block_m, v.M - t.row0()), cols = min(t.block_n, v.N - t.col0());
  if (rows <= 0 || cols <= 0) return;
  for (int i = threadIdx.x; i < rows * cols; i += blockDim.x) {
    const int r = i / cols, c = i - r * cols;
    f(t.row0() + r, t.col0() + c);
  }
}

// One elected thread waits for `*flag >= target` on rank `r`'s copy; the CTA gets the verdict.
IRIS_D bool cta_wait_remote(const DeviceContext& ctx, int32_t* flag, int r, int32_t target) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = wait_flag_ge(ctx, ctx.remote(flag, r), target) ? 1 : 0;
  __syncthreads();
  const bool ok = s_ok != 0;
  __syncthreads();
  return ok;
}

template <class T>
IRIS_D void all_reduce_atomic(const DeviceContext& ctx, const TileView& t, const TensorView<T>& src, const TensorView<T>& dst) {
  for_each(src, t, [&](int r, int c) {
    const float v = to_f32(*src.at(r, c));
    for (int k = 0; k < ctx.world; ++k) red_add<T>(ctx.remote(dst.at(r, c), k), v);
  });
}

// locks: int32[tiles] on the heap, 0 = free. tile_id indexes it.
template <class T>
IRIS_D bool all_reduce_spinlock(const DeviceContext& ctx, const TileView& t, int tile_id, const TensorView<T>& src,
                                const TensorView<T>& dst, int32_t* locks) {
  __shared__ int s_ok;
  for (int k = 0; k < ctx.world; ++k) {
    int rr = ctx.rank + k;
    if (rr >= ctx.world) rr -= ctx.world;
    int32_t* lock = ctx.remote(locks + tile_id, rr);
    if (threadIdx.x == 0) {
      const uint64_t t0 = now_ns();
      int ok = 1;
      while (atomicCAS_system((int*)lock, 0, 1) != 0) {
        if (now_ns() - t0 > ctx.timeout_ns) { ok = 0; ctx.fail(kTimeoutLock); break; }
        __nanosleep(100);
      }
      fence_sys();
      s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return false;
    for_each(src, t, [&](int r, int c) {
      T* d = ctx.remote(dst.at(r, c), rr);
      const float cur = to_f32(detail::bit_cast<T>(detail::ld_raw<CacheOp::cv, false>((const typename detail::Bits<sizeof(T)>::type*)d)));
      *d = from_f32<T>(cur + to_f32(*src.at(r, c)));
    });
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_sys();
      atomicExch_system((int*)lock, 0);
    }
    __syncthreads();
  }
  return true;
}

// Every rank has published `locks[tile_id] >= ready` after writing its tile of `src`.
template <class T>
IRIS_D bool all_reduce_one_shot(const DeviceContext& ctx, const TileView& t, int tile_id, const TensorView<T>& src,
                                const TensorView<T>& dst, int32_t* locks, int32_t ready = 1) {
  for (int k = 0; k < ctx.world; ++k)
    if (!cta_wait_remote(ctx, locks + tile_id, k, ready)) return false;
  for_each(src, t, [&](int r, int c) {
    float acc = 0.f;
    for (int k = 0; k < ctx.world; ++k) acc += to_f32(*ctx.remote(src.at(r, c), k));
    *dst.at(r, c) = from_f32<T>(acc);
  });
  return true;
}

// Owner of the tile (tile_id % W) reduces and stores the result on every rank; others skip.
template <class T>
IRIS_D bool all_reduce_two_shot(const DeviceContext& ctx, const TileView& t, int tile_id, const TensorView<T>& src,
                                const TensorView<T>& dst, int32_t* locks, int32_t ready = 1) {
  if (tile_id % ctx.world != ctx.rank) return true;
  for (int k = 0; k < ctx.world; ++k)
    if (!cta_wait_remote(ctx, locks + tile_id, k, ready)) return false;
  for_each(src, t, [&](int r, int c) {
    float acc = 0.f;
    for (int k = 0; k < ctx.world; ++k) acc += to_f32(*ctx.remote(src.at(r, c), k));
    const T o = from_f32<T>(acc);
    for (int k = 0; k < ctx.world; ++k) *ctx.remote(dst.at(r, c), k) = o;
  });
  return true;
}

// dim 0: my (M_local x N) tile lands at row offset rank*M_local of every rank's dst; dim 1: columns.
template <class T>
IRIS_D void all_gather(const DeviceContext& ctx, const TileView& t, const TensorView<T>& src, const TensorView<T>& dst, int dim) {
  const int ro = dim == 0 ? ctx.rank * src.M : 0, co = dim == 0 ? 0 : ctx.rank * src.N;
  for_each(src, t, [&](int r, int c) {
    const T v = *src.at(r, c);
    for (int k = 0; k < ctx.world; ++k) *ctx.remote(dst.at(r + ro, c + co), k) = v;
  });
}

// Pull `source_rank`'s tile of `src` into the local `out` (same coordinates).
template <class T>
IRIS_D void gather(const DeviceContext& ctx, const TileView& t, const TensorView<T>& src, const TensorView<T>& out, int source_rank) {
  for_each(src, t, [&](int r, int c) { *out.at(r, c) = *ctx.remote(src.at(r, c), source_rank); });
}

// src and dst are (M, N*W); the tile indexes the (M, N) chunk grid. Chunk d of my src goes to
// chunk `rank` of rank d's dst.
template <class T>
IRIS_D void all_to_all(const DeviceContext& ctx, const TileView& t, const TensorView<T>& src, const TensorView<T>& dst, int N_chunk) {
  TensorView<T> chunk_view{src.ptr, src.M, N_chunk, src.stride_m, src.stride_n};
  for_each(chunk_view, t, [&](int r, int c) {
    for (int d = 0; d < ctx.world; ++d)
      *ctx.remote(dst.at(r, ctx.rank * N_chunk + c), d) = *src.at(r, d * N_chunk + c);
  });
}

// Contiguous tile blocks of total/W per rank, last rank takes the remainder (row-major tile ids).
IRIS_HD int reduce_scatter_owner(int tile_id, int total_tiles, int world) {
  int per = total_tiles / world;
  if (per < 1) per = 1;
  int o = tile_id / per;
  return o >= world ? world - 1 : o;
}
template <class T>
IRIS_D bool reduce_scatter(const DeviceContext& ctx, const TileView& t, int tile_id, int total_tiles, const TensorView<T>& src,
                           const TensorView<T>& dst, int32_t* locks, int32_t ready = 1) {
  if (reduce_scatter_owner(tile_id, total_tiles, ctx.world) != ctx.rank) return true;
  for (int k = 0; k < ctx.world; ++k)
    if (!cta_wait_remote(ctx, locks + tile_id, k, ready)) return false;
  for_each(src, t, [&](int r, int c) {
    float acc = 0.f;
    for (int k = 0; k < ctx.world; ++k) acc += to_f32(*ctx.remote(src.at(r, c), k));
    *dst.at(r, c) = from_f32<T>(acc);
  });
  return true;
}

}  // namespace tile
}  // namespace iris
#endif
