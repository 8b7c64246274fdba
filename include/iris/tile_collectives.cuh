// Tile-level collectives for use INSIDE user kernels: one CTA moves or reduces one BLOCK_M x
// BLOCK_N tile of a row-major matrix that lives at the same heap offset on every rank.
// Same set and same ownership rules as the methods of the reference's DeviceContext
// (iris/mem/triton/context.py:687-997):
//   all_reduce_atomic     add my tile into every rank's destination (destination pre-zeroed)
//   all_reduce_spinlock   per-(tile, destination) lock, read-modify-write under the lock
//   all_reduce_one_shot   wait for every rank's "tile ready" lock, pull all W copies, sum, store
//   all_reduce_ring       pull the peers' copies in ring order (rank-1, rank-2, ...), sum, store
//   all_reduce_two_shot   owner (tile_id % W) pulls and sums, then stores the result to all ranks
//   all_gather            store my tile into every rank's destination at my rank's row/col block
//   gather                pull one rank's tile into local memory
//   all_to_all            exchange column chunks of a tile row block
//   reduce_scatter        owner of contiguous tile blocks (last rank takes the remainder) pulls+sums
// All threads of the CTA call the function. Waits are bounded (ctx.timeout_ns) and return false
// after recording a status; accumulation is fp32. Tiles whose rows are contiguous, start on a
// 16-byte boundary and are a whole number of 16-byte groups wide move 16 bytes per thread and access
// (vec_ok / for_each_vec); anything else takes the element-wise loop.
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

// 16-byte path: the tile's in-bounds part as rows of whole 16-byte groups (V elements each).
template <class T>
IRIS_D bool vec_ok(const TensorView<T>& v, const TileView& t) {
  constexpr int V = 16 / (int)sizeof(T);
  const int cols = min(t.block_n, v.N - t.col0());
  return v.stride_n == 1 && cols > 0 && cols % V == 0 && t.col0() % V == 0 && v.stride_m % V == 0 &&
         ((uintptr_t)v.ptr & 15) == 0;
}
template <class T, class F>
IRIS_D void for_each_vec(const TensorView<T>& v, const TileView& t, F f) {      // f(row, first column of the group)
  constexpr int V = 16 / (int)sizeof(T);
  const int rows = min(t.block_m, v.M - t.row0()), groups = min(t.block_n, v.N - t.col0()) / V;
  if (rows <= 0 || groups <= 0) return;
  for (int i = threadIdx.x; i < rows * groups; i += blockDim.x) {
    const int r = i / groups, g = i - r * groups;
    f(t.row0() + r, t.col0() + g * V);
  }
}
template <class T> struct alignas(16) Vec16 { T e[16 / sizeof(T)]; };
// Sum over the ranks (visited from `first`, stepping by `step` modulo W) of the 16-byte group at `p`.
template <class T>
IRIS_D Vec16<T> pull_sum_vec(const DeviceContext& ctx, const T* p, int first, int step) {
  constexpr int V = 16 / (int)sizeof(T);
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.f;
  int k = first;
  for (int n = 0; n < ctx.world; ++n) {
    const Vec16<T> x = *(const Vec16<T>*)ctx.remote(p, k);
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] += to_f32(x.e[j]);
    k += step;
    if (k >= ctx.world) k -= ctx.world;
    if (k < 0) k += ctx.world;
  }
  Vec16<T> o;
#pragma unroll
  for (int j = 0; j < V; ++j) o.e[j] = from_f32<T>(acc[j]);
  return o;
}
// dst tile = sum over ranks of the src tile (pulled), ranks visited from `first` with `step`.
template <class T>
IRIS_D void pull_sum_tile(const DeviceContext& ctx, const TileView& t, const TensorView<T>& src, const TensorView<T>& dst, int first,
                          int step, bool store_all) {
  if (vec_ok(src, t) && vec_ok(dst, t)) {
    for_each_vec(src, t, [&](int r, int c) {
      const Vec16<T> o = pull_sum_vec(ctx, src.at(r, c), first, step);
      if (store_all) {
        for (int k = 0; k < ctx.world; ++k) *(Vec16<T>*)ctx.remote(dst.at(r, c), k) = o;
      } else {
        *(Vec16<T>*)dst.at(r, c) = o;
      }
    });
    return;
  }
  for_each(src, t, [&](int r, int c) {
    float acc = 0.f;
    int k = first;
    for (int n = 0; n < ctx.world; ++n) {
      acc += to_f32(*ctx.remote(src.at(r, c), k));
      k += step;
      if (k >= ctx.world) k -= ctx.world;
      if (k < 0) k += ctx.world;
    }
    const T o = from_f32<T>(acc);
    if (store_all) {
      for (int k2 = 0; k2 < ctx.world; ++k2) *ctx.remote(dst.at(r, c), k2) = o;
    } else {
      *dst.at(r, c) = o;
    }
  });
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
  pull_sum_tile(ctx, t, src, dst, 0, 1, false);
  return true;
}

// Ring order (reference: iris/mem/triton/context.py:767-800): start from this rank's own copy and walk
// the ring backwards (rank - 1, rank - 2, ...), so that at any moment the W ranks read from W different
// peers; the sum is stored locally. The reference's second loop re-reads the peers' results, which are
// the same sum; it is left out.
template <class T>
IRIS_D bool all_reduce_ring(const DeviceContext& ctx, const TileView& t, int tile_id, const TensorView<T>& src,
                            const TensorView<T>& dst, int32_t* locks, int32_t ready = 1) {
  for (int k = 0; k < ctx.world; ++k) {
    int rr = ctx.rank - k;
    if (rr < 0) rr += ctx.world;
    if (!cta_wait_remote(ctx, locks + tile_id, rr, ready)) return false;
  }
  pull_sum_tile(ctx, t, src, dst, ctx.rank, -1, false);
  return true;
}

// Owner of the tile (tile_id % W) reduces and stores the result on every rank; others skip.
template <class T>
IRIS_D bool all_reduce_two_shot(const DeviceContext& ctx, const TileView& t, int tile_id, const TensorView<T>& src,
                                const TensorView<T>& dst, int32_t* locks, int32_t ready = 1) {
  if (tile_id % ctx.world != ctx.rank) return true;
  for (int k = 0; k < ctx.world; ++k)
    if (!cta_wait_remote(ctx, locks + tile_id, k, ready)) return false;
  pull_sum_tile(ctx, t, src, dst, 0, 1, true);
  return true;
}

// dim 0: my (M_local x N) tile lands at row offset rank*M_local of every rank's dst; dim 1: columns.
template <class T>
IRIS_D void all_gather(const DeviceContext& ctx, const TileView& t, const TensorView<T>& src, const TensorView<T>& dst, int dim) {
  const int ro = dim == 0 ? ctx.rank * src.M : 0, co = dim == 0 ? 0 : ctx.rank * src.N;
  constexpr int V = 16 / (int)sizeof(T);
  if (vec_ok(src, t) && dst.stride_n == 1 && dst.stride_m % V == 0 && co % V == 0 && ((uintptr_t)dst.ptr & 15) == 0) {
    for_each_vec(src, t, [&](int r, int c) {
      const Vec16<T> v = *(const Vec16<T>*)src.at(r, c);
      for (int k = 0; k < ctx.world; ++k) *(Vec16<T>*)ctx.remote(dst.at(r + ro, c + co), k) = v;
    });
    return;
  }
  for_each(src, t, [&](int r, int c) {
    const T v = *src.at(r, c);
    for (int k = 0; k < ctx.world; ++k) *ctx.remote(dst.at(r + ro, c + co), k) = v;
  });
}

// Pull `source_rank`'s tile of `src` into the local `out` (same coordinates).
template <class T>
IRIS_D void gather(const DeviceContext& ctx, const TileView& t, const TensorView<T>& src, const TensorView<T>& out, int source_rank) {
  if (vec_ok(src, t) && vec_ok(out, t)) {
    for_each_vec(src, t, [&](int r, int c) { *(Vec16<T>*)out.at(r, c) = *(const Vec16<T>*)ctx.remote(src.at(r, c), source_rank); });
    return;
  }
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
  pull_sum_tile(ctx, t, src, dst, 0, 1, false);
  return true;
}

}  // namespace tile
}  // namespace iris
#endif
