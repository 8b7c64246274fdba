// Collectives over the symmetric heap, each ONE persistent kernel that synchronises with its
// peers on the device: an entry round (every rank's input is final and its output may be
// written), the data movement over NVLink (peer loads / stores, or NVLS multimem through the
// switch), and an exit round run by the last CTA (every peer's stores into this rank have landed).
// The reference's kernels (iris/ccl/triton/*.py) move the same tiles but lean on a host barrier
// before and after each call; here no host synchronisation is involved.
//
//   all_gather      in (M,N) -> out (W*M, N), rank r's rows at [r*M, (r+1)*M)
//   all_to_all      in/out (M, N*W): column chunk d of rank s lands in column chunk s of rank d
//   all_reduce      in/out (M,N), SUM, fp32 accumulation (int32 for integers); variants atomic,
//                   spinlock, one_shot, two_shot, ring and nvls
//   reduce_scatter  out has the full (M,N) shape and a rank writes only the tiles it owns
//                   (block or strided distribution of BLOCK_M x BLOCK_N tiles), or, with
//                   `rows`, out is (M/W, N) holding this rank's row block of the sum
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <string.h>

#include "iris/host_api.h"
#include "iris/iris.cuh"

using namespace iris;

namespace {

constexpr int kThreads = 512;

struct CclArgs {
  DeviceContext ctx;
  SyncBlock* sb;
  const uint8_t* in;     // heap
  uint8_t* out;          // heap
  int M, N;              // all_gather/all_reduce/reduce_scatter: shape of `in`; all_to_all: chunk is (M, N)
  long long ld_in, ld_out;  // row pitches in elements
  int variant;
  int use_mc;
  int block_m, block_n, distribution, swizzle;  // reduce_scatter tile ownership
  uint8_t* ring_buf;     // ring: [2*(W-1)][slice bytes] on the heap
  int32_t* flags;        // ring: [2*(W-1)][ctas]; spinlock: [tiles]
  int rows_mode;         // reduce_scatter: 1 = row-block semantics
};

// ---- element helpers -------------------------------------------------------------------------
template <class T> struct Acc { using type = float; };
template <> struct Acc<int32_t> { using type = int32_t; };

template <class T> __device__ __forceinline__ typename Acc<T>::type to_acc(T v);
template <> __device__ __forceinline__ float to_acc<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ int32_t to_acc<int32_t>(int32_t v) { return v; }
template <class T> __device__ __forceinline__ T from_acc(typename Acc<T>::type v);
template <> __device__ __forceinline__ float from_acc<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_acc<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ int32_t from_acc<int32_t>(int32_t v) { return v; }

// A "unit" is 16 bytes when the rows allow it (VEC = 16 / sizeof(T) elements), else one element.
template <class T, int VEC> struct Unit;
template <class T> struct Unit<T, 1> {
  T v;
  using A = typename Acc<T>::type;
  __device__ __forceinline__ void accumulate(A* acc) const { acc[0] += to_acc<T>(v); }
  __device__ __forceinline__ static Unit pack(const A* acc) { return Unit{from_acc<T>(acc[0])}; }
};
template <class T, int VEC> struct Unit {
  uint4 raw;
  using A = typename Acc<T>::type;
  __device__ __forceinline__ void accumulate(A* acc) const {
    const T* e = (const T*)&raw;
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] += to_acc<T>(e[i]);
  }
  __device__ __forceinline__ static Unit pack(const A* acc) {
    Unit u;
    T* e = (T*)&u.raw;
#pragma unroll
    for (int i = 0; i < VEC; ++i) e[i] = from_acc<T>(acc[i]);
    return u;
  }
};

// Address of unit `u` of a row-major (rows x units_per_row) matrix with pitch `ld` elements.
template <class T, int VEC>
__device__ __forceinline__ Unit<T, VEC>* unit_ptr(const uint8_t* base, long long ld, int units_per_row, size_t u) {
  const size_t r = u / units_per_row, c = u - r * units_per_row;
  return (Unit<T, VEC>*)(base + ((size_t)r * ld + c * VEC) * sizeof(T));
}

// Uncached load of one unit (data another GPU may have just written under a lock).
template <class UT>
__device__ __forceinline__ UT load_unit_cv(const UT* p) {
  UT u;
  if constexpr (sizeof(UT) == 16) { uint4 v = __ldcv((const uint4*)p); memcpy(&u, &v, 16); }
  else if constexpr (sizeof(UT) == 4) { unsigned v = __ldcv((const unsigned*)p); memcpy(&u, &v, 4); }
  else { unsigned short v = __ldcv((const unsigned short*)p); memcpy(&u, &v, 2); }
  return u;
}

// Strided loop with kUnroll independent loads in flight per thread before the first store:
// `ld(u)` returns the value of unit u, `st(u, v)` consumes it. One NVLink round trip then covers
// kUnroll x 16 bytes per thread instead of 16.
template <int kUnroll, class V, class LD, class ST>
__device__ __forceinline__ void pipelined_loop(size_t first, size_t total, size_t stride, LD ld, ST st) {
  size_t u = first;
  for (; u + (kUnroll - 1) * stride < total; u += kUnroll * stride) {
    V v[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) v[k] = ld(u + k * stride);
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) st(u + k * stride, v[k]);
  }
  for (; u < total; u += stride) st(u, ld(u));
}

__device__ __forceinline__ int peer_of(const DeviceContext& ctx, int i) {  // i-th peer after me
  int r = ctx.rank + i;
  return r >= ctx.world ? r - ctx.world : r;
}

// ---- all_gather ------------------------------------------------------------------------------
// variant 0 "persistent": every CTA walks its share of the input and stores each unit to all
// ranks, starting with its right neighbour (destinations staggered across ranks).
// variant 1 "partitioned": CTAs are split over destinations, each pushes the whole input to one.
// use_mc: one multimem.st per unit reaches every rank through the switch.
template <int UB>
__global__ void __launch_bounds__(kThreads) all_gather_kernel(const __grid_constant__ CclArgs a) {
  using U = typename std::conditional<UB == 16, uint4, uint8_t>::type;
  const DeviceContext& ctx = a.ctx;
  const int32_t e0 = read_epoch(a.sb);
  const int W = ctx.world;
  if (!grid_entry_barrier(ctx, a.sb, e0)) { grid_exit_barrier(ctx, a.sb, e0, 1); return; }
  // element size travels in block_m (reused) for byte-typed movers
  const int esize = a.block_m;
  const size_t upr = (size_t)a.N * esize / UB;          // units per row
  const size_t total = (size_t)a.M * upr;
  const size_t in_pitch = (size_t)a.ld_in * esize, out_pitch = (size_t)a.ld_out * esize;
  uint8_t* out_mine = a.out + (size_t)ctx.rank * a.M * out_pitch;  // my row block inside `out`
  const int mode = a.block_n;  // 0 persistent, 1 partitioned
  if (a.use_mc) {
    uint8_t* dst = ctx.mc(out_mine);
    if constexpr (UB == 16) {
      pipelined_loop<8, uint4>((size_t)blockIdx.x * blockDim.x + threadIdx.x, total, (size_t)gridDim.x * blockDim.x,
          [&](size_t u) { const size_t r = u / upr, c = u - r * upr; return *(const uint4*)(a.in + r * in_pitch + c * 16); },
          [&](size_t u, uint4 v) {
            const size_t r = u / upr, c = u - r * upr;
            multimem::st_v4(dst + r * out_pitch + c * 16, multimem::V4{v.x, v.y, v.z, v.w});
          });
    }
  } else if (mode == 1 && (int)gridDim.x >= W) {
    const int per = gridDim.x / W;
    const int d = blockIdx.x / per;
    if (d < W) {
      const int dst_rank = peer_of(ctx, d);
      uint8_t* dst = ctx.remote(out_mine, dst_rank);
      const int j = blockIdx.x - d * per;
      pipelined_loop<8, U>((size_t)j * blockDim.x + threadIdx.x, total, (size_t)per * blockDim.x,
          [&](size_t u) { const size_t r = u / upr, c = u - r * upr; return *(const U*)(a.in + r * in_pitch + c * UB); },
          [&](size_t u, U v) { const size_t r = u / upr, c = u - r * upr; *(U*)(dst + r * out_pitch + c * UB) = v; });
    }
  } else {
    pipelined_loop<8, U>((size_t)blockIdx.x * blockDim.x + threadIdx.x, total, (size_t)gridDim.x * blockDim.x,
        [&](size_t u) { const size_t r = u / upr, c = u - r * upr; return *(const U*)(a.in + r * in_pitch + c * UB); },
        [&](size_t u, U v) {
          const size_t r = u / upr, c = u - r * upr;
          for (int i = 1; i <= W; ++i) {
            const int dst_rank = peer_of(ctx, i == W ? 0 : i);
            *(U*)(ctx.remote(out_mine, dst_rank) + r * out_pitch + c * UB) = v;
          }
        });
  }
  grid_exit_barrier(ctx, a.sb, e0, 1);
}

// ---- all_to_all ------------------------------------------------------------------------------
// Push: my column chunk d goes to column chunk `rank` of rank d. CTAs are spread over
// destinations so that all links are busy at once.
template <int UB>
__global__ void __launch_bounds__(kThreads) all_to_all_kernel(const __grid_constant__ CclArgs a) {
  using U = typename std::conditional<UB == 16, uint4, uint8_t>::type;
  const DeviceContext& ctx = a.ctx;
  const int32_t e0 = read_epoch(a.sb);
  const int W = ctx.world;
  if (!grid_entry_barrier(ctx, a.sb, e0)) { grid_exit_barrier(ctx, a.sb, e0, 1); return; }
  const int esize = a.block_m;
  const size_t upr = (size_t)a.N * esize / UB;  // units per chunk row
  const size_t total = (size_t)a.M * upr;
  const size_t in_pitch = (size_t)a.ld_in * esize, out_pitch = (size_t)a.ld_out * esize;
  const size_t chunk_bytes = (size_t)a.N * esize;
  const int per = max(1, (int)gridDim.x / W);
  for (int d0 = blockIdx.x / per; d0 < W; d0 += max(1, (int)gridDim.x / per)) {
    const int dst_rank = peer_of(ctx, d0);
    const uint8_t* src = a.in + (size_t)dst_rank * chunk_bytes;
    uint8_t* dst = ctx.remote(a.out, dst_rank) + (size_t)ctx.rank * chunk_bytes;
    const int j = blockIdx.x % per;
    pipelined_loop<8, U>((size_t)j * blockDim.x + threadIdx.x, total, (size_t)per * blockDim.x,
        [&](size_t u) { const size_t r = u / upr, c = u - r * upr; return *(const U*)(src + r * in_pitch + c * UB); },
        [&](size_t u, U v) { const size_t r = u / upr, c = u - r * upr; *(U*)(dst + r * out_pitch + c * UB) = v; });
  }
  grid_exit_barrier(ctx, a.sb, e0, 1);
}

// ---- all_reduce ------------------------------------------------------------------------------
enum ArVariant { kArAtomic = 0, kArRing = 1, kArOneShot = 2, kArTwoShot = 3, kArSpinlock = 4, kArNvls = 5, kArPush = 6 };

template <class T, int VEC>
__device__ __forceinline__ void reduce_unit_from_all(const CclArgs& a, size_t u, int upr, typename Acc<T>::type* acc, int start) {
  const DeviceContext& ctx = a.ctx;
  Unit<T, VEC> v[8];
  // issue the loads of up to 8 ranks before the first add (W-1 of them cross NVLink)
  for (int base = 0; base < ctx.world; base += 8) {
    const int cnt = min(8, ctx.world - base);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < cnt) {
        int r = start + base + i;
        r %= ctx.world;
        v[i] = *unit_ptr<T, VEC>(ctx.remote(a.in, r), a.ld_in, upr, u);
      }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < cnt) v[i].accumulate(acc);
  }
}

template <class T, int VEC>
__device__ void store_unit_everywhere(const CclArgs& a, size_t u, int upr, const Unit<T, VEC>& v) {
  const DeviceContext& ctx = a.ctx;
  Unit<T, VEC>* local = unit_ptr<T, VEC>(a.out, a.ld_out, upr, u);
  if constexpr (VEC > 1) {
    if (a.use_mc) {
      multimem::V4 m{v.raw.x, v.raw.y, v.raw.z, v.raw.w};
      multimem::st_v4(ctx.mc((uint8_t*)local), m);
      return;
    }
  }
  *local = v;
  for (int i = 1; i < ctx.world; ++i) *ctx.remote(local, peer_of(ctx, i)) = v;
}

template <class T> __device__ __forceinline__ void red_add_remote(T* p, T v);
template <> __device__ __forceinline__ void red_add_remote<float>(float* p, float v) {
  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
template <> __device__ __forceinline__ void red_add_remote<int32_t>(int32_t* p, int32_t v) {
  asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
template <> __device__ __forceinline__ void red_add_remote<__half>(__half* p, __half v) {
  asm volatile("red.relaxed.sys.global.add.noftz.f16 [%0], %1;" ::"l"(p), "h"(*(uint16_t*)&v) : "memory");
}
template <> __device__ __forceinline__ void red_add_remote<__nv_bfloat16>(__nv_bfloat16* p, __nv_bfloat16 v) {
  asm volatile("red.relaxed.sys.global.add.noftz.bf16 [%0], %1;" ::"l"(p), "h"(*(uint16_t*)&v) : "memory");
}

template <class T, int VEC>
__device__ __forceinline__ Unit<T, VEC> nvls_reduce(const void* mc_ptr) {
  Unit<T, VEC> u;
  if constexpr (VEC > 1) {
    multimem::V4 v;
    if constexpr (std::is_same<T, __nv_bfloat16>::value) v = multimem::ld_reduce_bf16x8(mc_ptr);
    else if constexpr (std::is_same<T, __half>::value) v = multimem::ld_reduce_f16x8(mc_ptr);
    else v = multimem::ld_reduce_f32x4(mc_ptr);
    u.raw = make_uint4(v.x, v.y, v.z, v.w);
  }
  return u;
}

template <class T, int VEC>
__global__ void __launch_bounds__(kThreads) all_reduce_kernel(const __grid_constant__ CclArgs a) {
  using A = typename Acc<T>::type;
  using UT = Unit<T, VEC>;
  const DeviceContext& ctx = a.ctx;
  const int W = ctx.world;
  const int32_t e0 = read_epoch(a.sb);
  const int upr = a.N / VEC;
  const size_t total = (size_t)a.M * upr;
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, gstride = (size_t)gridDim.x * blockDim.x;

  if (a.variant == kArAtomic) {
    // zero my output, then everyone adds its input into every rank's output
    for (size_t u = gtid; u < total; u += gstride) {
      A z[VEC] = {};
      *unit_ptr<T, VEC>(a.out, a.ld_out, upr, u) = UT::pack(z);
    }
    // every CTA's zeroes must be in place before CTA 0 tells the peers that they may add
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      atomicAdd(&a.sb->aux[0], 1);
      if (blockIdx.x == 0) {
        const uint64_t t0 = now_ns();
        while (*(volatile int32_t*)&a.sb->aux[0] < (int)gridDim.x) {
          if (now_ns() - t0 > ctx.timeout_ns) { ctx.fail(kTimeoutBarrier); break; }
        }
        a.sb->aux[0] = 0;
        __threadfence_system();
      }
    }
    __syncthreads();
  }
  if (!grid_entry_barrier(ctx, a.sb, e0)) { grid_exit_barrier(ctx, a.sb, e0, 1); return; }

  if (a.variant == kArOneShot) {
    for (size_t u = gtid; u < total; u += gstride) {
      A acc[VEC] = {};
      reduce_unit_from_all<T, VEC>(a, u, upr, acc, ctx.rank);
      *unit_ptr<T, VEC>(a.out, a.ld_out, upr, u) = UT::pack(acc);
    }
  } else if (a.variant == kArTwoShot || a.variant == kArNvls) {
    // this rank owns the units [lo, hi); start the pulls at a CTA-dependent rank to spread load
    const size_t lo = total * ctx.rank / W, hi = total * (ctx.rank + 1) / W;
    bool nvls_done = false;
    if constexpr (VEC > 1 && !std::is_same<T, int32_t>::value) {
      if (a.variant == kArNvls) {
        // reduce in the switch (one multimem.ld_reduce per 16 bytes, 4 in flight), broadcast back
        pipelined_loop<4, UT>(lo + gtid, hi, gstride,
            [&](size_t u) { return nvls_reduce<T, VEC>(ctx.mc((const uint8_t*)unit_ptr<T, VEC>(a.in, a.ld_in, upr, u))); },
            [&](size_t u, UT r) { store_unit_everywhere<T, VEC>(a, u, upr, r); });
        nvls_done = true;
      }
    }
    for (size_t u = lo + gtid; u < hi && !nvls_done; u += gstride) {
      UT r;
      if constexpr (VEC > 1 && !std::is_same<T, int32_t>::value) {
        if (a.variant == kArNvls) {
          r = nvls_reduce<T, VEC>(ctx.mc((const uint8_t*)unit_ptr<T, VEC>(a.in, a.ld_in, upr, u)));
          store_unit_everywhere<T, VEC>(a, u, upr, r);
          continue;
        }
      }
      A acc[VEC] = {};
      reduce_unit_from_all<T, VEC>(a, u, upr, acc, ctx.rank + blockIdx.x);
      r = UT::pack(acc);
      store_unit_everywhere<T, VEC>(a, u, upr, r);
    }
  } else if (a.variant == kArAtomic) {
    for (size_t u = gtid; u < total; u += gstride) {
      const UT v = *unit_ptr<T, VEC>(a.in, a.ld_in, upr, u);
      const T* e = (const T*)&v;
      T* dst0 = (T*)unit_ptr<T, VEC>(a.out, a.ld_out, upr, u);
      for (int i = 0; i < W; ++i) {
        T* dst = ctx.remote(dst0, peer_of(ctx, i));
#pragma unroll
        for (int k = 0; k < VEC; ++k) red_add_remote<T>(dst + k, e[k]);
      }
    }
  } else if (a.variant == kArSpinlock) {
    // One lock per 256-unit segment on the destination; a CTA takes the lock (CAS acquire,
    // bounded), adds its segment (read-modify-write) and releases it (exchange, release).
    // The output starts as the owner's own input: each rank first copies in -> out locally,
    // guarded by the same lock protocol through the entry round below.
    const size_t seg = 256;
    const size_t nseg = (total + seg - 1) / seg;
    __shared__ int s_ok;
    for (int i = 0; i < W; ++i) {
      const int dst_rank = peer_of(ctx, i);
      for (size_t sgi = blockIdx.x; sgi < nseg; sgi += gridDim.x) {
        int32_t* lock = ctx.remote(a.flags + sgi, dst_rank);
        if (threadIdx.x == 0) {
          const uint64_t t0 = now_ns();
          int ok = 1;
          unsigned n = 0;
          while (atomicCAS_system((int*)lock, 0, 1) != 0) {
            if ((++n & 15u) == 0 && now_ns() - t0 > ctx.timeout_ns) { ok = 0; ctx.fail(kTimeoutLock); break; }
            __nanosleep(100);
          }
          fence_sys();
          s_ok = ok;
        }
        __syncthreads();
        const bool ok = s_ok != 0;
        if (ok) {
          const size_t u = sgi * seg + threadIdx.x;
          if (threadIdx.x < seg && u < total) {
            const UT v = *unit_ptr<T, VEC>(a.in, a.ld_in, upr, u);
            UT* dst = ctx.remote(unit_ptr<T, VEC>(a.out, a.ld_out, upr, u), dst_rank);
            // aux[0] of the destination's sync block holds nothing; first writer is detected by a
            // per-segment "touched" count kept in the upper half of the flags array
            int32_t* touched = ctx.remote(a.flags + nseg + sgi, dst_rank);
            const int first = *(volatile int32_t*)touched == 0;
            A acc[VEC] = {};
            if (!first) load_unit_cv(dst).accumulate(acc);
            v.accumulate(acc);
            *dst = UT::pack(acc);
          }
        }
        __syncthreads();
        if (threadIdx.x == 0 && ok) {
          int32_t* touched = ctx.remote(a.flags + nseg + sgi, dst_rank);
          const int32_t t = *(volatile int32_t*)touched + 1;
          *(volatile int32_t*)touched = t == W ? 0 : t;  // last contributor resets for the next call
          fence_sys();
          atomicExch_system((int*)lock, 0);
        }
        __syncthreads();
      }
    }
  } else if (a.variant == kArRing) {
    // Ring: W-1 reduce-scatter steps then W-1 all-gather steps; each step has its own receive
    // slot in `ring_buf` and its own per-CTA arrival counter, so nothing is reused within a call.
    const int steps = 2 * (W - 1);
    const size_t slice = (total + W - 1) / W;                 // units per slice
    const size_t per_cta = (slice + gridDim.x - 1) / gridDim.x;
    const size_t c_lo = (size_t)blockIdx.x * per_cta, c_hi = min(slice, c_lo + per_cta);
    const int next = peer_of(ctx, 1);
    const int32_t target = (e0 >> 1) + 1;
    UT* rb = (UT*)a.ring_buf;
    __shared__ int s_ok2;
    auto slice_of = [&](int s) { int k = (ctx.rank - s) % W; return k < 0 ? k + W : k; };
    auto unit_in = [&](int sl, size_t i) -> const UT* { return unit_ptr<T, VEC>(a.in, a.ld_in, upr, (size_t)sl * slice + i); };
    auto valid = [&](int sl, size_t i) { return (size_t)sl * slice + i < total; };
    // step 0 send: my own slice `rank`
    for (size_t i = c_lo + threadIdx.x; i < c_hi; i += blockDim.x)
      if (valid(slice_of(0), i)) ctx.remote(rb, next)[(size_t)0 * slice + i] = *unit_in(slice_of(0), i);
    __syncthreads();
    if (threadIdx.x == 0) { fence_sys(); red_release_sys_add(ctx.remote(a.flags + 0 * gridDim.x + blockIdx.x, next), 1); }
    bool alive = true;
    for (int s = 0; s < steps && alive; ++s) {
      if (threadIdx.x == 0) s_ok2 = wait_flag_ge(ctx, a.flags + (size_t)s * gridDim.x + blockIdx.x, target) ? 1 : 0;
      __syncthreads();
      alive = s_ok2 != 0;
      __syncthreads();
      if (!alive) break;
      const bool rs_phase = s < W - 1;
      const int sl = slice_of(s + 1);  // slice that just arrived
      for (size_t i = c_lo + threadIdx.x; i < c_hi; i += blockDim.x) {
        if (!valid(sl, i)) continue;
        UT v = rb[(size_t)s * slice + i];
        if (rs_phase) {
          A acc[VEC] = {};
          v.accumulate(acc);
          unit_in(sl, i)->accumulate(acc);
          v = UT::pack(acc);
        }
        if (!rs_phase || s == W - 2) *unit_ptr<T, VEC>(a.out, a.ld_out, upr, (size_t)sl * slice + i) = v;
        if (s + 1 < steps) ctx.remote(rb, next)[(size_t)(s + 1) * slice + i] = v;
      }
      __syncthreads();
      if (threadIdx.x == 0 && s + 1 < steps) {
        fence_sys();
        red_release_sys_add(ctx.remote(a.flags + (size_t)(s + 1) * gridDim.x + blockIdx.x, next), 1);
      }
    }
  }
  grid_exit_barrier(ctx, a.sb, e0, 1);
}

// ---- all_reduce, one-shot push (latency path) -------------------------------------------------
// Every rank writes its whole (small) input into slot [rank] of every rank's staging area
// (multimem.st with NVLS, else one store per peer), raises a per-(source, CTA) counter there with
// release semantics (the counter is set to the call number), waits for the W counters of its own
// CTA index and sums the W slots locally.
// One NVLink traversal end to end, no entry or exit round: staging and counters are
// double-buffered by call parity, and seeing every source's counter in call k proves that all
// ranks left call k-1. ring_buf = staging [2][W][cap units], flags = [2][W][kPushMaxCtas],
// sb->aux[1] counts the calls.
constexpr int kPushMaxCtas = 32;
template <class T, int VEC>
__global__ void __launch_bounds__(kThreads) all_reduce_push_kernel(const __grid_constant__ CclArgs a, size_t cap_units) {
  using A = typename Acc<T>::type;
  using UT = Unit<T, VEC>;
  const DeviceContext& ctx = a.ctx;
  const int W = ctx.world;
  const int call = *(volatile int32_t*)&a.sb->aux[1];
  const int par = call & 1;
  const int32_t tag = (call >> 1) + 1;
  const int upr = a.N / VEC;
  const size_t total = (size_t)a.M * upr;
  const size_t per = (total + gridDim.x - 1) / gridDim.x;
  const size_t lo = min(total, (size_t)blockIdx.x * per), hi = min(total, lo + per);
  UT* stage = (UT*)a.ring_buf + (size_t)par * W * cap_units;
  UT* mine = stage + (size_t)ctx.rank * cap_units;
  for (size_t u = lo + threadIdx.x; u < hi; u += blockDim.x) {
    const UT v = *unit_ptr<T, VEC>(a.in, a.ld_in, upr, u);
    bool sent = false;
    if constexpr (VEC > 1) {
      if (a.use_mc) {
        multimem::st_v4(ctx.mc((uint8_t*)(mine + u)), multimem::V4{v.raw.x, v.raw.y, v.raw.z, v.raw.w});
        sent = true;
      }
    }
    if (!sent)
      for (int i = 0; i < W; ++i) *ctx.remote(mine + u, peer_of(ctx, i)) = v;
  }
  __syncthreads();
  int32_t* my_flag = a.flags + ((size_t)par * W + ctx.rank) * kPushMaxCtas + blockIdx.x;
  __shared__ int s_ok;
  if (threadIdx.x < 32) {
    // the flag carries the call number (one writer per flag), so CTA indices that were idle in
    // earlier, smaller calls need no catching up
    for (int r = threadIdx.x; r < W; r += 32) { fence_sys(); st_release_sys(ctx.remote(my_flag, r), tag); }
    bool ok = true;
    for (int r = threadIdx.x; r < W; r += 32)
      ok = wait_flag_ge(ctx, a.flags + ((size_t)par * W + r) * kPushMaxCtas + blockIdx.x, tag) && ok;
    ok = __all_sync(0xffffffffu, ok);
    if (threadIdx.x == 0) s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (s_ok) {
    for (size_t u = lo + threadIdx.x; u < hi; u += blockDim.x) {
      A acc[VEC] = {};
      for (int r = 0; r < W; ++r) load_unit_cv(stage + (size_t)r * cap_units + u).accumulate(acc);
      *unit_ptr<T, VEC>(a.out, a.ld_out, upr, u) = UT::pack(acc);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&a.sb->aux[2], 1) == (int)gridDim.x - 1) {
      a.sb->aux[2] = 0;
      a.sb->aux[1] = call + 1;
      __threadfence();
    }
  }
}

// ---- reduce_scatter --------------------------------------------------------------------------
// Tile ownership as in the reference (iris/ccl/triton/reduce_scatter.py:55-70): tiles are numbered
// row-major over (ceil(M/BM), ceil(N/BN)); distribution 0 = strided (tile % W == rank),
// 1 = contiguous blocks of ceil(T/W) tiles. The owner pulls the tile from all ranks, sums and
// writes it at the same position of its own output. rows_mode: plain row blocks into (M/W, N).
template <class T, int VEC>
__global__ void __launch_bounds__(kThreads) reduce_scatter_kernel(const __grid_constant__ CclArgs a) {
  using A = typename Acc<T>::type;
  using UT = Unit<T, VEC>;
  const DeviceContext& ctx = a.ctx;
  const int W = ctx.world;
  const int32_t e0 = read_epoch(a.sb);
  if (!grid_entry_barrier(ctx, a.sb, e0)) { grid_exit_barrier(ctx, a.sb, e0, 1); return; }
  const int upr = a.N / VEC;
  if (a.rows_mode) {
    const int rows = a.M / W;
    const size_t total = (size_t)rows * upr;
    const size_t base = (size_t)ctx.rank * rows * upr;
    const size_t first = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
    bool done = false;
    if constexpr (VEC > 1 && !std::is_same<T, int32_t>::value) {
      if (a.use_mc) {
        pipelined_loop<4, UT>(first, total, stride,
            [&](size_t u) { return nvls_reduce<T, VEC>(ctx.mc((const uint8_t*)unit_ptr<T, VEC>(a.in, a.ld_in, upr, base + u))); },
            [&](size_t u, UT r) { *unit_ptr<T, VEC>(a.out, a.ld_out, upr, u) = r; });
        done = true;
      }
    }
    if (!done) {
      // two units per thread and step: 2 x W independent peer loads in flight
      size_t u = first;
      for (; u + stride < total; u += 2 * stride) {
        A acc0[VEC] = {}, acc1[VEC] = {};
        reduce_unit_from_all<T, VEC>(a, base + u, upr, acc0, ctx.rank + blockIdx.x);
        reduce_unit_from_all<T, VEC>(a, base + u + stride, upr, acc1, ctx.rank + blockIdx.x);
        *unit_ptr<T, VEC>(a.out, a.ld_out, upr, u) = UT::pack(acc0);
        *unit_ptr<T, VEC>(a.out, a.ld_out, upr, u + stride) = UT::pack(acc1);
      }
      for (; u < total; u += stride) {
        A acc[VEC] = {};
        reduce_unit_from_all<T, VEC>(a, base + u, upr, acc, ctx.rank + blockIdx.x);
        *unit_ptr<T, VEC>(a.out, a.ld_out, upr, u) = UT::pack(acc);
      }
    }
  } else {
    const int tiles_m = (a.M + a.block_m - 1) / a.block_m, tiles_n = (a.N + a.block_n - 1) / a.block_n;
    const int T_total = tiles_m * tiles_n;
    const int per = (T_total + W - 1) / W;
    const int bn_units = a.block_n / VEC;
    for (int k = blockIdx.x;; k += gridDim.x) {
      int t;
      if (a.distribution == 0) t = ctx.rank + k * W;
      else t = ctx.rank * per + k;
      if (t >= T_total || (a.distribution != 0 && k >= per)) break;
      const int tm = t / tiles_n, tn = t % tiles_n;
      const int rows = min(a.block_m, a.M - tm * a.block_m);
      const int cu = min(bn_units, upr - tn * bn_units);
      for (int i = threadIdx.x; i < rows * cu; i += blockDim.x) {
        const int rr = i / cu, cc = i - rr * cu;
        const size_t u = (size_t)(tm * a.block_m + rr) * upr + (size_t)tn * bn_units + cc;
        A acc[VEC] = {};
        reduce_unit_from_all<T, VEC>(a, u, upr, acc, ctx.rank + blockIdx.x);
        *unit_ptr<T, VEC>(a.out, a.ld_out, upr, u) = UT::pack(acc);
      }
    }
  }
  grid_exit_barrier(ctx, a.sb, e0, 1);
}

template <class T>
int launch_reduce(const CclArgs& a, bool all_reduce, bool vec_ok, int grid, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  if (all_reduce) {
    if (vec_ok) all_reduce_kernel<T, V><<<grid, kThreads, 0, s>>>(a);
    else all_reduce_kernel<T, 1><<<grid, kThreads, 0, s>>>(a);
  } else {
    if (vec_ok) reduce_scatter_kernel<T, V><<<grid, kThreads, 0, s>>>(a);
    else reduce_scatter_kernel<T, 1><<<grid, kThreads, 0, s>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

extern "C" {

typedef struct IrisCclDesc {
  IrisCtx ctx;
  void* sync_block;
  const void* in;
  void* out;
  int32_t M, N;
  int64_t ld_in, ld_out;
  int32_t dtype;
  int32_t variant;       // all_gather: 0 persistent, 1 partitioned; all_reduce: ArVariant
  int32_t use_mc;
  int32_t comm_sms;
  int32_t block_m, block_n, distribution, swizzle;
  void* ring_buf;
  int32_t* flags;
  int32_t rows_mode;
  int32_t reserved;
} IrisCclDesc;

static int esize_of(int dtype) {
  switch (dtype) {
    case IRIS_F16: case IRIS_BF16: return 2;
    case IRIS_F32: case IRIS_I32: return 4;
    case IRIS_I8: case IRIS_F8E4M3: return 1;
    case IRIS_I64: return 8;
    default: return 0;
  }
}

static void fill_args(CclArgs& a, const IrisCclDesc* d) {
  memcpy(&a.ctx, &d->ctx, sizeof(DeviceContext));
  a.sb = (SyncBlock*)d->sync_block;
  a.in = (const uint8_t*)d->in;
  a.out = (uint8_t*)d->out;
  a.M = d->M; a.N = d->N; a.ld_in = d->ld_in; a.ld_out = d->ld_out;
  a.variant = d->variant;
  a.use_mc = d->use_mc && d->ctx.mc_base != 0 && d->ctx.world > 1;
  a.block_m = d->block_m; a.block_n = d->block_n; a.distribution = d->distribution; a.swizzle = d->swizzle;
  a.ring_buf = (uint8_t*)d->ring_buf; a.flags = d->flags; a.rows_mode = d->rows_mode;
}

static int grid_for(const IrisCclDesc* d, size_t bytes) {
  int g = d->comm_sms > 0 ? d->comm_sms : 64;
  // small messages: do not pay for CTAs that would have nothing to move
  const size_t per_cta = (size_t)kThreads * 16 * 4;
  const int need = (int)((bytes + per_cta - 1) / per_cta);
  if (need < g) g = need < 1 ? 1 : need;
  if (g > 148) g = 148;  // entry-round waiters must all be resident
  return g;
}

// op: 0 all_gather, 1 all_to_all, 2 all_reduce, 3 reduce_scatter
int iris_ccl_launch(int op, const IrisCclDesc* d, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  CclArgs a;
  fill_args(a, d);
  const int es = esize_of(d->dtype);
  if (!es) return -2;
  const int W = d->ctx.world;
  if (op == 0 || op == 1) {
    const size_t row_bytes = (size_t)d->N * es;
    const bool vec = row_bytes % 16 == 0 && aligned16(d->in) && aligned16(d->out) && (d->ld_in * es) % 16 == 0 &&
                     (d->ld_out * es) % 16 == 0;
    a.block_m = es;            // movers are typed by byte width only
    a.block_n = d->variant;    // all_gather mode
    if (!vec) a.use_mc = 0;
    // A multicast store also comes back to its sender through the switch: W / (W - 1) of the useful bytes enter
    // every GPU. With two ranks that doubles the traffic of an all-gather, which is bound by what a GPU can
    // take in; plain stores to the one peer move every byte once.
    if (op == 0 && W == 2) a.use_mc = 0;
    int grid = grid_for(d, row_bytes * d->M * (op == 0 ? 1 : W));
    if (op == 0) {
      if (a.block_n == 1 && grid >= W) grid = grid / W * W;
      if (vec) all_gather_kernel<16><<<grid, kThreads, 0, s>>>(a);
      else all_gather_kernel<1><<<grid, kThreads, 0, s>>>(a);
    } else {
      if (grid >= W) grid = grid / W * W;
      if (vec) all_to_all_kernel<16><<<grid, kThreads, 0, s>>>(a);
      else all_to_all_kernel<1><<<grid, kThreads, 0, s>>>(a);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -21;
  }
  const bool vec = ((size_t)d->N * es) % 16 == 0 && aligned16(d->in) && aligned16(d->out) && (d->ld_in * es) % 16 == 0 &&
                   (d->ld_out * es) % 16 == 0 && (op == 2 || d->rows_mode || (d->block_n * es) % 16 == 0);
  if (!vec) a.use_mc = 0;
  if (op == 2 && d->variant == kArNvls && !a.use_mc) a.variant = kArTwoShot;
  // two ranks, owner-reduces scheme: the multicast store of the result would also return to its sender through
  // the switch (measured at 1 GB: 2429 us with it, 1656 us with a plain store to the one peer; NCCL 1900 us)
  if (op == 2 && W == 2 && a.variant == kArTwoShot) a.use_mc = 0;
  if (op == 2 && W == 1) a.variant = kArOneShot;   // a single rank: every variant is a local copy
  if (op == 2 && a.variant == kArPush) {
    // d->block_m carries the staging capacity in bytes per (parity, source)
    const size_t bytes = (size_t)d->M * d->N * es;
    const size_t unit = vec ? 16 : es;
    if (bytes > (size_t)d->block_m * (size_t)1024 || !d->ring_buf || !d->flags) return -6;
    int g = (int)((bytes / unit + 1023) / 1024);
    if (g < 1) g = 1;
    if (g > kPushMaxCtas) g = kPushMaxCtas;
    const size_t cap_units = (size_t)d->block_m * 1024 / unit;
#define IRIS_PUSH(T)                                                                           \
    do {                                                                                         \
      if (vec) all_reduce_push_kernel<T, 16 / sizeof(T)><<<g, kThreads, 0, s>>>(a, cap_units);   \
      else all_reduce_push_kernel<T, 1><<<g, kThreads, 0, s>>>(a, cap_units);                    \
    } while (0)
    switch (d->dtype) {
      case IRIS_F16: IRIS_PUSH(__half); break;
      case IRIS_BF16: IRIS_PUSH(__nv_bfloat16); break;
      case IRIS_F32: IRIS_PUSH(float); break;
      case IRIS_I32: IRIS_PUSH(int32_t); break;
      default: return -2;
    }
#undef IRIS_PUSH
    return cudaGetLastError() == cudaSuccess ? 0 : -21;
  }
  int grid = grid_for(d, (size_t)d->M * d->N * es);
  // The two-shot all-reduce pulls its share from every peer: a CTA pulls about 15 GB/s, so large
  // messages take every SM unless the caller chose a count (measured on 2 GPUs at 256 MB:
  // 846 us with 64 CTAs, 619 us with 148; the NVLS variant is best at 64).
  if (op == 2 && a.variant == kArTwoShot && (d->comm_sms <= 0 || d->comm_sms == 64) && (size_t)d->M * d->N * es >= ((size_t)8 << 20))
    grid = 148;
  if (op == 2 && a.variant == kArRing) {
    grid = d->comm_sms > 0 ? d->comm_sms : 32;  // must match the flag layout chosen by the host
  }
  switch (d->dtype) {
    case IRIS_F16: return launch_reduce<__half>(a, op == 2, vec, grid, s);
    case IRIS_BF16: return launch_reduce<__nv_bfloat16>(a, op == 2, vec, grid, s);
    case IRIS_F32: return launch_reduce<float>(a, op == 2, vec, grid, s);
    case IRIS_I32: return launch_reduce<int32_t>(a, op == 2, vec, grid, s);
    default: return -2;
  }
}

}  // extern "C"
