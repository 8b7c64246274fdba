// Shared by the two ring-attention translation units (mma.sync attention CTAs in
// ring_attention.cu, tcgen05 attention CTAs in ring_attention_tc.cu): the kernel arguments, the
// ring-buffer addressing and the communication CTAs that pass K/V blocks round the ring.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <string.h>

#include "iris/host_api.h"
#include "iris/iris.cuh"

namespace iris_ring {
using namespace iris;

constexpr int kD = 128;
constexpr int kBQ = 64;            // queries per item (4 warps x 16 rows)
constexpr int kBKV = 64;           // keys per tile
constexpr int kStages = 2;
constexpr int kTileBytes = kBKV * kD * 2;    // 16 KB
constexpr int kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kPiece = 16 * 1024;

struct RingArgs {
  DeviceContext ctx;
  const uint8_t* q;       // [S, Hq, D]
  const uint8_t* k;       // [S, Hkv, D] own block
  const uint8_t* v;
  uint8_t* kv_buf;        // heap [2][W][2][S, Hkv, D]
  int32_t* flags;         // heap [2][W]
  int32_t* state;         // heap [0] call counter, [1] finished CTAs
  uint8_t* out;           // [S, Hq, D]
  float* lse;             // optional [S, Hq] natural log
  int S, Hq, Hkv, causal, n_comm, is_fp16;
  int zigzag;             // 1: this rank's block is [chunk r | chunk 2W-1-r] of 2W chunks (tcgen05 attention CTAs only)
  float sm_scale;
};

__device__ __forceinline__ void cp_async16(uint32_t smem, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool kFp16>
__device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kFp16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool kFp16> __device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (kFp16) { __half2 h = __floats2half2_rn(a, b); return *(uint32_t*)&h; }
  else { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *(uint32_t*)&h; }
}
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) { return row * (kD * 2) + ((chunk ^ (row & 7)) << 4); }

__device__ __forceinline__ size_t block_bytes(const RingArgs& a) { return (size_t)a.S * a.Hkv * kD * 2; }
// slot `origin` of the ring buffer of parity `par`: K at +0, V at +block_bytes
__device__ __forceinline__ uint8_t* slot_ptr(const RingArgs& a, int par, int origin) {
  return a.kv_buf + ((size_t)par * a.ctx.world + origin) * 2 * block_bytes(a);
}

// ------------------------------------------------------------------ communication CTAs
static __device__ void comm_main(const RingArgs& a, uint8_t* smem_raw, int smem_bytes, int call) {
  const DeviceContext& ctx = a.ctx;
  const int W = ctx.world, r = ctx.rank, c = blockIdx.x;
  if (W == 1) return;
  const int par = call & 1;
  const int32_t target = ((call >> 1) + 1) * a.n_comm;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  int nb = (smem_bytes - 512) / kPiece;
  if (nb > 8) nb = 8;
  uint64_t* bars = (uint64_t*)(smem + (size_t)nb * kPiece);
  if (threadIdx.x == 0) {
    for (int i = 0; i < nb; ++i) ptx::mbar_init(&bars[i], 1);
    ptx::fence_mbar_init();
    ptx::fence_proxy_async();
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const int next = r + 1 == W ? 0 : r + 1;
  const size_t bb = block_bytes(a);
  // this CTA's byte range of a block (K and V handled as two ranges of the same shape)
  const size_t per = ((bb + a.n_comm - 1) / a.n_comm + 15) & ~(size_t)15;
  const size_t lo = min(bb, (size_t)c * per), hi = min(bb, lo + per);
  int seq = 0;
  for (int i = 0; i + 1 < W; ++i) {
    int origin = r - i;
    if (origin < 0) origin += W;
    const uint8_t* src_k;
    const uint8_t* src_v;
    if (i == 0) { src_k = a.k; src_v = a.v; }
    else {
      if (!wait_flag_ge(ctx, a.flags + (size_t)par * W + origin, target)) return;
      ptx::fence_proxy_async();
      src_k = slot_ptr(a, par, origin); src_v = src_k + bb;
    }
    uint8_t* dst_k = ctx.remote(slot_ptr(a, par, origin), next);
    uint8_t* dst_v = dst_k + bb;
    const int n_half = (int)((hi - lo + kPiece - 1) / kPiece);
    const int total = 2 * n_half;
    auto src_of = [&](int q) { return (q < n_half ? src_k : src_v) + lo + (size_t)(q % max(n_half, 1)) * kPiece; };
    auto dst_of = [&](int q) { return (q < n_half ? dst_k : dst_v) + lo + (size_t)(q % max(n_half, 1)) * kPiece; };
    auto len_of = [&](int q) { const size_t o = lo + (size_t)(q % max(n_half, 1)) * kPiece; return (uint32_t)min((size_t)kPiece, hi - o); };
    auto issue = [&](int q) {
      const int slot = (seq + q) % nb;
      ptx::mbar_expect_tx(&bars[slot], len_of(q));
      ptx::bulk_load(smem + (size_t)slot * kPiece, src_of(q), len_of(q), &bars[slot]);
    };
    int nxt = min(nb, total);
    for (int q = 0; q < nxt; ++q) issue(q);
    for (int q = 0; q < total; ++q) {
      const int slot = (seq + q) % nb;
      if (!ptx::mbar_wait(&bars[slot], (uint32_t)(((seq + q) / nb) & 1))) { ctx.fail(kTimeoutPipeline); return; }
      ptx::bulk_store(dst_of(q), smem + (size_t)slot * kPiece, len_of(q));
      ptx::bulk_commit();
      if (q == total - 1) ptx::bulk_wait<0>();
      else ptx::bulk_wait_read<1>();
      const int free_upto = q == total - 1 ? q : q - 1;
      while (nxt <= free_upto + nb && nxt < total) issue(nxt++);
    }
    seq += total;
    ptx::fence_proxy_async();
    fence_sys();
    red_release_sys_add(ctx.remote(a.flags + (size_t)par * W + origin, next), 1);
  }
}


// Last step of both kernels: count finished CTAs; the last one advances the call counter.
__device__ __forceinline__ void finish_call(const RingArgs& a, int call) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&a.state[1], 1) == (int)gridDim.x - 1) {
      a.state[1] = 0;
      a.state[0] = call + 1;
      __threadfence();
    }
  }
}

// Launches the kernel whose attention CTAs use tcgen05 (ring_attention_tc.cu). Returns 1 when the
// shape is not covered (S not a multiple of 128), 0 on success, < 0 on a launch error.
int launch_ring_attention_tc(const RingArgs& a, cudaStream_t stream);

}  // namespace iris_ring
