// Distributed flash-decode: one query token per sequence, the KV cache sharded along the sequence
// over the ranks (reference: examples/13_flash_decode/decode_kernels.py:141-415 and
// flash_decode_fused_layer.py:38-148).
//
//   1. splitk kernel  grid (splits, kv_heads * head_groups, batch): attention of the query heads
//      of one KV head over one slice of the LOCAL KV shard, paged KV gathered through the block
//      table, online softmax; writes a normalised partial output and its log-sum-exp per split.
//      K/V stream through a ring of swizzled shared-memory tiles; QK^T and PV run on tensor
//      cores with the query heads of the group as the M dimension (each K/V byte is read from HBM
//      exactly once; the kernel is bound by HBM bandwidth). Two ways of filling the ring: one
//      thread issuing TMA box loads per page through a tensor map over the cache (page sizes 8,
//      16, 32 or a multiple of 64; completion on an mbarrier per stage), or all threads issuing
//      16-byte cp.async copies (any page size).
//   2. exchange kernel (persistent): phase A combines the local splits of every (batch, head) and
//      stores (o, lse) into slot [my_rank] of every rank's gathered buffer, then raises that
//      rank's flag for (my_rank, batch, head) with release semantics; phase B waits (acquire,
//      bounded) for the flags of all source ranks and merges the W partials into the final output.
//      All pushes are issued before any wait, so ranks never wait on each other in a cycle; the
//      buffers are double-buffered by call parity and flags carry the call number, so nothing is
//      cleared between calls (the reference zeroes its flags and runs a host barrier per call).
// lse is kept in fp32 (the reference stores it in the fp16 payload).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <string.h>

#include <cuda.h>

#include "iris/host_api.h"
#include "iris/iris.cuh"
#include "iris/ptx.cuh"
#include "flash_decode_static.h"
#include <stdio.h>
#include <mutex>

using namespace iris;

namespace {

constexpr int kD = 128;            // head dimension
constexpr int kBlockN = 64;        // KV positions per pipeline stage
constexpr int kStages = 3;
constexpr int kWarps = 4;
constexpr int kRowBytes = kD * 2;  // one position of one head
constexpr int kTileBytes = kBlockN * kRowBytes;   // 16 KB per K or V tile
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeArgs {
  alignas(64) CUtensorMap tmK;     // TMA path: 2-D maps over the caches seen as [num_blocks * page, Hkv * D],
  alignas(64) CUtensorMap tmV;     // box = 64 columns (128 bytes, swizzled) x box_rows positions
  int box_rows;                    // min(page, 64)
  int32_t* status;                 // context status word (a TMA wait that runs out is recorded there)
  const __nv_bfloat16* q;          // [B, Hq, D]
  const __nv_bfloat16* k_cache;    // [num_blocks, page, Hkv, D]
  const __nv_bfloat16* v_cache;
  const int32_t* block_table;      // [B, max_blocks]
  const int32_t* kv_lens;          // [B] local lengths
  float* partial;                  // [B, Hq, splits, D + 1]  (o normalised, lse in log2 units)
  int B, Hq, Hkv, page, max_blocks, splits, group, head_groups;
  float sm_scale, soft_cap;
  int is_fp16;
};

__device__ __forceinline__ void cp_async16(uint32_t smem, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool kFp16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
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

// Shared-memory tile of kBlockN positions x 16 chunks of 16 B.
// cp.async path: [position][16 chunks], chunk index XOR-swizzled by row & 7.
// TMA path: two halves of the head dimension, each [position][128 bytes] in the 128-byte swizzle
// TMA writes (chunk index within the half XOR row & 7; tiles are 1024-byte aligned).
template <bool kTma>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  if constexpr (kTma) return (chunk >> 3) * (kBlockN * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
  else return row * kRowBytes + ((chunk ^ (row & 7)) << 4);
}

constexpr uint64_t kTmaWaitNs = 2000000000ull;

template <bool kFp16, bool kTma>
__global__ void __launch_bounds__(kWarps * 32, 2) decode_splitk_kernel(const __grid_constant__ DecodeArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // the TMA path needs 1024-byte aligned tiles (the launch adds the slack)
  uint8_t* smem = kTma ? (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023) : smem_raw;
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / a.head_groups, hg = blockIdx.y % a.head_groups;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_here = min(16, a.group - hg * 16);   // query heads of this KV head handled by this CTA
  const int h0 = kvh * a.group + hg * 16;

  const int len = a.kv_lens[b];
  const int per = ((len + a.splits - 1) / a.splits + kBlockN - 1) / kBlockN * kBlockN;   // positions per split, tile aligned
  const int lo = min(len, split * per), hi = min(len, lo + per);
  const int n_tiles = (hi - lo + kBlockN - 1) / kBlockN;

  // ---- Q fragments (A operand, rows = heads, padded to 16 with zeros)
  uint32_t qf[8][4];
  {
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
    const uint32_t* qrow0 = (const uint32_t*)(a.q + ((size_t)b * a.Hq + h0 + r0) * kD);
    const uint32_t* qrow1 = (const uint32_t*)(a.q + ((size_t)b * a.Hq + h0 + r0 + 8) * kD);
    const bool v0 = r0 < heads_here, v1 = r0 + 8 < heads_here;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int c = (ks * 16 + c0) >> 1;
      qf[ks][0] = v0 ? qrow0[c] : 0u;
      qf[ks][1] = v1 ? qrow1[c] : 0u;
      qf[ks][2] = v0 ? qrow0[c + 4] : 0u;
      qf[ks][3] = v1 ? qrow1[c + 4] : 0u;
    }
  }
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float scale2 = a.sm_scale * kLog2e;

  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
  const int32_t* bt = a.block_table + (size_t)b * a.max_blocks;
  const size_t pos_stride = (size_t)a.Hkv * kD;   // elements between consecutive positions of a page

  auto issue_tile = [&](int t) {
    const int stage = t % kStages;
    const uint32_t ks = smem_base + stage * 2 * kTileBytes, vs = ks + kTileBytes;
    // 64 rows x 16 chunks for K and for V = 2048 chunks, 128 threads -> 16 each
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = threadIdx.x + i * 128;     // 0..1023
      const int row = idx >> 4, chunk = idx & 15;
      const int pos = lo + t * kBlockN + row;
      if (pos < hi) {
        const int blk = bt[pos / a.page];
        const size_t e = ((size_t)blk * a.page + pos % a.page) * pos_stride + (size_t)kvh * kD + chunk * 8;
        cp_async16(ks + tile_off<false>(row, chunk), a.k_cache + e);
        cp_async16(vs + tile_off<false>(row, chunk), a.v_cache + e);
      } else {
        *(uint4*)(smem + stage * 2 * kTileBytes + tile_off<false>(row, chunk)) = make_uint4(0, 0, 0, 0);
        *(uint4*)(smem + stage * 2 * kTileBytes + kTileBytes + tile_off<false>(row, chunk)) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  // TMA path, one thread: one box per page piece and half of the head dimension, for K and for V.
  // Tiles start at multiples of 64 positions, so a box never straddles a page.
  uint64_t* full = (uint64_t*)(smem + kStages * 2 * kTileBytes);
  auto issue_tile_tma = [&](int t) {
    const int stage = t % kStages;
    uint8_t* kdst = smem + stage * 2 * kTileBytes;
    uint8_t* vdst = kdst + kTileBytes;
    const int pos0 = lo + t * kBlockN;
    const int rows = min(kBlockN, hi - pos0);
    const int nbox = (rows + a.box_rows - 1) / a.box_rows;
    ptx::mbar_expect_tx(&full[stage], (uint32_t)(nbox * a.box_rows * 128 * 4));
    for (int j = 0; j < nbox; ++j) {
      const int pos = pos0 + j * a.box_rows;
      const int y = bt[pos / a.page] * a.page + pos % a.page;
      const int off = j * a.box_rows * 128;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        ptx::tma_load_2d(kdst + half * (kBlockN * 128) + off, &a.tmK, &full[stage], kvh * kD + half * 64, y);
        ptx::tma_load_2d(vdst + half * (kBlockN * 128) + off, &a.tmV, &full[stage], kvh * kD + half * 64, y);
      }
    }
  };

  if constexpr (kTma) {
    if (threadIdx.x == 0) {
      for (int i = 0; i < kStages; ++i) ptx::mbar_init(&full[i], 1);
      ptx::fence_mbar_init();
      ptx::fence_proxy_async();
    }
    __syncthreads();
    if (threadIdx.x == 0)
      for (int t = 0; t < kStages - 1 && t < n_tiles; ++t) issue_tile_tma(t);
  } else {
    for (int t = 0; t < kStages - 1; ++t) {
      if (t < n_tiles) issue_tile(t);
      cp_async_commit();
    }
  }
  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t % kStages;
    if constexpr (kTma) {
      if (!ptx::mbar_wait(&full[stage], (uint32_t)((t / kStages) & 1), kTmaWaitNs)) {
        if (a.status) atomicCAS(a.status, 0, (int)kTimeoutPipeline);
        break;     // every thread of the CTA waits on the same barrier, so all of them leave here
      }
      __syncthreads();   // everybody is done with tile t-1: its stage can be refilled
      if (threadIdx.x == 0 && t + kStages - 1 < n_tiles) issue_tile_tma(t + kStages - 1);
      const int rows = hi - (lo + t * kBlockN);
      if (rows < kBlockN) {
        // last, partial tile: rows past the end hold whatever the page (or an older tile) held;
        // their scores are masked below, and their V rows are cleared so that 0 * NaN cannot arise
        uint8_t* vt = smem + stage * 2 * kTileBytes + kTileBytes;
        for (int idx = threadIdx.x; idx < (kBlockN - rows) * 16; idx += blockDim.x) {
          const int row = rows + (idx >> 4), chunk = idx & 15;
          *(uint4*)(vt + tile_off<true>(row, chunk)) = make_uint4(0, 0, 0, 0);
        }
        __syncthreads();
      }
    } else {
      cp_async_wait<kStages - 2>();
      __syncthreads();
      if (t + kStages - 1 < n_tiles) issue_tile(t + kStages - 1);
      cp_async_commit();
    }
    const uint32_t ks = smem_base + stage * 2 * kTileBytes, vs = ks + kTileBytes;
    const int p0 = warp * 16;   // this warp's 16 positions of the tile

    // ---- S = Q K^T for 16 heads x 16 positions
    float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t kf[4];
      const int j = lane >> 3, r = lane & 7;
      ldmatrix_x4(kf, ks + tile_off<kTma>(p0 + (j >> 1) * 8 + r, kk * 2 + (j & 1)));
      mma16816<kFp16>(s[0], qf[kk], kf[0], kf[1]);
      mma16816<kFp16>(s[1], qf[kk], kf[2], kf[3]);
    }
    // ---- online softmax (rows lane/4 and lane/4 + 8; columns: nb * 8 + (lane % 4) * 2 + {0, 1})
    const int pos_base = lo + t * kBlockN + p0 + (lane & 3) * 2;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nb][e] * scale2;
        if (a.soft_cap > 0.f) v = a.soft_cap * kLog2e * tanhf(s[nb][e] * a.sm_scale / a.soft_cap);
        const int pos = pos_base + nb * 8 + (e & 1);
        v = pos < hi ? v : -INFINITY;
        s[nb][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      alpha[r] = m_new == -INFINITY ? 1.f : exp2f(m_run[r] - m_new);
      m_run[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mr = m_run[e >> 1];
        p[e] = mr == -INFINITY ? 0.f : exp2f(s[nb][e] - mr);
        rs[e >> 1] += p[e];
      }
      pf[nb * 2 + 0] = pack2<kFp16>(p[0], p[1]);
      pf[nb * 2 + 1] = pack2<kFp16>(p[2], p[3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
      l_run[r] = l_run[r] * alpha[r] + rs[r];
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
    // ---- O += P V   (A = P: 16 heads x 16 positions, B = V: 16 positions x 128 dims)
#pragma unroll
    for (int nb2 = 0; nb2 < 8; ++nb2) {
      uint32_t vf[4];
      const int j = lane >> 3, r = lane & 7;
      ldmatrix_x4_trans(vf, vs + tile_off<kTma>(p0 + (j & 1) * 8 + r, nb2 * 2 + (j >> 1)));
      mma16816<kFp16>(o[nb2 * 2], pf, vf[0], vf[1]);
      mma16816<kFp16>(o[nb2 * 2 + 1], pf, vf[2], vf[3]);
    }
  }
  if constexpr (!kTma) cp_async_wait<0>();
  __syncthreads();

  // ---- merge the 4 warps (each saw a quarter of the positions), write the partial for this split
  float* sm_o = (float*)smem;                         // [warps][8 rows... 16][128]
  float* sm_ml = sm_o + kWarps * 16 * kD;             // [warps][16][2]
  {
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float* base = sm_o + (warp * 16) * kD + i * 8 + c0;
      base[r0 * kD] = o[i][0]; base[r0 * kD + 1] = o[i][1];
      base[(r0 + 8) * kD] = o[i][2]; base[(r0 + 8) * kD + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      sm_ml[(warp * 16 + r0) * 2] = m_run[0]; sm_ml[(warp * 16 + r0) * 2 + 1] = l_run[0];
      sm_ml[(warp * 16 + r0 + 8) * 2] = m_run[1]; sm_ml[(warp * 16 + r0 + 8) * 2 + 1] = l_run[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < heads_here * kD; idx += blockDim.x) {
    const int h = idx / kD, d = idx - h * kD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, sm_ml[(w * 16 + h) * 2]);
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = sm_ml[(w * 16 + h) * 2];
      const float sc = mw == -INFINITY ? 0.f : exp2f(mw - m);
      l += sm_ml[(w * 16 + h) * 2 + 1] * sc;
      acc += sm_o[(w * 16 + h) * kD + d] * sc;
    }
    float* dst = a.partial + (((size_t)b * a.Hq + h0 + h) * a.splits + split) * (kD + 1);
    dst[d] = l > 0.f ? acc / l : 0.f;
    if (d == 0) dst[kD] = l > 0.f ? m + log2f(l) : -INFINITY;
  }
}

// ------------------------------------------------------------------------------ exchange + merge
struct ExchangeArgs {
  DeviceContext ctx;
  const float* partial;     // [B, Hq, splits, D+1]
  float* gathered;          // heap: [2][W][Bmax][Hq][D+1]
  int32_t* flags;           // heap: [2][W][Bmax][Hq]
  int32_t* state;           // heap: [0] call counter, [1] finished CTAs
  void* out;                // [B, Hq, D] 16-bit
  float* out_lse;           // optional [B, Hq] natural-log lse of the full attention
  int B, Bmax, Hq, splits;
  int is_fp16;
};

__global__ void __launch_bounds__(kD) decode_exchange_kernel(const __grid_constant__ ExchangeArgs a) {
  const DeviceContext& ctx = a.ctx;
  const int W = ctx.world;
  const int call = *(volatile int32_t*)&a.state[0];
  const int buf = call & 1;
  const int32_t tag = (call >> 1) + 1;
  const int items = a.B * a.Hq;
  const int d = threadIdx.x;
  __shared__ float s_w[64];
  __shared__ int s_ok;
  // phase A: combine local splits, push to every rank
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int b = it / a.Hq, h = it - b * a.Hq;
    const float* p = a.partial + (size_t)it * a.splits * (kD + 1);
    float m = -INFINITY;
    for (int s = 0; s < a.splits; ++s) m = fmaxf(m, p[s * (kD + 1) + kD]);
    float l = 0.f, acc = 0.f;
    for (int s = 0; s < a.splits; ++s) {
      const float ls = p[s * (kD + 1) + kD];
      const float w = ls == -INFINITY ? 0.f : exp2f(ls - m);
      l += w;
      acc += w * p[s * (kD + 1) + d];
    }
    const float o = l > 0.f ? acc / l : 0.f;
    const float lse = l > 0.f ? m + log2f(l) : -INFINITY;
    float* slot = a.gathered + ((((size_t)buf * W + ctx.rank) * a.Bmax + b) * a.Hq + h) * (kD + 1);
    int32_t* flag = a.flags + (((size_t)buf * W + ctx.rank) * a.Bmax + b) * a.Hq + h;
    for (int i = 0; i < W; ++i) {
      int r = ctx.rank + i;
      if (r >= W) r -= W;
      float* dst = ctx.remote(slot, r);
      dst[d] = o;
      if (d == 0) dst[kD] = lse;
    }
    __syncthreads();
    if (d < W) {
      int r = ctx.rank + d;
      if (r >= W) r -= W;
      fence_sys();
      st_release_sys(ctx.remote(flag, r), tag);
    }
  }
  // phase B: wait for every source rank, merge
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int b = it / a.Hq, h = it - b * a.Hq;
    if (d == 0) s_ok = 1;
    __syncthreads();
    if (d < W) {
      const int32_t* flag = a.flags + (((size_t)buf * W + d) * a.Bmax + b) * a.Hq + h;
      if (!wait_flag_ge(ctx, flag, tag)) s_ok = 0;
      const float* slot = a.gathered + ((((size_t)buf * W + d) * a.Bmax + b) * a.Hq + h) * (kD + 1);
      s_w[d] = __ldcv(slot + kD);
    }
    __syncthreads();
    if (!s_ok) break;
    float m = -INFINITY;
    for (int r = 0; r < W; ++r) m = fmaxf(m, s_w[r]);
    float l = 0.f, acc = 0.f;
    for (int r = 0; r < W; ++r) {
      const float w = s_w[r] == -INFINITY ? 0.f : exp2f(s_w[r] - m);
      const float* slot = a.gathered + ((((size_t)buf * W + r) * a.Bmax + b) * a.Hq + h) * (kD + 1);
      l += w;
      acc += w * __ldcv(slot + d);
    }
    const float o = l > 0.f ? acc / l : 0.f;
    if (a.is_fp16) ((__half*)a.out)[(size_t)it * kD + d] = __float2half_rn(o);
    else ((__nv_bfloat16*)a.out)[(size_t)it * kD + d] = __float2bfloat16_rn(o);
    if (a.out_lse && d == 0) a.out_lse[it] = l > 0.f ? (m + log2f(l)) / kLog2e : -INFINITY;
    __syncthreads();
  }
  __syncthreads();
  if (d == 0) {
    __threadfence();
    if (atomicAdd(&a.state[1], 1) == (int)gridDim.x - 1) {
      a.state[1] = 0;
      a.state[0] = call + 1;
      __threadfence();
    }
  }
}

// Local-only finish (exchange == 2): fold this rank's splits into (o, lse) without talking to any peer.
// What a decode over a KV shard returns when the cross-rank merge is done elsewhere, e.g. by an
// all-gather of the partial results as in the reference's RCCL baseline
// (examples/benchmark/reference/flash_decode_rccl/flash_decode_layer_rccl.py:100-130).
__global__ void __launch_bounds__(kD) decode_local_finish_kernel(const float* partial, void* out, float* out_lse, int splits, int is_fp16) {
  const int it = blockIdx.x, d = threadIdx.x;
  const float* p = partial + (size_t)it * splits * (kD + 1);
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, p[s * (kD + 1) + kD]);
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ls = p[s * (kD + 1) + kD];
    const float w = ls == -INFINITY ? 0.f : exp2f(ls - m);
    l += w;
    acc += w * p[s * (kD + 1) + d];
  }
  const float o = l > 0.f ? acc / l : 0.f;
  if (is_fp16) ((__half*)out)[(size_t)it * kD + d] = __float2half_rn(o);
  else ((__nv_bfloat16*)out)[(size_t)it * kD + d] = __float2bfloat16_rn(o);
  if (out_lse && d == 0) out_lse[it] = l > 0.f ? (m + log2f(l)) / kLog2e : -INFINITY;
}

}  // namespace

extern "C" {

typedef struct IrisDecodeDesc {
  IrisCtx ctx;
  const void* q; const void* k_cache; const void* v_cache;
  const int32_t* block_table; const int32_t* kv_lens;
  float* partial;
  float* gathered; int32_t* flags; int32_t* state;
  void* out; float* out_lse;
  int32_t B, Bmax, Hq, Hkv, D, page, max_blocks, splits;
  float sm_scale, soft_cap;
  int32_t dtype;
  int32_t exchange;   // 0: only the local split-K pass, 1: also combine + exchange + merge, 2: combine locally (out, lse of this rank's shard)
  int32_t num_blocks; // pages in each cache tensor (0: unknown, the TMA path is not used)
} IrisDecodeDesc;

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// 2-D map over a cache seen as [num_blocks * page positions, Hkv * D] 16-bit elements.
bool make_cache_map(CUtensorMap* m, const void* base, int dtype, uint64_t positions, uint64_t row_elems, uint32_t box_rows) {
  static EncodeTiledFn enc = nullptr;
  if (!enc) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return false;
    enc = (EncodeTiledFn)p;
  }
  if (((uint64_t)base & 15) || ((row_elems * 2) & 15)) return false;
  cuuint64_t dims[2] = {row_elems, positions};
  cuuint64_t strides[1] = {row_elems * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = dtype == IRIS_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return enc(m, dt, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

int iris_flash_decode(const IrisDecodeDesc* d, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (d->D != kD) return -3;
  if (d->Hq % d->Hkv) return -3;
  if (d->dtype != IRIS_BF16 && d->dtype != IRIS_F16) return -2;
  DecodeArgs a;
  a.q = (const __nv_bfloat16*)d->q; a.k_cache = (const __nv_bfloat16*)d->k_cache; a.v_cache = (const __nv_bfloat16*)d->v_cache;
  a.block_table = d->block_table; a.kv_lens = d->kv_lens; a.partial = d->partial;
  a.B = d->B; a.Hq = d->Hq; a.Hkv = d->Hkv; a.page = d->page; a.max_blocks = d->max_blocks; a.splits = d->splits;
  a.group = d->Hq / d->Hkv; a.head_groups = (a.group + 15) / 16;
  a.sm_scale = d->sm_scale; a.soft_cap = d->soft_cap; a.is_fp16 = d->dtype == IRIS_F16;
  a.status = d->ctx.status; a.box_rows = 0;
  // TMA fill when a 64-position tile is a whole number of page pieces
  bool tma = d->num_blocks > 0 && (d->page == 8 || d->page == 16 || d->page == 32 || d->page % 64 == 0);
  if (tma) {
    a.box_rows = d->page < kBlockN ? d->page : kBlockN;
    const uint64_t positions = (uint64_t)d->num_blocks * d->page, row = (uint64_t)d->Hkv * kD;
    tma = make_cache_map(&a.tmK, d->k_cache, d->dtype, positions, row, a.box_rows) &&
          make_cache_map(&a.tmV, d->v_cache, d->dtype, positions, row, a.box_rows);
  }
  const int smem = kStages * 2 * kTileBytes > (int)((kWarps * 16 * kD + kWarps * 32) * sizeof(float))
                       ? kStages * 2 * kTileBytes : (int)((kWarps * 16 * kD + kWarps * 32) * sizeof(float));
  const int smem_tma = smem + 64 + 1024;     // stage barriers, alignment slack
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(decode_splitk_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -20;
    if (cudaFuncSetAttribute(decode_splitk_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -20;
    if (cudaFuncSetAttribute(decode_splitk_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_tma) != cudaSuccess) return -20;
    if (cudaFuncSetAttribute(decode_splitk_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_tma) != cudaSuccess) return -20;
    attr = true;
  }
  dim3 grid(d->splits, d->Hkv * a.head_groups, d->B);
  if (tma) {
    if (a.is_fp16) decode_splitk_kernel<true, true><<<grid, kWarps * 32, smem_tma, s>>>(a);
    else decode_splitk_kernel<false, true><<<grid, kWarps * 32, smem_tma, s>>>(a);
  } else {
    if (a.is_fp16) decode_splitk_kernel<true, false><<<grid, kWarps * 32, smem, s>>>(a);
    else decode_splitk_kernel<false, false><<<grid, kWarps * 32, smem, s>>>(a);
  }
  if (cudaGetLastError() != cudaSuccess) return -21;
  if (!d->exchange) return 0;
  if (d->exchange == 2) {
    decode_local_finish_kernel<<<d->B * d->Hq, kD, 0, s>>>(d->partial, d->out, d->out_lse, d->splits, a.is_fp16);
    return cudaGetLastError() == cudaSuccess ? 0 : -21;
  }
  ExchangeArgs x;
  memcpy(&x.ctx, &d->ctx, sizeof(DeviceContext));
  if (x.ctx.world > 64) return -4;
  x.partial = d->partial; x.gathered = d->gathered; x.flags = d->flags; x.state = d->state;
  x.out = d->out; x.out_lse = d->out_lse; x.B = d->B; x.Bmax = d->Bmax; x.Hq = d->Hq; x.splits = d->splits;
  x.is_fp16 = a.is_fp16;
  int items = d->B * d->Hq;
  int grid2 = items < 148 * 8 ? items : 148 * 8;   // every CTA resident: pushes precede all waits anyway
  decode_exchange_kernel<<<grid2, kD, 0, s>>>(x);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // extern "C"

// ------------------------------------------------------------------ entry point that allocates nothing
// See flash_decode_static.h. The split-K kernel above is launched unchanged with its partial
// results directed into the file-scope array below; a small kernel then folds the splits into
// the output. Host code never uses `g_decode_static_scratch` as an address: the name is only a
// handle on the host side, the device address comes from cudaGetSymbolAddress.
namespace {

static __device__ __align__(256) unsigned char g_decode_static_scratch[IRIS_DECODE_STATIC_SCRATCH_BYTES];

constexpr int kStaticMaxDevices = 64;
float* g_static_scratch_addr[kStaticMaxDevices] = {};
bool g_static_attr_done[kStaticMaxDevices] = {};   // shared-memory limit raised on that device's function handles
std::mutex g_static_setup_mutex;

__global__ void __launch_bounds__(kD) decode_local_combine_kernel(const float* partial, void* out, int splits, int is_fp16) {
  const int it = blockIdx.x, d = threadIdx.x;
  const float* p = partial + (size_t)it * splits * (kD + 1);
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, p[s * (kD + 1) + kD]);
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ls = p[s * (kD + 1) + kD];
    const float w = ls == -INFINITY ? 0.f : exp2f(ls - m);
    l += w;
    acc += w * p[s * (kD + 1) + d];
  }
  const float o = l > 0.f ? acc / l : 0.f;
  if (is_fp16) ((__half*)out)[(size_t)it * kD + d] = __float2half_rn(o);
  else ((__nv_bfloat16*)out)[(size_t)it * kD + d] = __float2bfloat16_rn(o);
}

void static_err(char* err, int32_t errlen, const char* msg) {
  if (err && errlen > 0) snprintf(err, (size_t)errlen, "%s", msg);
}

}  // namespace

extern "C" uint64_t iris_flash_decode_static_scratch_needed(int32_t B, int32_t Hq, int32_t splits, int32_t D) {
  return (uint64_t)B * (uint64_t)Hq * (uint64_t)splits * (uint64_t)(D + 1);
}

extern "C" int iris_flash_decode_static(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                                        const int32_t* kv_lens, void* out, int32_t B, int32_t Hq, int32_t Hkv, int32_t D,
                                        int32_t page, int32_t max_blocks, int32_t splits, float sm_scale, float soft_cap,
                                        int32_t dtype, void* stream, char* err, int32_t errlen) {
  cudaStream_t s = (cudaStream_t)stream;
  if (D != kD || Hkv <= 0 || Hq % Hkv || B <= 0 || splits <= 0 || page <= 0) {
    static_err(err, errlen, "iris_flash_decode_static: head_dim must be 128, q_heads a multiple of kv_heads, sizes positive");
    return -3;
  }
  if (dtype != IRIS_BF16 && dtype != IRIS_F16) {
    static_err(err, errlen, "iris_flash_decode_static: dtype must be fp16 (0) or bf16 (1)");
    return -2;
  }
  const uint64_t need = iris_flash_decode_static_scratch_needed(B, Hq, splits, D) * sizeof(float);
  if (need > IRIS_DECODE_STATIC_SCRATCH_BYTES) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "iris_flash_decode_static: batch %d x q_heads %d x splits %d needs %llu bytes of scratch, the built-in array holds %u; "
             "lower splits or call iris_flash_decode with your own buffer",
             B, Hq, splits, (unsigned long long)need, IRIS_DECODE_STATIC_SCRATCH_BYTES);
    static_err(err, errlen, msg);
    return IRIS_DECODE_STATIC_TOO_LARGE;
  }
  // set-up, once per device: the array's address on the device that is current now
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) {
    static_err(err, errlen, "iris_flash_decode_static: no current CUDA device");
    return -4;
  }
  // Both tables below are per device: the array's address differs from GPU to GPU, and the raised
  // shared-memory limit belongs to the function handle of the device that was current when it was
  // set. One mutex covers the set-up, so that two host threads making a device's first call agree.
  const int smem = kStages * 2 * kTileBytes > (int)((kWarps * 16 * kD + kWarps * 32) * sizeof(float))
                       ? kStages * 2 * kTileBytes : (int)((kWarps * 16 * kD + kWarps * 32) * sizeof(float));
  {
    std::lock_guard<std::mutex> guard(g_static_setup_mutex);
    if (!g_static_scratch_addr[dev]) {
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
      if (e != cudaSuccess || !p) {
        static_err(err, errlen, "iris_flash_decode_static: cudaGetSymbolAddress failed for the scratch array");
        return -5;
      }
      g_static_scratch_addr[dev] = (float*)p;
    }
    if (!g_static_attr_done[dev]) {
      if (cudaFuncSetAttribute(decode_splitk_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
          cudaFuncSetAttribute(decode_splitk_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        static_err(err, errlen, "iris_flash_decode_static: cannot raise the kernel's shared-memory limit");
        return -20;
      }
      g_static_attr_done[dev] = true;
    }
  }
  float* scratch = g_static_scratch_addr[dev];

  DecodeArgs a;
  a.q = (const __nv_bfloat16*)q; a.k_cache = (const __nv_bfloat16*)k_cache; a.v_cache = (const __nv_bfloat16*)v_cache;
  a.block_table = block_table; a.kv_lens = kv_lens; a.partial = scratch;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.page = page; a.max_blocks = max_blocks; a.splits = splits;
  a.group = Hq / Hkv; a.head_groups = (a.group + 15) / 16;
  a.sm_scale = sm_scale; a.soft_cap = soft_cap; a.is_fp16 = dtype == IRIS_F16;
  a.status = nullptr; a.box_rows = 0;     // the cp.async instantiation: no tensor maps
  dim3 grid(splits, Hkv * a.head_groups, B);
  if (a.is_fp16) decode_splitk_kernel<true, false><<<grid, kWarps * 32, smem, s>>>(a);
  else decode_splitk_kernel<false, false><<<grid, kWarps * 32, smem, s>>>(a);
  if (cudaGetLastError() != cudaSuccess) {
    static_err(err, errlen, "iris_flash_decode_static: split-K kernel launch failed");
    return -21;
  }
  decode_local_combine_kernel<<<B * Hq, kD, 0, s>>>(scratch, out, splits, a.is_fp16);
  if (cudaGetLastError() != cudaSuccess) {
    static_err(err, errlen, "iris_flash_decode_static: combine kernel launch failed");
    return -21;
  }
  return 0;
}
