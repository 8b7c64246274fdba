// GEMM kernels of iris_b200 for sm_100a: the local GEMM and the fused compute+collective ops
//   all_gather_matmul      (reference iris/ops/all_gather_matmul.py:27-159, examples/14 push variant)
//   matmul_all_gather      (iris/ops/matmul_all_gather.py:28-105; examples/07 all-scatter layout)
//   matmul_reduce_scatter  (iris/ops/matmul_reduce_scatter.py:26-118; examples/22 row-chunk ownership)
//   matmul_all_reduce      (iris/ops/matmul_all_reduce.py:26-144)
// all built on include/iris/gemm/sm100_mainloop.cuh (TMA -> smem ring -> tcgen05.mma -> TMEM).
// The collective half of each op runs inside the same kernel: peer stores / NVLS multimem stores
// issued from the epilogue warps or from dedicated communication CTAs, per-tile flags on the
// symmetric heap, bounded waits.
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>
#include <stdio.h>

#include "iris/host_api.h"
#include "iris/context.cuh"
#include "iris/rma.cuh"
#include "iris/sync.cuh"
#include "iris/multimem.cuh"
#include "iris/gemm/sm100_mainloop.cuh"

using namespace iris;
using namespace iris::gemm;

#include "gemm_host.cuh"

namespace {

// ------------------------------------------------------------------------------------ local GEMM
struct LocalGemm : Common {
  uint8_t* C;
  int64_t ldc;
  struct State {};
  IRIS_D void tile(int t, int& tm, int& tn) const { swizzled_tile(t, order_m, tiles_n, group_m, tm, tn); }
  IRIS_D bool a_source(State&, int tm, int kb, ASource& s) const {
    s.map = &tmA; s.x = kb * kBK; s.y = tm * kBM; s.bk = kb * kBK;
    return true;
  }
  IRIS_D void begin_tile(State&, int, int, uint8_t*) const {}
  IRIS_D int row_origin(State&, int tm) const { return tm * kBM; }
  static constexpr bool kSwiGLU = false;
  IRIS_D void store16(State&, int row, int col, uint4 v) const {
    if (row < sh.M && col < sh.N) *(uint4*)(C + ((int64_t)row * ldc + col) * 2) = v;
  }
  static constexpr bool kBulkEpilogue = false;
  IRIS_D void store_chunk(State&, int, int, int, const uint8_t*) const {}
  IRIS_D bool reduce_here(State&) const { return false; }
  IRIS_D void add_partials(State&, int, int, int, uint32_t (&)[32]) const {}
  IRIS_D void tile_done(State&, int, int) const {}
  IRIS_D void comm_main(uint8_t*, int) const {}
  IRIS_D void post_main() const {}
};

// ------------------------------------------------------------------------------------ AG + GEMM
// A is sharded over ranks (rows: mode 0, K: mode 1). Communication CTAs push this rank's shard
// into every peer's inbox (one multimem.st through the switch when NVLS is on, else one store per
// peer) and bump a per-(source, 128-row chunk) arrival counter with release semantics. The TMA
// producer of a GEMM CTA polls the counter of the chunk it is about to read (acquire) and then
// loads from its OWN memory: a remote tile crosses NVLink once, whatever the number of N tiles.
// The inbox and the counters are double-buffered by call parity; waiting for every source's
// counters in call k proves every rank left call k-1, so buffer reuse needs no extra barrier.
struct AllGatherGemm : Common {
  CUtensorMap tmInbox;     // rows = 2 * W * rows_per_src, cols = cols_per_src
  DeviceContext ctx;
  SyncBlock* sb;
  const uint8_t* A_local;  // this rank's shard, row pitch lda (elements)
  int64_t lda;
  uint8_t* inbox;          // heap, buffer 0 of [2][W][rows_per_src][cols_per_src]
  int32_t* flags;          // heap, [2][W][chunks]
  uint8_t* C;
  int64_t ldc;
  int mode;                // 0: rows sharded, 1: K sharded
  int rows_per_src;        // mode 0: M_local, mode 1: M
  int cols_per_src;        // mode 0: K, mode 1: K_local
  int chunks;              // 128-row chunks per source
  int n_comm_ctas;
  int use_mc;

  struct State {
    int key = -1;        // (source, chunk) whose arrival has been confirmed
    int epoch = -1;
    int tm = -1;         // tile row the cached values below belong to
    int src = 0, chunk = 0, g = 0, kb_next_src = 0, kb0 = 0;
    const CUtensorMap* map = nullptr;
    int y = 0;
  };
  IRIS_D int src_of_group(int g) const {  // own shard first, then the order the pushes arrive in
    int s = ctx.rank - g;
    return s < 0 ? s + ctx.world : s;
  }
  // Row-sharded A: this rank's own shard first (nothing to wait for), then the peers' shards in
  // the order their data lands: every source streams its 128-row chunks in order and all sources
  // stream at once, so chunk c of every peer is complete before chunk c+1 of any peer. Visiting
  // (chunk, source) in that order keeps the GEMM behind the transfer instead of waiting for one
  // source's last chunk.
  IRIS_D void tile(int t, int& tm, int& tn) const {
    if (mode == 0) {
      const int oc = chunks >> pair;          // row tiles per source in tile-order units
      const int per_src = oc * tiles_n;
      if (t < per_src || ctx.world == 1) {
        int lm, ln;
        swizzled_tile(t, oc, tiles_n, group_m, lm, ln);
        tm = ctx.rank * oc + lm;
        tn = ln;
        return;
      }
      const int u = t - per_src;
      const int per_chunk = (ctx.world - 1) * tiles_n;
      const int c = u / per_chunk;
      const int v = u - c * per_chunk;
      const int si = v / tiles_n;
      tm = src_of_group(si + 1) * oc + c;
      tn = v - si * tiles_n;
    } else {
      swizzled_tile(t, order_m, tiles_n, group_m, tm, tn);
    }
  }
  // Select the map / row of (source, chunk) and make sure the chunk has arrived. The divisions
  // and the flag poll happen once per (tile, source), not per K block.
  IRIS_D bool select(State& st, int src, int chunk) const {
    st.src = src; st.chunk = chunk;
    if (src == ctx.rank) {       // own shard: read in place, nothing to wait for
      st.map = &tmA; st.y = chunk * kBM;
      return true;
    }
    const int buf = st.epoch & 1;
    const int key = src * chunks + chunk;
    if (key != st.key) {
      const int target = ((st.epoch >> 1) + 1) * n_comm_ctas;
      if (!wait_flag_ge(ctx, flags + ((size_t)buf * ctx.world + src) * chunks + chunk, target)) return false;
      st.key = key;
      // The data was written by another GPU (generic proxy, remote); order the TMA (async proxy)
      // reads after the acquire.
      ptx::fence_proxy_async();
    }
    st.map = &tmInbox; st.y = ((buf * ctx.world + src) * rows_per_src) + chunk * kBM;
    return true;
  }
  IRIS_D bool a_source(State& st, int tm, int kb, ASource& s) const {
    if (st.epoch < 0) st.epoch = read_epoch(sb);
    if (mode == 0) {
      if (tm != st.tm) {
        st.tm = tm;
        const int src = tm / chunks;
        if (!select(st, src, tm - src * chunks)) return false;
      }
      s.map = st.map; s.x = kb * kBK; s.y = st.y; s.bk = s.x;
      return true;
    }
    // K-sharded: walk the sources along K, own shard first
    if (kb == 0 || kb == st.kb_next_src) {
      const int kb_per_src = cols_per_src / kBK;
      st.g = kb == 0 ? 0 : st.g + 1;
      st.kb0 = st.g * kb_per_src;
      st.kb_next_src = st.kb0 + kb_per_src;
      if (!select(st, src_of_group(st.g), tm)) return false;
    }
    s.map = st.map; s.x = (kb - st.kb0) * kBK; s.y = st.y; s.bk = st.src * cols_per_src + s.x;
    return true;
  }
  IRIS_D void begin_tile(State&, int, int, uint8_t*) const {}
  IRIS_D int row_origin(State&, int tm) const { return tm * kBM; }
  static constexpr bool kSwiGLU = false;
  IRIS_D void store16(State&, int row, int col, uint4 v) const {
    if (row < sh.M && col < sh.N) *(uint4*)(C + ((int64_t)row * ldc + col) * 2) = v;
  }
  static constexpr bool kBulkEpilogue = false;
  IRIS_D void store_chunk(State&, int, int, int, const uint8_t*) const {}
  IRIS_D bool reduce_here(State&) const { return false; }
  IRIS_D void add_partials(State&, int, int, int, uint32_t (&)[32]) const {}
  IRIS_D void tile_done(State&, int, int) const {}

  // Communication CTAs: CTA j moves slice j (of n_comm_ctas) of every 128-row chunk, chunk by
  // chunk, so chunk 0 is complete everywhere first. The slice streams through a ring of shared
  // memory buffers filled by bulk async copies (cp.async.bulk, local HBM read once); from there it
  // goes either to each peer with bulk async stores issued by one thread (unicast), or to all
  // ranks at once with multimem.st issued by every thread (NVLS). After the last piece of a chunk
  // the stores are drained and the chunk's arrival counter is raised on the receivers.
  static constexpr int kPiece = 32 * 1024;
  // wait until at most `n` of the most recent bulk groups are still pending
  IRIS_D static void bulk_wait_upto(int n) {
    switch (n) {
      case 0: ptx::bulk_wait<0>(); break;
      case 1: ptx::bulk_wait<1>(); break;
      case 2: ptx::bulk_wait<2>(); break;
      case 3: ptx::bulk_wait<3>(); break;
      case 4: ptx::bulk_wait<4>(); break;
      case 5: ptx::bulk_wait<5>(); break;
      case 6: ptx::bulk_wait<6>(); break;
      case 7: ptx::bulk_wait<7>(); break;
      case 8: ptx::bulk_wait<8>(); break;
      default: ptx::bulk_wait<0>(); break;   // more groups than cases: drain everything
    }
  }
  IRIS_D void signal_chunk(int buf, int c) const {
    int32_t* flag_local = flags + ((size_t)buf * ctx.world + ctx.rank) * chunks + c;
    ptx::fence_proxy_async();
    fence_sys();
    for (int p = 1; p < ctx.world; ++p) {
      int dst_rank = ctx.rank + p;
      if (dst_rank >= ctx.world) dst_rank -= ctx.world;
      red_release_sys_add(ctx.remote(flag_local, dst_rank), 1);
    }
  }
  IRIS_D void comm_main(uint8_t* smem_raw, int smem_bytes) const {
    const int j = blockIdx.x - n_gemm_ctas;
    const int epoch = read_epoch(sb);
    const int buf = epoch & 1;
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
    int nb = (smem_bytes - 1024) / kPiece;
    if (nb > 6) nb = 6;
    uint64_t* bars = (uint64_t*)(smem + (size_t)nb * kPiece);
    if (threadIdx.x == 0) {
      for (int i = 0; i < nb; ++i) ptx::mbar_init(&bars[i], 1);
      ptx::fence_mbar_init();
      ptx::fence_proxy_async();
    }
    __syncthreads();
    const size_t row_bytes = (size_t)cols_per_src * 2;
    const size_t src_pitch = (size_t)lda * 2;
    const bool flat = src_pitch == row_bytes;
    const int pieces_per_row = (int)((row_bytes + kPiece - 1) / kPiece);
    // piece i of a slice of `nrows` rows starting at byte offsets (src0, dst0): (src, dst, bytes)
    auto piece = [&](int i, size_t slice_bytes, size_t& soff, size_t& doff, uint32_t& bytes) {
      if (flat) {
        soff = doff = (size_t)i * kPiece;
        bytes = (uint32_t)min((size_t)kPiece, slice_bytes - soff);
      } else {
        const int r = i / pieces_per_row, k = i - r * pieces_per_row;
        soff = (size_t)r * src_pitch + (size_t)k * kPiece;
        doff = (size_t)r * row_bytes + (size_t)k * kPiece;
        bytes = (uint32_t)min((size_t)kPiece, row_bytes - (size_t)k * kPiece);
      }
    };
    __shared__ int s_abort;
    if (threadIdx.x == 0) s_abort = 0;
    __syncthreads();
    int it_global = 0;   // pieces issued so far by this CTA (selects ring slot and barrier parity)
    for (int c = 0; c < chunks; ++c) {
      const int r0 = c * kBM;
      const int nrows_c = min(kBM, rows_per_src - r0);
      const int rows_lo = (int)((int64_t)nrows_c * j / n_comm_ctas), rows_hi = (int)((int64_t)nrows_c * (j + 1) / n_comm_ctas);
      const int nrows = rows_hi - rows_lo;
      const size_t slice_bytes = (size_t)nrows * row_bytes;
      const int n = nrows == 0 ? 0 : (flat ? (int)((slice_bytes + kPiece - 1) / kPiece) : nrows * pieces_per_row);
      const uint8_t* src0 = A_local + (size_t)(r0 + rows_lo) * src_pitch;
      uint8_t* dst_local = inbox + (((size_t)buf * ctx.world + ctx.rank) * rows_per_src + r0 + rows_lo) * row_bytes;
      int32_t* flag_local = flags + ((size_t)buf * ctx.world + ctx.rank) * chunks + c;
      const int base = it_global;
      auto issue_load = [&](int i) {   // thread 0 only
        size_t so, d_o; uint32_t by;
        piece(i, slice_bytes, so, d_o, by);
        const int slot = (base + i) % nb;
        ptx::mbar_expect_tx(&bars[slot], by);
        ptx::bulk_load(smem + (size_t)slot * kPiece, src0 + so, by, &bars[slot]);
      };
      if (use_mc) {
        uint8_t* dst_mc = ctx.mc(dst_local);
        if (threadIdx.x == 0)
          for (int i = 0; i < min(nb, n); ++i) issue_load(i);
        for (int i = 0; i < n; ++i) {
          const int slot = (base + i) % nb;
          const uint32_t parity = (uint32_t)(((base + i) / nb) & 1);
          if (!ptx::mbar_wait(&bars[slot], parity, kPipeTimeoutNs)) { fail(kTimeoutPipeline); s_abort = 1; }
          __syncthreads();
          if (s_abort) break;
          size_t so, d_o; uint32_t by;
          piece(i, slice_bytes, so, d_o, by);
          const uint8_t* sp = smem + (size_t)slot * kPiece;
          for (uint32_t u = threadIdx.x * 16; u < by; u += blockDim.x * 16) {
            const multimem::V4 v = *(const multimem::V4*)(sp + u);
            multimem::st_v4(dst_mc + d_o + u, v);
          }
          __syncthreads();
          if (threadIdx.x == 0 && i + nb < n) {
            ptx::fence_proxy_async();   // generic reads of the slot precede the async refill
            issue_load(i + nb);
          }
        }
        __syncthreads();
        if (threadIdx.x == 0 && !s_abort) {
          fence_sys();
          multimem::red_release_add_u32(ctx.mc(flag_local), 1);
        }
      } else if (threadIdx.x == 0) {
        int next_load = min(nb, n);
        for (int i = 0; i < next_load; ++i) issue_load(i);
        bool ok = true;
        for (int i = 0; i < n && ok; ++i) {
          const int slot = (base + i) % nb;
          const uint32_t parity = (uint32_t)(((base + i) / nb) & 1);
          if (!ptx::mbar_wait(&bars[slot], parity, kPipeTimeoutNs)) { fail(kTimeoutPipeline); ok = false; break; }
          size_t so, d_o; uint32_t by;
          piece(i, slice_bytes, so, d_o, by);
          for (int p = 1; p < ctx.world; ++p) {
            int dst_rank = ctx.rank + p;
            if (dst_rank >= ctx.world) dst_rank -= ctx.world;
            ptx::bulk_store(ctx.remote(dst_local, dst_rank) + d_o, smem + (size_t)slot * kPiece, by);
          }
          ptx::bulk_commit();
          ptx::bulk_wait_read<1>();
          while (next_load <= i - 1 + nb && next_load < n) issue_load(next_load++);
        }
        if (!ok) { s_abort = 1; }
        // The stores of chunk c are only known complete once all but the groups committed after
        // them have drained: raise chunk c-1's counter now (its groups are older than the n just
        // committed), and the last chunk's after a full drain. Keeps the pipe busy across chunks.
        if (!s_abort) {
          if (c > 0) {
            bulk_wait_upto(n);
            signal_chunk(buf, c - 1);
          }
          if (c == chunks - 1) {
            ptx::bulk_wait<0>();
            signal_chunk(buf, c);
          }
        }
      }
      it_global += n;
      if (threadIdx.x == 0 && j == 0) stamp(tiles_m * tiles_n + c, 3);
    }
    finish();
  }
  IRIS_D void post_main() const { finish(); }
  // Count finished CTAs; the last one advances the call counter (no cross-rank round needed).
  IRIS_D void finish() const {
    __syncthreads();
    if (threadIdx.x == 0) {
      const int e = read_epoch(sb);
      __threadfence();
      if (atomicAdd(&sb->done, 1) == (int)gridDim.x - 1) {
        sb->done = 0;
        sb->epoch = e + 1;
        __threadfence();
      }
    }
  }
};

// ------------------------------------------------------------------------- GEMM + push epilogues
// mode ALL_GATHER / ALL_SCATTER: the epilogue stores each 16-byte output fragment to every rank
// (multimem.st, or one store per peer). The last CTA runs one cross-rank round before the kernel
// ends, so every rank's output is complete when its kernel completes.
// mode REDUCE_SCATTER / ALL_REDUCE / RS_TILES: each output tile has an owner rank. Every rank
// stores its partial tile (16-bit) into the owner's staging slot for (source, tile) and adds 1 to
// the owner's arrival counter for that tile (release, system scope). After its own GEMM tiles a
// CTA turns reducer: it waits (acquire) until a tile it owns has W arrivals, sums the W partials
// in fp32 and writes the result: to its own output (reduce-scatter) or to all ranks (all-reduce).
// Staging and counters are double-buffered by call parity, as in AllGatherGemm.
template <bool kReduce>
struct ScatterGemmT : Common {
  static constexpr bool kBulkEpilogue = kReduce;
  DeviceContext ctx;
  SyncBlock* sb;
  int mode;               // IrisGemmOp
  uint8_t* out;           // final output; heap pointer when peers write it (AG / AR / ALL_SCATTER)
  int64_t ld_out;
  uint8_t* staging;       // heap: [2][W][max_owned][128*bn] 16-bit
  int32_t* flags;         // heap: [2][max_owned]
  int max_owned;          // owned tiles per rank (upper bound used for addressing)
  int tiles_m_per_rank;   // REDUCE_SCATTER: row tiles per owner
  int tiles_per_rank;     // RS_TILES: contiguous tile block per owner
  int use_mc;

  struct State {
    int buf = -1;
    int32_t target = 0;
    int owner = 0, lt = 0;
    bool mine = false;         // this rank finishes the tile (adds the peers' partials)
    bool have = true;          // the peers' partials arrived in time
    uint8_t* slot = nullptr;   // not mine: owner's staging slot for (me, tile), translated
    const uint8_t* part0 = nullptr;  // mine: staging slot of source 0 for this tile (local)
  };
  IRIS_D size_t slot_bytes() const { return (size_t)kBM * bn * 2; }
  IRIS_D int total_tiles() const { return tiles_m * tiles_n; }
  // tiles owned by rank o
  // (in the unit the tile order walks: 256-row tiles for CTA pairs)
  IRIS_D int owned_count(int o) const {
    if (mode == IRIS_GEMM_REDUCE_SCATTER) return (tiles_m_per_rank >> pair) * tiles_n;
    if (mode == IRIS_GEMM_ALL_REDUCE) return (order_m * tiles_n - o + ctx.world - 1) / ctx.world;
    const int T = total_tiles();
    if (o == ctx.world - 1) return max(0, T - tiles_per_rank * (ctx.world - 1));
    return min(tiles_per_rank, max(0, T - tiles_per_rank * o));
  }
  // owner rank and the tile's index among the owner's tiles
  IRIS_D void owner_of(int tm, int tn, int& owner, int& lt) const {
    if (mode == IRIS_GEMM_REDUCE_SCATTER) {
      owner = tm / tiles_m_per_rank;
      lt = (tm - owner * tiles_m_per_rank) * tiles_n + tn;
    } else if (mode == IRIS_GEMM_ALL_REDUCE) {
      // round-robin over the tiles the order walks; both 128-row halves of a pair tile share an owner
      const int t = (tm >> pair) * tiles_n + tn;
      owner = t % ctx.world;
      lt = pair ? (t / ctx.world) * 2 + (tm & 1) : t / ctx.world;
    } else {  // RS_TILES: contiguous blocks, last rank takes the remainder
      const int t = tm * tiles_n + tn;
      owner = min(t / tiles_per_rank, ctx.world - 1);
      lt = t - owner * tiles_per_rank;
    }
  }
  // Reducing modes visit the tiles owner by owner: the next rank's tiles first, this rank's own
  // tiles last, so that by the time a rank finishes its own tiles every peer's partial for them
  // has long been delivered.
  IRIS_D void tile(int t, int& tm, int& tn) const {
    if (!reducing()) {
      swizzled_tile(t, order_m, tiles_n, group_m, tm, tn);
      return;
    }
    int o = ctx.rank, k = t;
    for (int g = 0; g < ctx.world; ++g) {
      o = ctx.rank + 1 + g;
      if (o >= ctx.world) o -= ctx.world;
      const int cnt = owned_count(o);
      if (k < cnt) break;
      k -= cnt;
    }
    if (mode == IRIS_GEMM_REDUCE_SCATTER) {
      int lm, ln;
      swizzled_tile(k, tiles_m_per_rank >> pair, tiles_n, group_m, lm, ln);
      tm = o * (tiles_m_per_rank >> pair) + lm;
      tn = ln;
    } else {
      const int id = mode == IRIS_GEMM_ALL_REDUCE ? o + k * ctx.world : o * tiles_per_rank + k;
      tm = id / tiles_n;
      tn = id - tm * tiles_n;
    }
  }
  IRIS_D bool a_source(State&, int tm, int kb, ASource& s) const {
    s.map = &tmA; s.x = kb * kBK; s.y = tm * kBM; s.bk = kb * kBK;
    return true;
  }
  IRIS_D bool reducing() const {
    return mode == IRIS_GEMM_REDUCE_SCATTER || mode == IRIS_GEMM_ALL_REDUCE || mode == IRIS_GEMM_RS_TILES;
  }
  static constexpr bool kSwiGLU = false;
  IRIS_D int row_origin(State&, int tm) const { return tm * kBM; }
  IRIS_D void begin_tile(State& st, int tm, int tn, uint8_t*) const {
    if (!reducing()) return;
    if (st.buf < 0) {
      const int e = read_epoch(sb);
      st.buf = e & 1;
      st.target = ((e >> 1) + 1) * (ctx.world - 1);
    }
    owner_of(tm, tn, st.owner, st.lt);
    st.mine = st.owner == ctx.rank;
    uint8_t* slot0 = staging + (((size_t)st.buf * ctx.world) * max_owned + st.lt) * slot_bytes();
    if (st.mine) {
      st.part0 = slot0;
      st.have = true;
      if (ctx.world > 1) {
        int ok = 1;
        if ((threadIdx.x & 31) == 0) ok = wait_flag_ge(ctx, flags + (size_t)st.buf * max_owned + st.lt, st.target) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        st.have = ok != 0;
      }
    } else {
      st.slot = ctx.remote(slot0 + (size_t)ctx.rank * max_owned * slot_bytes(), st.owner);
    }
  }
  IRIS_D bool reduce_here(State& st) const { return st.mine; }
  // Staging slot layout (private to this kernel): [64-col chunk][quarter][32 rows][width cols],
  // 16-byte groups XOR-swizzled by row exactly as staged in shared memory by the epilogue.
  IRIS_D void add_partials(State& st, int quarter, int c32, int lane, uint32_t (&acc)[32]) const {
    if (!st.have || ctx.world == 1) return;
    const int chunk = c32 >> 1, hlf = c32 & 1;
    const int width = (bn - chunk * 64) >= 64 ? 64 : 32;
    const size_t off = (size_t)chunk * (kBM * 64 * 2) + (size_t)quarter * (32 * width * 2) + (size_t)lane * (width * 2);
    const size_t src_stride = (size_t)max_owned * slot_bytes();
    const int g0 = width == 64 ? hlf * 4 : 0;
    const int swz = width == 64 ? (lane & 7) : ((lane >> 1) & 3);
#pragma unroll
    for (int half = 0; half < 2; ++half) {        // 16 columns = two 16-byte groups per source
#pragma unroll 1
      for (int s0 = 0; s0 < ctx.world; s0 += 8) {
        uint4 v[8][2];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int src = s0 + k;
          if (src < ctx.world && src != ctx.rank) {
            const uint8_t* p = st.part0 + (size_t)src * src_stride + off;
            v[k][0] = __ldcg((const uint4*)(p + (((g0 + half * 2 + 0) ^ swz) << 4)));
            v[k][1] = __ldcg((const uint4*)(p + (((g0 + half * 2 + 1) ^ swz) << 4)));
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int src = s0 + k;
          if (src < ctx.world && src != ctx.rank) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const uint32_t w4[4] = {v[k][q].x, v[k][q].y, v[k][q].z, v[k][q].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = bf16 ? __bfloat1622float2(*(const __nv_bfloat162*)&w4[e]) : __half22float2(*(const __half2*)&w4[e]);
                const int idx = half * 16 + q * 8 + e * 2;
                acc[idx] = __float_as_uint(__uint_as_float(acc[idx]) + f.x);
                acc[idx + 1] = __float_as_uint(__uint_as_float(acc[idx + 1]) + f.y);
              }
            }
          }
        }
      }
    }
  }
  IRIS_D void store_everywhere(uint8_t* local_ptr, uint4 v) const {
    if (use_mc) {
      multimem::V4 m{v.x, v.y, v.z, v.w};
      multimem::st_v4(ctx.mc(local_ptr), m);
    } else {
      *(uint4*)local_ptr = v;
      for (int p = 1; p < ctx.world; ++p) {
        int r = ctx.rank + p;
        if (r >= ctx.world) r -= ctx.world;
        *(uint4*)ctx.remote(local_ptr, r) = v;
      }
    }
  }
  IRIS_D void store16(State&, int row, int col, uint4 v) const {
    if (row >= sh.M || col >= sh.N) return;
    switch (mode) {
      case IRIS_GEMM_ALL_GATHER:
        store_everywhere(out + (((int64_t)ctx.rank * sh.M + row) * ld_out + col) * 2, v);
        break;
      case IRIS_GEMM_ALL_SCATTER:
        store_everywhere(out + ((int64_t)row * ld_out + (int64_t)ctx.rank * sh.N + col) * 2, v);
        break;
      case IRIS_GEMM_REDUCE_SCATTER:   // finished tile of my row block
        *(uint4*)(out + ((int64_t)(row - ctx.rank * tiles_m_per_rank * kBM) * ld_out + col) * 2) = v;
        break;
      case IRIS_GEMM_RS_TILES:
        *(uint4*)(out + ((int64_t)row * ld_out + col) * 2) = v;
        break;
      default:                         // ALL_REDUCE: the finished tile goes to every rank
        store_everywhere(out + ((int64_t)row * ld_out + col) * 2, v);
        break;
    }
  }
  // A tile finished elsewhere: rows [32*quarter, +32) x columns [64*chunk, +width) go to the
  // owner's staging slot as one contiguous piece.
  IRIS_D void store_chunk(State& st, int quarter, int chunk, int width, const uint8_t* smem) const {
    uint8_t* dst = st.slot + (size_t)chunk * (kBM * 64 * 2) + (size_t)quarter * (32 * width * 2);
    ptx::bulk_store(dst, smem, 32 * width * 2);
  }
  IRIS_D void tile_done(State& st, int, int) const {
    if (!reducing() || st.mine) return;
    fence_sys();
    red_release_sys_add(ctx.remote(flags + (size_t)st.buf * max_owned + st.lt, st.owner), 1);
  }
  IRIS_D void comm_main(uint8_t*, int) const {}
  IRIS_D void post_main() const {
    const int epoch = read_epoch(sb);
    // Outputs written by peers (AG, all-scatter, AR) need the cross-rank round; RS_TILES takes it
    // too because a rank that owns no tile would otherwise never learn that its peers moved on.
    // Row reduce-scatter needs none: waiting for every peer's partials in call k proves that all
    // ranks left call k-1, which is what makes the double-buffered staging safe to reuse.
    if (mode != IRIS_GEMM_REDUCE_SCATTER) {
      grid_exit_barrier(ctx, sb, epoch, 0);
    } else {
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&sb->done, 1) == (int)gridDim.x - 1) {
          sb->done = 0;
          sb->epoch = epoch + 1;
          __threadfence();
        }
      }
    }
  }
};

// ------------------------------------------------------------------------------------ host side
// Tile shape: least estimated time over `ctas` persistent CTAs; ties go to the candidate listed
// first. `bn_fixed` > 0 pins the width; pair_mode 0 = choose, 1 = single CTAs, 2 = CTA pairs (when
// `pair_ok`). The estimate is waves x tile width x a per-shape factor. Under the power cap a
// partly idle last wave costs little (the busy SMs clock higher; measured: 6.05 waves of 256-wide
// pair tiles beat 6.92 waves of 224-wide ones), so the wave count is the fractional one, at least
// one. Factors are measured: a pair tile saves 4 to 7 % (B leaves L2 once per pair), a 128-wide
// tile costs about 12 % more.
void choose_tile(int M, int N, int ctas, int bn_fixed, int pair_mode, bool pair_ok, int& bn_out, int& pair_out) {
  const int cand[3] = {256, 224, 128};
  double best = 1e30;
  bn_out = bn_fixed > 0 ? bn_fixed : 256;
  pair_out = 0;
  for (int pr = 1; pr >= 0; --pr) {
    if (pr == 1 && (!pair_ok || pair_mode == 1 || ctas < 2)) continue;
    if (pr == 0 && pair_mode == 2 && pair_ok && ctas >= 2 && (bn_fixed == 0 || bn_fixed >= 224)) continue;
    for (int i = 0; i < 3; ++i) {
      const int bn = cand[i];
      if (bn_fixed > 0 && bn != bn_fixed) continue;
      if (pr == 1 && bn == 128) continue;
      const int tiles = ceil_div(M, kBM << pr) * ceil_div(N, bn);
      const int slots = ctas >> pr;
      const double frac = (double)tiles / slots;
      const double waves = frac < 1.0 ? 1.0 : frac;
      // (a 224-wide pair tile measured 2 to 12 % slower per flop than a 256-wide one: its B halves are 112 wide)
      const double cost = waves * bn * (bn == 128 ? 1.12 : 1.0) * (pr ? (bn == 224 ? 1.05 : 0.95) : 1.0);
      if (cost < best - 1e-9) { best = cost; bn_out = bn; pair_out = pr; }
    }
  }
}

template <class Policy>
int dispatch(const Policy& pol, int bn, bool kmajor, int grid, cudaStream_t stream) {
  if (pol.pair) {
    if (kmajor) {
      if (bn == 256) return launch<Config<256, true, 6, true>>(pol, grid, stream);
      if (bn == 224) return launch<Config<224, true, 6, true>>(pol, grid, stream);
    } else {
      if (bn == 256) return launch<Config<256, false, 6, true>>(pol, grid, stream);
      if (bn == 224) return launch<Config<224, false, 6, true>>(pol, grid, stream);
    }
    return -30;
  }
  if (kmajor) {
    if (bn == 256) return launch<Config<256, true, 4>>(pol, grid, stream);
    if (bn == 224) return launch<Config<224, true, 4>>(pol, grid, stream);
    if (bn == 128) return launch<Config<128, true, 6>>(pol, grid, stream);
  } else {
    if (bn == 256) return launch<Config<256, false, 4>>(pol, grid, stream);
    if (bn == 224) return launch<Config<224, false, 4>>(pol, grid, stream);
    if (bn == 128) return launch<Config<128, false, 6>>(pol, grid, stream);
  }
  return -30;
}

int fill_common(Common& c, const IrisGemmDesc* d, int bn, int pair, int gemm_ctas, const void* A, uint64_t a_rows,
                uint64_t a_cols, int64_t lda) {
  if (d->dtype != IRIS_BF16 && d->dtype != IRIS_F16) return -2;
  if (d->N % 8 || d->K % 8) return -3;
  int r = make_map(&c.tmA, A, d->dtype, a_rows, a_cols, lda, kBK, kBM);
  if (r) return r;
  if (d->b_kmajor) r = make_map(&c.tmB, d->B, d->dtype, d->N, d->K, d->ldb, kBK, pair ? bn / 2 : bn);
  else r = make_map(&c.tmB, d->B, d->dtype, d->K, d->N, d->ldb, 64, 64);
  if (r) return r;
  c.sh = Shape{d->M, d->N, d->K};
  c.tiles_m = ceil_div(d->M, kBM);
  c.pair = pair;
  c.order_m = pair ? ceil_div(d->M, 2 * kBM) : c.tiles_m;
  c.tiles_n = ceil_div(d->N, bn);
  c.group_m = d->group_m > 0 ? d->group_m : 8;
  c.n_gemm_ctas = gemm_ctas;
  c.bf16 = d->dtype == IRIS_BF16;
  c.bn = bn;
  c.bias_row = d->bias_row;
  c.bias_col = d->bias_col;
  c.status = d->ctx.status;
  c.timeline = (int64_t*)d->timeline;
  return 0;
}

struct Plan {
  int bn, pair, gemm_ctas, comm_ctas;
  int chunks, rows_per_src, cols_per_src;
  int max_owned, tiles_m_per_rank, tiles_per_rank;
  uint64_t inbox_bytes, flags_bytes, staging_bytes;
};

int make_plan(const IrisGemmDesc* d, Plan& p) {
  memset(&p, 0, sizeof(p));
  const int W = d->ctx.world > 0 ? d->ctx.world : 1;
  const int sms = sm_count();
  const bool ag = d->op == IRIS_GEMM_AG_M || d->op == IRIS_GEMM_AG_K;
  p.comm_ctas = ag && W > 1 ? (d->comm_ctas > 0 ? d->comm_ctas : 8) : 0;
  if (ag && W > 1 && d->comm_ctas <= 0 && d->gemm_ctas <= 0) {
    // Communication CTAs are free as long as the GEMM keeps its number of waves: give them every
    // SM the last wave would leave idle (between 8 and 32).
    const int bn0 = d->bn > 0 ? d->bn : 256;
    const int tiles = ceil_div(d->M, kBM) * ceil_div(d->N, bn0);
    const int waves = ceil_div(tiles, sms - 8);
    int spare = sms - ceil_div(tiles, waves);
    if (spare > 32) spare = 32;
    if (spare < 8) spare = 8;
    spare += spare & 1;            // even, so that CTA pairs stay possible
    p.comm_ctas = spare;
  }
  p.gemm_ctas = d->gemm_ctas > 0 ? d->gemm_ctas : sms - p.comm_ctas;
  if (p.gemm_ctas + p.comm_ctas > sms) return -4;  // every CTA must be resident: consumers wait on producers
  if (d->bn != 0 && d->bn != 256 && d->bn != 224 && d->bn != 128) return -5;
  // CTA pairs need whole 256-row tiles wherever a tile's rows belong to one source or owner
  const int tiles_m = ceil_div(d->M, kBM);
  bool pair_ok = d->N >= 224 && p.comm_ctas % 2 == 0;
  switch (d->op) {
    case IRIS_GEMM_LOCAL: break;
    case IRIS_GEMM_AG_M: pair_ok = pair_ok && d->M_local % (2 * kBM) == 0; break;
    case IRIS_GEMM_REDUCE_SCATTER: pair_ok = pair_ok && d->M % (2 * kBM * W) == 0; break;
    case IRIS_GEMM_RS_TILES: pair_ok = false; break;
    default: pair_ok = pair_ok && d->M % (2 * kBM) == 0; break;
  }
  choose_tile(d->M, d->N, p.gemm_ctas, d->bn, d->two_sm, pair_ok, p.bn, p.pair);
  if (p.pair) p.gemm_ctas &= ~1;
  const int tiles_n = ceil_div(d->N, p.bn);
  if (d->op == IRIS_GEMM_AG_M) {
    if (d->M_local % kBM || d->M != d->M_local * W) return -6;
    p.rows_per_src = d->M_local; p.cols_per_src = d->K; p.chunks = d->M_local / kBM;
  } else if (d->op == IRIS_GEMM_AG_K) {
    if (d->K_local % kBK || d->K != d->K_local * W) return -6;
    p.rows_per_src = d->M; p.cols_per_src = d->K_local; p.chunks = tiles_m;
  }
  if (ag) {
    p.inbox_bytes = 2ull * W * p.rows_per_src * p.cols_per_src * 2;
    p.flags_bytes = 2ull * W * p.chunks * 4;
  }
  if (d->op == IRIS_GEMM_REDUCE_SCATTER) {
    if (tiles_m % W || d->M % (W * kBM)) return -7;
    p.tiles_m_per_rank = tiles_m / W;
    p.max_owned = p.tiles_m_per_rank * tiles_n;
  } else if (d->op == IRIS_GEMM_ALL_REDUCE) {
    p.max_owned = p.pair ? 2 * ceil_div((tiles_m / 2) * tiles_n, W) : ceil_div(tiles_m * tiles_n, W);
  } else if (d->op == IRIS_GEMM_RS_TILES) {
    p.tiles_per_rank = (tiles_m * tiles_n) / W;
    if (p.tiles_per_rank == 0) p.tiles_per_rank = 1;
    p.max_owned = tiles_m * tiles_n - p.tiles_per_rank * (W - 1);
    if (p.max_owned < p.tiles_per_rank) p.max_owned = p.tiles_per_rank;
  }
  if (p.max_owned) {
    p.staging_bytes = 2ull * W * p.max_owned * kBM * p.bn * 2;
    p.flags_bytes = 2ull * p.max_owned * 4;
  }
  return 0;
}

}  // namespace

extern "C" int iris_gemm_workspace(const IrisGemmDesc* d, uint64_t* inbox_bytes, uint64_t* flags_bytes,
                                   uint64_t* staging_bytes, int32_t* bn_out, int32_t* pair_out) {
  Plan p;
  int r = make_plan(d, p);
  if (r) return r;
  if (inbox_bytes) *inbox_bytes = p.inbox_bytes;
  if (flags_bytes) *flags_bytes = p.flags_bytes;
  if (staging_bytes) *staging_bytes = p.staging_bytes;
  if (bn_out) *bn_out = p.bn;
  if (pair_out) *pair_out = p.pair;
  return 0;
}

extern "C" int iris_gemm_launch(const IrisGemmDesc* d, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  Plan p;
  int r = make_plan(d, p);
  if (r) return r;
  const int grid = p.gemm_ctas + p.comm_ctas;
  const bool use_mc = d->use_mc && d->ctx.mc_base != 0 && d->ctx.world > 1;
  DeviceContext ctx;
  memcpy(&ctx, &d->ctx, sizeof(ctx));

  if (d->op == IRIS_GEMM_LOCAL) {
    LocalGemm pol;
    r = fill_common(pol, d, p.bn, p.pair, p.gemm_ctas, d->A, d->M, d->K, d->lda);
    if (r) return r;
    pol.C = (uint8_t*)d->C; pol.ldc = d->ldc;
    const int ctas = (pol.order_m * pol.tiles_n) << p.pair;   // no more CTAs than tiles
    return dispatch(pol, p.bn, d->b_kmajor != 0, ctas < grid ? ctas : grid, stream);
  }
  if (d->op == IRIS_GEMM_AG_M || d->op == IRIS_GEMM_AG_K) {
    AllGatherGemm pol;
    // tmA covers this rank's shard only
    r = fill_common(pol, d, p.bn, p.pair, p.gemm_ctas, d->A, p.rows_per_src, p.cols_per_src, d->lda);
    if (r) return r;
    if (ctx.world > 1) {
      r = make_map(&pol.tmInbox, d->inbox, d->dtype, 2ull * ctx.world * p.rows_per_src, p.cols_per_src, p.cols_per_src,
                   kBK, kBM);
      if (r) return r;
    } else {
      pol.tmInbox = pol.tmA;
    }
    pol.ctx = ctx; pol.sb = (SyncBlock*)d->sync_block;
    pol.A_local = (const uint8_t*)d->A; pol.lda = d->lda;
    pol.inbox = (uint8_t*)d->inbox; pol.flags = d->flags;
    pol.C = (uint8_t*)d->C; pol.ldc = d->ldc;
    pol.mode = d->op == IRIS_GEMM_AG_M ? 0 : 1;
    pol.rows_per_src = p.rows_per_src; pol.cols_per_src = p.cols_per_src; pol.chunks = p.chunks;
    pol.n_comm_ctas = p.comm_ctas; pol.use_mc = use_mc;
    if ((p.cols_per_src * 2) % 16) return -8;
    return dispatch(pol, p.bn, d->b_kmajor != 0, grid, stream);
  }
  auto fill = [&](auto& pol) -> int {
    int rr = fill_common(pol, d, p.bn, p.pair, p.gemm_ctas, d->A, d->M, d->K, d->lda);
    if (rr) return rr;
    pol.ctx = ctx; pol.sb = (SyncBlock*)d->sync_block; pol.mode = d->op;
    pol.out = (uint8_t*)d->C; pol.ld_out = d->ldc;
    pol.staging = (uint8_t*)d->staging; pol.flags = d->flags;
    pol.max_owned = p.max_owned; pol.tiles_m_per_rank = p.tiles_m_per_rank; pol.tiles_per_rank = p.tiles_per_rank;
    pol.use_mc = use_mc;
    return 0;
  };
  // reducers stride over all GEMM CTAs, so launch the full grid even for few tiles
  if (d->op == IRIS_GEMM_ALL_GATHER || d->op == IRIS_GEMM_ALL_SCATTER) {
    ScatterGemmT<false> pol;
    r = fill(pol);
    if (r) return r;
    return dispatch(pol, p.bn, d->b_kmajor != 0, grid, stream);
  }
  ScatterGemmT<true> pol;
  r = fill(pol);
  if (r) return r;
  return dispatch(pol, p.bn, d->b_kmajor != 0, grid, stream);
}
