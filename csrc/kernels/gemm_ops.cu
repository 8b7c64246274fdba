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
#include <stdlib.h>

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
    s.map = &tmA; s.x = kb * bk; s.y = tm * kBM; s.bk = kb * bk;
    s.sf_map = &tmSFA; s.sf_row = tm * kblocks + kb;
    return true;
  }
  IRIS_D void begin_tile(State&, int, int, uint8_t*) const {}
  IRIS_D int row_origin(State&, int tm) const { return tm * kBM; }
  static constexpr bool kSwiGLU = false;
  IRIS_D void store16(State&, int row, int col, uint4 v) const {
    if (row < sh.M && col < sh.N) *(uint4*)(C + ((int64_t)row * ldc + col) * 2) = v;
  }
  static constexpr bool kBulkEpilogue = true;
  IRIS_D bool bulk_tile(State&) const { return c_bulk != 0; }
  IRIS_D void store_chunk(State&, int, int, int width, const uint8_t* smem, int row, int col) const { store_chunk_local(width, smem, row, col); }
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
  // fp8: the shard's scale atoms [chunks][K blocks per source][512 B] travel with it into a second inbox
  int esz;                 // bytes per element of A: 2, or 1 (e4m3)
  int kb_per_src;          // K blocks (stages) per source column range
  CUtensorMap tmSFInbox;   // [2][W][chunks][kb_per_src] atoms
  const uint8_t* sf_local;
  uint8_t* sf_inbox;

  struct State {
    int key = -1;        // (source, chunk) whose arrival has been confirmed
    int epoch = -1;
    int tm = -1;         // tile row the cached values below belong to
    int src = 0, chunk = 0, g = 0, kb_next_src = 0, kb0 = 0;
    const CUtensorMap* map = nullptr;
    int y = 0;
    const CUtensorMap* sf_map = nullptr;
    int sf_row0 = 0;
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
      st.sf_map = &tmSFA; st.sf_row0 = chunk * kb_per_src;
      return true;
    }
    const int buf = st.epoch & 1;
    const int key = src * chunks + chunk;
    if (key != st.key) {
      const int target = ((st.epoch >> 1) + 1) * arrivals_per_chunk();
      if (!wait_flag_ge(ctx, flags + ((size_t)buf * ctx.world + src) * chunks + chunk, target)) return false;
      st.key = key;
      // The data was written by another GPU (generic proxy, remote); order the TMA (async proxy)
      // reads after the acquire.
      ptx::fence_proxy_async();
    }
    st.map = &tmInbox; st.y = ((buf * ctx.world + src) * rows_per_src) + chunk * kBM;
    st.sf_map = &tmSFInbox; st.sf_row0 = ((buf * ctx.world + src) * chunks + chunk) * kb_per_src;
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
      s.map = st.map; s.x = kb * bk; s.y = st.y; s.bk = s.x;
      s.sf_map = st.sf_map; s.sf_row = st.sf_row0 + kb;
      return true;
    }
    // K-sharded: walk the sources along K, own shard first
    if (kb == 0 || kb == st.kb_next_src) {
      st.g = kb == 0 ? 0 : st.g + 1;
      st.kb0 = st.g * kb_per_src;
      st.kb_next_src = st.kb0 + kb_per_src;
      if (!select(st, src_of_group(st.g), tm)) return false;
    }
    s.map = st.map; s.x = (kb - st.kb0) * bk; s.y = st.y; s.bk = st.src * cols_per_src + s.x;
    s.sf_map = st.sf_map; s.sf_row = st.sf_row0 + (kb - st.kb0);
    return true;
  }
  IRIS_D void begin_tile(State&, int, int, uint8_t*) const {}
  IRIS_D int row_origin(State&, int tm) const { return tm * kBM; }
  static constexpr bool kSwiGLU = false;
  IRIS_D void store16(State&, int row, int col, uint4 v) const {
    if (row < sh.M && col < sh.N) *(uint4*)(C + ((int64_t)row * ldc + col) * 2) = v;
  }
  static constexpr bool kBulkEpilogue = true;
  IRIS_D bool bulk_tile(State&) const { return c_bulk != 0; }
  IRIS_D void store_chunk(State&, int, int, int width, const uint8_t* smem, int row, int col) const { store_chunk_local(width, smem, row, col); }
  IRIS_D void tile_done(State&, int, int) const {}

  // Communication CTAs: CTA j moves slice j (of n_comm_ctas) of every 128-row chunk, chunk by chunk,
  // so chunk 0 is complete everywhere first. Three roles inside the CTA:
  //   mover    (warp 0, one thread)  streams the CTA's pieces (32 KB) through a ring of shared-memory
  //            slots without ever draining it: bulk async copy HBM -> slot, then one bulk async store per
  //            peer, loads running ahead across chunk boundaries. It never fences. A chunk whose stores
  //            were all issued is handed to the signaller once enough later traffic has been issued that
  //            waiting for its bulk groups no longer stalls (a store completes only after everything
  //            queued in front of it on the link: several microseconds), or at the end.
  //   signaller (warp 1)             waits for the hand-over, then lane p raises the chunk's arrival counter
  //            on peer p (release, system scope). The fences this needs cost a link round trip each; here
  //            they delay only the signal, not the data.
  //   scales   (warp 2, fp8 only)    copies the CTA's share of the chunk's scale atoms to the peers.
  // A chunk has arrived at a receiver when its counter shows n_comm_ctas arrivals for this call.
  static constexpr int kPiece = 32 * 1024;
  static constexpr int kSlots = 6;
  static constexpr int kMaxChunksTracked = 1024;
  IRIS_D int arrivals_per_chunk() const { return n_comm_ctas; }
  IRIS_D static void bulk_wait_upto(int n) {      // wait until at most `n` of the most recent bulk groups are pending
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
      case 9: ptx::bulk_wait<9>(); break;
      case 10: ptx::bulk_wait<10>(); break;
      case 11: ptx::bulk_wait<11>(); break;
      case 12: ptx::bulk_wait<12>(); break;
      case 13: ptx::bulk_wait<13>(); break;
      case 14: ptx::bulk_wait<14>(); break;
      case 15: ptx::bulk_wait<15>(); break;
      default: ptx::bulk_wait<16>(); break;        // more recent groups than that may stay pending either way
    }
  }
  IRIS_D void comm_main(uint8_t* smem_raw, int smem_bytes) const {
    const int j = blockIdx.x - n_gemm_ctas;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int epoch = read_epoch(sb);
    const int buf = epoch & 1;
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
    uint64_t* bars = (uint64_t*)(smem + (size_t)kSlots * kPiece);
    volatile int* handed = (volatile int*)(bars + kSlots);          // chunks handed to the signaller
    volatile int* sf_done = handed + 1;                              // chunks whose scale atoms were written (fp8)
    volatile int* aborted = handed + 2;
    int* g_last = (int*)(handed + 4);                                // per chunk: bulk groups committed when its last piece was
    if (threadIdx.x == 0) {
      for (int i = 0; i < kSlots; ++i) ptx::mbar_init(&bars[i], 1);
      *handed = 0; *sf_done = 0; *aborted = 0;
      ptx::fence_mbar_init();
      ptx::fence_proxy_async();
    }
    __syncthreads();
    const size_t row_bytes = (size_t)cols_per_src * esz;
    const size_t src_pitch = (size_t)lda * esz;
    const bool flat = src_pitch == row_bytes;
    const int pieces_per_row = (int)((row_bytes + kPiece - 1) / kPiece);
    const int tracked = min(chunks, kMaxChunksTracked);
    // this CTA's slice of chunk c: first row, rows, pieces
    auto slice = [&](int c, int& row_lo, int& nrows, int& n) {
      const int r0 = c * kBM;
      const int nrows_c = min(kBM, rows_per_src - r0);
      const int lo = (int)((int64_t)nrows_c * j / n_comm_ctas), hi = (int)((int64_t)nrows_c * (j + 1) / n_comm_ctas);
      row_lo = r0 + lo; nrows = hi - lo;
      n = nrows == 0 ? 0 : (flat ? (int)(((size_t)nrows * row_bytes + kPiece - 1) / kPiece) : nrows * pieces_per_row);
    };
    auto piece = [&](int i, int nrows, size_t& soff, size_t& doff, uint32_t& bytes) {
      if (flat) {
        soff = doff = (size_t)i * kPiece;
        bytes = (uint32_t)min((size_t)kPiece, (size_t)nrows * row_bytes - soff);
      } else {
        const int r = i / pieces_per_row, k = i - r * pieces_per_row;
        soff = (size_t)r * src_pitch + (size_t)k * kPiece;
        doff = (size_t)r * row_bytes + (size_t)k * kPiece;
        bytes = (uint32_t)min((size_t)kPiece, row_bytes - (size_t)k * kPiece);
      }
    };
    if (w == 0 && lane == 0) {
      // ---------------------------------------------------------------- mover
      // two cursors over the CTA's pieces in (chunk, piece) order: `ld` runs ahead of `st` by up to kSlots
      int ld_c = 0, ld_i = 0, ld_seq = 0;
      int st_seq = 0;
      int groups = 0, next_hand = 0;
      bool ok = true;
      // a chunk is handed over once this many groups were committed after its last one
      const int depth = max(1, min(16, (12 + ctx.world - 2) / (ctx.world - 1)));
      auto advance_ld = [&]() -> bool {           // move `ld` to the next existing piece; false at the end
        while (ld_c < chunks) {
          int row_lo, nrows, n;
          slice(ld_c, row_lo, nrows, n);
          if (ld_i < n) return true;
          ++ld_c; ld_i = 0;
        }
        return false;
      };
      auto issue_load = [&]() {
        int row_lo, nrows, n;
        slice(ld_c, row_lo, nrows, n);
        size_t so, d_o; uint32_t by;
        piece(ld_i, nrows, so, d_o, by);
        const int s = ld_seq % kSlots;
        ptx::mbar_expect_tx(&bars[s], by);
        ptx::bulk_load(smem + (size_t)s * kPiece, A_local + (size_t)row_lo * src_pitch + so, by, &bars[s]);
        ++ld_seq; ++ld_i;
      };
      auto hand_over = [&](bool all) {
        const int before = next_hand;
        while (next_hand < chunks) {
          const int gl = next_hand < tracked ? g_last[next_hand] : groups;
          if (gl < 0) break;                                       // its last piece has not been issued yet
          if (!all && groups - gl < depth) break;
          bulk_wait_upto(groups - gl);
          ++next_hand;
        }
        if (next_hand == before) return;
        ptx::fence_proxy_async();
        asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(ptx::smem_u32((const void*)handed)), "r"(next_hand) : "memory");
      };
      for (int c = 0; c < tracked; ++c) g_last[c] = -1;
      while (ld_seq < kSlots && advance_ld()) issue_load();
      for (int c = 0; c < chunks && ok; ++c) {
        int row_lo, nrows, n;
        slice(c, row_lo, nrows, n);
        uint8_t* dst_local = inbox + (((size_t)buf * ctx.world + ctx.rank) * rows_per_src + row_lo) * row_bytes;
        for (int i = 0; i < n; ++i) {
          const int s = st_seq % kSlots;
          if (!ptx::mbar_wait(&bars[s], (uint32_t)((st_seq / kSlots) & 1), kPipeTimeoutNs)) { fail(kTimeoutPipeline); ok = false; break; }
          size_t so, d_o; uint32_t by;
          piece(i, nrows, so, d_o, by);
          for (int p = 1; p < ctx.world; ++p) {
            int dst_rank = ctx.rank + p;
            if (dst_rank >= ctx.world) dst_rank -= ctx.world;
            ptx::bulk_store(ctx.remote(dst_local, dst_rank) + d_o, smem + (size_t)s * kPiece, by);
          }
          ptx::bulk_commit();
          ++groups; ++st_seq;
          ptx::bulk_wait_read<1>();                  // every slot but the one just sent has been read out
          while (ld_seq < st_seq - 1 + kSlots && advance_ld()) issue_load();
          if (i == n - 1 && c < tracked) g_last[c] = groups;
          hand_over(false);
        }
        if (n == 0 && c < tracked) { g_last[c] = groups; hand_over(false); }
      }
      if (ok) hand_over(true);
      else *aborted = 1;
    } else if (w == 1) {
      // ---------------------------------------------------------------- signaller
      const uint64_t t0 = now_ns();
      for (int c = 0; c < chunks; ++c) {
        bool ok = true;
        unsigned spins = 0;
        while (true) {
          int h, sfd = chunks;
          asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(h) : "r"(ptx::smem_u32((const void*)handed)) : "memory");
          if (sf_local) asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(sfd) : "r"(ptx::smem_u32((const void*)sf_done)) : "memory");
          if (h > c && sfd > c) break;
          if (*aborted || ((++spins & 1023u) == 0 && now_ns() - t0 > 2 * kPipeTimeoutNs)) { ok = false; break; }
          __nanosleep(64);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        int32_t* flag_local = flags + ((size_t)buf * ctx.world + ctx.rank) * chunks + c;
        fence_sys();
        for (int r = lane; r < ctx.world; r += 32)
          if (r != ctx.rank) red_release_sys_add(ctx.remote(flag_local, r), 1);
        if (lane == 0 && j == 0) stamp(tiles_m * tiles_n + c, 3);
      }
    } else if (w == 2 && sf_local) {
      // ---------------------------------------------------------------- scale atoms (fp8)
      const size_t sf_chunk = (size_t)kb_per_src * 512;
      const size_t sf_lo = (sf_chunk / 16 * j / n_comm_ctas) * 16, sf_hi = (sf_chunk / 16 * (j + 1) / n_comm_ctas) * 16;
      for (int c = 0; c < chunks; ++c) {
        const uint8_t* sf_src = sf_local + (size_t)c * sf_chunk;
        uint8_t* sf_dst = sf_inbox + (((size_t)buf * ctx.world + ctx.rank) * chunks + c) * sf_chunk;
        for (size_t u = sf_lo + lane * 16; u < sf_hi; u += 32 * 16) {
          const uint4 v = *(const uint4*)(sf_src + u);
          for (int p = 1; p < ctx.world; ++p) {
            int dst_rank = ctx.rank + p;
            if (dst_rank >= ctx.world) dst_rank -= ctx.world;
            *(uint4*)(ctx.remote(sf_dst, dst_rank) + u) = v;
          }
        }
        __threadfence_system();
        __syncwarp();
        if (lane == 0) asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(ptx::smem_u32((const void*)sf_done)), "r"(c + 1) : "memory");
      }
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
  static constexpr bool kBulkEpilogue = true;
  DeviceContext ctx;
  SyncBlock* sb;
  int mode;               // IrisGemmOp
  // ALL_GATHER / ALL_SCATTER with communication CTAs ("workgroup specialised", the reference's
  // examples/10_gemm_all_scatter_wg_specialization): the GEMM CTAs store each tile into THIS rank's
  // copy of the output (tensor stores at row / column offset out_roff / out_coff) and publish a per-tile
  // flag; the communication CTAs wait for the flag and forward the tile to every peer.
  int wg_spec;
  int out_roff, out_coff;
  int n_comm_ctas;
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
    s.map = &tmA; s.x = kb * bk; s.y = tm * kBM; s.bk = kb * bk;
    s.sf_map = &tmSFA; s.sf_row = tm * kblocks + kb;
    return true;
  }
  IRIS_D bool reducing() const {
    return mode == IRIS_GEMM_REDUCE_SCATTER || mode == IRIS_GEMM_ALL_REDUCE || mode == IRIS_GEMM_RS_TILES;
  }
  static constexpr bool kSwiGLU = false;
  IRIS_D int row_origin(State&, int tm) const { return tm * kBM; }
  IRIS_D void begin_tile(State& st, int tm, int tn, uint8_t*) const {
    if ((mode == IRIS_GEMM_AR_ONE_SHOT || wg_spec) && st.buf < 0) {
      const int e = read_epoch(sb);
      st.buf = e & 1;
      st.target = (e >> 1) + 1;
    }
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
  // A tile finished elsewhere always leaves as bulk stores into the owner's staging; a tile finished here
  // leaves through the output's tensor maps when it stays on this rank (reduce-scatter), and by rows
  // when every rank gets it (all-reduce: multimem / per-peer stores).
  IRIS_D bool bulk_tile(State& st) const {
    if (!reducing()) return wg_spec != 0;
    return !st.mine || (c_bulk != 0 && mode != IRIS_GEMM_ALL_REDUCE);
  }
  IRIS_D bool signals_tile(State& st) const { return reducing() ? !st.mine : wg_spec != 0; }
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
  // Add the 8 16-bit values to the same place of every rank's output (remote atomics; in the switch with NVLS).
  IRIS_D void add_everywhere(uint8_t* local_ptr, uint4 v) const {
    if (use_mc) {
      multimem::V4 m{v.x, v.y, v.z, v.w};
      if (bf16) multimem::red_add_bf16x8(ctx.mc(local_ptr), m);
      else multimem::red_add_f16x8(ctx.mc(local_ptr), m);
      return;
    }
    const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
    for (int p = 0; p < ctx.world; ++p) {
      int r = ctx.rank + p;
      if (r >= ctx.world) r -= ctx.world;
      uint8_t* dst = ctx.remote(local_ptr, r);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (bf16) asm volatile("red.relaxed.sys.global.add.noftz.bf16x2 [%0], %1;" ::"l"(dst + 4 * e), "r"(w4[e]) : "memory");
        else asm volatile("red.relaxed.sys.global.add.noftz.f16x2 [%0], %1;" ::"l"(dst + 4 * e), "r"(w4[e]) : "memory");
      }
    }
  }
  IRIS_D void store16(State& st, int row, int col, uint4 v) const {
    if (row >= sh.M || col >= sh.N) return;
    switch (mode) {
      case IRIS_GEMM_AR_ONE_SHOT:      // my partial, into slot [call parity][my rank] of every rank's staging
        store_everywhere(staging + ((((size_t)st.buf * ctx.world + ctx.rank) * sh.M + row) * sh.N + col) * 2, v);
        break;
      case IRIS_GEMM_AR_ATOMIC:
        add_everywhere(out + ((int64_t)row * ld_out + col) * 2, v);
        break;
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
  IRIS_D void store_chunk(State& st, int quarter, int chunk, int width, const uint8_t* smem, int row, int col) const {
    if (!reducing()) {            // workgroup-specialised gather / scatter: into this rank's own copy of the output
      store_chunk_local(width, smem, row + out_roff, col + out_coff);
      return;
    }
    if (st.mine) {
      store_chunk_local(width, smem, mode == IRIS_GEMM_REDUCE_SCATTER ? row - ctx.rank * tiles_m_per_rank * kBM : row, col);
      return;
    }
    uint8_t* dst = st.slot + (size_t)chunk * (kBM * 64 * 2) + (size_t)quarter * (32 * width * 2);
    ptx::bulk_store(dst, smem, 32 * width * 2);
  }
  IRIS_D void tile_done(State& st, int tm, int tn) const {
    if (mode == IRIS_GEMM_AR_ONE_SHOT) {       // this tile of my partial is on its way to every rank: count it everywhere
      int32_t* fl = flags + (size_t)st.buf * max_owned + (tm * tiles_n + tn);
      fence_sys();
      if (use_mc) {
        multimem::red_release_add_u32(ctx.mc(fl), 1);
      } else {
        for (int p = 0; p < ctx.world; ++p) {
          int r = ctx.rank + p;
          if (r >= ctx.world) r -= ctx.world;
          red_release_sys_add(ctx.remote(fl, r), 1);
        }
      }
      return;
    }
    if (wg_spec && !reducing()) {   // the tile is in this rank's output (its stores have completed): tell the communication CTAs
      __threadfence();
      st_release_gpu(flags + (size_t)st.buf * max_owned + (tm * tiles_n + tn), st.target);
      return;
    }
    if (!reducing() || st.mine) return;
    fence_sys();
    red_release_sys_add(ctx.remote(flags + (size_t)st.buf * max_owned + st.lt, st.owner), 1);
  }
  // One-shot all-reduce, second half: the CTAs share out the output tiles; a tile is summed (fp32) over
  // the W partials in this rank's staging once its counter shows W arrivals for this call. Only this
  // rank's own output is written, so the kernel needs no cross-rank round at its end: collecting every
  // rank's partials for call k proves that all ranks have left call k - 1 (the parity double-buffering).
  IRIS_D void one_shot_reduce(int epoch) const {
    __shared__ int s_ok;
    const int buf = epoch & 1;
    const int32_t target = ((epoch >> 1) + 1) * ctx.world;
    const int units_per_row = bn / 8;
    for (int t = blockIdx.x; t < tiles_m * tiles_n; t += gridDim.x) {
      __syncthreads();
      if (threadIdx.x == 0) s_ok = wait_flag_ge(ctx, flags + (size_t)buf * max_owned + t, target) ? 1 : 0;
      __syncthreads();
      if (!s_ok) return;
      const int tm = t / tiles_n, tn = t - tm * tiles_n;
      for (int u = threadIdx.x; u < kBM * units_per_row; u += blockDim.x) {
        const int r = u / units_per_row, row = tm * kBM + r, col = tn * bn + (u - r * units_per_row) * 8;
        if (row >= sh.M || col >= sh.N) continue;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int src = 0; src < ctx.world; ++src) {
          const uint4 v = __ldcg((const uint4*)(staging + ((((size_t)buf * ctx.world + src) * sh.M + row) * sh.N + col) * 2));
          const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = bf16 ? __bfloat1622float2(*(const __nv_bfloat162*)&w4[e]) : __half22float2(*(const __half2*)&w4[e]);
            acc[2 * e] += f.x; acc[2 * e + 1] += f.y;
          }
        }
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (bf16) { __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]); o[e] = *(uint32_t*)&h; }
          else { __half2 h = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]); o[e] = *(uint32_t*)&h; }
        }
        *(uint4*)(out + ((int64_t)row * ld_out + col) * 2) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  // Communication CTAs of the workgroup-specialised gather / scatter: CTA j forwards the 128-row tiles
  // j, j + n, ... in the order the GEMM CTAs finish them. For each it waits for the tile's flag (acquire),
  // then every thread moves 16-byte pieces of the tile from this rank's output to the same place on every
  // peer (one multimem.st with NVLS, else one store per peer), eight loads in flight per thread.
  IRIS_D void comm_main(uint8_t*, int) const {
    if (!wg_spec) return;
    __shared__ int s_ok;
    const int j = blockIdx.x - n_gemm_ctas;
    const int epoch = read_epoch(sb);
    const int buf = epoch & 1;
    const int32_t target = (epoch >> 1) + 1;
    const int units_per_row = bn / 8;
    const int n_order = order_m * tiles_n;
    for (int q = j; q < (n_order << pair); q += n_comm_ctas) {
      // 128-row tiles in the order of the tile walk; a pair tile contributes its two halves one after the other
      int om, tn;
      swizzled_tile(q >> pair, order_m, tiles_n, group_m, om, tn);
      const int tm = pair ? 2 * om + (q & 1) : om;
      if (tm >= tiles_m) continue;
      __syncthreads();
      if (threadIdx.x == 0) {
        const int32_t* fl = flags + (size_t)buf * max_owned + (tm * tiles_n + tn);
        bool ok = true;
        const uint64_t t0 = now_ns();
        unsigned n = 0;
        while (ld_acquire_gpu(fl) - target < 0) {
          if ((++n & 63u) == 0) {
            if (now_ns() - t0 > ctx.timeout_ns) { ok = false; fail(kTimeoutFlag); break; }
            backoff(64);
          }
        }
        s_ok = ok ? 1 : 0;
      }
      __syncthreads();
      if (!s_ok) return;
      constexpr int kUnroll = 8;
      for (int u0 = threadIdx.x; u0 < kBM * units_per_row; u0 += blockDim.x * kUnroll) {
        uint4 v[kUnroll];
        uint8_t* dst[kUnroll];
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
          const int u = u0 + k * blockDim.x;
          dst[k] = nullptr;
          if (u < kBM * units_per_row) {
            const int r = u / units_per_row, row = tm * kBM + r, col = tn * bn + (u - r * units_per_row) * 8;
            if (row < sh.M && col < sh.N) {
              dst[k] = out + ((int64_t)(row + out_roff) * ld_out + col + out_coff) * 2;
              v[k] = __ldcg((const uint4*)dst[k]);
            }
          }
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
          if (!dst[k]) continue;
          if (use_mc) {
            multimem::st_v4(ctx.mc(dst[k]), multimem::V4{v[k].x, v[k].y, v[k].z, v[k].w});
          } else {
            for (int p = 1; p < ctx.world; ++p) {
              int r = ctx.rank + p;
              if (r >= ctx.world) r -= ctx.world;
              *(uint4*)ctx.remote(dst[k], r) = v[k];
            }
          }
        }
      }
    }
    grid_exit_barrier(ctx, sb, epoch, 0);
  }
  IRIS_D void post_main() const {
    const int epoch = read_epoch(sb);
    // Outputs written by peers (AG, all-scatter, AR) need the cross-rank round; RS_TILES takes it
    // too because a rank that owns no tile would otherwise never learn that its peers moved on.
    // Row reduce-scatter needs none: waiting for every peer's partials in call k proves that all
    // ranks left call k-1, which is what makes the double-buffered staging safe to reuse.
    if (mode == IRIS_GEMM_AR_ONE_SHOT) one_shot_reduce(epoch);
    if (mode != IRIS_GEMM_REDUCE_SCATTER && mode != IRIS_GEMM_AR_ONE_SHOT) {
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
// `pair_ok`). The estimate is waves x tile width x a per-shape factor. Factors are measured with every
// configuration interleaved under one power state: a pair tile saves about 11 % (B leaves L2 once per
// pair and every stage holds less, so more K blocks are in flight), a single 224-wide tile costs 5 % more
// per flop than a single 256-wide one, a 128-wide tile about 12 % more.
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
      // a partly filled last wave costs about half of what its idle slots would suggest: the mean of the
      // fractional and the whole wave count reproduces the measured order of the 256- and 224-wide tiles
      // (8192 x 3584: 6.05 against 6.92 waves, the 224-wide tiles 9 % faster; equal wave products: equal times)
      const double waves = frac < 1.0 ? 1.0 : 0.5 * (frac + ceil(frac - 1e-9));
      // (measured with every configuration interleaved under the same power state: a pair tile costs 0.89 of a
      // single one per flop at either width; a single 224-wide tile 1.05 of a single 256-wide one)
      const double cost = waves * bn * (bn == 128 ? 1.12 : 1.0) * (pr ? 0.89 : (bn == 224 ? 1.05 : 1.0));
      if (cost < best * 0.99) { best = cost; bn_out = bn; pair_out = pr; }   // a later candidate has to win by 1 %
    }
  }
}

template <class Policy>
int dispatch(const Policy& pol, int bn, bool kmajor, int grid, cudaStream_t stream) {
  if (pol.fp8) {      // e4m3 with hardware block scaling: K-major B, tiles at most 240 wide
    if (!kmajor) return -30;
    if (pol.pair) {
      if (bn == 224) return launch<Config<224, true, 6, true, true>>(pol, grid, stream);
      return -30;
    }
    if (bn == 224) return launch<Config<224, true, 4, false, true>>(pol, grid, stream);
    if (bn == 128) return launch<Config<128, true, 5, false, true>>(pol, grid, stream);
    return -30;
  }
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

bool is_fp8(const IrisGemmDesc* d) { return d->in_dtype == IRIS_F8E4M3; }

// `sf_a_atoms`: scale atoms behind d->sf_a (rows of A this call reads directly, in 128-row tiles, times
// the K blocks of those rows).
int fill_common(Common& c, const IrisGemmDesc* d, int bn, int pair, int gemm_ctas, const void* A, uint64_t a_rows,
                uint64_t a_cols, int64_t lda) {
  if (d->dtype != IRIS_BF16 && d->dtype != IRIS_F16) return -2;
  const bool f8 = is_fp8(d);
  if (d->in_dtype != 0 && !f8 && d->in_dtype != d->dtype) return -2;
  if (d->N % 8 || d->K % (f8 ? 16 : 8)) return -3;
  const int in_dt = f8 ? IRIS_F8E4M3 : d->dtype;
  const int bk = f8 ? 128 : kBK;
  int r = make_map(&c.tmA, A, in_dt, a_rows, a_cols, lda, bk, kBM);
  if (r) return r;
  if (f8 && !d->b_kmajor) return -13;       // e4m3 weights are taken as [N, K]
  if (d->b_kmajor) r = make_map(&c.tmB, d->B, in_dt, d->N, d->K, d->ldb, bk, pair ? bn / 2 : bn);
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
  c.fp8 = f8;
  c.bk = bk;
  c.kblocks = ceil_div(d->K, bk);
  c.sfb_atoms = ceil_div(bn, 128);
  if (f8) {
    if (!d->sf_a || !d->sf_b) return -14;
    r = make_sf_map(&c.tmSFA, d->sf_a, (uint64_t)ceil_div((int)a_rows, kBM) * ceil_div((int)a_cols, bk), 1);
    if (r) return r;
    r = make_sf_map(&c.tmSFB, d->sf_b, (uint64_t)c.tiles_n * c.kblocks * c.sfb_atoms, c.sfb_atoms);
    if (r) return r;
  }
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
  uint64_t inbox_bytes, flags_bytes, staging_bytes, sf_inbox_bytes;
  int kb_per_src;
};

// Workgroup-specialised gather / scatter applies when this rank's block of the output is made of whole
// store boxes (a tensor store that overlapped the next rank's block would race with that rank's data).
bool wg_specialised(const IrisGemmDesc* d) {
  const int W = d->ctx.world > 0 ? d->ctx.world : 1;
  if (d->overlap != 1 || W < 2) return false;
  if (d->op == IRIS_GEMM_ALL_GATHER) return d->M % kBM == 0;
  if (d->op == IRIS_GEMM_ALL_SCATTER) return d->N % 64 == 0;
  return false;
}

int make_plan(const IrisGemmDesc* d, Plan& p) {
  memset(&p, 0, sizeof(p));
  const int W = d->ctx.world > 0 ? d->ctx.world : 1;
  const int sms = sm_count();
  const bool ag = d->op == IRIS_GEMM_AG_M || d->op == IRIS_GEMM_AG_K;
  p.comm_ctas = ag && W > 1 ? (d->comm_ctas > 0 ? d->comm_ctas : 8) : 0;
  // With NVLS the gather is done by a warp of every GEMM CTA: no communication CTAs unless asked for.
  if (ag && W > 1 && d->comm_ctas <= 0 && d->gemm_ctas <= 0) {
    // Communication CTAs are free as long as the GEMM keeps its number of waves: give them every
    // SM the last wave would leave idle (between 8 and 32).
    const int bn0 = d->bn > 0 ? d->bn : (is_fp8(d) ? 224 : 256);
    const int tiles = ceil_div(d->M, kBM) * ceil_div(d->N, bn0);
    const int waves = ceil_div(tiles, sms - 8);
    int spare = sms - ceil_div(tiles, waves);
    if (spare > 32) spare = 32;
    if (spare < 8) spare = 8;
    spare += spare & 1;            // even, so that CTA pairs stay possible
    p.comm_ctas = spare;
  }
  const bool wg = wg_specialised(d);
  if (wg) p.comm_ctas = d->comm_ctas > 0 ? d->comm_ctas : 16;
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
  if (is_fp8(d)) {
    // block-scaled e4m3 tiles are 224 (or 128) wide: two accumulator buffers plus the scale cells fill TMEM.
    // CTA pairs only on request.
    if (d->bn != 0 && d->bn != 224 && d->bn != 128) return -5;
    choose_tile(d->M, d->N, p.gemm_ctas, d->bn == 128 ? 128 : 224, d->two_sm == 2 ? 2 : 1, pair_ok && d->bn != 128, p.bn, p.pair);
  } else {
    choose_tile(d->M, d->N, p.gemm_ctas, d->bn, d->two_sm, pair_ok, p.bn, p.pair);
  }
  if (p.pair) p.gemm_ctas &= ~1;
  const int tiles_n = ceil_div(d->N, p.bn);
  if (d->op == IRIS_GEMM_AG_M) {
    if (d->M_local % kBM || d->M != d->M_local * W) return -6;
    p.rows_per_src = d->M_local; p.cols_per_src = d->K; p.chunks = d->M_local / kBM;
  } else if (d->op == IRIS_GEMM_AG_K) {
    if (d->K_local % (is_fp8(d) ? 128 : kBK) || d->K != d->K_local * W) return -6;
    p.rows_per_src = d->M; p.cols_per_src = d->K_local; p.chunks = tiles_m;
  }
  if (ag) {
    p.inbox_bytes = 2ull * W * p.rows_per_src * p.cols_per_src * (is_fp8(d) ? 1 : 2);
    p.flags_bytes = 2ull * W * p.chunks * 4;
    if (is_fp8(d)) {
      if (p.cols_per_src % 128 || p.rows_per_src % kBM) return -6;     // whole scale atoms per source
      p.kb_per_src = p.cols_per_src / 128;
      p.sf_inbox_bytes = 2ull * W * p.chunks * p.kb_per_src * 512;
    }
  }
  if (d->op == IRIS_GEMM_REDUCE_SCATTER) {
    if (tiles_m % W || d->M % (W * kBM)) return -7;
    p.tiles_m_per_rank = tiles_m / W;
    p.max_owned = p.tiles_m_per_rank * tiles_n;
  } else if (d->op == IRIS_GEMM_ALL_REDUCE) {
    p.max_owned = p.pair ? 2 * ceil_div((tiles_m / 2) * tiles_n, W) : ceil_div(tiles_m * tiles_n, W);
  } else if (d->op == IRIS_GEMM_AR_ONE_SHOT || wg) {
    if (d->N % 8) return -3;
    p.max_owned = tiles_m * tiles_n;            // one arrival counter / flag per 128-row tile
  } else if (d->op == IRIS_GEMM_RS_TILES) {
    p.tiles_per_rank = (tiles_m * tiles_n) / W;
    if (p.tiles_per_rank == 0) p.tiles_per_rank = 1;
    p.max_owned = tiles_m * tiles_n - p.tiles_per_rank * (W - 1);
    if (p.max_owned < p.tiles_per_rank) p.max_owned = p.tiles_per_rank;
  }
  if (p.max_owned) {
    p.staging_bytes = d->op == IRIS_GEMM_AR_ONE_SHOT ? 2ull * W * d->M * d->N * 2 : wg ? 0 : 2ull * W * p.max_owned * kBM * p.bn * 2;
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

extern "C" uint64_t iris_gemm_sf_inbox_bytes(const IrisGemmDesc* d) {
  Plan p;
  return make_plan(d, p) ? 0 : p.sf_inbox_bytes;
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
    pol.c_bulk = make_out_maps(&pol.tmC, &pol.tmC32, d->C, d->dtype, d->M, d->N, d->ldc);
    const int ctas = (pol.order_m * pol.tiles_n) << p.pair;   // no more CTAs than tiles
    return dispatch(pol, p.bn, d->b_kmajor != 0, ctas < grid ? ctas : grid, stream);
  }
  if (d->op == IRIS_GEMM_AG_M || d->op == IRIS_GEMM_AG_K) {
    AllGatherGemm pol;
    // tmA covers this rank's shard only
    r = fill_common(pol, d, p.bn, p.pair, p.gemm_ctas, d->A, p.rows_per_src, p.cols_per_src, d->lda);
    if (r) return r;
    const bool f8 = is_fp8(d);
    pol.tmSFInbox = pol.tmSFA;
    if (ctx.world > 1) {
      r = make_map(&pol.tmInbox, d->inbox, f8 ? (int)IRIS_F8E4M3 : d->dtype, 2ull * ctx.world * p.rows_per_src, p.cols_per_src,
                   p.cols_per_src, f8 ? 128 : kBK, kBM);
      if (r) return r;
      if (f8) {
        if (!d->sf_inbox) return -14;
        r = make_sf_map(&pol.tmSFInbox, d->sf_inbox, 2ull * ctx.world * p.chunks * p.kb_per_src, 1);
        if (r) return r;
      }
    } else {
      pol.tmInbox = pol.tmA;
    }
    pol.esz = f8 ? 1 : 2;
    pol.kb_per_src = p.cols_per_src / pol.bk;
    pol.sf_local = f8 ? (const uint8_t*)d->sf_a : nullptr;
    pol.sf_inbox = (uint8_t*)d->sf_inbox;
    pol.ctx = ctx; pol.sb = (SyncBlock*)d->sync_block;
    pol.A_local = (const uint8_t*)d->A; pol.lda = d->lda;
    pol.inbox = (uint8_t*)d->inbox; pol.flags = d->flags;
    pol.C = (uint8_t*)d->C; pol.ldc = d->ldc;
    pol.c_bulk = make_out_maps(&pol.tmC, &pol.tmC32, d->C, d->dtype, d->M, d->N, d->ldc);
    pol.mode = d->op == IRIS_GEMM_AG_M ? 0 : 1;
    pol.rows_per_src = p.rows_per_src; pol.cols_per_src = p.cols_per_src; pol.chunks = p.chunks;
    pol.n_comm_ctas = p.comm_ctas; pol.use_mc = use_mc;
    if ((p.cols_per_src * pol.esz) % 16) return -8;
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
    pol.c_bulk = 0;
    pol.wg_spec = 0; pol.out_roff = 0; pol.out_coff = 0; pol.n_comm_ctas = p.comm_ctas;
    if (wg_specialised(d)) {
      // this rank's block of the gathered output, as a tensor-store target
      const bool rows = d->op == IRIS_GEMM_ALL_GATHER;
      pol.out_roff = rows ? ctx.rank * d->M : 0;
      pol.out_coff = rows ? 0 : ctx.rank * d->N;
      pol.c_bulk = make_out_maps(&pol.tmC, &pol.tmC32, d->C, d->dtype, rows ? (uint64_t)ctx.world * d->M : (uint64_t)d->M,
                                 rows ? (uint64_t)d->N : (uint64_t)ctx.world * d->N, d->ldc);
      if (!pol.c_bulk || !d->flags) return -15;
      pol.wg_spec = 1;
    }
    if (d->op == IRIS_GEMM_REDUCE_SCATTER)
      pol.c_bulk = make_out_maps(&pol.tmC, &pol.tmC32, d->C, d->dtype, (uint64_t)p.tiles_m_per_rank * kBM, d->N, d->ldc);
    else if (d->op == IRIS_GEMM_RS_TILES)
      pol.c_bulk = make_out_maps(&pol.tmC, &pol.tmC32, d->C, d->dtype, d->M, d->N, d->ldc);
    return 0;
  };
  // reducers stride over all GEMM CTAs, so launch the full grid even for few tiles
  if (d->op == IRIS_GEMM_ALL_GATHER || d->op == IRIS_GEMM_ALL_SCATTER || d->op == IRIS_GEMM_AR_ONE_SHOT || d->op == IRIS_GEMM_AR_ATOMIC) {
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
