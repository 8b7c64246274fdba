// Persistent, warp-specialised GEMM main loop for sm_100a:
//   warp 0      TMA producer: cp.async.bulk.tensor (no multicast) into a ring of swizzled smem stages
//   warp 1      MMA issuer: tcgen05.mma, fp32 accumulators in TMEM, two accumulator buffers so the
//               epilogue of tile i overlaps the main loop of tile i+1
//   warps 2..5  epilogue: tcgen05.ld TMEM -> registers -> 16-bit -> smem transpose -> 16-byte stores
//
// What differs between a local GEMM and the fused compute+collective kernels is injected through
// a Policy object (tile order, where an A tile comes from and which flag guards it, where an
// output fragment goes and who is told about it, what extra "communication CTAs" do). It stands in
// for the reference's use of tritonblas' GemmContext/ScheduleContext (iris/ops/matmul_all_reduce.py:
// 95-105) plus the tile collectives of iris/mem/triton/context.py:687-997 used as GEMM epilogues.
//
// Operand layouts: A is [M, K] row-major ("K-major"). B is either [N, K] row-major (K-major, the
// nn.Linear weight layout, passed as a transposed view) or [K, N] row-major ("MN-major").
// 16-bit inputs (bf16 or fp16), fp32 accumulation, 16-bit output.
#pragma once
#include "../common.cuh"
#include "../ptx.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace iris {
namespace gemm {

constexpr int kBM = 128;         // rows of an output tile = TMEM lanes
constexpr int kBK = 64;          // K per stage: 64 x 2 B = one 128-byte swizzle row
constexpr int kUmmaK = 16;       // K of one tcgen05.mma for 16-bit inputs
constexpr int kThreads = 192;    // 6 warps
constexpr int kEpiWarps = 4;
constexpr uint64_t kPipeTimeoutNs = 4000000000ull;

// kPair_: two CTAs of a cluster compute one 256 x BN tile with tcgen05.mma.cta_group::2. Each CTA
// stages its own 128 rows of A and HALF of the B tile (so a stage is at most 32 KB, six fit, and B
// leaves L2 once per pair); the even CTA issues the MMAs for both, each CTA's 128 accumulator rows
// live in its own TMEM and each CTA runs its own epilogue.
//
// kFp8_: e4m3 operands with block scales applied by the tensor core (tcgen05.mma.kind::mxf8f6f4.
// block_scale). A stage still holds 128 bytes of K per row, i.e. 128 elements = one scale block of
// the 1 x 128 / 128 x 128 quantisation; it is consumed by four MMAs of K 32, each with its own
// UE8M0 scale byte per row (the four bytes of a block are equal when the scales come from a 128-wide
// quantiser). Per stage the producer also brings one scale atom for the tile's 128 rows of A and
// ceil(BN / 128) atoms for B (512 bytes each: row r of the atom at byte (r % 32) * 16 + (r / 32) * 4,
// four bytes = the four K groups); the MMA thread copies them to TMEM (tcgen05.cp) in front of the
// block's MMAs. The two accumulator buffers are packed BN columns apart and the scales use 16
// columns behind them, so BN is at most 240.
template <int BN_, bool kBKMajor_, int kStages_, bool kPair_ = false, bool kFp8_ = false, int kAccBufs_ = 2, int kEpiStage_ = 8192>
struct Config {
  static constexpr int kEpiStageBytes = kEpiStage_;                     // staging per epilogue warp: 8 KB, or 0 for an epilogue that stores from registers
  static constexpr int kAccBufs = kAccBufs_;                             // accumulator buffers in TMEM: 2 (the epilogue of a tile overlaps
                                                                        // the next tile's main loop) or 1 (a 256-wide fp8 tile: two would not
                                                                        // leave room for the scale cells)
  static constexpr int BN = BN_;
  static constexpr bool kBKMajor = kBKMajor_;
  static constexpr int kStages = kStages_;
  static constexpr bool kPair = kPair_;
  static constexpr bool kFp8 = kFp8_;
  static constexpr int kBKElems = kFp8_ ? 128 : kBK;                    // elements of K per stage (128 bytes per row either way)
  static constexpr int kUmmaKElems = kFp8_ ? 32 : kUmmaK;               // K of one MMA (32 bytes per row either way)
  static constexpr int kBCols = kPair_ ? BN_ / 2 : BN_;                 // columns of B staged by one CTA
  static constexpr int kABytes = kBM * kBK * 2;                         // 16 KB
  static constexpr int kBBoxes = kBKMajor_ ? 1 : (kBCols + 63) / 64;    // MN-major: 64(n) x 64(k) boxes
  static constexpr int kBBytes = kBKMajor_ ? kBCols * kBK * 2 : kBBoxes * 8192;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSfbAtoms = kFp8_ ? (BN_ + 127) / 128 : 0;       // scale atoms of B per stage (every CTA of a pair holds all of them)
  static constexpr int kSfBytes = kFp8_ ? (1 + kSfbAtoms) * 512 : 0;    // scale bytes per stage
  static constexpr int kAccCols = kFp8_ ? BN_ : 256;                    // column pitch of an accumulator buffer
  static constexpr int kSfaCol = kAccBufs_ * kAccCols;                        // TMEM columns of the scales (fp8 only): A 4, then B 4 per atom;
  static constexpr int kSfbCol = kSfaCol + 4;                           // two such sets, used by alternate K blocks, so that the copy
  static constexpr int kSfSetCols = 4 + 4 * kSfbAtoms;                  // for block kb + 1 does not wait for the MMAs of block kb
  static constexpr int kTmemCols = 512;
  static constexpr int kEpiWarpBytes = kEpiStage_ + 256;                 // per warp: 8 KB of staging (two 32-row x 64-col chunks,
                                                                        // or one 32-row x 128-col round) + 256 B of policy scratch
                                                                        // (all staging first, 1024-byte aligned, then the scratch)
  static constexpr int kEpiBytes = kEpiWarps * kEpiWarpBytes;
  static constexpr int kSmemBytes = 1024 + kStages_ * (kStageBytes + kSfBytes) + kEpiBytes + 256;
  static_assert(BN_ % 32 == 0 && BN_ >= 32 && BN_ <= 256, "BN must be a multiple of 32 up to 256");
  static_assert(!kPair_ || kBCols % 16 == 0, "a pair splits B into two halves of whole 16-column groups");
  static_assert(kStageBytes % 1024 == 0, "stages keep the 1024-byte alignment of the 128-byte swizzle");
  static_assert(kAccBufs_ == 1 || kAccBufs_ == 2, "one or two accumulator buffers");
  static_assert(!kFp8_ || (kBKMajor_ && kAccBufs_ * BN_ + 2 * (4 + 4 * kSfbAtoms) <= 512), "fp8: K-major B, and accumulators plus scales must fit TMEM");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
// K-major tile [rows][64] of 16-bit: 8-row groups are 1024 B apart (SBO); LBO unused.
IRIS_D uint64_t desc_kmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand stored as 64(k) x 64(n) boxes of 8 KB: k groups of 8 rows are 1024 B apart
// (SBO), the next 64 columns of n are one box = 8192 B further (LBO).
IRIS_D uint64_t desc_mnmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(8192 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: fp32 accumulate, A K-major, M = 128 (256 for a CTA pair).
IRIS_HD uint32_t make_idesc(int n, bool bf16, bool b_mn_major, int m = kBM) {
  uint32_t fmt = bf16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// Instruction descriptor, kind::mxf8f6f4.block_scale: e4m3 x e4m3, both K-major, UE8M0 scales.
// `sf_id` (0..3) selects which byte of the 32-bit scale cells in TMEM this MMA uses, for A and for B.
IRIS_HD uint32_t make_idesc_mxf8(int n, int m, uint32_t sf_id) {
  return (sf_id << 4) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(m >> 4) << 24) | (sf_id << 29);
}
// Shared-memory descriptor of one scale atom for tcgen05.cp: K-major, no swizzle, 8-row x 16-byte
// core matrices stacked 128 bytes apart (SBO); a single core matrix along K, so LBO is unused.
IRIS_D uint64_t desc_sf(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}

struct Shape {
  int M, N, K;
};

// Where the producer gets the A tile of (m_tile, k_block) from.
struct ASource {
  const CUtensorMap* map;
  int x, y;   // coordinates of the A box in `map`
  int bk;     // K offset of the matching B rows/columns (differs from x when A is gathered along K)
  int bn0;    // first output column of the tile inside B's N dimension (grouped GEMMs offset it per group)
  // fp8 only: where the scale atom of this (128-row tile, K block) is: row of a [atoms, 128 x u32] map
  const CUtensorMap* sf_map;
  int sf_row;
  int sfb_off;   // added to the row of B's scale atoms (grouped GEMMs: the group's first atom)
};

// GROUP_M swizzled tile order (same idea as the reference's GROUP_SIZE_M, all_reduce.py:182-187).
IRIS_D void swizzled_tile(int t, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  int per_group = group_m * tiles_n;
  int g = t / per_group;
  int first_m = g * group_m;
  int gsz = min(tiles_m - first_m, group_m);
  int r = t - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

struct Pipeline {
  uint64_t* full;        // [stages]  TMA bytes landed
  uint64_t* empty;       // [stages]  MMAs that read the stage retired
  uint64_t* tmem_full;   // [2]       accumulator complete
  uint64_t* tmem_empty;  // [2]       accumulator drained by the epilogue
};

// The kernel body. `Policy` must provide:
//   Shape shape() const;  int gemm_ctas() const;  int num_tiles() const;
//   void tile(int t, int& m_tile, int& n_tile) const;
//   struct State;                                          (mutable per-thread scratch of the hooks)
//   bool a_source(State&, int m_tile, int kb, ASource& s) const;   (producer warp, all lanes; false = abort)
//   const CUtensorMap* b_map() const;  bool is_bf16() const;
//   void begin_tile(State&, int m_tile, int n_tile, uint8_t* warp_scratch) const;
//        (every epilogue thread, before a tile's stores; warp_scratch: 256 bytes of shared memory
//         private to the warp)
//   int row_origin(State&, int m_tile) const;              (first output row of the tile: m_tile*128
//        for a plain GEMM, the group's row offset for a grouped one)
//   static constexpr bool kSwiGLU;                         (row-major path: the tile's columns are
//        [gate 128 | up 128]; emit silu(gate) * up, 128 columns per 256-wide tile)
//   void store16(State&, int row, int col, uint4 v) const; (8 consecutive outputs of one row)
//   float row_bias(int row) const;  float col_bias(int col) const;  bool has_bias() const;
//   static constexpr bool kSfaFromRows;  void sfa_fill(State&, int m_tile, int kb, uint8_t* atom, int lane) const;
//        (fp8: the producer warp builds A's 512-byte scale atom itself, lane l writing bytes [16 l, 16 l + 16))
//   static constexpr bool kQuantOut;  void store_q32(State&, int row, int col, uint4, uint4) const;
//        void store_row_scale(State&, int row, int n_tile, uint32_t ue8m0) const;
//        (SwiGLU epilogue that writes e4m3 values, 32 per call, and one scale byte per row and tile)
//   static constexpr bool kBulkEpilogue;                   (true: tiles may leave through store_chunk)
//   bool bulk_tile(State&) const;                          (this tile leaves in 64-column chunks staged in
//        shared memory in the 128-byte-swizzle layout, each stored by ONE asynchronous bulk / tensor store)
//   void store_chunk(State&, int quarter, int chunk, int width, const uint8_t* smem, int row, int col) const;
//        (lane 0 of an epilogue warp: issue the store of rows [32*quarter, +32) x columns
//         [64*chunk, +width) of the current tile, i.e. output rows [row, +32) x columns [col, +width))
//   bool signals_tile(State&) const;                       (tile_done tells a peer about the tile, so its
//        stores must be complete, not just issued, before that)
//   bool reduce_here(State&) const;                        (this tile is finished on this rank: the other
//        ranks' partials are added to the accumulators first)
//   void add_partials(State&, int quarter, int c32, int lane, uint32_t (&acc)[32]) const;
//        (add to the fp32 accumulators of row `lane` of the quarter, columns [32*c32, +32))
//   void tile_done(State&, int m_tile, int n_tile) const;  (one thread, after the tile's stores)
//   void comm_main(uint8_t* smem, int smem_bytes) const;    (CTAs with blockIdx.x >= gemm_ctas())
//   void post_main() const;                                 (GEMM CTAs, all threads, after their tiles)
//   void fail(int code) const;
//   void stamp(int tile_seq, int what) const;              (optional per-tile timestamps: 0 tile
//        start, 1 first A tile available, 2 tile stored; reference examples collect the same with
//        COLLECT_TIMESTAMPS, examples/07_gemm_all_scatter/gemm_all_scatter.py:64-66)
// The policy is a __grid_constant__ kernel parameter (its tensor maps are used in place), so every
// hook is const.
//
// Pair configurations (Cfg::kPair): tile() is asked for PAIR tiles (its m index counts 256-row
// tiles); every other hook sees 128-row tile indices (2 * pair_m + cluster rank). Barrier wiring
// (L = even CTA, P = odd CTA):
//   full[s]        lives in L; both CTAs' TMA loads complete_tx on it (the .cta_group::2 load form
//                  with L's barrier address, no multicast); L arms it with both CTAs' byte count.
//   empty[s]       one per CTA; L's MMA thread releases both with one multicast tcgen05.commit.
//   tmem_full[b]   one per CTA, signalled by a multicast commit; tmem_empty[b] lives in L and
//                  counts the epilogue warps of both CTAs (P arrives remotely).
template <class Cfg, class Policy>
IRIS_D void gemm_cta_main(const Policy& pol, uint8_t* smem_raw) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const Shape sh = pol.shape();
  constexpr bool kPair = Cfg::kPair;
  uint32_t cta = 0;
  if constexpr (kPair) cta = ptx::cluster_ctarank();
  const bool leader = cta == 0;

  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  // epilogue staging: 8 KB per warp, 1024-byte aligned (tensor stores apply the hardware swizzle to
  // absolute shared-memory addresses), then 256 bytes of policy scratch per warp, then the scales
  uint8_t* epi_base = smem + Cfg::kStages * Cfg::kStageBytes;
  uint8_t* scratch_base = epi_base + kEpiWarps * Cfg::kEpiStageBytes;
  uint8_t* sf_base = scratch_base + kEpiWarps * 256;               // fp8: per stage one scale atom of A, then B's
  uint64_t* bars = (uint64_t*)(sf_base + Cfg::kStages * Cfg::kSfBytes);
  Pipeline pipe{bars, bars + Cfg::kStages, bars + 2 * Cfg::kStages, bars + 2 * Cfg::kStages + 2};
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * Cfg::kStages + 4);

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      ptx::mbar_init(&pipe.full[s], 1);
      ptx::mbar_init(&pipe.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&pipe.tmem_full[b], 1);
      ptx::mbar_init(&pipe.tmem_empty[b], kEpiWarps * (kPair ? 2 : 1));
    }
    ptx::fence_mbar_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    if constexpr (kPair) {
      ptx::tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);   // one warp of each CTA of the pair
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (kPair) ptx::cluster_sync();   // both CTAs' barriers exist before anyone signals remotely
  ptx::tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;

  const int num_tiles = pol.num_tiles();
  const int k_blocks = (sh.K + Cfg::kBKElems - 1) / Cfg::kBKElems;
  const int first = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int step = kPair ? pol.gemm_ctas() >> 1 : pol.gemm_ctas();
  // the epilogue warp's arrival that hands an accumulator buffer back to the MMA issuer
  auto release_acc = [&](int buf) {
    if (!kPair || leader) ptx::mbar_arrive(&pipe.tmem_empty[buf]);
    else ptx::mbar_arrive_cluster(&pipe.tmem_empty[buf], 0);
  };

  const uint32_t stage0 = ptx::smem_u32(stage_base), sf0 = ptx::smem_u32(sf_base);
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) ptx::prefetch_tmap(pol.b_map());
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    typename Policy::State st;
    for (int t = first; t < num_tiles && ok; t += step) {
      int tm, tn;
      pol.tile(t, tm, tn);
      if constexpr (kPair) tm = 2 * tm + (int)cta;
      if (lane == 0) pol.stamp(t, 0);
      for (int kb = 0; kb < k_blocks; ++kb) {
        ASource as;
        as.bn0 = tn * Cfg::BN;
        as.sfb_off = 0;
        if (!__all_sync(0xffffffffu, pol.a_source(st, tm, kb, as))) { ok = false; break; }
        if (kb == 0 && lane == 0) pol.stamp(t, 1);
        if (!__all_sync(0xffffffffu, ptx::mbar_wait<kPair>(&pipe.empty[s], ph ^ 1, kPipeTimeoutNs))) { pol.fail(kTimeoutPipeline); ok = false; break; }
        if constexpr (Cfg::kFp8 && Policy::kSfaFromRows) {
          // A's scale atom is put together here from one scale byte per row (rows that arrived one by one,
          // e.g. dispatched tokens, have no ready-made atom): lane l writes the 16 bytes of rows l, l + 32,
          // l + 64, l + 96. Generic-proxy stores, made visible to tcgen05.cp by the proxy fence; the arrive
          // below (after the warp barrier) publishes them together with the TMA bytes.
          static_assert(!kPair, "scale atoms built from rows: single-CTA tiles only");
          pol.sfa_fill(st, tm, kb, sf_base + s * Cfg::kSfBytes, lane);
          ptx::fence_proxy_async_smem();
          __syncwarp();
        }
        // the warp stays converged and every instruction elects its issuing lane (see the MMA issuer)
        const uint32_t sa = stage0 + s * Cfg::kStageBytes;
        const uint32_t sb = sa + Cfg::kABytes;
        if constexpr (kPair) {
          if (leader) ptx::mbar_expect_tx_elect(&pipe.full[s], 2 * (Cfg::kStageBytes + Cfg::kSfBytes));
          const int n0 = as.bn0 + (int)cta * Cfg::kBCols;
          ptx::tma_load_2d_pair_elect(sa, as.map, &pipe.full[s], as.x, as.y);
          if constexpr (Cfg::kBKMajor) {
            ptx::tma_load_2d_pair_elect(sb, pol.b_map(), &pipe.full[s], as.bk, n0);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::kBBoxes; ++j)
              ptx::tma_load_2d_pair_elect(sb + j * 8192, pol.b_map(), &pipe.full[s], n0 + j * 64, as.bk);
          }
        } else {
          ptx::mbar_expect_tx_elect(&pipe.full[s], Cfg::kStageBytes + Cfg::kSfBytes - ((Cfg::kFp8 && Policy::kSfaFromRows) ? 512 : 0));
          ptx::tma_load_2d_elect(sa, as.map, &pipe.full[s], as.x, as.y);
          if constexpr (Cfg::kBKMajor) {
            ptx::tma_load_2d_elect(sb, pol.b_map(), &pipe.full[s], as.bk, as.bn0);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::kBBoxes; ++j)
              ptx::tma_load_2d_elect(sb + j * 8192, pol.b_map(), &pipe.full[s], as.bn0 + j * 64, as.bk);
          }
        }
        if constexpr (Cfg::kFp8) {
          // scale atoms: this tile's 128 rows of A, and all of the tile's columns of B (each
          // CTA of a pair keeps the whole of B's scales: its MMA half multiplies every column)
          const uint32_t ssf = sf0 + s * Cfg::kSfBytes;
          const int brow = pol.b_sf_row(tn, as.bk / Cfg::kBKElems) + as.sfb_off;   // B's K block: not kb when A is gathered along K
          if constexpr (kPair) {
            ptx::tma_load_2d_pair_elect(ssf, as.sf_map, &pipe.full[s], 0, as.sf_row);
            ptx::tma_load_2d_pair_elect(ssf + 512, pol.sfb_map(), &pipe.full[s], 0, brow);
          } else {
            if constexpr (!Policy::kSfaFromRows) ptx::tma_load_2d_elect(ssf, as.sf_map, &pipe.full[s], 0, as.sf_row);
            ptx::tma_load_2d_elect(ssf + 512, pol.sfb_map(), &pipe.full[s], 0, brow);
          }
        }
        if (++s == Cfg::kStages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The warp stays converged: every lane computes the (warp-uniform) descriptors and each tensor-core
    // instruction elects the lane that issues it. Issued from inside `if (lane == 0)` every instruction
    // cost this warp 100 to 150 cycles, more than a fifth of a K block's MMA time.
    const uint32_t idesc = make_idesc(Cfg::BN, pol.is_bf16(), !Cfg::kBKMajor, kPair ? 2 * kBM : kBM);
    // warp reductions and votes give the compiler values it knows to be the same in every lane (the TMEM
    // base comes out of shared memory, the waits return per lane), which keeps the loop state uniform
    const uint32_t tmem_u = __reduce_or_sync(0xffffffffu, tmem_base);
    int s = 0;
    uint32_t ph = 0;
    int it = 0;
    bool ok = leader;      // the even CTA of a pair issues for both
    for (int t = first; t < num_tiles && ok; t += step, ++it) {
      const int buf = Cfg::kAccBufs == 2 ? (it & 1) : 0;
      const uint32_t acc_ph = Cfg::kAccBufs == 2 ? ((it >> 1) & 1) : (it & 1);
      if (!__all_sync(0xffffffffu, ptx::mbar_wait<kPair>(&pipe.tmem_empty[buf], acc_ph ^ 1, kPipeTimeoutNs))) { pol.fail(kTimeoutPipeline); break; }
      ptx::tc_fence_after();
      const uint32_t d_tmem = tmem_u + buf * Cfg::kAccCols;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait<kPair>(&pipe.full[s], ph, kPipeTimeoutNs))) { pol.fail(kTimeoutPipeline); ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t sa = stage0 + s * Cfg::kStageBytes;
        const uint32_t sb = sa + Cfg::kABytes;
        if constexpr (Cfg::kFp8) {
          // this block's scales: shared memory -> TMEM, in front of the MMAs that use them (the
          // copies and the MMAs of one thread execute in issue order, so the cells are rewritten
          // only after the previous block's MMAs have read them)
          const uint32_t ssf = sf0 + s * Cfg::kSfBytes;
          const uint32_t t_sfa = tmem_u + Cfg::kSfaCol + (kb & 1) * Cfg::kSfSetCols, t_sfb = t_sfa + 4;
          if constexpr (kPair) {
            ptx::tmem_cp_sf_pair_elect(t_sfa, desc_sf(ssf));
#pragma unroll
            for (int j = 0; j < Cfg::kSfbAtoms; ++j) ptx::tmem_cp_sf_pair_elect(t_sfb + 4 * j, desc_sf(ssf + 512 + 512 * j));
          } else {
            ptx::tmem_cp_sf_elect(t_sfa, desc_sf(ssf));
#pragma unroll
            for (int j = 0; j < Cfg::kSfbAtoms; ++j) ptx::tmem_cp_sf_elect(t_sfb + 4 * j, desc_sf(ssf + 512 + 512 * j));
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {     // four MMAs of K 32, each with its own scale byte
            const uint64_t ad = desc_kmajor(sa + k * 32), bd = desc_kmajor(sb + k * 32);
            const uint32_t id8 = make_idesc_mxf8(Cfg::BN, kPair ? 2 * kBM : kBM, (uint32_t)k);
            if constexpr (kPair) ptx::mma_mxf8_pair_elect(d_tmem, ad, bd, id8, (kb | k) != 0, t_sfa, t_sfb);
            else ptx::mma_mxf8_elect(d_tmem, ad, bd, id8, (kb | k) != 0, t_sfa, t_sfb);
          }
        } else {
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t ad = desc_kmajor(sa + k * (kUmmaK * 2));
            const uint64_t bd = Cfg::kBKMajor ? desc_kmajor(sb + k * (kUmmaK * 2)) : desc_mnmajor(sb + k * (kUmmaK * 128));
            if constexpr (kPair) ptx::mma_f16_pair_elect(d_tmem, ad, bd, idesc, (kb | k) != 0);
            else ptx::mma_f16_elect(d_tmem, ad, bd, idesc, (kb | k) != 0);
          }
        }
        if constexpr (kPair) {
          ptx::mma_commit_pair_elect(&pipe.empty[s], 3);
          if (kb == k_blocks - 1) ptx::mma_commit_pair_elect(&pipe.tmem_full[buf], 3);
        } else {
          ptx::mma_commit_elect(&pipe.empty[s]);
          if (kb == k_blocks - 1) ptx::mma_commit_elect(&pipe.tmem_full[buf]);
        }
        if (++s == Cfg::kStages) { s = 0; ph ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    uint8_t* my_epi = epi_base + (warp - 2) * Cfg::kEpiStageBytes;
    uint32_t chunk_seq = 0;   // bulk epilogue: chunks issued by this warp (selects the staging half)
    const bool bf16 = pol.is_bf16();
    const bool has_bias = pol.has_bias();
    typename Policy::State est;
    int it = 0;
    for (int t = first; t < num_tiles; t += step, ++it) {
      const int buf = Cfg::kAccBufs == 2 ? (it & 1) : 0;
      const uint32_t acc_ph = Cfg::kAccBufs == 2 ? ((it >> 1) & 1) : (it & 1);
      int tm, tn;
      pol.tile(t, tm, tn);
      if constexpr (kPair) tm = 2 * tm + (int)cta;
      // A wait that runs out still goes through this tile's named barrier (the other epilogue
      // warps may have got through) and leaves afterwards.
      const bool live = ptx::mbar_wait<kPair>(&pipe.tmem_full[buf], acc_ph, kPipeTimeoutNs);
      if (!live) {
        pol.fail(kTimeoutPipeline);
        ptx::named_barrier(1, kEpiWarps * 32);
        break;
      }
      ptx::tc_fence_after();
      pol.begin_tile(est, tm, tn, scratch_base + (warp - 2) * 256);
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * Cfg::kAccCols;
      const int row0 = pol.row_origin(est, tm) + quarter * 32;
      const float rb = has_bias ? pol.row_bias(row0 + lane) : 0.f;
      // fp32 accumulators of 32 columns -> 16-bit pairs (bias added)
      auto pack32 = [&](const uint32_t (&r)[32], int col0, uint32_t (&packed)[16]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float a = __uint_as_float(r[2 * j]) + rb, b = __uint_as_float(r[2 * j + 1]) + rb;
          if (has_bias) { a += pol.col_bias(col0 + 2 * j); b += pol.col_bias(col0 + 2 * j + 1); }
          if (bf16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            packed[j] = *(uint32_t*)&h;
          } else {
            __half2 h = __floats2half2_rn(a, b);
            packed[j] = *(uint32_t*)&h;
          }
        }
      };
      bool bulk = false;
      if constexpr (Policy::kBulkEpilogue) bulk = pol.bulk_tile(est);
      if (bulk) {
        // The tile leaves in 64-column chunks: TMEM -> registers -> swizzled shared memory, then
        // ONE bulk async store per chunk (4 KB, or 2 KB for a 32-column tail) issued by lane 0
        // through the policy. Two staging halves per warp: a half is rewritten only after the
        // store that read it has finished reading (wait_group.read).
        constexpr int kChunks = (Cfg::BN + 63) / 64;
#pragma unroll 1
        for (int cc = 0; cc < kChunks; ++cc) {
          const int w = (Cfg::BN - cc * 64) >= 64 ? 64 : 32;   // columns in this chunk
          uint8_t* stage = my_epi + (chunk_seq & 1) * 4096;
          if (lane == 0) ptx::bulk_wait_read<1>();
          __syncwarp();
#pragma unroll 1
          for (int hlf = 0; hlf < w / 32; ++hlf) {
            uint32_t r[32];
            ptx::tmem_ld_32x32(t_addr + cc * 64 + hlf * 32, r);
            ptx::tmem_ld_wait();
            if (cc == kChunks - 1 && hlf == w / 32 - 1) {
              ptx::tc_fence_before();
              __syncwarp();
              if (lane == 0) release_acc(buf);
            }
            if (pol.reduce_here(est)) pol.add_partials(est, quarter, cc * 2 + hlf, lane, r);
            uint32_t packed[16];
            pack32(r, tn * Cfg::BN + cc * 64 + hlf * 32, packed);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
              const int c16 = hlf * 4 + j;   // 16-byte column group inside the chunk
              const int pos = w == 64 ? (c16 ^ (lane & 7)) : (c16 ^ ((lane >> 1) & 3));
              *(uint4*)(stage + lane * (w * 2) + pos * 16) = v;
            }
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            pol.store_chunk(est, quarter, cc, w, stage, row0, tn * Cfg::BN + cc * 64);
            ptx::bulk_commit();
          }
          ++chunk_seq;
        }
        if (lane == 0 && pol.signals_tile(est)) {
          ptx::bulk_wait<0>();          // a peer is told about this tile: this warp's stores of it are complete first
          ptx::fence_proxy_async();
        }
        __syncwarp();
      } else {
        // 32 columns at a time: TMEM -> registers (-> plus the other ranks' partials when this
        // rank reduces the tile) -> 16-bit -> shared-memory transpose -> 16-byte row-major stores.
        uint8_t* stage = my_epi;
        if constexpr (Policy::kBulkEpilogue) {
          if (lane == 0) ptx::bulk_wait_read<0>();   // earlier bulk stores may still read the staging
          __syncwarp();
        }
        if constexpr (Policy::kSwiGLU && Policy::kQuantOut) {
          // SwiGLU whose output feeds a block-scaled fp8 GEMM: the tile's 128 outputs of a row are exactly one
          // 1 x 128 quantisation block. The outputs are computed once and kept as bf16 pairs in registers while
          // the row's amax is found, then written as e4m3 values; the row's scale leaves as one UE8M0 byte.
          static_assert(Cfg::BN == 256, "the SwiGLU epilogue pairs columns c and c + 128 of a 256-wide tile");
          float amax = 0.f;
          // gate and up values leave TMEM as bf16 pairs (128 registers) and the accumulator buffer is released
          // before any SiLU is computed: with one accumulator buffer the next tile's MMAs wait for this release
          uint32_t hreg[64], ureg[64];
#pragma unroll
          for (int c = 0; c < 8; ++c) {        // chunks 0..3: gate columns, 4..7: up columns (32 at a time)
            uint32_t r[32];
            ptx::tmem_ld_32x32(t_addr + c * 32, r);
            ptx::tmem_ld_wait();
            if (c == 7) {
              ptx::tc_fence_before();
              __syncwarp();
              if (lane == 0) release_acc(buf);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const __nv_bfloat162 pb = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
              if (c < 4) hreg[c * 16 + j] = *(const uint32_t*)&pb;
              else ureg[(c - 4) * 16 + j] = *(const uint32_t*)&pb;
            }
          }
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            const float2 gf = __bfloat1622float2(*(const __nv_bfloat162*)&hreg[j]);
            const float2 uf = __bfloat1622float2(*(const __nv_bfloat162*)&ureg[j]);
            const float h0 = gf.x / (1.f + __expf(-gf.x)) * uf.x, h1 = gf.y / (1.f + __expf(-gf.y)) * uf.y;
            amax = fmaxf(amax, fmaxf(fabsf(h0), fabsf(h1)));
            const __nv_bfloat162 hb = __floats2bfloat162_rn(h0, h1);
            hreg[j] = *(const uint32_t*)&hb;
          }
          int e8 = (int)ceilf(log2f(fmaxf(amax, 1e-12f) * (1.0f / 448.0f)));
          e8 = max(-127, min(127, e8));
          const float inv = exp2f((float)-e8);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&hreg[c * 16 + 2 * j]);
              const float2 b = __bfloat1622float2(*(const __nv_bfloat162*)&hreg[c * 16 + 2 * j + 1]);
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv, b.y * inv), __NV_SATFINITE, __NV_E4M3);
              q[j] = lo | (hi << 16);
            }
            pol.store_q32(est, row0 + lane, tn * 128 + c * 32, make_uint4(q[0], q[1], q[2], q[3]), make_uint4(q[4], q[5], q[6], q[7]));
          }
          pol.store_row_scale(est, row0 + lane, tn, (uint32_t)(e8 + 127));
        } else if constexpr (Policy::kSwiGLU) {
          static_assert(!Policy::kSwiGLU || Cfg::BN == 256, "the SwiGLU epilogue pairs columns c and c + 128 of a 256-wide tile");
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t g[32], u[32];
            ptx::tmem_ld_32x32(t_addr + c * 32, g);
            ptx::tmem_ld_32x32(t_addr + 128 + c * 32, u);
            ptx::tmem_ld_wait();
            if (c == 3) {
              ptx::tc_fence_before();
              __syncwarp();
              if (lane == 0) release_acc(buf);
            }
            uint32_t r[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float gv = __uint_as_float(g[j]), uv = __uint_as_float(u[j]);
              r[j] = __float_as_uint(gv / (1.f + __expf(-gv)) * uv);
            }
            const int col0 = tn * 128 + c * 32;
            uint32_t packed[16];
            pack32(r, col0, packed);
            const int sw = (lane >> 1) & 3;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
              *(uint4*)(stage + lane * 64 + ((j ^ sw) * 16)) = v;
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int rr = i * 8 + (lane >> 2), cc = lane & 3;
              uint4 v = *(uint4*)(stage + rr * 64 + ((cc ^ ((rr >> 1) & 3)) * 16));
              pol.store16(est, row0 + rr, col0 + cc * 8, v);
            }
            __syncwarp();
          }
        } else {
          // Rounds of 128 columns: four tcgen05.ld of 32 columns are packed into a [32 rows][256 B]
          // staging tile (16-byte groups XOR-swizzled by row), then read back so that 16 consecutive
          // lanes hold 256 contiguous bytes of one output row: remote stores (multimem, peer
          // pointers, the per-row destinations of the MoE combine) leave as 256-byte runs.
          constexpr int kRounds = (Cfg::BN + 127) / 128;
#pragma unroll 1
          for (int rd = 0; rd < kRounds; ++rd) {
            const int wr = (Cfg::BN - rd * 128) >= 128 ? 128 : (Cfg::BN - rd * 128);    // columns of this round
            const int col_rd = tn * Cfg::BN + rd * 128;
#pragma unroll 1
            for (int q = 0; q < wr / 32; ++q) {
              const int c = rd * 4 + q;
              uint32_t r[32];
              ptx::tmem_ld_32x32(t_addr + c * 32, r);
              ptx::tmem_ld_wait();
              if (c == Cfg::BN / 32 - 1) {
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) release_acc(buf);
              }
              if constexpr (Policy::kBulkEpilogue) { if (pol.reduce_here(est)) pol.add_partials(est, quarter, c, lane, r); }
              uint32_t packed[16];
              pack32(r, col_rd + q * 32, packed);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                *(uint4*)(stage + lane * 256 + (((q * 4 + j) ^ (lane & 15)) * 16)) = v;
              }
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int rr = i * 2 + (lane >> 4), cc = lane & 15;
              if (cc * 8 < wr) {
                uint4 v = *(uint4*)(stage + rr * 256 + ((cc ^ (rr & 15)) * 16));
                pol.store16(est, row0 + rr, col_rd + cc * 8, v);
              }
            }
            __syncwarp();
          }
        }
      }
      ptx::named_barrier(1, kEpiWarps * 32);
      if (warp == 2 && lane == 0) {
        pol.tile_done(est, tm, tn);
        pol.stamp(t, 2);
      }
    }
    if constexpr (Policy::kBulkEpilogue) {
      if (lane == 0) ptx::bulk_wait<0>();   // stores still reading the staging buffers finish before the CTA leaves
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (kPair) ptx::cluster_sync();   // the peer's shared memory and barriers stay alive until both are done
  ptx::tc_fence_after();
  if (warp == 1) {
    if constexpr (kPair) ptx::tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    else ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  pol.post_main();
}

template <class Cfg, class Policy>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ Policy pol_in) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x >= pol_in.gemm_ctas()) {
    pol_in.comm_main(smem_raw, Cfg::kSmemBytes);
    return;
  }
  gemm_cta_main<Cfg, Policy>(pol_in, smem_raw);
}

// Pair configurations: clusters of two CTAs. gemm_ctas() and the grid are even, so a cluster is
// either two GEMM CTAs or two communication CTAs (which never touch the cluster barrier).
template <class Cfg, class Policy>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) gemm_pair_kernel(const __grid_constant__ Policy pol_in) {
  static_assert(Cfg::kPair, "pair kernel needs a pair configuration");
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x >= pol_in.gemm_ctas()) {
    pol_in.comm_main(smem_raw, Cfg::kSmemBytes);
    return;
  }
  gemm_cta_main<Cfg, Policy>(pol_in, smem_raw);
}

}  // namespace gemm
}  // namespace iris
