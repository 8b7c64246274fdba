// Ring attention with tcgen05 attention CTAs (the communication CTAs are those of
// ring_attention_common.cuh). One attention CTA works on items of 128 queries x one head and walks
// the key blocks in arrival order in tiles of 128 keys:
//
//   warp 0      TMA producer: K and V tiles (three stages each) from this rank's own K/V or from
//               the ring-buffer slot of the block's origin, after the slot's arrival counter has
//               been seen (acquire, bounded)
//   warp 1      MMA issuer: S = Q K^T (tcgen05.mma, M 128, N 128, K 128) into one of two TMEM
//               buffers, and O += P V (M 128, N 128 = head_dim, K 128 keys) into a third. Q and P
//               are read from TMEM (the A operand of both MMAs), only K and V come from shared
//               memory, whose bandwidth is what bounds this kernel. S of tile j+1 is issued before
//               P V of tile j, so the tensor pipe works while the softmax of tile j runs
//   warps 2..9  softmax, two threads per query row (warp w: TMEM lanes 32 * (w % 4) .. +32, keys
//               64 * ((w - 2) / 4) .. +64 of the tile). At the start of an item they copy their
//               part of the Q row from global memory into TMEM (tcgen05.st). Per tile:
//               tcgen05.ld of the 64 scores, the row maximum agreed between the two threads
//               through shared memory, P = exp2(s - max) (one packed FMA per two scores, one
//               ex2.approx each) written as packed 16-bit pairs over the first 64 columns of the
//               SAME S buffer (both threads have read their scores by then; the tensor pipe runs
//               its MMAs in issue order, so the buffer is not overwritten before P V has read it);
//               running sum kept per thread; when a row's maximum moved, its O row in TMEM is
//               rescaled (tcgen05.ld / st, each thread its 64 columns), which after the first tiles
//               is rare; at the end of an item O / sum is stored
//
// TMEM: S0 / P0 columns [0, 128), S1 / P1 [128, 256), O [256, 384), Q [384, 448) (128 values as 64
// columns of 16-bit pairs). Shared memory: K 3 x 32 KB, V 3 x 32 KB. Every wait (mbarriers, arrival
// counters) is bounded.
#include "ring_attention_common.cuh"

#include "iris/gemm/sm100_mainloop.cuh"

using namespace iris;
using namespace iris_ring;
using iris::gemm::desc_kmajor;
using iris::gemm::desc_mnmajor;
using iris::gemm::make_idesc;

namespace {

constexpr int kTQ = 128;                 // queries per item = TMEM lanes
constexpr int kTK = 128;                 // keys per tile
constexpr int kTcThreads = 320;
constexpr int kHalf = 128 * 128;         // bytes of a [128 rows][64 columns] 16-bit half tile
constexpr int kTile = 2 * kHalf;         // 32 KB
constexpr int kKvStages = 3;
constexpr int kTcSmem = 1024 + kTile * 2 * kKvStages + 256 + 3072;    // K and V stages, barriers, row exchange
constexpr uint64_t kWaitNs = 4000000000ull;
static_assert(kTcSmem <= 227 * 1024, "shared memory budget");

struct TcArgs {
  RingArgs a;
  CUtensorMap tmKown;    // [S, Hkv * D], box 64 x 128
  CUtensorMap tmVown;    // [S, Hkv * D], box 64 x 64
  CUtensorMap tmKbuf;    // ring buffer seen as [2 * W * 2 * S, Hkv * D], box 64 x 128
  CUtensorMap tmVbuf;    // same, box 64 x 64
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem desc]: A is read from TMEM (lane = row, 16-bit pairs along K per column).
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same for a converged warp: every lane executes it with warp-uniform operands and one elected lane issues.
__device__ __forceinline__ void mma_f16_ts_elect(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\telect.sync _|q, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The key tiles of one item, in the order every role walks them: blocks in arrival order (own,
// r-1, r-2, ...), tiles inside a block in order; causal items skip what lies after their queries.
//
// Contiguous layout: rank r holds tokens [r*S, (r+1)*S). A causal item of query tile qt takes all
// tiles of earlier blocks, tiles 0..qt of its own block (the last one masked on the diagonal) and
// nothing of later blocks - so the last rank does W times the work of the first.
// Zigzag layout: the sequence is cut into 2W chunks of S/2 tokens and rank r holds chunks r and
// 2W-1-r (its block = [chunk r | chunk 2W-1-r]). Under a causal mask a query of chunk r sees
// chunks 0..r, a query of chunk 2W-1-r sees every first-half chunk and the second-half chunks
// of origins >= r: every rank does the same amount of work.
struct TileWalk {
  int W, r, T, causal, zigzag, qt;
  int step = 0, t = -1, origin = 0;
  int a0 = 0, a1 = 0, b0 = 0, b1 = 0;      // tile ranges [a0, a1) and [b0, b1) of the current block (b0 >= a1)
  int diag = -1;                           // tile of the block that needs the diagonal mask
  bool first = false;                      // the current tile is the first one taken from its block
  __device__ TileWalk(const RingArgs& a, int qt_)
      : W(a.ctx.world), r(a.ctx.rank), T(a.S / kTK), causal(a.causal), zigzag(a.zigzag), qt(qt_) { open_block(); }
  __device__ void ranges() {
    a0 = 0; a1 = T; b0 = b1 = T; diag = -1;
    if (!causal) return;
    if (!zigzag) {
      if (origin > r) a1 = 0;
      else if (origin == r) { a1 = qt + 1; diag = qt; }
      return;
    }
    const int Th = T / 2;
    if (qt < Th) {                  // query chunk r: first halves of origins <= r
      if (origin > r) a1 = 0;
      else if (origin == r) { a1 = qt + 1; diag = qt; }
      else a1 = Th;
    } else {                        // query chunk 2W-1-r: every first half, second halves of origins >= r
      a1 = Th;
      if (origin > r) { b0 = Th; b1 = T; }
      else if (origin == r) { b0 = Th; b1 = qt + 1; diag = qt; }
    }
  }
  __device__ void open_block() {
    for (; step < W; ++step) {
      origin = r - step;
      if (origin < 0) origin += W;
      ranges();
      if (a1 > a0 || b1 > b0) { t = -1; return; }
    }
  }
  // advances to the next tile; false when the item is finished
  __device__ bool next() {
    while (step < W) {
      first = t < 0;
      if (t < 0) t = a1 > a0 ? a0 : b0;
      else if (++t == a1 && b1 > b0) t = b0;
      if ((t >= a0 && t < a1) || (t >= b0 && t < b1)) return true;
      ++step;
      open_block();
    }
    return false;
  }
  __device__ bool diagonal() const { return t == diag; }
};

template <bool kFp16>
__device__ void attn_main_tc(const TcArgs& g, uint8_t* smem_raw, int call) {
  const RingArgs& a = g.a;
  const DeviceContext& ctx = a.ctx;
  const int W = ctx.world, r = ctx.rank;
  const int par = call & 1;
  const int32_t target = ((call >> 1) + 1) * a.n_comm;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = a.S / kTQ;
  const int items = q_tiles * a.Hq;
  const int group = a.Hq / a.Hkv;

  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* k_s = smem;                                   // [stages][kTile]
  uint8_t* v_s = k_s + kKvStages * kTile;
  uint64_t* bars = (uint64_t*)(v_s + kKvStages * kTile);
  uint64_t* q_full = bars;              // 8 softmax warps: the item's Q is in TMEM
  uint64_t* q_free = bars + 1;          // 1: every S MMA of the item has read Q
  uint64_t* k_full = bars + 2;          // [3]
  uint64_t* k_empty = bars + 5;         // [3]
  uint64_t* v_full = bars + 8;          // [3]
  uint64_t* v_empty = bars + 11;        // [3]
  uint64_t* s_full = bars + 14;         // [2]
  uint64_t* p_full = bars + 16;         // [2] 8 softmax warps
  uint64_t* o_ready = bars + 18;        // [2] by tile parity: O holds every tile up to that one
  uint64_t* o_free = bars + 20;         // 8 softmax warps: the item's O has been read out
  uint32_t* tmem_slot = (uint32_t*)(bars + 21);
  // exchange between the two threads of a row (bounded waits, no bar.sync: a thread that gave up
  // must not leave its partner blocked): values [2 parities][2 halves][128 rows], then the number
  // of the last exchange each (half, row) published
  float* xchg = (float*)(bars + 22);
  uint32_t* xseq = (uint32_t*)(xchg + 512);

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 8);
    ptx::mbar_init(q_free, 1);
    for (int i = 0; i < kKvStages; ++i) {
      ptx::mbar_init(&k_full[i], 1); ptx::mbar_init(&k_empty[i], 1);
      ptx::mbar_init(&v_full[i], 1); ptx::mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&s_full[i], 1);
      ptx::mbar_init(&p_full[i], 8);
      ptx::mbar_init(&o_ready[i], 1);
    }
    ptx::mbar_init(o_free, 8);
    ptx::fence_mbar_init();
    ptx::fence_proxy_async();
  }
  for (int i = threadIdx.x; i < 256; i += blockDim.x) xseq[i] = 0;
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;
  const int first = blockIdx.x - a.n_comm, stride = gridDim.x - a.n_comm;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    unsigned arrived_mask = 1u << r;
    uint32_t n_item = 0, n_tile = 0;        // items / tiles issued so far (barrier phases)
    bool ok = true;
    for (int it = first; it < items && ok; it += stride, ++n_item) {
      const int h = it % a.Hq, qt = it / a.Hq, kvh = h / group;
      TileWalk w(a, qt);
      while (w.next()) {
        if (w.first && !((arrived_mask >> w.origin) & 1u)) {
          int seen = 1;
          if (lane == 0) seen = wait_flag_ge(ctx, a.flags + (size_t)par * W + w.origin, target) ? 1 : 0;
          seen = __shfl_sync(0xffffffffu, seen, 0);
          if (!seen) { ok = false; break; }
          ptx::fence_proxy_async();
          arrived_mask |= 1u << w.origin;
        }
        const int st = n_tile % kKvStages;
        const uint32_t ph = ((n_tile / kKvStages) & 1) ^ 1;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&k_empty[st], ph, kWaitNs) && ptx::mbar_wait(&v_empty[st], ph, kWaitNs))) {
          ctx.fail(kTimeoutPipeline); ok = false; break;
        }
        {   // converged warp, one elected lane per instruction
          const bool own = w.origin == r;
          const CUtensorMap* mk = own ? &g.tmKown : &g.tmKbuf;
          const CUtensorMap* mv = own ? &g.tmVown : &g.tmVbuf;
          // ring buffer rows: ((parity * W + origin) * 2 + {K: 0, V: 1}) * S + position
          const int rowk = own ? 0 : ((par * W + w.origin) * 2) * a.S;
          const int rowv = own ? 0 : rowk + a.S;
          const int pos0 = w.t * kTK;
          const uint32_t kd = ptx::smem_u32(k_s + st * kTile);
          const uint32_t vd = ptx::smem_u32(v_s + st * kTile);
          ptx::mbar_expect_tx_elect(&k_full[st], kTile);
          ptx::tma_load_2d_elect(kd, mk, &k_full[st], kvh * kD, rowk + pos0);
          ptx::tma_load_2d_elect(kd + kHalf, mk, &k_full[st], kvh * kD + 64, rowk + pos0);
          ptx::mbar_expect_tx_elect(&v_full[st], kTile);
#pragma unroll
          for (int kh = 0; kh < 2; ++kh)
#pragma unroll
            for (int nb = 0; nb < 2; ++nb)
              ptx::tma_load_2d_elect(vd + kh * kHalf + nb * 8192, mv, &v_full[st], kvh * kD + nb * 64, rowv + pos0 + kh * 64);
        }
        ++n_tile;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc_s = make_idesc(kTK, !kFp16, false);     // B = K tile, K-major
    const uint32_t idesc_o = make_idesc(kD, !kFp16, true);       // B = V tile, [keys, d] row-major
    uint32_t n_item = 0, n_s = 0, n_pv = 0;     // items, S tiles and P V tiles issued so far
    bool ok = true;
    // The warp stays converged: every lane computes the warp-uniform operands and each tensor-core instruction
    // elects its issuing lane (issued from inside `if (lane == 0)` they cost about 100 cycles apiece). Votes and
    // the warp reduction make the loop state and the TMEM base uniform for the compiler too.
    const uint32_t tmem_u = __reduce_or_sync(0xffffffffu, tmem_base);
    // The S buffer of tile j also holds P of tile j (its first 64 columns) until the P V MMA of
    // tile j has read it; S of tile j + 2 is issued after that MMA and the tensor pipe runs MMAs in
    // issue order, so no barrier guards the reuse of the buffer.
    auto issue_s = [&]() -> bool {
      const int sb = n_s & 1, st = n_s % kKvStages;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&k_full[st], (n_s / kKvStages) & 1, kWaitNs))) return false;
      ptx::tc_fence_after();
      {
        const uint32_t kb = ptx::smem_u32(k_s + st * kTile);
#pragma unroll
        for (int k = 0; k < 8; ++k) {        // 16 of the 128 head dimensions per step: 8 columns of Q in TMEM
          const uint32_t off = (k >> 2) * kHalf + (k & 3) * 32;
          mma_f16_ts_elect(tmem_u + sb * 128, tmem_u + 384 + k * 8, desc_kmajor(kb + off), idesc_s, k != 0);
        }
        ptx::mma_commit_elect(&k_empty[st]);
        ptx::mma_commit_elect(&s_full[sb]);
      }
      ++n_s;
      return true;
    };
    auto issue_pv = [&](bool first_of_item) -> bool {
      const int sb = n_pv & 1, st = n_pv % kKvStages;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&p_full[sb], (n_pv >> 1) & 1, kWaitNs))) return false;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&v_full[st], (n_pv / kKvStages) & 1, kWaitNs))) return false;
      ptx::tc_fence_after();
      {
        const uint32_t vb = ptx::smem_u32(v_s + st * kTile);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t boff = (k >> 2) * kHalf + (k & 3) * 2048;        // V: 64-key halves, 16 keys = 2048 B
          // P: 16 keys = 8 columns of 16-bit pairs at the start of the tile's S buffer
          mma_f16_ts_elect(tmem_u + 256, tmem_u + sb * 128 + k * 8, desc_mnmajor(vb + boff), idesc_o, !(first_of_item && k == 0));
        }
        ptx::mma_commit_elect(&v_empty[st]);
        ptx::mma_commit_elect(&o_ready[sb]);
      }
      ++n_pv;
      return true;
    };
    for (int it = first; it < items && ok; it += stride, ++n_item) {
      const int qt = it / a.Hq;
      int n = 0;
      {
        TileWalk w(a, qt);
        while (w.next()) ++n;
      }
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(q_full, n_item & 1, kWaitNs))) { ctx.fail(kTimeoutPipeline); break; }
      if (!issue_s()) { ctx.fail(kTimeoutPipeline); break; }
      for (int j = 0; j < n; ++j) {
        if (j + 1 < n && !issue_s()) { ctx.fail(kTimeoutPipeline); ok = false; break; }
        if (j + 1 == n) ptx::mma_commit_elect(q_free);       // every S MMA of the item is issued
        // the previous item's O must have been read out before this item's first P V overwrites it
        if (j == 0 && !__all_sync(0xffffffffu, ptx::mbar_wait(o_free, (n_item & 1) ^ 1, kWaitNs))) { ctx.fail(kTimeoutPipeline); ok = false; break; }
        if (!issue_pv(j == 0)) { ctx.fail(kTimeoutPipeline); ok = false; break; }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;                         // which 64 keys of a tile / 64 columns of O
    const int row = quarter * 32 + lane;                      // query row inside the tile
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float scale2 = a.sm_scale * kLog2e;
    uint32_t n_item = 0, n_tile = 0, xtag = 0;
    bool ok = true;
    // publishes `v`, returns the partner's value of the same exchange (false in `ok` after 4 s)
    auto exchange = [&](float v) -> float {
      ++xtag;
      volatile float* val = xchg + (xtag & 1) * 256;
      volatile uint32_t* seq = xseq;
      val[half * 128 + row] = v;
      __threadfence_block();
      seq[half * 128 + row] = xtag;
      const int other = (half ^ 1) * 128 + row;
      if ((int)(seq[other] - xtag) < 0) {
        const uint64_t t0 = ptx::globaltimer();
        uint32_t spins = 0;
        while ((int)(seq[other] - xtag) < 0) {
          if ((++spins & 1023u) == 0 && ptx::globaltimer() - t0 > kWaitNs) { ok = false; break; }
        }
      }
      __threadfence_block();
      return val[other];
    };
    for (int it = first; it < items && ok; it += stride, ++n_item) {
      const int h = it % a.Hq, qt = it / a.Hq;
      const int qpos = qt * kTQ + row;                        // position inside this rank's block
      float m_run = -INFINITY, l_run = 0.f;                   // l_run: this thread's half of the row sum
      // this thread's 64 values of the Q row -> TMEM (16-bit pairs), once every S MMA of the previous item is done
      {
        uint32_t qw[32];
        const uint4* qsrc = (const uint4*)(a.q + ((size_t)(qt * kTQ + row) * a.Hq + h) * kD * 2 + half * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 v = __ldg(qsrc + i);
          qw[4 * i] = v.x; qw[4 * i + 1] = v.y; qw[4 * i + 2] = v.z; qw[4 * i + 3] = v.w;
        }
        if (!ptx::mbar_wait(q_free, (n_item & 1) ^ 1, kWaitNs)) { ctx.fail(kTimeoutPipeline); break; }
        ptx::tc_fence_after();
        tmem_st_32x32(lane_addr + 384 + half * 32, qw);
        tmem_st_wait();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(q_full);
      }
      TileWalk w(a, qt);
      int j = 0;
      while (w.next()) {
        const int st = n_tile & 1;
        if (!ptx::mbar_wait(&s_full[st], (n_tile >> 1) & 1, kWaitNs)) { ctx.fail(kTimeoutPipeline); ok = false; break; }
        ptx::tc_fence_after();
        uint32_t s[64];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t (&chunk)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[c * 32]);
          ptx::tmem_ld_32x32(lane_addr + st * 128 + half * 64 + c * 32, chunk);
        }
        ptx::tmem_ld_wait();
        // causal mask on the diagonal tile, maximum of this thread's 64 raw scores
        const bool diag = w.diagonal();
        const int kpos0 = w.t * kTK + half * 64;
        if (diag) {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (kpos0 + c > qpos) s[c] = 0xff800000u;     // -inf
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains: the maximum is latency bound otherwise
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
#pragma unroll
          for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(mx4[u], __uint_as_float(s[c + u]));
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // agree on the row maximum with the thread that holds the other 64 keys
        mx = fmaxf(mx, exchange(mx));
        if (!__all_sync(0xffffffffu, ok)) { ctx.fail(kTimeoutPipeline); ok = false; break; }
        const float m_new = fmaxf(m_run, mx * scale2);     // finite: the diagonal tile holds the row's own key
        const float alpha = j == 0 ? 1.f : ex2_approx(m_run - m_new);
        m_run = m_new;
        // P goes over the first 64 columns of this tile's S buffer: both threads of the row have read
        // their scores (the partner published its maximum after its loads)
        uint32_t pw[32];        // this thread's 64 probabilities as 16-bit pairs
        // p = exp2(s * scale - max): packed FMA for two scores at a time, one ex2.approx each, four sum chains
        unsigned long long scale_pair, negm_pair;
        asm("mov.b64 %0, {%1, %1};" : "=l"(scale_pair) : "f"(scale2));
        asm("mov.b64 %0, {%1, %1};" : "=l"(negm_pair) : "f"(-m_new));
        float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16) {       // groups of 8 keys
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            unsigned long long sp, xp;
            asm("mov.b64 %0, {%1, %2};" : "=l"(sp) : "r"(s[c16 * 8 + 2 * e]), "r"(s[c16 * 8 + 2 * e + 1]));
            asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(xp) : "l"(sp), "l"(scale_pair), "l"(negm_pair));
            float x0, x1;
            asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(xp));
            const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
            rs4[e] += p0 + p1;
            pw[c16 * 4 + e] = pack2<kFp16>(p0, p1);
          }
        }
        tmem_st_32x32(lane_addr + st * 128 + half * 32, pw);
        l_run = l_run * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
        // rescale O when some row of this warp moved its maximum (O then holds every earlier tile)
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          // (the barrier of the previous tile's parity: this tile's S was issued after the P V of two
          //  tiles ago and MMAs complete in issue order, so between "two tiles ago" and "the previous
          //  tile" a phase parity is unambiguous)
          if (!ptx::mbar_wait(&o_ready[(n_tile - 1) & 1], ((n_tile - 1) >> 1) & 1, kWaitNs)) { ctx.fail(kTimeoutPipeline); ok = false; break; }
          ptx::tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t o[32];
            ptx::tmem_ld_32x32(lane_addr + 256 + half * 64 + c * 32, o);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(lane_addr + 256 + half * 64 + c * 32, o);
          }
        }
        tmem_st_wait();                         // P (and a rescaled O) are in TMEM before the MMA is told
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&p_full[st]);
        ++n_tile;
        ++j;
      }
      if (!ok) break;
      // ---- item epilogue: the row sum of both halves, the last P V, O / sum -> 16-bit -> global
      const float l_all = l_run + exchange(l_run);
      if (!__all_sync(0xffffffffu, ok)) { ctx.fail(kTimeoutPipeline); break; }
      if (!ptx::mbar_wait(&o_ready[(n_tile - 1) & 1], ((n_tile - 1) >> 1) & 1, kWaitNs)) { ctx.fail(kTimeoutPipeline); break; }
      ptx::tc_fence_after();
      const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
      uint8_t* orow = a.out + ((size_t)(qt * kTQ + row) * a.Hq + h) * kD * 2 + half * 128;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        ptx::tmem_ld_32x32(lane_addr + 256 + half * 64 + c * 32, o);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 v;
          v.x = pack2<kFp16>(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
          v.y = pack2<kFp16>(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
          v.z = pack2<kFp16>(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
          v.w = pack2<kFp16>(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
          *(uint4*)(orow + c * 64 + i * 16) = v;
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(o_free);
      if (a.lse && half == 0) a.lse[(size_t)(qt * kTQ + row) * a.Hq + h] = l_all > 0.f ? (m_run + log2f(l_all)) / kLog2e : -INFINITY;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, 512);
}

template <bool kFp16>
__global__ void __launch_bounds__(kTcThreads, 1) ring_attention_tc_kernel(const __grid_constant__ TcArgs g) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int call = *(volatile int32_t*)&g.a.state[0];
  if ((int)blockIdx.x < g.a.n_comm) comm_main(g.a, smem, kTcSmem, call);
  else attn_main_tc<kFp16>(g, smem, call);
  finish_call(g.a, call);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
bool make_map16(CUtensorMap* m, const void* base, bool fp16, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  static EncodeTiledFn enc = nullptr;
  if (!enc) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return false;
    enc = (EncodeTiledFn)p;
  }
  if (((uint64_t)base & 15) || ((cols * 2) & 15)) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

namespace iris_ring {

int launch_ring_attention_tc(const RingArgs& a, cudaStream_t stream) {
  if (a.S % kTQ || a.S <= 0) return 1;
  const int W = a.ctx.world;
  TcArgs g;
  g.a = a;
  const bool f16 = a.is_fp16 != 0;
  const uint64_t kvc = (uint64_t)a.Hkv * kD;
  if ((uint64_t)a.q & 15) return 1;      // Q rows are read with 16-byte loads
  if (!make_map16(&g.tmKown, a.k, f16, a.S, kvc, kTK)) return 1;
  if (!make_map16(&g.tmVown, a.v, f16, a.S, kvc, 64)) return 1;
  if (W > 1) {
    if (!make_map16(&g.tmKbuf, a.kv_buf, f16, 4ull * W * a.S, kvc, kTK)) return 1;
    if (!make_map16(&g.tmVbuf, a.kv_buf, f16, 4ull * W * a.S, kvc, 64)) return 1;
  } else {
    g.tmKbuf = g.tmKown;
    g.tmVbuf = g.tmVown;
  }
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(ring_attention_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem) != cudaSuccess) return -20;
    if (cudaFuncSetAttribute(ring_attention_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem) != cudaSuccess) return -20;
    attr = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int items = (a.S / kTQ) * a.Hq;
  int attn = sms - a.n_comm;                 // one CTA per SM (196 KB of shared memory), all resident
  if (attn > items) attn = items;
  if (attn < 1) return 1;
  const int grid = a.n_comm + attn;
  if (f16) ring_attention_tc_kernel<true><<<grid, kTcThreads, kTcSmem, stream>>>(g);
  else ring_attention_tc_kernel<false><<<grid, kTcThreads, kTcSmem, stream>>>(g);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace iris_ring
