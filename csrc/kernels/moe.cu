// Expert-sharded mixture-of-experts layer (reference: examples/31_expert_sharded_moe/*: topk.py,
// dispatch.py, grouped_matmul.py, fused_exp_matmul_ep_to_dp.py, combine.py, reduce.py).
//
// Launch sequence of one forward pass, all on one stream, no host round trips (the reference
// synchronises with .item() and a Python loop per expert, moe.py:262, ragged_metadata.py:52-78):
//   1 router     warp per token: top-k of the logits, softmax over the selected k, histogram
//   2 meta       one CTA: push this rank's expert histogram to every rank, cross-rank round, then
//                all offsets: where my rows for expert e start on e's owner, row range and tile
//                range of every local expert, expected arrivals
//   3 sort       (token, k) pairs bucketed by expert (list per expert)
//   4 dispatch + grouped GEMM 1 + SwiGLU, ONE kernel: communication CTAs walk the experts by local
//                index (so every rank's expert j fills up at the same time), stream each token row
//                HBM -> shared memory -> owner's inbox with bulk async copies and add the row
//                count to the owner's arrival counter for that expert; GEMM CTAs (tcgen05 main
//                loop) wait for an expert's arrivals, then multiply its rows by the expert's fused
//                gate|up weight and write silu(gate) * up
//                (the fusion the reference leaves as NotImplementedError, moe.py:285-286)
//   5 grouped GEMM 2 + combine, ONE kernel: down projection whose epilogue stores every output row
//                straight into the (token, k) slot of the token's home rank; cross-rank round at exit
//   6 reduce     out[t] = sum_k weight[t, k] * slot[t, k]   (the reference's sum is unweighted)
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <math.h>
#include <string.h>

#include "gemm_host.cuh"

namespace {

constexpr int kMaxTopK = 16;

struct MoeDims {
  int T, K, E, El, D, F, capacity;
};

// Device-resident metadata of one layer (all int32 unless noted; "heap" = symmetric heap).
struct MoeMeta {
  int32_t* topk_idx;       // [T, K]
  float* topk_w;           // [T, K]
  int32_t* counts_local;   // [E]      my tokens per expert
  int32_t* counts_all;     // heap [W, E]
  int32_t* cursor;         // [E]
  int32_t* list_off;       // [E + 1]  bucket boundaries in sorted_pairs
  int32_t* sorted_pairs;   // [T * K]
  int32_t* my_off;         // [E]      first inbox row (on the owner) of my rows for expert e
  int32_t* expert_rows;    // [El]     rows this rank receives per local expert
  int32_t* expert_row0;    // [El + 1] prefix of expert_rows
  int32_t* tile_prefix;    // [El + 1] prefix of ceil(rows / 128)
  int32_t* expected_cum;   // [El]     arrivals expected so far (all calls)
  int32_t* arrived;        // heap [El] arrivals so far (all calls)
  long long* inbox_meta;   // heap [capacity]  (source rank << 32) | pair id
};

// ------------------------------------------------------------------------------------ 1 router
__global__ void router_topk_kernel(const float* __restrict__ logits, MoeDims dm, MoeMeta m) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= dm.T) return;
  const float* row = logits + (size_t)warp * dm.E;
  constexpr int kPer = 32;   // up to 1024 experts
  float v[kPer];
  const int per = (dm.E + 31) / 32;
#pragma unroll
  for (int i = 0; i < kPer; ++i) v[i] = (i < per && lane + i * 32 < dm.E) ? row[lane + i * 32] : -INFINITY;
  float sel_v[kMaxTopK];
  int sel_i[kMaxTopK];
  for (int k = 0; k < dm.K; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPer; ++i)
      if (i < per && v[i] > best) { best = v[i]; bi = lane + i * 32; }
    // warp arg-max, ties to the lower expert index
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    sel_v[k] = best; sel_i[k] = bi;
    if ((bi & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kPer; ++i)
        if (i == (bi >> 5)) v[i] = -INFINITY;
    }
  }
  if (lane == 0) {
    float mx = sel_v[0], sum = 0.f;
    for (int k = 0; k < dm.K; ++k) sum += __expf(sel_v[k] - mx);
    for (int k = 0; k < dm.K; ++k) {
      m.topk_idx[(size_t)warp * dm.K + k] = sel_i[k];
      m.topk_w[(size_t)warp * dm.K + k] = __expf(sel_v[k] - mx) / sum;
      atomicAdd(&m.counts_local[sel_i[k]], 1);
    }
  }
}

// ------------------------------------------------------------------------------------ 2 meta
__global__ void __launch_bounds__(1024) moe_meta_kernel(const __grid_constant__ DeviceContext ctx, SyncBlock* sb, MoeDims dm,
                                                          MoeMeta m) {
  const int W = ctx.world, E = dm.E, El = dm.El;
  const int32_t e0 = read_epoch(sb);
  __shared__ int s_ok;
  // publish my histogram on every rank, then one cross-rank round
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    const int32_t c = m.counts_local[i];
    for (int r = 0; r < W; ++r) *ctx.remote(m.counts_all + (size_t)ctx.rank * E + i, r) = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    bool ok = true;
    if (W > 1) {
      __threadfence_system();
      barrier_signal(ctx, sb);
      ok = barrier_wait(ctx, sb, e0 + 1);
    }
    sb->epoch = e0 + 1;
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  // per global expert: total rows, my offset inside the owner's block
  __shared__ int32_t tot[1024];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < W; ++s) t += __ldcv(m.counts_all + (size_t)s * E + e);
    tot[e] = t;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int owner = e / El;
    int off = 0;
    for (int e2 = owner * El; e2 < e; ++e2) off += tot[e2];
    for (int s = 0; s < ctx.rank; ++s) off += __ldcv(m.counts_all + (size_t)s * E + e);
    m.my_off[e] = off;
    m.cursor[e] = 0;
  }
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) { m.list_off[e] = acc; acc += m.counts_local[e]; }
    m.list_off[E] = acc;
    int rows = 0, tiles = 0;
    for (int j = 0; j < El; ++j) {
      const int r = tot[ctx.rank * El + j];
      m.expert_rows[j] = r;
      m.expert_row0[j] = rows;
      m.tile_prefix[j] = tiles;
      m.expected_cum[j] += r;
      rows += r;
      tiles += (r + kBM - 1) / kBM;
    }
    m.expert_row0[El] = rows;
    m.tile_prefix[El] = tiles;
    if (rows > dm.capacity) ctx.fail(kBadTranslate);   // more rows routed here than the inbox holds
  }
}

// ------------------------------------------------------------------------------------ 3 sort
__global__ void moe_sort_kernel(MoeDims dm, MoeMeta m) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= dm.T * dm.K) return;
  const int e = m.topk_idx[p];
  const int pos = atomicAdd(&m.cursor[e], 1);
  m.sorted_pairs[m.list_off[e] + pos] = p;
}
__global__ void moe_clear_kernel(MoeDims dm, MoeMeta m) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < dm.E) m.counts_local[i] = 0;
}

// ------------------------------------------------------------------ 4/5 grouped GEMM policies
// kStage 1: A = inbox rows (dispatch runs in the communication CTAs of the same kernel), B = fused
// gate|up weight, SwiGLU epilogue into H. kStage 2: A = H, B = down weight, the epilogue sends
// every row to its token's home rank.
// kFp8: block-scaled e4m3. Tokens travel as e4m3 rows plus one scale byte per 128 columns; the inbox rows of
// a tile arrive one by one, so the producer warp puts the tile's scale atoms together from those bytes
// (kSfaFromRows). Stage 1's SwiGLU epilogue writes H as e4m3 with one scale byte per row and 128 columns
// (kQuantOut), which stage 2 reads the same way. Weights carry 128 x 128 block scales packed per expert.
template <int kStage, bool kFp8 = false>
struct GroupedGemm : Common {
  static constexpr bool kBulkEpilogue = false;
  static constexpr bool kSwiGLU = kStage == 1;
  static constexpr bool kSfaFromRows = kFp8;
  static constexpr bool kQuantOut = kFp8 && kStage == 1;
  static constexpr int kEsz = kFp8 ? 1 : 2;        // bytes per element of the tokens / of H
  const uint8_t* a_sf;     // fp8: scale bytes of this GEMM's A rows, [capacity][a_sf_ld] (inbox_sf or H_sf)
  int a_sf_ld;
  const uint8_t* x_sf;     // fp8 stage 1: scale bytes of this rank's tokens [T][a_sf_ld] (dispatch source)
  uint8_t* inbox_sf;       // fp8 stage 1: heap [capacity][a_sf_ld]
  uint8_t* h_sf;           // fp8 stage 1: [capacity][h_sf_ld] scale bytes of H
  int h_sf_ld;
  int sfb_per_expert;      // fp8: scale atoms of B per expert (tiles_n * kblocks * sfb_atoms)
  DeviceContext ctx;
  SyncBlock* sb;
  MoeDims dm;
  MoeMeta meta;
  const uint8_t* x;        // [T, D] tokens of this rank (stage 1: dispatch source)
  uint8_t* inbox;          // heap [capacity, D]
  uint8_t* H;              // [capacity, F]
  uint8_t* comb;           // heap [T * K, D]
  int n_comm_ctas;
  int k_per_expert;        // rows of B per expert (K of this GEMM)
  int n_per_expert;        // columns of B per expert when B is stored [El * N, K] (K-major)
  int b_kmajor;

  struct State {
    int j = -1;            // local expert of the current tile
    int key = -1;          // expert whose arrivals were confirmed
    int row0 = 0, rows_end = 0;
    unsigned long long* tab = nullptr;   // stage 2: destination row pointers of this warp's 32 rows
    uint32_t sf_cur[4] = {0, 0, 0, 0};   // fp8 producer: scale bytes of rows lane + 32 a for K blocks [4 g, 4 g + 4)
    uint32_t sf_nxt[4] = {0, 0, 0, 0};   //               and for the next four
  };
  IRIS_D int num_tiles() const { return meta.tile_prefix[dm.El] * tiles_n; }
  // tile -> (virtual m index = global 128-row tile counter, n tile); experts in order
  IRIS_D void tile(int t, int& tm, int& tn) const {
    tm = t / tiles_n;
    tn = t - tm * tiles_n;
  }
  IRIS_D int expert_of(int tm) const {
    int j = 0;
    while (j + 1 < dm.El && meta.tile_prefix[j + 1] <= tm) ++j;
    return j;
  }
  IRIS_D bool a_source(State& st, int tm, int kb, ASource& s) const {
    if (kb == 0) {
      st.j = expert_of(tm);
      st.row0 = meta.expert_row0[st.j] + (tm - meta.tile_prefix[st.j]) * kBM;
      if (kStage == 1 && st.key != st.j) {
        if (!wait_flag_ge(ctx, meta.arrived + st.j, meta.expected_cum[st.j])) return false;
        st.key = st.j;
        ptx::fence_proxy_async();
      }
    }
    s.map = &tmA; s.x = kb * bk; s.y = st.row0;
    if (b_kmajor) { s.bk = kb * bk; s.bn0 += st.j * n_per_expert; }
    else s.bk = st.j * k_per_expert + kb * bk;
    s.sf_map = nullptr; s.sf_row = 0;
    s.sfb_off = st.j * sfb_per_expert;
    return true;
  }
  // fp8: the scale atom of (128-row tile at st.row0, K block kb). Lane l owns rows l, l + 32, l + 64, l + 96:
  // their scale bytes come four K blocks at a time (one 32-bit load per row, the following group prefetched),
  // and the lane writes bytes [16 l, 16 l + 16) of the atom: for each of its rows the byte of this block, four times.
  IRIS_D void sfa_fill(State& st, int, int kb, uint8_t* atom, int lane) const {
    auto ld = [&](int a, int k) -> uint32_t {
      const int row = min(st.row0 + lane + 32 * a, dm.capacity - 1);
      return __ldcg((const uint32_t*)(a_sf + (size_t)row * a_sf_ld + k));
    };
    if (kb == 0) {
#pragma unroll
      for (int a = 0; a < 4; ++a) { st.sf_cur[a] = ld(a, 0); st.sf_nxt[a] = 4 < a_sf_ld ? ld(a, 4) : 0; }
    } else if ((kb & 3) == 0) {
#pragma unroll
      for (int a = 0; a < 4; ++a) { st.sf_cur[a] = st.sf_nxt[a]; st.sf_nxt[a] = kb + 4 < a_sf_ld ? ld(a, kb + 4) : 0; }
    }
    const int sh8 = (kb & 3) * 8;
    uint4 v;
    v.x = ((st.sf_cur[0] >> sh8) & 0xffu) * 0x01010101u;
    v.y = ((st.sf_cur[1] >> sh8) & 0xffu) * 0x01010101u;
    v.z = ((st.sf_cur[2] >> sh8) & 0xffu) * 0x01010101u;
    v.w = ((st.sf_cur[3] >> sh8) & 0xffu) * 0x01010101u;
    *(uint4*)(atom + lane * 16) = v;
  }
  // fp8 stage 1: 32 e4m3 values of H, and the row's scale byte for the tile's 128 columns
  IRIS_D void store_q32(State& st, int row, int col, uint4 a, uint4 b) const {
    if (row >= st.rows_end || col >= dm.F) return;
    uint4* p = (uint4*)(H + (size_t)row * dm.F + col);
    p[0] = a; p[1] = b;
  }
  IRIS_D void store_row_scale(State& st, int row, int n_tile, uint32_t byte) const {
    if (row < st.rows_end) h_sf[(size_t)row * h_sf_ld + n_tile] = (uint8_t)byte;
  }
  IRIS_D int row_origin(State& st, int) const { return st.row0; }
  IRIS_D void begin_tile(State& st, int tm, int, uint8_t* warp_scratch) const {
    st.j = expert_of(tm);
    st.row0 = meta.expert_row0[st.j] + (tm - meta.tile_prefix[st.j]) * kBM;
    st.rows_end = min(meta.expert_row0[st.j] + meta.expert_rows[st.j], dm.capacity);
    if (kStage == 2) {
      st.tab = (unsigned long long*)warp_scratch;
      const int lane = threadIdx.x & 31, quarter = (threadIdx.x >> 5) & 3;
      const int row = st.row0 + quarter * 32 + lane;
      unsigned long long ptr = 0;
      if (row < st.rows_end) {
        const long long mt = meta.inbox_meta[row];
        const int src = (int)(mt >> 32), pair = (int)(mt & 0xffffffffll);
        ptr = (unsigned long long)ctx.remote(comb + (size_t)pair * dm.D * 2, src);      // the combine buffer stays 16-bit
      }
      __syncwarp();
      st.tab[lane] = ptr;
      __syncwarp();
    }
  }
  IRIS_D void store16(State& st, int row, int col, uint4 v) const {
    if (row >= st.rows_end) return;
    if (kStage == 1) {
      if (col < dm.F) *(uint4*)(H + ((size_t)row * dm.F + col) * 2) = v;
    } else {
      const int quarter = (threadIdx.x >> 5) & 3;
      const unsigned long long p = st.tab[row - st.row0 - quarter * 32];
      if (p && col < dm.D) *(uint4*)(p + (size_t)col * 2) = v;
    }
  }
  IRIS_D void tile_done(State&, int, int) const {}

  // Dispatch (stage 1 only): groups (local expert j, destination) in j-major order, the order in
  // which the GEMM CTAs consume the experts. Every communication CTA pushes its slice of the rows
  // of EVERY group, so the first expert's rows are complete after 1 / El of the dispatch instead
  // of after a whole group per CTA. Rows go HBM -> shared memory -> destination inbox by bulk
  // async copies driven by one thread; the 8-byte routing record of each row is stored by the
  // other threads; each CTA adds its slice's row count to the expert's arrival counter.
  static constexpr int kSlot = 16 * 1024;
  IRIS_D void comm_main(uint8_t* smem_raw, int smem_bytes) const {
    if (kStage != 1) return;
    const int c = blockIdx.x - n_gemm_ctas;
    const int W = ctx.world;
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
    const uint32_t row_bytes = (uint32_t)dm.D * kEsz;
    const int pieces = (int)((row_bytes + kSlot - 1) / kSlot);      // pieces per row
    int nb = (smem_bytes - 1024) / kSlot;
    if (nb > 12) nb = 12;
    uint64_t* bars = (uint64_t*)(smem + (size_t)nb * kSlot);
    if (threadIdx.x == 0) {
      for (int i = 0; i < nb; ++i) ptx::mbar_init(&bars[i], 1);
      ptx::fence_mbar_init();
      ptx::fence_proxy_async();
    }
    __syncthreads();
    int seq = 0;   // pieces issued so far (ring slot / parity)
    for (int g = 0; g < dm.El * W; ++g) {
      const int j = g / W;
      int r = ctx.rank + g % W;
      if (r >= W) r -= W;
      const int e = r * dm.El + j;
      const int n_all = meta.list_off[e + 1] - meta.list_off[e];
      const int i0 = (int)((long long)n_all * c / n_comm_ctas), i1 = (int)((long long)n_all * (c + 1) / n_comm_ctas);
      const int n = i1 - i0;
      if (n == 0) continue;                      // uniform over the CTA
      const int lo = meta.list_off[e] + i0;
      const int dst0 = meta.my_off[e] + i0;
      uint8_t* dst_inbox = ctx.remote(inbox, r);
      long long* dst_meta = ctx.remote(meta.inbox_meta, r);
      // routing records
      for (int i = threadIdx.x; i < n; i += blockDim.x)
        if (dst0 + i < dm.capacity) dst_meta[dst0 + i] = ((long long)ctx.rank << 32) | (long long)meta.sorted_pairs[lo + i];
      if constexpr (kFp8) {       // and the rows' scale bytes, 16 at a time
        uint8_t* dst_sf = ctx.remote(inbox_sf, r);
        const int per_row = a_sf_ld / 16;
        for (int u = threadIdx.x; u < n * per_row; u += blockDim.x) {
          const int i = u / per_row, c16 = u - i * per_row;
          if (dst0 + i >= dm.capacity) continue;
          const int tok = meta.sorted_pairs[lo + i] / dm.K;
          *(uint4*)(dst_sf + (size_t)(dst0 + i) * a_sf_ld + c16 * 16) = *(const uint4*)(x_sf + (size_t)tok * a_sf_ld + c16 * 16);
        }
      }
      if (threadIdx.x == 0) {
        const int total = n * pieces;
        auto src_of = [&](int q) -> const uint8_t* {
          const int i = q / pieces, k = q - i * pieces;
          const int pair = meta.sorted_pairs[lo + i];
          return x + (size_t)(pair / dm.K) * row_bytes + (size_t)k * kSlot;
        };
        auto len_of = [&](int q) -> uint32_t {
          const int k = q % pieces;
          return min((uint32_t)kSlot, row_bytes - (uint32_t)k * kSlot);
        };
        auto issue = [&](int q) {
          const int slot = (seq + q) % nb;
          ptx::mbar_expect_tx(&bars[slot], len_of(q));
          ptx::bulk_load(smem + (size_t)slot * kSlot, src_of(q), len_of(q), &bars[slot]);
        };
        int next = min(nb, total);
        for (int q = 0; q < next; ++q) issue(q);
        bool ok = true;
        for (int q = 0; q < total; ++q) {
          const int slot = (seq + q) % nb;
          if (!ptx::mbar_wait(&bars[slot], (uint32_t)(((seq + q) / nb) & 1), kPipeTimeoutNs)) { fail(kTimeoutPipeline); ok = false; break; }
          const int i = q / pieces, k = q - i * pieces;
          if (dst0 + i < dm.capacity)
            ptx::bulk_store(dst_inbox + (size_t)(dst0 + i) * row_bytes + (size_t)k * kSlot, smem + (size_t)slot * kSlot, len_of(q));
          ptx::bulk_commit();
          if (q == total - 1) ptx::bulk_wait<0>();
          else ptx::bulk_wait_read<1>();
          const int free_upto = q == total - 1 ? q : q - 1;
          while (next <= free_upto + nb && next < total) issue(next++);
        }
        seq += total;
        if (ok) {
          ptx::fence_proxy_async();
        }
      }
      __syncthreads();   // routing records of all threads + data of thread 0 precede the release below
      if (threadIdx.x == 0) {
        fence_sys();
        red_release_sys_add(ctx.remote(meta.arrived + j, r), n);
      }
    }
  }
  IRIS_D void post_main() const {
    if (kStage == 2) {
      grid_exit_barrier(ctx, sb, read_epoch(sb), 0);
    }
  }
};

// ------------------------------------------------------------------------------------ 6 reduce
__global__ void moe_reduce_kernel(const __nv_bfloat16* __restrict__ comb, const float* __restrict__ w, __nv_bfloat16* out,
                                  int T, int K, int D) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < D; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < K; ++k) {
      const float wk = w[(size_t)t * K + k];
      const uint4 v = __ldcg((const uint4*)(comb + ((size_t)t * K + k) * D + c));
      const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += wk * f.x;
        acc[2 * q + 1] += wk * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = (__nv_bfloat162*)&o;
#pragma unroll
    for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    *(uint4*)(out + (size_t)t * D + c) = o;
  }
}

}  // namespace

extern "C" {

typedef struct IrisMoeDesc {
  IrisCtx ctx;
  int32_t T, K, E, El, D, F, capacity, comm_ctas;
  const void* x;            // [T, D] bf16
  const float* logits;      // [T, E]
  const void* w13;          // [El, D, 2F] bf16, columns in blocks of [gate 128 | up 128]
  const void* w2;           // [El, F, D] bf16
  void* out;                // [T, D] bf16
  void* inbox; void* H; void* comb;
  void* sync_meta; void* sync_gemm2;
  int32_t* topk_idx; float* topk_w;
  int32_t* counts_local; int32_t* counts_all; int32_t* cursor; int32_t* list_off; int32_t* sorted_pairs; int32_t* my_off;
  int32_t* expert_rows; int32_t* expert_row0; int32_t* tile_prefix; int32_t* expected_cum; int32_t* arrived;
  void* inbox_meta;
  int32_t weights_kmajor;   // 1: w13 is [El, 2F, D] and w2 is [El, D, F] (each expert's weight transposed: K contiguous)
  // Block-scaled e4m3 mode (fp8 != 0; weights_kmajor must be 1): x is the e4m3 form of the tokens [T, D] bytes,
  // w13 / w2 are e4m3, inbox is [capacity, D] bytes, H is [capacity, F] bytes; comb and out stay bf16.
  int32_t fp8;
  int32_t sf_ld1;           // bytes per row of x_sf / inbox_sf: >= D / 128, multiple of 16
  int32_t sf_ld2;           // bytes per row of H_sf: >= F / 128, multiple of 16
  const void* x_sf;         // [T, sf_ld1] one UE8M0 byte per token and 128 columns
  void* inbox_sf;           // heap [capacity, sf_ld1]
  void* H_sf;               // [capacity, sf_ld2]
  const void* w13_sf;       // scale atoms of w13: [El][2F / 256][D / 128][2][512]
  const void* w2_sf;        // scale atoms of w2:  [El][ceil(D / 224)][F / 128][2][512]
} IrisMoeDesc;

int iris_moe_forward(const IrisMoeDesc* d, void* stream_) {
  cudaStream_t s = (cudaStream_t)stream_;
  if (d->K > kMaxTopK || d->E > 1024 || d->E % d->ctx.world || d->D % 64 || d->F % 128 || d->D % 256) return -3;
  DeviceContext ctx;
  memcpy(&ctx, &d->ctx, sizeof(ctx));
  MoeDims dm{d->T, d->K, d->E, d->El, d->D, d->F, d->capacity};
  MoeMeta m{d->topk_idx, d->topk_w, d->counts_local, d->counts_all, d->cursor, d->list_off, d->sorted_pairs, d->my_off,
            d->expert_rows, d->expert_row0, d->tile_prefix, d->expected_cum, d->arrived, (long long*)d->inbox_meta};
  moe_clear_kernel<<<(d->E + 255) / 256, 256, 0, s>>>(dm, m);
  router_topk_kernel<<<(d->T * 32 + 255) / 256, 256, 0, s>>>(d->logits, dm, m);
  moe_meta_kernel<<<1, 1024, 0, s>>>(ctx, (SyncBlock*)d->sync_meta, dm, m);
  moe_sort_kernel<<<(d->T * d->K + 255) / 256, 256, 0, s>>>(dm, m);
  if (cudaGetLastError() != cudaSuccess) return -21;

  const int sms = sm_count();
  const int comm = ctx.world > 0 ? (d->comm_ctas > 0 ? d->comm_ctas : 16) : 0;
  const bool km = d->weights_kmajor != 0;
  auto common = [&](auto& pol, int bn, int N, int Kdim, bool f8) {
    pol.sh = Shape{d->capacity, N, Kdim};
    pol.tiles_m = 0; pol.tiles_n = ceil_div(N, bn); pol.group_m = 1;
    pol.bf16 = 1; pol.bn = bn; pol.fp8 = f8; pol.bk = f8 ? 128 : kBK; pol.kblocks = ceil_div(Kdim, pol.bk);
    pol.sfb_atoms = f8 ? ceil_div(bn, 128) : 0; pol.c_bulk = 0;
    pol.bias_row = nullptr; pol.bias_col = nullptr; pol.status = d->ctx.status; pol.timeline = nullptr;
    pol.ctx = ctx; pol.dm = dm; pol.meta = m;
    pol.inbox = (uint8_t*)d->inbox; pol.H = (uint8_t*)d->H; pol.comb = (uint8_t*)d->comb;
    pol.b_kmajor = km;
    pol.a_sf = nullptr; pol.a_sf_ld = 0; pol.x_sf = nullptr; pol.inbox_sf = nullptr; pol.h_sf = nullptr; pol.h_sf_ld = 0;
    pol.sfb_per_expert = pol.tiles_n * pol.kblocks * pol.sfb_atoms;
  };
  if (d->fp8) {
    if (!km || d->sf_ld1 % 16 || d->sf_ld2 % 16 || d->sf_ld1 * 128 < d->D || d->sf_ld2 * 128 < d->F || d->D % 128 || d->F % 128) return -3;
    {
      GroupedGemm<1, true> pol;
      common(pol, 256, 2 * d->F, d->D, true);
      int r = make_map(&pol.tmA, d->inbox, IRIS_F8E4M3, d->capacity, d->D, d->D, 128, kBM);
      if (r) return r;
      r = make_map(&pol.tmB, d->w13, IRIS_F8E4M3, (uint64_t)d->El * 2 * d->F, d->D, d->D, 128, 256);
      if (r) return r;
      r = make_sf_map(&pol.tmSFB, d->w13_sf, (uint64_t)d->El * pol.sfb_per_expert, pol.sfb_atoms);
      if (r) return r;
      pol.tmSFA = pol.tmSFB;      // unused: A's atoms are built from the rows' scale bytes
      pol.n_gemm_ctas = sms - comm; pol.sb = nullptr;
      pol.x = (const uint8_t*)d->x; pol.n_comm_ctas = comm; pol.k_per_expert = d->D; pol.n_per_expert = 2 * d->F;
      pol.a_sf = (const uint8_t*)d->inbox_sf; pol.a_sf_ld = d->sf_ld1; pol.x_sf = (const uint8_t*)d->x_sf;
      pol.inbox_sf = (uint8_t*)d->inbox_sf; pol.h_sf = (uint8_t*)d->H_sf; pol.h_sf_ld = d->sf_ld2;
      r = launch<Config<256, true, 4, false, true, 1, 0>>(pol, sms, s);
      if (r) return r;
    }
    {
      GroupedGemm<2, true> pol;
      common(pol, 224, d->D, d->F, true);
      int r = make_map(&pol.tmA, d->H, IRIS_F8E4M3, d->capacity, d->F, d->F, 128, kBM);
      if (r) return r;
      r = make_map(&pol.tmB, d->w2, IRIS_F8E4M3, (uint64_t)d->El * d->D, d->F, d->F, 128, 224);
      if (r) return r;
      r = make_sf_map(&pol.tmSFB, d->w2_sf, (uint64_t)d->El * pol.sfb_per_expert, pol.sfb_atoms);
      if (r) return r;
      pol.tmSFA = pol.tmSFB;
      pol.n_gemm_ctas = sms; pol.sb = (SyncBlock*)d->sync_gemm2;
      pol.x = nullptr; pol.n_comm_ctas = 0; pol.k_per_expert = d->F; pol.n_per_expert = d->D;
      pol.a_sf = (const uint8_t*)d->H_sf; pol.a_sf_ld = d->sf_ld2;
      r = launch<Config<224, true, 4, false, true, 2>>(pol, sms, s);
      if (r) return r;
    }
  } else {
  {
    GroupedGemm<1> pol;
    common(pol, 256, 2 * d->F, d->D, false);
    int r = make_map(&pol.tmA, d->inbox, IRIS_BF16, d->capacity, d->D, d->D, kBK, kBM);
    if (r) return r;
    if (km) r = make_map(&pol.tmB, d->w13, IRIS_BF16, (uint64_t)d->El * 2 * d->F, d->D, d->D, kBK, 256);
    else r = make_map(&pol.tmB, d->w13, IRIS_BF16, (uint64_t)d->El * d->D, 2 * d->F, 2 * d->F, 64, 64);
    if (r) return r;
    pol.n_gemm_ctas = sms - comm; pol.sb = nullptr;
    pol.x = (const uint8_t*)d->x; pol.n_comm_ctas = comm; pol.k_per_expert = d->D; pol.n_per_expert = km ? 2 * d->F : 0;
    r = km ? launch<Config<256, true, 4>>(pol, sms, s) : launch<Config<256, false, 4>>(pol, sms, s);
    if (r) return r;
  }
  {
    GroupedGemm<2> pol;
    common(pol, 256, d->D, d->F, false);
    int r = make_map(&pol.tmA, d->H, IRIS_BF16, d->capacity, d->F, d->F, kBK, kBM);
    if (r) return r;
    if (km) r = make_map(&pol.tmB, d->w2, IRIS_BF16, (uint64_t)d->El * d->D, d->F, d->F, kBK, 256);
    else r = make_map(&pol.tmB, d->w2, IRIS_BF16, (uint64_t)d->El * d->F, d->D, d->D, 64, 64);
    if (r) return r;
    pol.n_gemm_ctas = sms; pol.sb = (SyncBlock*)d->sync_gemm2;
    pol.x = nullptr; pol.n_comm_ctas = 0; pol.k_per_expert = d->F; pol.n_per_expert = km ? d->D : 0;
    r = km ? launch<Config<256, true, 4>>(pol, sms, s) : launch<Config<256, false, 4>>(pol, sms, s);
    if (r) return r;
  }
  }
  moe_reduce_kernel<<<d->T, 256, 0, s>>>((const __nv_bfloat16*)d->comb, d->topk_w, (__nv_bfloat16*)d->out, d->T, d->K, d->D);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // extern "C"
