// C ABI shared by the kernel library (libiris_b200_kernels.so) and its Python loader
// (iris_b200/_lib.py mirrors these structs with ctypes). Every entry point returns 0 or a
// negative error code, launches on the given stream and never synchronises or allocates unless
// its comment says so.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IRIS_MAX_RANKS 72

// Host copy of iris::DeviceContext (same field order).
typedef struct IrisCtx {
  int32_t rank;
  int32_t world;
  uint64_t heap_size;
  uint64_t mc_base;
  int32_t* status;
  uint64_t timeout_ns;
  // trace block (see include/iris/context.cuh TraceBuffers)
  int32_t trace_enabled;
  int32_t trace_max_events;
  void* trace_ptrs[15];
  uint64_t bases[IRIS_MAX_RANKS];
} IrisCtx;

enum IrisDType { IRIS_F16 = 0, IRIS_BF16 = 1, IRIS_F32 = 2, IRIS_I32 = 3, IRIS_I8 = 4, IRIS_F8E4M3 = 5, IRIS_I64 = 6 };

enum IrisGemmOp {
  IRIS_GEMM_LOCAL = 0,          // C = A @ B (+ bias)
  IRIS_GEMM_AG_M = 1,           // all-gather A (sharded by rows) then GEMM
  IRIS_GEMM_AG_K = 2,           // all-gather A (sharded along K) then GEMM
  IRIS_GEMM_ALL_GATHER = 3,     // GEMM then all-gather of C rows (rank r's rows at r*M)
  IRIS_GEMM_REDUCE_SCATTER = 4, // GEMM then sum over ranks, rank r keeps rows [r*M/W, (r+1)*M/W)
  IRIS_GEMM_ALL_REDUCE = 5,     // GEMM then sum over ranks, everyone gets [M, N]
  IRIS_GEMM_ALL_SCATTER = 6,    // GEMM then all-gather of C columns (rank r's columns at r*N)
  IRIS_GEMM_RS_TILES = 7,       // GEMM then sum over ranks; output [M, N], rank r writes only the
                                // tiles it owns (contiguous tile blocks, last rank takes the remainder)
  IRIS_GEMM_AR_ONE_SHOT = 8,    // all-reduce, one traversal: every rank sends its partial tiles to ALL ranks
                                // (staging [2][W][M][N]) and every rank sums the W partials itself
  IRIS_GEMM_AR_ATOMIC = 9,      // all-reduce by remote atomic adds of the partial tiles into every rank's
                                // (pre-zeroed) output; 16-bit accumulation in memory, order not fixed
};

typedef struct IrisGemmDesc {
  int32_t op;
  int32_t M, N, K;        // problem of the MMA loop on this rank (gathered sizes for AG_*)
  int32_t dtype;          // IRIS_F16 or IRIS_BF16 (inputs and output)
  int32_t b_kmajor;       // 1: B given as [N, K] row-major, 0: B given as [K, N] row-major
  int32_t bn;             // tile width: 128, 224 or 256; 0 = choose
  int32_t group_m;        // tile-order swizzle, 0 = default
  int32_t gemm_ctas;      // 0 = all SMs minus comm_ctas
  int32_t comm_ctas;      // CTAs that only move data (AG_M / AG_K), 0 = default
  int32_t use_mc;         // use the NVLS multicast window when the context has one
  int32_t two_sm;         // CTA pairs on 256-row tiles (tcgen05 cta_group::2): 0 = plan decides, 1 = never, 2 = whenever the shape allows
  const void* A; int64_t lda;
  const void* B; int64_t ldb;
  void* C; int64_t ldc;
  const float* bias_row;  // [M] or null
  const float* bias_col;  // [N] or null
  IrisCtx ctx;
  void* sync_block;       // iris::SyncBlock on the heap
  void* inbox;            // AG_*: [2][W][rows][cols] staging of gathered A (heap)
  int32_t* flags;         // AG_*: [2][W][chunks]; RS/AR: [2][tiles] arrival counters (heap)
  void* staging;          // RS/AR: [2][W][owned tiles][128*bn] partial tiles (heap)
  int32_t M_local;        // AG_M: rows per rank; ALL_GATHER: rows per rank (= M)
  int32_t K_local;        // AG_K: K per rank
  void* timeline;         // optional int64 [tiles + chunks][4]: per-tile timestamps in ns (0 start,
                          // 1 operands available, 2 stored; comm CTA 0 stamps slot tiles+c, col 3)
  // Block-scaled fp8 inputs (in_dtype == IRIS_F8E4M3; 0 means "same as dtype"): A [.., K] and B [N, K]
  // are e4m3 bytes (B K-major only), `dtype` is the 16-bit output format, lda / ldb count bytes.
  // Scales are UE8M0 bytes (power-of-two factors) packed in 512-byte atoms of 128 rows x 4 K groups of
  // 32 (row r at byte (r % 32) * 16 + (r / 32) * 4):
  //   sf_a  [ceil(rows / 128)][K / 128] atoms over the rows of A this rank holds (its shard for AG_*)
  //   sf_b  [ceil(N / bn)][K / 128][ceil(bn / 128)] atoms, rows counted from each column tile's first column
  //   sf_inbox (AG_*): [2][W][chunks][K blocks per source] atoms of the gathered shards (heap)
  int32_t in_dtype;
  const void* sf_a;
  const void* sf_b;
  void* sf_inbox;
  // ALL_GATHER / ALL_SCATTER: how the collective half overlaps the GEMM. 0: every epilogue warp stores its
  // fragment to all ranks itself ("fused sequential"); 1: the GEMM CTAs write the tile to this rank's own
  // output and raise a per-tile flag, `comm_ctas` communication CTAs of the same kernel wait for the flags
  // and forward the tiles to the peers ("workgroup specialised"; flags: [2][128-row tiles x column tiles]).
  int32_t overlap;
} IrisGemmDesc;

// Block-scaled fp8 (e4m3) GEMM: C = (A * scale_a) @ (B * scale_b)^T with A [M, K] and B [N, K]
// row-major bytes, scale_a [M, ceil(K/128)] (one per row and 128-wide K block), scale_b
// [ceil(N/128), ceil(K/128)] (one per 128 x 128 block), fp32 accumulation, 16-bit output.
typedef struct IrisFp8GemmDesc {
  const void* A;          // e4m3, pitch lda bytes (multiple of 16)
  const void* B;          // e4m3, pitch ldb bytes (multiple of 16)
  const float* scale_a;
  const float* scale_b;
  void* C;                // [M, N] 16-bit, pitch ldc elements
  int64_t lda, ldb, ldc;
  int32_t M, N, K;
  int32_t out_dtype;      // IRIS_BF16 or IRIS_F16
  int32_t* status;        // optional status word (a pipeline wait that runs out is recorded there)
} IrisFp8GemmDesc;
int iris_gemm_fp8_launch(const IrisFp8GemmDesc* d, void* stream);

// Bytes of workspace the op needs for this shape (inbox / flags / staging) and the tile the plan
// picked (width, and whether CTA pairs run 256-row tiles). Pure arithmetic.
int iris_gemm_workspace(const IrisGemmDesc* d, uint64_t* inbox_bytes, uint64_t* flags_bytes, uint64_t* staging_bytes,
                        int32_t* bn_out, int32_t* pair_out);
int iris_gemm_launch(const IrisGemmDesc* d, void* stream);
// Bytes of the scale inbox of an fp8 AG_* op (0 for every other op).
uint64_t iris_gemm_sf_inbox_bytes(const IrisGemmDesc* d);

#ifdef __cplusplus
}
#endif
