// Pieces shared by the translation units that instantiate the sm_100a GEMM main loop
// (gemm_ops.cu, moe.cu): the fields every policy carries, TMA tensor-map encoding through the
// driver entry point, and the launch helper. Everything lives in an unnamed namespace, so each
// translation unit gets its own copy.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>

#include "iris/host_api.h"
#include "iris/context.cuh"
#include "iris/rma.cuh"
#include "iris/sync.cuh"
#include "iris/multimem.cuh"
#include "iris/gemm/sm100_mainloop.cuh"

using namespace iris;
using namespace iris::gemm;

static_assert(sizeof(IrisCtx) == sizeof(DeviceContext), "IrisCtx must mirror iris::DeviceContext");

namespace {

struct Common {
  CUtensorMap tmA;
  CUtensorMap tmB;
  Shape sh;
  int tiles_m, tiles_n, group_m;   // tiles_m counts 128-row tiles
  int pair;                        // 1: CTA pairs walk 256-row tiles (order_m = tiles_m / 2)
  int order_m;                     // row tiles in the unit the tile order walks
  int n_gemm_ctas;
  int bf16;                        // output (and 16-bit input) format: 1 bf16, 0 fp16
  int bn;
  // e4m3 operands with block scales (Config::kFp8): K elements per stage, K blocks, and the maps of the
  // scale atoms. tmSFA: [128-row tiles of A][K blocks] atoms; tmSFB: [column tiles][K blocks][atoms per
  // tile] (packed for this tile width), both as rows of 128 x u32.
  int fp8;
  int bk;                          // K elements per stage: 64 (16-bit) or 128 (fp8)
  int kblocks;
  int sfb_atoms;
  CUtensorMap tmSFA;
  CUtensorMap tmSFB;
  const float* bias_row;
  const float* bias_col;
  int32_t* status;
  int64_t* timeline;   // optional [tiles + chunks][4] nanosecond stamps (globaltimer)

  IRIS_D void stamp(int slot, int what) const {
    if (timeline) timeline[(size_t)slot * 4 + what] = (int64_t)now_ns();
  }
  IRIS_D Shape shape() const { return sh; }
  IRIS_D int gemm_ctas() const { return n_gemm_ctas; }
  IRIS_D int num_tiles() const { return order_m * tiles_n; }
  IRIS_D const CUtensorMap* b_map() const { return &tmB; }
  IRIS_D const CUtensorMap* sfb_map() const { return &tmSFB; }
  IRIS_D int b_sf_row(int tn, int kb) const { return (tn * kblocks + kb) * sfb_atoms; }
  IRIS_D bool is_bf16() const { return bf16 != 0; }
  IRIS_D bool has_bias() const { return bias_row != nullptr || bias_col != nullptr; }
  IRIS_D float row_bias(int row) const { return (bias_row && row < sh.M) ? bias_row[row] : 0.f; }
  IRIS_D float col_bias(int col) const { return (bias_col && col < sh.N) ? bias_col[col] : 0.f; }
  IRIS_D void fail(int code) const {
    if (status) atomicCAS(status, 0, code);
  }
  // Output of this rank as tensor maps for the chunked epilogue (64-column chunks with the 128-byte
  // swizzle, a 32-column tail chunk with the 64-byte one); c_bulk = 0 when the output cannot be mapped
  // (pitch or base not 16-byte aligned) and the tiles take the row-major path instead.
  CUtensorMap tmC;
  CUtensorMap tmC32;
  int c_bulk;
  IRIS_D void store_chunk_local(int width, const uint8_t* smem, int row, int col) const {
    ptx::tma_store_2d(width == 64 ? &tmC : &tmC32, smem, col, row);
  }
  static constexpr bool kSfaFromRows = false;
  static constexpr bool kQuantOut = false;
  // defaults of the epilogue hooks a policy may leave out
  struct NoState {};
  template <class S> IRIS_D bool bulk_tile(S&) const { return false; }
  template <class S> IRIS_D bool signals_tile(S&) const { return false; }
  template <class S> IRIS_D bool reduce_here(S&) const { return false; }
  template <class S> IRIS_D void store_chunk(S&, int, int, int, const uint8_t*, int, int) const {}
  template <class S> IRIS_D void add_partials(S&, int, int, int, uint32_t (&)[32]) const {}
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeTiledFn)p;
  }
  return fn;
}
// 2-D map over a row-major [rows, cols] matrix of 16-bit (IRIS_BF16 / IRIS_F16) or 8-bit (IRIS_F8E4M3)
// elements with pitch `ld` elements; box = box_cols x box_rows (box_cols elements = 128 bytes), 128-byte swizzle.
int make_map(CUtensorMap* m, const void* base, int dtype, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
             uint32_t box_rows, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -10;
  const uint64_t esz = dtype == IRIS_F8E4M3 ? 1 : 2;
  if (((uint64_t)base & 15) || ((ld * esz) & 15)) return -11;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esz};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = dtype == IRIS_F8E4M3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : dtype == IRIS_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(m, dt, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}
// The two output maps of the chunked epilogue over a row-major 16-bit [rows, cols] matrix. Returns 1 when both exist.
int make_out_maps(CUtensorMap* m64, CUtensorMap* m32, const void* base, int dtype, uint64_t rows, uint64_t cols, uint64_t ld) {
  if (!base || rows == 0 || cols == 0) return 0;
  if (make_map(m64, base, dtype, rows, cols, ld, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B)) return 0;
  if (make_map(m32, base, dtype, rows, cols, ld, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B)) return 0;
  return 1;
}
// Map over `atoms` scale atoms of 512 bytes each (rows of 128 x u32, contiguous); a box is `box_atoms` atoms, no swizzle.
int make_sf_map(CUtensorMap* m, const void* base, uint64_t atoms, uint32_t box_atoms) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -10;
  if (((uint64_t)base & 15) || atoms == 0) return -11;
  cuuint64_t dims[2] = {128, atoms};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, box_atoms};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;     // no device (plan queries on a machine without a GPU): a B200's count
  }
  return n;
}

int ceil_div(int a, int b) { return (a + b - 1) / b; }

template <class Cfg, class Policy>
int launch(const Policy& pol, int grid, cudaStream_t stream) {
  void (*kern)(const Policy);
  if constexpr (Cfg::kPair) kern = gemm_pair_kernel<Cfg, Policy>;
  else kern = gemm_kernel<Cfg, Policy>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return -20;
    attr_set = true;
  }
  kern<<<grid, kThreads, Cfg::kSmemBytes, stream>>>(pol);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}


}  // namespace
