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
  int bf16;
  int bn;
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
  IRIS_D bool is_bf16() const { return bf16 != 0; }
  IRIS_D bool has_bias() const { return bias_row != nullptr || bias_col != nullptr; }
  IRIS_D float row_bias(int row) const { return (bias_row && row < sh.M) ? bias_row[row] : 0.f; }
  IRIS_D float col_bias(int col) const { return (bias_col && col < sh.N) ? bias_col[col] : 0.f; }
  IRIS_D void fail(int code) const {
    if (status) atomicCAS(status, 0, code);
  }
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
// 2-D map over a row-major [rows, cols] 16-bit matrix with pitch `ld` elements; box = box_cols x box_rows.
int make_map(CUtensorMap* m, const void* base, int dtype, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
             uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -10;
  if (((uint64_t)base & 15) || ((ld * 2) & 15)) return -11;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = dtype == IRIS_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(m, dt, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
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
