// Block-scaled fp8 (e4m3) GEMM for sm_100a: C[m, n] = sum_kb sA[m, kb] * sB[n / 128, kb] *
// (sum over the 128 k of block kb of A[m, k] * B[n, k]), 16-bit output.
//
// The scale layout is the one of block-quantised transformer weights: activations carry one fp32
// scale per row and 128-wide K block (1 x 128), weights one per 128 x 128 block. The reference
// has no fp8 path (its GEMM main loop, iris/ops/matmul_all_reduce.py:95-105, is 16-bit); this
// kernel is the local building block for fp8 variants of the fused ops.
//
// tcgen05.mma.kind::f8f6f4 accumulates in fp32 but knows nothing about per-block scales, so one
// K block (128 elements = one 128-byte swizzle row = four MMAs of K 32) is accumulated into a
// fresh TMEM buffer and then "promoted": the epilogue warps read the partial sums with tcgen05.ld,
// multiply by sA * sB and add them to accumulators they keep in REGISTERS for the whole tile.
// Two TMEM buffers of 256 columns alternate, so the MMAs of block kb + 1 run while block kb is
// promoted. Roles (384 threads = three warpgroups): warpgroup 0 holds the TMA producer (warp 0)
// and the MMA issuer (warp 1) and gives its registers away (setmaxnreg 40); warpgroups 1 and 2
// (setmaxnreg 232) promote and store: warp w reads TMEM lanes 32 * (w % 4) .. +32 and owns output
// columns 128 * (w / 4 - 1) .. +128, i.e. 128 accumulators per thread. Per K block a thread issues
// 64 packed FMAs (fma.rn.f32x2) and four tcgen05.ld (32 columns each, two in flight at a time).
// The MMAs of a block take about 520 cycles; reading the 128 KB of partial sums back from TMEM
// takes about twice that (measured: with the FMAs removed the kernel tops out at 2.2 PFLOP/s),
// so this formulation is bound by tcgen05.ld, at about 60 % of the unscaled fp8 rate.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <string.h>

#include "iris/host_api.h"
#include "iris/common.cuh"
#include "iris/ptx.cuh"
#include "iris/gemm/sm100_mainloop.cuh"

using namespace iris;
using namespace iris::gemm;

namespace {

constexpr int kBN8 = 256;
constexpr int kBK8 = 128;                 // fp8 elements = bytes per swizzle row = the scale block
constexpr int kStages8 = 4;
constexpr int kThreads8 = 384;
constexpr int kPromoWarps = 8;
constexpr int kABytes8 = kBM * kBK8;      // 16 KB
constexpr int kBBytes8 = kBN8 * kBK8;     // 32 KB
constexpr int kStageBytes8 = kABytes8 + kBBytes8;
constexpr int kEpiBytes8 = kPromoWarps * 2048;
constexpr int kSmemBytes8 = 1024 + kStages8 * kStageBytes8 + kEpiBytes8 + 256;
static_assert(kSmemBytes8 <= 227 * 1024, "shared memory budget");

struct Fp8Args {
  CUtensorMap tmA;          // [M, K] bytes, box 128 x 128
  CUtensorMap tmB;          // [N, K] bytes, box 128 x 256
  const float* sA;          // [M, kblocks]
  const float* sB;          // [ceil(N / 128), kblocks]
  uint8_t* C;               // [M, N] 16-bit, pitch ldc elements
  int64_t ldc;
  int M, N, K;
  int tiles_m, tiles_n, group_m;
  int out_bf16;
  int32_t* status;
};

// kind::f8f6f4 instruction descriptor: fp32 accumulate, A and B e4m3 (format 0), both K-major.
__host__ __device__ constexpr uint32_t idesc_fp8(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

// tcgen05.wait::ld with the loaded registers as in/out operands: the compiler cannot move a use
// of them above the wait.
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                 "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                 "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}
// acc[kOff / 2 .. +16) += scale * r, two columns per instruction (packed fp32 FMA).
template <int kOff>
__device__ __forceinline__ void promote32(unsigned long long (&acc)[64], const uint32_t (&r)[32], unsigned long long scale2) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(r[2 * j]), "r"(r[2 * j + 1]));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc[kOff / 2 + j]) : "l"(scale2), "l"(v));
  }
}

__global__ void __launch_bounds__(kThreads8, 1) gemm_fp8_kernel(const __grid_constant__ Fp8Args a) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* epi_base = smem + kStages8 * kStageBytes8;
  uint64_t* bars = (uint64_t*)(epi_base + kEpiBytes8);
  uint64_t* full = bars;                      // [stages]  TMA bytes landed
  uint64_t* empty = bars + kStages8;          // [stages]  MMAs that read the stage retired
  uint64_t* acc_full = bars + 2 * kStages8;   // [2]       partial sums of one K block complete
  uint64_t* acc_empty = acc_full + 2;         // [2]       partial sums promoted by all 8 warps
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages8; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full[b], 1);
      ptx::mbar_init(&acc_empty[b], kPromoWarps);
    }
    ptx::fence_mbar_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;

  const int num_tiles = a.tiles_m * a.tiles_n;
  const int k_blocks = (a.K + kBK8 - 1) / kBK8;
  const int first = blockIdx.x, step = gridDim.x;
  auto fail = [&]() {
    if (a.status) atomicCAS(a.status, 0, (int)kTimeoutPipeline);
  };

  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      ptx::prefetch_tmap(&a.tmA);
      ptx::prefetch_tmap(&a.tmB);
    }
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int t = first; t < num_tiles && ok; t += step) {
      int tm, tn;
      swizzled_tile(t, a.tiles_m, a.tiles_n, a.group_m, tm, tn);
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&empty[s], ph ^ 1, kPipeTimeoutNs))) { fail(); ok = false; break; }
        {   // converged warp: each instruction elects its issuing lane, operands stay warp-uniform
          const uint32_t sa = ptx::smem_u32(stage_base + s * kStageBytes8);
          ptx::mbar_expect_tx_elect(&full[s], kStageBytes8);
          ptx::tma_load_2d_elect(sa, &a.tmA, &full[s], kb * kBK8, tm * kBM);
          ptx::tma_load_2d_elect(sa + kABytes8, &a.tmB, &full[s], kb * kBK8, tn * kBN8);
        }
        if (++s == kStages8) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = idesc_fp8(kBN8);
    int s = 0;
    uint32_t ph = 0;
    uint32_t blk = 0;      // K blocks issued so far by this CTA: selects the TMEM buffer and its phase
    bool ok = true;
    const uint32_t tmem_u = __reduce_or_sync(0xffffffffu, tmem_base);   // the same value, known to be warp-uniform
    for (int t = first; t < num_tiles && ok; t += step) {
      for (int kb = 0; kb < k_blocks; ++kb, ++blk) {
        const int buf = blk & 1;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&acc_empty[buf], ((blk >> 1) & 1) ^ 1, kPipeTimeoutNs))) { fail(); ok = false; break; }
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&full[s], ph, kPipeTimeoutNs))) { fail(); ok = false; break; }
        ptx::tc_fence_after();
        {
          const uint32_t sa = ptx::smem_u32(stage_base + s * kStageBytes8);
          const uint32_t sb = sa + kABytes8;
          const uint32_t d_tmem = tmem_u + buf * 256;
#pragma unroll
          for (int k = 0; k < kBK8 / 32; ++k)
            ptx::mma_f8_elect(d_tmem, desc_kmajor(sa + k * 32), desc_kmajor(sb + k * 32), idesc, k != 0);
          ptx::mma_commit_elect(&empty[s]);
          ptx::mma_commit_elect(&acc_full[buf]);
        }
        if (++s == kStages8) { s = 0; ph ^= 1; }
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ promotion + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int pw = warp - 4;
    const int quarter = warp & 3;           // TMEM lanes this warp may read
    const int half = pw >> 2;               // which 128 output columns
    uint8_t* my_epi = epi_base + pw * 2048;
    const int sb_rows = (a.N + 127) / 128;
    uint32_t blk = 0;
    bool ok = true;
    for (int t = first; t < num_tiles && ok; t += step) {
      int tm, tn;
      swizzled_tile(t, a.tiles_m, a.tiles_n, a.group_m, tm, tn);
      const int row = tm * kBM + quarter * 32 + lane;
      const int srow = row < a.M ? row : a.M - 1;
      const int sbr = min(tn * 2 + half, sb_rows - 1);
      const float* sa_row = a.sA + (size_t)srow * k_blocks;
      const float* sb_row = a.sB + (size_t)sbr * k_blocks;
      unsigned long long acc[64];      // 128 fp32 accumulators as pairs
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = 0ull;
      float scale_next = __ldg(sa_row) * __ldg(sb_row);
      for (int kb = 0; kb < k_blocks; ++kb, ++blk) {
        const int buf = blk & 1;
        unsigned long long scale;
        asm("mov.b64 %0, {%1, %1};" : "=l"(scale) : "f"(scale_next));
        if (kb + 1 < k_blocks) scale_next = __ldg(sa_row + kb + 1) * __ldg(sb_row + kb + 1);
        if (!ptx::mbar_wait(&acc_full[buf], (blk >> 1) & 1, kPipeTimeoutNs)) { fail(); ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * 256 + half * 128;
        // two loads of 32 columns in flight at a time: the latency of tcgen05.ld, not its
        // bandwidth, bounds this loop
        uint32_t ra[32], rb[32];
        ptx::tmem_ld_32x32(t_addr, ra);
        ptx::tmem_ld_32x32(t_addr + 32, rb);
        tmem_ld_wait_on(ra);
        tmem_ld_wait_on(rb);
        promote32<0>(acc, ra, scale);
        ptx::tmem_ld_32x32(t_addr + 64, ra);
        promote32<32>(acc, rb, scale);
        ptx::tmem_ld_32x32(t_addr + 96, rb);
        tmem_ld_wait_on(ra);
        tmem_ld_wait_on(rb);
        ptx::tc_fence_before();                  // every load of this buffer has completed: hand it back
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
        promote32<64>(acc, ra, scale);
        promote32<96>(acc, rb, scale);
      }
      if (!ok) break;
      // ---- tile epilogue: 16-bit, shared-memory transpose, 16-byte row-major stores
      const int row0 = tm * kBM + quarter * 32;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int col0 = tn * kBN8 + half * 128 + c * 32;
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float lo, hi;
          asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[c * 16 + j]));
          if (a.out_bf16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
            packed[j] = *(uint32_t*)&h;
          } else {
            __half2 h = __floats2half2_rn(lo, hi);
            packed[j] = *(uint32_t*)&h;
          }
        }
        const int sw = (lane >> 1) & 3;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          *(uint4*)(my_epi + lane * 64 + ((j ^ sw) * 16)) = v;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int rr = i * 8 + (lane >> 2), cc = lane & 3;
          uint4 v = *(uint4*)(my_epi + rr * 64 + ((cc ^ ((rr >> 1) & 3)) * 16));
          const int orow = row0 + rr, ocol = col0 + cc * 8;
          if (orow < a.M && ocol < a.N) *(uint4*)(a.C + ((int64_t)orow * a.ldc + ocol) * 2) = v;
        }
        __syncwarp();
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, 512);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// 2-D map over a row-major [rows, cols] byte matrix with pitch `ld` bytes; box = 128 bytes x box_rows.
int make_map_u8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  static EncodeTiledFn enc = nullptr;
  if (!enc) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return -10;
    enc = (EncodeTiledFn)p;
  }
  if (((uint64_t)base & 15) || (ld & 15)) return -11;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

}  // namespace

extern "C" int iris_gemm_fp8_launch(const IrisFp8GemmDesc* d, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return -3;
  if (d->K % 16 || d->N % 8 || d->lda % 16 || d->ldb % 16) return -3;   // TMA pitch and 16-byte output stores
  if (d->out_dtype != IRIS_BF16 && d->out_dtype != IRIS_F16) return -2;
  Fp8Args a;
  int r = make_map_u8(&a.tmA, d->A, d->M, d->K, d->lda, kBM);
  if (r) return r;
  r = make_map_u8(&a.tmB, d->B, d->N, d->K, d->ldb, kBN8);
  if (r) return r;
  a.sA = d->scale_a; a.sB = d->scale_b;
  a.C = (uint8_t*)d->C; a.ldc = d->ldc;
  a.M = d->M; a.N = d->N; a.K = d->K;
  a.tiles_m = (d->M + kBM - 1) / kBM;
  a.tiles_n = (d->N + kBN8 - 1) / kBN8;
  a.group_m = 8;
  a.out_bf16 = d->out_dtype == IRIS_BF16;
  a.status = d->status;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes8) != cudaSuccess) return -20;
    attr_set = true;
  }
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = a.tiles_m * a.tiles_n;
  gemm_fp8_kernel<<<tiles < sms ? tiles : sms, kThreads8, kSmemBytes8, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
