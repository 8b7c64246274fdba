// Activation quantiser for the block-scaled fp8 paths: x [M, K] (fp32 / bf16 / fp16) -> e4m3 values with
// one power-of-two scale per row and 128-wide K block, written in the three forms the kernels use:
//   q      [M, K] e4m3
//   scale  [M, KB] fp32 (optional; what the PyTorch oracle multiplies by)
//   atoms  [ceil(M / 128), KB, 512] UE8M0 bytes in the layout tcgen05.cp copies into TMEM: row r of a
//          128-row tile at byte (r % 32) * 16 + (r / 32) * 4, four equal bytes (the four 32-element K
//          groups of the block share the scale).
//   rows   [M, ld_rows] one UE8M0 byte per row and K block (optional): the form that travels with a row when
//          rows are routed one by one (MoE dispatch); the consumer builds the atoms of its tiles from it.
// The reference has no quantised path; this plays the role of the activation cast in front of its
// 16-bit GEMMs (iris/ops/matmul_all_reduce.py:95-105 consumes 16-bit tiles directly).
// One warp per (row, K block): four elements per lane, amax by shuffles, scale = 2^ceil(log2(amax / 448)).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "iris/host_api.h"

namespace {

template <typename T>
__device__ __forceinline__ void load4(const T* p, int n_valid, bool vec, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, int n_valid, bool vec, float (&v)[4]) {
  if (vec && n_valid >= 4) {
    const float4 f = *(const float4*)p;
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
  } else {
    for (int i = 0; i < 4; ++i) v[i] = i < n_valid ? p[i] : 0.f;
  }
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, int n_valid, bool vec, float (&v)[4]) {
  if (vec && n_valid >= 4) {
    const uint2 u = *(const uint2*)p;
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&u.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&u.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    for (int i = 0; i < 4; ++i) v[i] = i < n_valid ? __bfloat162float(p[i]) : 0.f;
  }
}
template <>
__device__ __forceinline__ void load4<__half>(const __half* p, int n_valid, bool vec, float (&v)[4]) {
  if (vec && n_valid >= 4) {
    const uint2 u = *(const uint2*)p;
    const float2 a = __half22float2(*(const __half2*)&u.x), b = __half22float2(*(const __half2*)&u.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    for (int i = 0; i < 4; ++i) v[i] = i < n_valid ? __half2float(p[i]) : 0.f;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_1x128_pow2_kernel(const T* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q, int64_t ldq,
                                                                   float* __restrict__ scale, uint8_t* __restrict__ atoms,
                                                                   uint8_t* __restrict__ rows, int64_t ld_rows, int M, int K, int KB,
                                                                   int aligned) {
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (int64_t)M * KB) return;
  const int row = (int)(warp / KB), kb = (int)(warp - (int64_t)row * KB);
  const int k0 = kb * 128 + lane * 4;
  const int n_valid = max(0, min(4, K - k0));
  float v[4];
  load4<T>(x + (int64_t)row * ldx + k0, n_valid, aligned != 0, v);   // unaligned rows take the element-wise path
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax = fmaxf(amax, 1e-12f);
  // smallest power of two >= amax / 448, as an exponent
  int e = (int)ceilf(log2f(amax * (1.0f / 448.0f)));
  e = max(-127, min(127, e));
  const float s = exp2f((float)e), inv = exp2f((float)-e);
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_fp8_e4m3 f(fminf(fmaxf(v[i] * inv, -448.f), 448.f));
    packed |= (uint32_t)f.__x << (8 * i);
  }
  uint8_t* dst = q + (int64_t)row * ldq + k0;
  if (n_valid == 4 && (ldq & 3) == 0) *(uint32_t*)dst = packed;
  else for (int i = 0; i < n_valid; ++i) dst[i] = (uint8_t)(packed >> (8 * i));
  if (lane == 0) {
    if (scale) scale[(int64_t)row * KB + kb] = s;
    if (rows) rows[(int64_t)row * ld_rows + kb] = (uint8_t)(e + 127);
    if (atoms) {
      const uint32_t b = (uint32_t)(e + 127);
      const int tile = row >> 7, r = row & 127;
      *(uint32_t*)(atoms + ((int64_t)tile * KB + kb) * 512 + (r & 31) * 16 + (r >> 5) * 4) = b * 0x01010101u;
    }
  }
}

}  // namespace

// x: [M, K] of `dtype` (IRIS_F32 / IRIS_BF16 / IRIS_F16), row pitch ldx elements. q: [M, K] bytes, pitch ldq.
// scale (may be null): [M, ceil(K / 128)] fp32. atoms (may be null): [ceil(M / 128), ceil(K / 128), 512] bytes;
// rows past M inside the last 128-row tile are NOT written (pre-fill the buffer with 127 = scale 1 if M is ragged).
static int quantize_launch(const void* x, int64_t ldx, int32_t dtype, void* q, int64_t ldq, float* scale, void* atoms, void* rows,
                           int64_t ld_rows, int32_t M, int32_t K, void* stream) {
  if (M <= 0 || K <= 0) return 0;
  const int KB = (K + 127) / 128;
  const int64_t warps = (int64_t)M * KB;
  const int64_t blocks = (warps * 32 + 255) / 256;
  if (blocks > 0x7fffffffll) return -3;
  cudaStream_t s = (cudaStream_t)stream;
  const int esz = dtype == IRIS_F32 ? 4 : 2;
  const int aligned = (((uintptr_t)x % (4 * esz)) == 0 && (ldx * esz) % (4 * esz) == 0) ? 1 : 0;
  if (dtype == IRIS_F32)
    quantize_1x128_pow2_kernel<float><<<(unsigned)blocks, 256, 0, s>>>((const float*)x, ldx, (uint8_t*)q, ldq, scale, (uint8_t*)atoms, (uint8_t*)rows, ld_rows, M, K, KB, aligned);
  else if (dtype == IRIS_BF16)
    quantize_1x128_pow2_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, scale, (uint8_t*)atoms, (uint8_t*)rows, ld_rows, M, K, KB, aligned);
  else if (dtype == IRIS_F16)
    quantize_1x128_pow2_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>((const __half*)x, ldx, (uint8_t*)q, ldq, scale, (uint8_t*)atoms, (uint8_t*)rows, ld_rows, M, K, KB, aligned);
  else
    return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int iris_quantize_1x128_pow2(const void* x, int64_t ldx, int32_t dtype, void* q, int64_t ldq, float* scale, void* atoms,
                                        int32_t M, int32_t K, void* stream) {
  return quantize_launch(x, ldx, dtype, q, ldq, scale, atoms, nullptr, 0, M, K, stream);
}
// Same, writing one scale byte per row and K block into rows [M, ld_rows] (bytes past ceil(K / 128) of a row are left alone).
extern "C" int iris_quantize_1x128_pow2_rows(const void* x, int64_t ldx, int32_t dtype, void* q, int64_t ldq, void* rows, int64_t ld_rows,
                                             int32_t M, int32_t K, void* stream) {
  return quantize_launch(x, ldx, dtype, q, ldq, nullptr, nullptr, rows, ld_rows, M, K, stream);
}
