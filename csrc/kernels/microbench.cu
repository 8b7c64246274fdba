// Bandwidth micro-benchmarks of the primitives everything else is built from (reference:
// examples/00_load .. 05_atomic_xchg). Each kernel moves `bytes` between a source and a
// destination that the host picks to be local or a peer's heap, with a chosen number of CTAs, so
// the same kernels measure local HBM, NVLink loads, NVLink stores, NVLS multimem stores, remote
// atomics and the TMA bulk-copy path, per SM and in aggregate.
#include <cuda_runtime.h>
#include <string.h>

#include "iris/host_api.h"
#include "iris/iris.cuh"

using namespace iris;

namespace {

// mode 0: dst[i] = src[i] with 16-byte vectors, UNROLL independent loads in flight per thread
template <int UNROLL>
__global__ void __launch_bounds__(512) copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (UNROLL - 1) * stride < n; i += UNROLL * stride) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) dst[i + u * stride] = v[u];
  }
  for (; i < n; i += stride) dst[i] = src[i];
}

// mode 1: read only (sum into a sink so the loads are not removed)
template <int UNROLL>
__global__ void __launch_bounds__(512) read_kernel(const uint4* __restrict__ src, size_t n, uint32_t* sink) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  uint32_t acc = 0;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (UNROLL - 1) * stride < n; i += UNROLL * stride) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  for (; i < n; i += stride) acc ^= src[i].x;
  if (acc == 0x12345678u) *sink = acc;
}

// mode 2: write only
__global__ void __launch_bounds__(512) write_kernel(uint4* __restrict__ dst, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const uint4 v = make_uint4(1, 2, 3, 4);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = v;
}

// mode 3: multimem.st broadcast of src to the multicast address mc_dst
template <int UNROLL>
__global__ void __launch_bounds__(512) mc_store_kernel(uint8_t* mc_dst, const uint4* __restrict__ src, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (UNROLL - 1) * stride < n; i += UNROLL * stride) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      multimem::V4 m{v[u].x, v[u].y, v[u].z, v[u].w};
      multimem::st_v4(mc_dst + (i + u * stride) * 16, m);
    }
  }
  for (; i < n; i += stride) {
    uint4 v = src[i];
    multimem::V4 m{v.x, v.y, v.z, v.w};
    multimem::st_v4(mc_dst + i * 16, m);
  }
}

// mode 4: relaxed atomic add of 1 to every 32-bit word of dst (system scope)
__global__ void __launch_bounds__(512) atomic_kernel(int32_t* dst, size_t n_words, int xchg) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += stride) {
    if (xchg) atomicExch_system(dst + i, 1);
    else asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(dst + i), "r"(1) : "memory");
  }
}

// mode 5: TMA bulk path, one thread per CTA: global -> shared ring -> global (dst may be a peer).
// `piece` bytes per copy, `nbuf` ring slots. Bounded mbarrier waits.
__global__ void __launch_bounds__(128) bulk_copy_kernel(uint8_t* dst, const uint8_t* src, size_t bytes, int piece, int nbuf,
                                                        int32_t* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = (uint64_t*)(smem + (size_t)nbuf * piece);
  if (threadIdx.x == 0) {
    for (int i = 0; i < nbuf; ++i) ptx::mbar_init(&bars[i], 1);
    ptx::fence_mbar_init();
    ptx::fence_proxy_async();
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const size_t n_pieces = (bytes + piece - 1) / piece;
  // CTA c handles pieces c, c + grid, ...
  const size_t mine = n_pieces > blockIdx.x ? (n_pieces - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  auto off = [&](size_t k) { return ((size_t)blockIdx.x + k * gridDim.x) * piece; };
  auto len = [&](size_t k) { size_t o = off(k); return (uint32_t)(bytes - o < (size_t)piece ? bytes - o : piece); };
  auto issue = [&](size_t k) {
    const int slot = (int)(k % nbuf);
    ptx::mbar_expect_tx(&bars[slot], len(k));
    ptx::bulk_load(smem + (size_t)slot * piece, src + off(k), len(k), &bars[slot]);
  };
  size_t next = mine < (size_t)nbuf ? mine : nbuf;
  for (size_t k = 0; k < next; ++k) issue(k);
  for (size_t k = 0; k < mine; ++k) {
    const int slot = (int)(k % nbuf);
    if (!ptx::mbar_wait(&bars[slot], (uint32_t)((k / nbuf) & 1))) {
      atomicCAS(status, 0, kTimeoutPipeline);
      break;
    }
    ptx::bulk_store(dst + off(k), smem + (size_t)slot * piece, len(k));
    ptx::bulk_commit();
    long free_upto;
    if (k == mine - 1) { ptx::bulk_wait<0>(); free_upto = (long)k; }
    else { ptx::bulk_wait_read<1>(); free_upto = (long)k - 1; }
    while ((long)next <= free_upto + nbuf && next < mine) issue(next++);
  }
}

}  // namespace

extern "C" {

// mode: 0 copy, 1 read, 2 write, 3 multimem store, 4 atomic add, 5 atomic xchg, 6 TMA bulk copy.
// Returns 0; timing is done by the caller with CUDA events around the launch.
int iris_microbench(int mode, void* dst, const void* src, unsigned long long bytes, int ctas, int unroll, int piece,
                    int nbuf, int32_t* status, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const size_t n = bytes / 16;
  if (ctas <= 0) ctas = 148;
  switch (mode) {
    case 0:
      if (unroll >= 8) copy_kernel<8><<<ctas, 512, 0, s>>>((uint4*)dst, (const uint4*)src, n);
      else if (unroll >= 4) copy_kernel<4><<<ctas, 512, 0, s>>>((uint4*)dst, (const uint4*)src, n);
      else copy_kernel<1><<<ctas, 512, 0, s>>>((uint4*)dst, (const uint4*)src, n);
      break;
    case 1:
      if (unroll >= 8) read_kernel<8><<<ctas, 512, 0, s>>>((const uint4*)src, n, (uint32_t*)status);
      else read_kernel<1><<<ctas, 512, 0, s>>>((const uint4*)src, n, (uint32_t*)status);
      break;
    case 2: write_kernel<<<ctas, 512, 0, s>>>((uint4*)dst, n); break;
    case 3:
      if (unroll >= 8) mc_store_kernel<8><<<ctas, 512, 0, s>>>((uint8_t*)dst, (const uint4*)src, n);
      else mc_store_kernel<1><<<ctas, 512, 0, s>>>((uint8_t*)dst, (const uint4*)src, n);
      break;
    case 4: atomic_kernel<<<ctas, 512, 0, s>>>((int32_t*)dst, bytes / 4, 0); break;
    case 5: atomic_kernel<<<ctas, 512, 0, s>>>((int32_t*)dst, bytes / 4, 1); break;
    case 6: {
      if (piece <= 0) piece = 32768;
      if (nbuf <= 0) nbuf = 6;
      const int smem = nbuf * piece + 256;
      static int configured = 0;
      if (smem > configured) {
        if (cudaFuncSetAttribute(bulk_copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -20;
        configured = smem;
      }
      bulk_copy_kernel<<<ctas, 128, smem, s>>>((uint8_t*)dst, (const uint8_t*)src, bytes, piece, nbuf, status);
      break;
    }
    default: return -2;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // extern "C"
