// User-style kernels for the tests: written only against <iris/iris.cuh>, compiled by
// iris_b200.jit, launched through extern "C" functions. They exercise the functional and the
// object-oriented device API, masks, the message-passing protocol and the tile collectives.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <string.h>

#include <iris/host_api.h>
#include <iris/iris.cuh>

using namespace iris;

static DeviceContext to_ctx(const IrisCtx* c) {
  DeviceContext ctx;
  memcpy(&ctx, c, sizeof(ctx));
  return ctx;
}

// README example of the reference: store a value into a peer's buffer block by block.
__global__ void store_blocks_kernel(DeviceContext ctx, float* buf, int n, float value, int to_rank) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  store(buf + i, value, ctx.rank, to_rank, ctx.bases, i < n);
}
extern "C" int store_blocks(const IrisCtx* c, float* buf, int n, float value, int to_rank, void* stream) {
  store_blocks_kernel<<<(n + 1023) / 1024, 1024, 0, (cudaStream_t)stream>>>(to_ctx(c), buf, n, value, to_rank);
  return (int)cudaGetLastError();
}

// Context built on the device from the int64 context tensor, masked load with `other`.
__global__ void masked_load_kernel(const int64_t* ctx_tensor, const int* src, int* out, int n, int valid, int from_rank) {
  DeviceContext ctx = DeviceContext::initialize(ctx_tensor);
  Ctx c(ctx);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = c.load(src + i, from_rank, i < valid, -7);
}
extern "C" int masked_load(const int64_t* ctx_tensor, const int* src, int* out, int n, int valid, int from_rank, void* stream) {
  masked_load_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(ctx_tensor, src, out, n, valid, from_rank);
  return (int)cudaGetLastError();
}

// Atomic counter: every thread of every rank adds 1 to `counter` on `to_rank` (release, sys).
__global__ void count_kernel(DeviceContext ctx, int* counter, int to_rank) {
  Ctx(ctx).atomic_add<Sem::release, Scope::sys>(counter, 1, to_rank);
}
extern "C" int count(const IrisCtx* c, int* counter, int threads, int to_rank, void* stream) {
  count_kernel<<<1, threads, 0, (cudaStream_t)stream>>>(to_ctx(c), counter, to_rank);
  return (int)cudaGetLastError();
}

// Tile collectives on an (M, N) fp32 matrix, one CTA per tile. op: 0 atomic, 1 spinlock,
// 2 one_shot, 3 two_shot, 4 all_gather(dim 0), 5 gather(from `arg`), 6 all_to_all (chunk N = arg),
// 7 reduce_scatter. For 2, 3, 7 the kernel first publishes "tile ready" on its own lock.
__global__ void tile_kernel(DeviceContext ctx, int op, float* src, float* dst, int32_t* locks, int M, int N, int dst_M,
                            int dst_N, int bm, int bn, int arg, int32_t ready) {
  const int tiles_n = ((op == 6 ? arg : N) + bn - 1) / bn;
  const int tiles_m = (M + bm - 1) / bm;
  const int tile_id = blockIdx.x;
  if (tile_id >= tiles_m * tiles_n) return;
  TileView t{tile_id / tiles_n, tile_id % tiles_n, bm, bn};
  TensorView<float> s = make_tensor_view(src, M, N, (int64_t)N);
  TensorView<float> d = make_tensor_view(dst, dst_M, dst_N, (int64_t)dst_N);
  if (op == 2 || op == 3 || op == 7 || op == 8) {
    __syncthreads();
    if (threadIdx.x == 0) { fence_sys(); st_release_sys(locks + tile_id, ready); }
  }
  switch (op) {
    case 0: tile::all_reduce_atomic(ctx, t, s, d); break;
    case 1: tile::all_reduce_spinlock(ctx, t, tile_id, s, d, locks); break;
    case 2: tile::all_reduce_one_shot(ctx, t, tile_id, s, d, locks, ready); break;
    case 3: tile::all_reduce_two_shot(ctx, t, tile_id, s, d, locks, ready); break;
    case 4: tile::all_gather(ctx, t, s, d, 0); break;
    case 5: tile::gather(ctx, t, s, d, arg); break;
    case 6: tile::all_to_all(ctx, t, s, d, arg); break;
    case 7: tile::reduce_scatter(ctx, t, tile_id, tiles_m * tiles_n, s, d, locks, ready); break;
    case 8: tile::all_reduce_ring(ctx, t, tile_id, s, d, locks, ready); break;
  }
}
extern "C" int tile_collective(const IrisCtx* c, int op, float* src, float* dst, int32_t* locks, int M, int N, int dst_M,
                               int dst_N, int bm, int bn, int arg, int ready, void* stream) {
  const int tiles = ((M + bm - 1) / bm) * (((op == 6 ? arg : N) + bn - 1) / bn);
  tile_kernel<<<tiles, 128, 0, (cudaStream_t)stream>>>(to_ctx(c), op, src, dst, locks, M, N, dst_M, dst_N, bm, bn, arg, ready);
  return (int)cudaGetLastError();
}
