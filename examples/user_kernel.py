#!/usr/bin/env python3
"""Write your own kernel against the device library (the README example of the reference: rank 0
stores into rank 1's buffer from inside a kernel).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/user_kernel.py
"""
import torch

from _common import finish, init

SOURCE = r"""
#include <cuda_runtime.h>
#include <string.h>
#include <iris/host_api.h>
#include <iris/iris.cuh>

__global__ void fill_remote(iris::DeviceContext ctx, float* buf, int n, float value, int to_rank) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  iris::Ctx(ctx).store(buf + i, value, to_rank, i < n);     // translate + st.global on the peer's heap
}
extern "C" int launch(const IrisCtx* c, float* buf, int n, float value, int to_rank, void* stream) {
  iris::DeviceContext ctx;
  memcpy(&ctx, c, sizeof(ctx));
  fill_remote<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(ctx, buf, n, value, to_rank);
  return (int)cudaGetLastError();
}
"""

if __name__ == "__main__":
    ctx = init()
    from iris_b200 import jit

    mod = jit.compile_source(SOURCE, name="fill_remote")
    buf = ctx.zeros(4096, dtype=torch.float32)
    ctx.barrier()
    if ctx.get_rank() == 0 and ctx.get_num_ranks() > 1:
        mod.fn("launch")(ctx, buf, buf.numel(), 1.0, 1)
    ctx.barrier()
    expect = 1.0 if (ctx.get_rank() == 1) else 0.0
    assert torch.all(buf == expect)
    ctx.info(f"buffer is all {expect}")
    finish(ctx)
