#!/usr/bin/env python3
"""Per-tile timeline of the fused all_gather_matmul and matmul_reduce_scatter kernels on the shapes of
`bench.py` (8192 x 3584 x 8192 and 8192 x 8192 x 3584 per rank, bf16), at any world size.

    python benchmark/ops/timeline_fused_ops.py                                          (1 GPU)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmark/ops/timeline_fused_ops.py

For each op: device time per call (CUDA events around 20 back-to-back calls after 3 warm-up calls,
maximum over ranks), then ONE call with the kernel's own timestamps switched on
(`FusedWorkspace.extra["timeline"]`, %globaltimer per tile: start, first operand available, stored;
the reference's examples collect the same with COLLECT_TIMESTAMPS, examples/07_gemm_all_scatter/
gemm_all_scatter.py:64-66). Printed per wave of tiles: when the wave started, how long its tiles waited
for their gathered operand, when they were done; and the times at which the communication CTAs had
signalled every eighth chunk. `DIAG_COMM=8,32` adds runs with that many communication CTAs.
"""
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch, torch.distributed as dist, numpy as np
rank = int(os.environ.get("RANK", 0)); world = int(os.environ.get("WORLD_SIZE", 1)); local = int(os.environ.get("LOCAL_RANK", 0))
torch.cuda.set_device(local)
os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29577")
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
import iris_b200 as iris
from iris_b200.ops import FusedConfig
ctx = iris.iris(8 << 30)
dtype = torch.bfloat16; W = world
Ml, K, N = 8192 // W, 8192, 3584


def timed(fn, iters=20):
    for _ in range(3): fn()
    ctx.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier(); torch.cuda.synchronize()
    s.record()
    for _ in range(iters): fn()
    e.record(); torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


A = torch.randn(Ml, K, device="cuda", dtype=dtype); B = (torch.randn(N, K, device="cuda", dtype=dtype) * 0.02).t()
C = ctx.zeros((W * Ml, N), dtype=dtype)
variants = [(0, True)]
extra = [int(x) for x in os.environ.get("DIAG_COMM", "").split(",") if x]
for cc in extra:
    variants += [(cc, True)]
for comm, mc in variants:
    cfg = FusedConfig(comm_sms=comm, use_multicast=mc)
    ws = ctx.ops.all_gather_matmul(C, A, B, shard_dim=0, config=cfg)
    ms = timed(lambda: ctx.ops.all_gather_matmul(C, A, B, shard_dim=0, workspace=ws, config=cfg, async_op=True))
    pair = ws.extra.get("two_sm", 1) == 2
    tiles128 = 64 * (-(-N // ws.bn)); chunks = Ml // 128
    order_tiles = tiles128 // 2 if pair else tiles128
    tl = torch.zeros((tiles128 + chunks, 4), dtype=torch.int64, device="cuda")
    ctx.barrier()
    ws.extra["timeline"] = tl
    ctx.ops.all_gather_matmul(C, A, B, shard_dim=0, workspace=ws, config=cfg, async_op=True)
    torch.cuda.synchronize()
    ws.extra.pop("timeline")
    t = tl.cpu().numpy().astype(np.float64)
    tt = t[:order_tiles]
    t0 = tt[:, 0][tt[:, 0] > 0].min()
    if rank == 0:
        start = (tt[:, 0] - t0) / 1e3; avail = (tt[:, 1] - t0) / 1e3; done = (tt[:, 2] - t0) / 1e3
        sig = (t[tiles128:, 3] - t0) / 1e3
        cc_used = ws.extra.get("comm_ctas")
        print(f"AG W={W} comm_req={comm} mc={mc} bn={ws.bn} pair={pair}: {ms*1e3:.1f} us/call; span {done.max():.1f} us; chunk issue-done times: {np.round(sig[::max(1, chunks // 8)], 1)}")
        slots = max(1, (148 - (20 if W > 1 else 0)) // (2 if pair else 1))
        nw = -(-order_tiles // slots)
        for wv in range(nw):
            idx = np.arange(wv * slots, min((wv + 1) * slots, order_tiles))
            print(f"  wave {wv}: start {start[idx].mean():7.1f} wait mean {np.mean(avail[idx]-start[idx]):6.1f} max {np.max(avail[idx]-start[idx]):6.1f} done mean {done[idx].mean():7.1f} max {done[idx].max():7.1f}")
    ctx.barrier()

M, Kl, N2 = 8192, 3584, 8192
A2 = torch.randn(M, Kl, device="cuda", dtype=dtype); B2 = (torch.randn(N2, Kl, device="cuda", dtype=dtype) * 0.02).t()
C2 = ctx.zeros((M // W, N2), dtype=dtype)
ws2 = ctx.ops.matmul_reduce_scatter(C2, A2, B2, scatter_rows=True)
ms = timed(lambda: ctx.ops.matmul_reduce_scatter(C2, A2, B2, scatter_rows=True, workspace=ws2, async_op=True))
pair = ws2.extra.get("two_sm", 1) == 2
tiles128 = 64 * (N2 // ws2.bn); order_tiles = tiles128 // 2 if pair else tiles128
tl = torch.zeros((tiles128 + 148, 4), dtype=torch.int64, device="cuda")
ctx.barrier()
ws2.extra["timeline"] = tl
ctx.ops.matmul_reduce_scatter(C2, A2, B2, scatter_rows=True, workspace=ws2, async_op=True)
torch.cuda.synchronize()
ws2.extra.pop("timeline")
t = tl.cpu().numpy().astype(np.float64)
tt = t[:order_tiles]
t0 = tt[:, 0][tt[:, 0] > 0].min()
if rank == 0:
    start = (tt[:, 0] - t0) / 1e3; done = (tt[:, 2] - t0) / 1e3
    print(f"RS W={W} bn={ws2.bn} pair={pair}: {ms*1e3:.1f} us/call; span {done.max():.1f}")
    slots = 148 // (2 if pair else 1)
    for wv in range(-(-order_tiles // slots)):
        idx = np.arange(wv * slots, min((wv + 1) * slots, order_tiles))
        print(f"  wave {wv}: start {start[idx].mean():7.1f} done mean {done[idx].mean():7.1f} max {done[idx].max():7.1f} dur {np.mean(done[idx]-start[idx]):6.1f}")
ctx.barrier()
ctx.close()
dist.barrier(); dist.destroy_process_group()
