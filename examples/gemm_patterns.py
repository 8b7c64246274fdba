#!/usr/bin/env python3
"""The overlap patterns of the reference's GEMM examples, each as the fused op that covers it here:

    07 gemm_all_scatter, 10 (workgroup specialisation), 11 (producer/consumer), 20 (independent)  -> matmul_all_gather(scatter_cols=True)
    12 gemm_all_scatter bulk-synchronous                                                            -> local matmul + ccl.all_gather
    08 gemm_all_reduce_atomics, 09 / 21 gemm_one_shot_all_reduce, 15 gemm_all_reduce_ring_based     -> matmul_all_reduce
    22 gemm_one_shot_reduce_scatter                                                                 -> matmul_reduce_scatter
    14 all_gather_gemm (pull / push)                                                                -> all_gather_matmul
    23 gemm_all_scatter_tracing                                                                     -> per-tile timeline of a fused op

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/gemm_patterns.py
"""
import torch
import torch.distributed as dist

from _common import finish, init

if __name__ == "__main__":
    ctx = init(2 << 30)
    W, r = ctx.get_num_ranks(), ctx.get_rank()
    dev = ctx.get_device()
    dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
    torch.manual_seed(r)
    M, K, N = 256, 512, 256
    A = torch.randn(M, K, device=dev, dtype=dt)
    B = torch.randn(K, N, device=dev, dtype=dt) * 0.05
    local = A.float() @ B.float()
    parts = [torch.empty_like(local) for _ in range(W)]
    dist.all_gather(parts, local)
    tol = 0.05 * max(p.abs().max().item() for p in parts) * W

    # GEMM + all-scatter: rank r's [M, N] product lands in columns [r*N, (r+1)*N) on every rank
    C = ctx.zeros((M, W * N), dtype=dt)
    ctx.ops.matmul_all_gather(C, A, B, scatter_cols=True)
    assert (C.float() - torch.cat(parts, dim=1)).abs().max().item() < tol
    # the same result under each selectable overlap pattern (examples 07 / 10 / 11 / 12 of the reference):
    # epilogue stores, communication CTAs forwarding finished tiles, GEMM kernel followed by the collective
    from iris_b200.ops import FusedConfig, matmul
    for pattern in ("fused", "wg_specialized", "producer_consumer", "bulk_synchronous"):
        Cp = ctx.zeros((M, W * N), dtype=dt)
        ctx.ops.matmul_all_gather(Cp, A, B, scatter_cols=True, config=FusedConfig(overlap=pattern))
        assert (Cp.float() - torch.cat(parts, dim=1)).abs().max().item() < tol, pattern
    # the bulk-synchronous form by hand: GEMM, then the collective
    loc = ctx.as_symmetric((matmul(A, B) if A.is_cuda else (A @ B)).contiguous())
    rows = ctx.zeros((W * M, N), dtype=dt)
    ctx.ccl.all_gather(rows, loc)
    assert (rows.float() - torch.cat(parts, dim=0)).abs().max().item() < tol
    # GEMM + all-reduce and GEMM + reduce-scatter of the partial products
    total = torch.stack(parts).sum(0)
    C2 = ctx.zeros((M, N), dtype=dt)
    ctx.ops.matmul_all_reduce(C2, A, B)
    assert (C2.float() - total).abs().max().item() < tol
    # every all-reduce variant (examples 08: atomics, 09 / 21: one shot; two_shot: owner reduces, then broadcasts)
    for variant in ("two_shot", "one_shot", "atomic"):
        Cv = ctx.zeros((M, N), dtype=dt)
        ctx.ops.matmul_all_reduce(Cv, A, B, config=FusedConfig(all_reduce_variant=variant))
        assert (Cv.float() - total).abs().max().item() < tol, variant
    if M % (128 * W) == 0:
        C3 = ctx.zeros((M // W, N), dtype=dt)
        ctx.ops.matmul_reduce_scatter(C3, A, B, scatter_rows=True)
        assert (C3.float() - total[r * (M // W):(r + 1) * (M // W)]).abs().max().item() < tol
    # all-gather + GEMM: A sharded along K
    Ak = torch.randn(M, K // W, device=dev, dtype=dt)
    Bk = torch.randn(K, N, device=dev, dtype=dt) * 0.05
    dist.broadcast(Bk, 0)
    shards = [torch.empty_like(Ak) for _ in range(W)]
    dist.all_gather(shards, Ak)
    C4 = ctx.zeros((M, N), dtype=dt)
    ctx.ops.all_gather_matmul(C4, Ak, Bk)
    ref = torch.cat(shards, dim=1).float() @ Bk.float()
    assert (C4.float() - ref).abs().max().item() < 0.05 * ref.abs().max().item()
    ctx.check()
    ctx.info("GEMM + collective patterns validated")
    finish(ctx)
