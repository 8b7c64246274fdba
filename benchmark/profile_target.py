#!/usr/bin/env python3
"""Small, self-terminating workloads for `ncu` captures (one GPU, a few launches, < 1 GB held).

    python benchmark/profile_target.py gemm      # 3 launches of the local tcgen05 GEMM 4096x3584x8192 bf16
    python benchmark/profile_target.py decode    # 3 flash-decode steps, batch 8, 16384 keys, 64/8 heads
    python benchmark/profile_target.py fused     # world-size-1 all_gather_matmul + matmul_reduce_scatter
    python benchmark/profile_target.py moe       # one MoE layer pass, 1024 tokens, 8 experts
    python benchmark/profile_target.py moe_fp8   # the same with e4m3 tokens, weights and hidden activations
    python benchmark/profile_target.py fp8       # 3 launches of the block-scaled fp8 GEMM 4096x4096x7168
    python benchmark/profile_target.py ring      # 3 ring-attention calls, world size 1, 4096 tokens, 32/8 heads
    python benchmark/profile_target.py fp8hw     # 3 launches of the hardware block-scaled fp8 GEMM 4096x3584x8192
    python benchmark/profile_target.py ar        # world-size-1 matmul_all_reduce (two_shot, one_shot) and matmul_all_gather
    python benchmark/profile_target.py ccl       # world-size-1 all_reduce / all_gather / reduce_scatter kernels, 256 MB
    python benchmark/profile_target.py moe_full  # two passes of the benchmark-size MoE layer (4096 tokens, hidden 7168, 32 experts, top-8):
    python benchmark/profile_target.py moe_fp8_full   # for a launch list (`--metrics gpu__time_duration.sum`, one pass) only, about 6 GB held

The fused ops and collectives run here with ONE rank: the same kernel templates as on several GPUs
(policy code, epilogues, flag protocol) with no peer to wait for, which is the form a replaying
profiler can capture safely.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def ctx_world1(heap=2 << 30):
    import iris_b200 as iris

    torch.cuda.set_device(0)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    return iris.iris(heap)


def main():
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    dt = torch.bfloat16
    if what == "gemm":
        from iris_b200.ops.gemm import matmul

        A = torch.randn(4096, 8192, device="cuda", dtype=dt)
        B = torch.randn(8192, 3584, device="cuda", dtype=dt) * 0.02
        C = torch.empty(4096, 3584, device="cuda", dtype=dt)
        for _ in range(3):
            matmul(A, B, out=C)
        torch.cuda.synchronize()
        return
    if what == "fp8":
        from iris_b200.ops.gemm_fp8 import matmul_fp8, quantize_1x128, quantize_128x128

        aq, asc = quantize_1x128(torch.randn(4096, 7168, device="cuda"))
        bq, bsc = quantize_128x128(torch.randn(4096, 7168, device="cuda") * 0.05)
        out = torch.empty(4096, 4096, device="cuda", dtype=dt)
        for _ in range(3):
            matmul_fp8(aq, asc, bq, bsc, out=out)
        torch.cuda.synchronize()
        return
    if what == "fp8hw":
        from iris_b200.ops import matmul, quantize_activation, quantize_weight

        a = quantize_activation(torch.randn(4096, 8192, device="cuda"))
        b = quantize_weight(torch.randn(3584, 8192, device="cuda") * 0.05)
        out = torch.empty(4096, 3584, device="cuda", dtype=dt)
        for _ in range(3):
            matmul(a, b, out=out)
        torch.cuda.synchronize()
        return
    ctx = ctx_world1(8 << 30 if what.endswith("_full") else 2 << 30)
    if what == "ar":
        from iris_b200.ops import FusedConfig

        A = torch.randn(4096, 3584, device="cuda", dtype=dt)
        B = torch.randn(3584, 8192, device="cuda", dtype=dt) * 0.02
        C = ctx.zeros((4096, 8192), dtype=dt)
        for variant in ("two_shot", "one_shot"):
            for _ in range(2):
                ctx.ops.matmul_all_reduce(C, A, B, config=FusedConfig(all_reduce_variant=variant), async_op=True)
        for _ in range(2):
            ctx.ops.matmul_all_gather(C, A, B, async_op=True)
    elif what == "ccl":
        x = ctx.zeros((8192, 16384), dtype=dt)            # 256 MB
        y = ctx.zeros((8192, 16384), dtype=dt)
        for _ in range(2):
            ctx.ccl.all_reduce(y, x, async_op=True)
            ctx.ccl.all_gather(y, x, async_op=True)
            ctx.ccl.reduce_scatter(y, x, async_op=True)
    elif what == "decode":
        from iris_b200.models import FlashDecodeLayer

        B_, L, Hq, Hkv, page = 8, 16384, 64, 8, 64
        nb = L // page
        kc = torch.randn(B_ * nb, page, Hkv, 128, device="cuda", dtype=dt)
        vc = torch.randn(B_ * nb, page, Hkv, 128, device="cuda", dtype=dt)
        table = torch.arange(B_ * nb, device="cuda", dtype=torch.int32).view(B_, nb)
        lens = torch.full((1, B_), L, device="cuda", dtype=torch.int32)
        q = torch.randn(B_, Hq, 128, device="cuda", dtype=dt)
        layer = FlashDecodeLayer(ctx, Hq, Hkv, 128, max_batch=B_)
        for _ in range(3):
            layer(q, kc, vc, lens, table)
    elif what == "ring":
        from iris_b200.models import RingAttention

        S, Hq, Hkv = 4096, 32, 8
        q = torch.randn(S, Hq, 128, device="cuda", dtype=dt)
        k = torch.randn(S, Hkv, 128, device="cuda", dtype=dt)
        v = torch.randn(S, Hkv, 128, device="cuda", dtype=dt)
        layer = RingAttention(ctx, S, Hq, Hkv)
        for _ in range(3):
            layer(q, k, v, causal=False)
    elif what == "fused":
        X = torch.randn(4096, 8192, device="cuda", dtype=dt)
        W1 = torch.randn(8192, 3584, device="cuda", dtype=dt) * 0.02
        W2 = torch.randn(3584, 8192, device="cuda", dtype=dt) * 0.02
        H = torch.empty(4096, 3584, device="cuda", dtype=dt)
        Y = torch.empty(4096, 8192, device="cuda", dtype=dt)
        for _ in range(2):
            ctx.ops.all_gather_matmul(H, X, W1, shard_dim=0, async_op=True)
            ctx.ops.matmul_reduce_scatter(Y, H, W2, scatter_rows=True, async_op=True)
    elif what in ("moe", "moe_fp8", "moe_full", "moe_fp8_full"):
        from iris_b200.models import MoELayer

        T, D, F, E, K = (4096, 7168, 2048, 32, 8) if what.endswith("_full") else (1024, 2048, 1024, 8, 2)
        wg = (torch.randn(E, D, F, device="cuda") * 0.02).to(dt)
        wu = (torch.randn(E, D, F, device="cuda") * 0.02).to(dt)
        wd = (torch.randn(E, F, D, device="cuda") * 0.02).to(dt)
        layer = MoELayer(ctx, D, F, E, K, max_tokens=T, w_gate=wg, w_up=wu, w_down=wd, fp8="fp8" in what,
                         **({"capacity_factor": 2.0} if what.endswith("_full") else {}))
        x = torch.randn(T, D, device="cuda", dtype=dt)
        logits = torch.randn(T, E, device="cuda")
        for _ in range(2):
            layer(x, logits)
    torch.cuda.synchronize()
    ctx.check()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
