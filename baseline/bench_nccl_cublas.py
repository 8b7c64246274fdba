#!/usr/bin/env python3
"""The step of `bench.py` done the unfused way: NCCL all-gather, two cuBLAS GEMMs, NCCL
reduce-scatter (what a stock PyTorch tensor-parallel MLP runs). Same shapes, same timing rules
(W warm-up steps, K timed steps between barriers, CUDA events, maximum over ranks), same JSON keys.

    python baseline/bench_nccl_cublas.py --steps 100 --warmup 10                     (1 GPU)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 baseline/bench_nccl_cublas.py --gpus N --steps 100 --warmup 10
"""
import argparse
import json
import os
import sys

M_TOTAL, K_DIM, F_LOCAL = 8192, 8192, 3584


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    args = ap.parse_args()
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    import torch
    import torch.distributed as dist

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    dev, dt = torch.device("cuda", local), torch.bfloat16
    M_local = M_TOTAL // world
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    W1 = (torch.randn(F_LOCAL, K_DIM, device=dev, generator=g) * 0.02).to(dt).t()
    W2 = (torch.randn(K_DIM, F_LOCAL, device=dev, generator=g) * 0.02).to(dt).t()
    X = torch.randn(M_local, K_DIM, device=dev, generator=g).to(dt)
    Xall = torch.empty(M_TOTAL, K_DIM, device=dev, dtype=dt)
    H = torch.empty(M_TOTAL, F_LOCAL, device=dev, dtype=dt)
    P = torch.empty(M_TOTAL, K_DIM, device=dev, dtype=dt)
    Y = torch.empty(M_local, K_DIM, device=dev, dtype=dt)

    def step():
        if world > 1:
            dist.all_gather_into_tensor(Xall, X)
            torch.matmul(Xall, W1, out=H)
            torch.matmul(H, W2, out=P)
            dist.reduce_scatter_tensor(Y, P)
        else:
            torch.matmul(X, W1, out=H)
            torch.matmul(H, W2, out=Y)

    for _ in range(max(args.warmup, 3)):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.steps):
        step()
    e.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([s.elapsed_time(e) / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    flops = 2.0 * M_TOTAL * K_DIM * F_LOCAL * 2 * world
    if rank == 0:
        print(json.dumps({"metric": "NCCL all-gather + cuBLAS GEMMs + NCCL reduce-scatter TFLOPS (aggregate, device time, max over ranks)",
                          "value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
                          "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "dtype": "bf16", "impl": "nccl+cublas"}))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
