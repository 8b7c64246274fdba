#!/usr/bin/env python3
"""Point-to-point and one-to-all bandwidth of the heap primitives (reference: examples/00_load,
01_store, 02_all_load, 03_all_store, 04_atomic_add, 05_atomic_xchg).

Run with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmark/p2p_bandwidth.py --size-mb 256 --json out.json

Rank 0 measures (the other ranks only provide their heaps and idle at a barrier), with CUDA events,
after warm-up: local copy / read / write, remote load (pull), remote store (push), NVLS multimem
store, remote atomics and the TMA bulk path, each for several CTA counts.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import iris_b200 as iris  # noqa: E402
from iris_b200 import _lib  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size-mb", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    nbytes = args.size_mb << 20
    ctx = iris.iris(3 * nbytes + (64 << 20))
    lib = _lib.kernels()
    lib.iris_microbench.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_ulonglong, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_void_p, C.c_void_p]
    lib.iris_microbench.restype = C.c_int
    a = ctx.zeros(nbytes, dtype=torch.uint8)
    b = ctx.zeros(nbytes, dtype=torch.uint8)
    a.fill_(1)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ctx.barrier()
    peer = (rank + 1) % world
    peer_a = ctx.heap.peer_view(a, peer).data_ptr()
    peer_b = ctx.heap.peer_view(b, peer).data_ptr()
    mc_b = ctx.heap.mc_base + ctx.heap.offset_of(b) if ctx.has_multicast() else 0
    results = []

    def timeit(mode, dst, src, ctas, unroll=8, piece=0, nbuf=0, size=nbytes):
        def launch():
            rc = lib.iris_microbench(mode, dst, src, size, ctas, unroll, piece, nbuf, status.data_ptr(), _lib.current_stream_ptr())
            assert rc == 0, rc
        for _ in range(3):
            launch()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.iters):
            launch()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / args.iters

    def report(name, ms, ctas, size=nbytes, **extra):
        gbs = size / ms / 1e6
        row = {"test": name, "ctas": ctas, "ms": round(ms, 4), "GBps": round(gbs, 1), **extra}
        results.append(row)
        print(f"{name:<34} ctas={ctas:<4} {ms * 1e3:9.1f} us  {gbs:8.1f} GB/s  {extra if extra else ''}", flush=True)

    if rank == 0:
        for ctas in (148, 296):
            report("local copy (read+write counted once)", timeit(0, b.data_ptr(), a.data_ptr(), ctas), ctas)
        report("local read", timeit(1, None, a.data_ptr(), 296), 296)
        report("local write", timeit(2, b.data_ptr(), None, 296), 296)
        if world > 1:
            for ctas in (4, 8, 16, 32, 64, 148):
                for unroll in (1, 8):
                    report("remote store (push, st.v4)", timeit(0, peer_b, a.data_ptr(), ctas, unroll), ctas, unroll=unroll)
            for ctas in (4, 8, 16, 32, 64, 148):
                for unroll in (1, 8):
                    report("remote load (pull, ld.v4)", timeit(0, b.data_ptr(), peer_a, ctas, unroll), ctas, unroll=unroll)
            for ctas in (1, 2, 4, 8, 16, 32):
                for piece, nbuf in ((16384, 8), (32768, 6), (65536, 3)):
                    report("remote store (TMA bulk)", timeit(6, peer_b, a.data_ptr(), ctas, 0, piece, nbuf), ctas, piece=piece, nbuf=nbuf)
            for ctas in (4, 16):
                report("local copy (TMA bulk)", timeit(6, b.data_ptr(), a.data_ptr(), ctas, 0, 32768, 6), ctas)
                report("remote load (TMA bulk)", timeit(6, b.data_ptr(), peer_a, ctas, 0, 32768, 6), ctas)
            if mc_b:
                for ctas in (4, 8, 16, 32, 64, 148):
                    report("NVLS multimem.st (to all ranks)", timeit(3, mc_b, a.data_ptr(), ctas, 8), ctas)
            small = 64 << 20
            for ctas in (16, 148):
                report("remote atomic add (4 B words)", timeit(4, peer_b, None, ctas, size=small), ctas, size=small)
                report("remote atomic xchg (4 B words)", timeit(5, peer_b, None, ctas, size=small), ctas, size=small)
            report("local atomic add (4 B words)", timeit(4, b.data_ptr(), None, 148, size=small), 148, size=small)
        if args.json:
            with open(args.json, "w") as f:
                json.dump({"world": world, "size_mb": args.size_mb, "multicast": bool(mc_b), "results": results}, f, indent=1)
    ctx.barrier()
    del ctx
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
