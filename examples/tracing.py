#!/usr/bin/env python3
"""Device event tracing to a Perfetto / chrome://tracing file (reference:
examples/23_gemm_all_scatter_tracing, examples/32_gluon_all_gather_tracing).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/tracing.py
"""
import os
import tempfile

import torch

from _common import finish, init

if __name__ == "__main__":
    ctx = init()
    ctx.tracing.enable(max_events=100_000)
    buf = ctx.zeros(8192, dtype=torch.float32)
    ctx.barrier()
    peer = (ctx.get_rank() + 1) % ctx.get_num_ranks()
    ctx.rma.store(buf, 2.0, to_rank=peer)        # every element records a "store" event with its target rank
    ctx.rma.atomic_add(buf, 1.0, to_rank=peer)
    ctx.barrier()
    out_dir = os.environ.get("IRIS_TRACE_DIR") or tempfile.gettempdir()
    path = os.path.join(out_dir, "trace.json")
    ctx.tracing.export(path, merge=True)          # trace_rank<r>.json per rank + merged trace.json on rank 0
    ctx.info(f"{ctx.tracing.num_events()} events recorded, written next to {path}")
    finish(ctx)
