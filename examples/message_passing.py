#!/usr/bin/env python3
"""Producer / consumer message passing with put + flag (reference: examples/06_message_passing,
examples/31_message_passing). Rank 0 puts blocks into rank 1's buffer and raises one flag per block
(release, system scope); rank 1 waits for each flag (acquire, bounded) and reads the block.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/message_passing.py
"""
import ctypes as C

import torch

from _common import finish, init

if __name__ == "__main__":
    ctx = init()
    from iris_b200 import _lib

    lib = _lib.kernels()
    n, block = 1 << 20, 4096
    buf = ctx.zeros(n, dtype=torch.float32)
    flags = ctx.zeros(n // block, dtype=torch.int32)
    ctx.barrier()
    stream = C.c_void_p(_lib.current_stream_ptr())
    c = ctx.ctx_struct()
    if ctx.get_num_ranks() >= 2:
        if ctx.get_rank() == 0:
            src = torch.arange(n, device="cuda", dtype=torch.float32)
            lib.iris_msg_producer(C.byref(c), C.c_void_p(src.data_ptr()), C.c_void_p(buf.data_ptr()), C.c_void_p(flags.data_ptr()),
                                  C.c_ulonglong(n), block, 1, stream)
        elif ctx.get_rank() == 1:
            out = torch.zeros(n, device="cuda", dtype=torch.float32)
            lib.iris_msg_consumer(C.byref(c), C.c_void_p(buf.data_ptr()), C.c_void_p(out.data_ptr()), C.c_void_p(flags.data_ptr()),
                                  C.c_ulonglong(n), block, stream)
            torch.cuda.synchronize()
            assert torch.equal(out, torch.arange(n, device="cuda", dtype=torch.float32))
            ctx.info("consumer received every block")
    ctx.check()
    finish(ctx)
