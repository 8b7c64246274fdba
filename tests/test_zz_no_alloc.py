"""The decode entry point that allocates nothing, called through its exported C symbol.

Who needs it: code that must not allocate device memory when it decodes (a serving loop living
inside a fixed start-up budget, a plugin inside a host application that owns the GPU's memory).
Such a caller hands in inputs and the output buffer only; the split-K scratch is an 8 MiB array
compiled into the library. The test checks, twice in a row (the array keeps the first call's
contents), that the result equals the regular entry point's, and that a problem too large for the
array is refused with a message instead of being launched.

The file name sorts last on purpose: a run that stops at the first failure has by then run every
other test.
"""
import ctypes as C
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from iris_b200 import _lib

    lib = _lib.kernels()
    fn = lib.iris_flash_decode_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 6 + [C.c_int32] * 7 + [C.c_float, C.c_float, C.c_int32, C.c_void_p, C.c_char_p, C.c_int32]
    need = lib.iris_flash_decode_static_scratch_needed
    need.restype = C.c_uint64
    need.argtypes = [C.c_int32] * 4
    return fn, need


def _context():
    import torch.distributed as dist

    from helpers import free_port

    torch.cuda.set_device(0)
    if not dist.is_initialized():
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(free_port())
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    import iris_b200 as iris

    return iris.iris(1 << 28)


@pytest.mark.parametrize("dt,code", [(torch.bfloat16, 1), (torch.float16, 0)], ids=["bf16", "fp16"])
def test_static_scratch_decode_matches_regular_entry_point_twice(dt, code):
    from iris_b200.models import FlashDecodeLayer

    fn, need = _symbol()
    ctx = _context()
    B, Hq, Hkv, D, page, splits = 3, 32, 4, 128, 64, 6
    torch.manual_seed(11)
    lens = [900, 64, 1531]
    max_blocks = -(-max(lens) // page)
    nblocks = B * max_blocks
    kc = torch.randn(nblocks, page, Hkv, D, device="cuda", dtype=dt)
    vc = torch.randn(nblocks, page, Hkv, D, device="cuda", dtype=dt)
    table = torch.randperm(nblocks, device="cuda").to(torch.int32).view(B, max_blocks).contiguous()
    kv_lens = torch.tensor(lens, device="cuda", dtype=torch.int32)
    layer = FlashDecodeLayer(ctx, Hq, Hkv, D, max_batch=4)
    stream = torch.cuda.current_stream().cuda_stream
    err = C.create_string_buffer(512)
    assert need(B, Hq, splits, D) * 4 <= 8 << 20
    for call in range(2):                                   # second call sees the first call's leftovers
        q = torch.randn(B, Hq, D, device="cuda", dtype=dt)
        expected = layer(q, kc, vc, kv_lens.view(1, B), table)        # the existing entry point
        out = torch.full((B, Hq, D), float("nan"), device="cuda", dtype=dt)
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), kv_lens.data_ptr(), out.data_ptr(),
                B, Hq, Hkv, D, page, max_blocks, splits, 1.0 / D ** 0.5, 0.0, code, stream, err, 512)
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20)  # nothing was allocated by the call
        assert torch.isfinite(out.float()).all()
        assert (out.float() - expected.float()).abs().max().item() < 2e-2, f"call {call}"
    ctx.check()


def test_static_scratch_refuses_what_does_not_fit():
    fn, need = _symbol()
    _context()
    B, Hq, Hkv, D, splits = 64, 64, 8, 128, 64             # 64*64*64*129 floats = 135 MB > 8 MiB
    assert need(B, Hq, splits, D) * 4 > 8 << 20
    err = C.create_string_buffer(512)
    dummy = torch.zeros(16, device="cuda")
    rc = fn(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
            B, Hq, Hkv, D, 64, 4, splits, 0.1, 0.0, 1, torch.cuda.current_stream().cuda_stream, err, 512)
    assert rc == -100
    msg = err.value.decode()
    assert "scratch" in msg and "splits" in msg
    torch.cuda.synchronize()
