"""Single-GPU tests of the sm_100a kernels against plain PyTorch fp32 references.

One process, world size 1: the heap, the device context, the collectives and the fused ops all run
their real kernels (peer loops degenerate to the local rank), so every CUDA path is exercised on
one B200. Multi-rank behaviour is covered by test_gpu_multi.py.
"""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import torch.distributed as dist

    from helpers import free_port

    torch.cuda.set_device(0)
    if not dist.is_initialized():
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(free_port())
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    import iris_b200 as iris

    c = iris.iris(2 << 30)
    yield c
    c.barrier()


def _rel_err(a, ref):
    return (a.float() - ref.float()).abs().max().item() / max(ref.float().abs().max().item(), 1e-6)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kmajor", [True, False])
@pytest.mark.parametrize("shape,bn", [((128, 256, 64), 256), ((256, 512, 512), 128), ((256, 448, 512), 224),
                                      ((200, 264, 328), 0), ((1024, 3584, 1024), 0)])
def test_gemm_matches_fp32_reference(dtype, kmajor, shape, bn):
    from iris_b200.ops.gemm import matmul

    M, N, K = shape
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda", dtype=dtype)
    B = (torch.randn(N, K, device="cuda", dtype=dtype) * 0.05).t() if kmajor else torch.randn(K, N, device="cuda", dtype=dtype) * 0.05
    bias = torch.randn(N, device="cuda", dtype=dtype)
    C = matmul(A, B, bias=bias, bn=bn)
    ref = A.float() @ B.float() + bias.float()
    assert _rel_err(C, ref) < 1e-2
    rows = torch.randn(M, device="cuda", dtype=dtype)
    C2 = matmul(A, B, bias=rows, bias_dim=0, bn=bn)
    assert _rel_err(C2, A.float() @ B.float() + rows.float()[:, None]) < 1e-2


def test_context_basics(ctx):
    assert ctx.get_rank() == 0 and ctx.get_num_ranks() == 1
    assert ctx.get_cu_count() >= 100
    bases = ctx.get_heap_bases()
    assert bases.dtype == torch.int64 and bases.numel() == 1 and int(bases[0]) == ctx.heap.base
    dc = ctx.get_device_context()
    assert dc.dtype == torch.int64 and dc.numel() == 2 + 1 + 17
    assert int(dc[0]) == 0 and int(dc[1]) == 1 and int(dc[2]) == ctx.heap.base
    t = ctx.zeros(3, 5, dtype=torch.float16)
    assert ctx.is_symmetric(t) and t.shape == (3, 5) and torch.all(t == 0)
    assert not ctx.is_symmetric(torch.zeros(4, device="cuda"))
    s = ctx.as_symmetric(torch.arange(10, device="cuda"))
    assert ctx.is_symmetric(s) and torch.equal(s, torch.arange(10, device="cuda"))
    assert t.data_ptr() % 1024 == 0


def test_heap_out_of_memory(ctx):
    with pytest.raises(MemoryError):
        ctx.empty(1 << 40, dtype=torch.uint8)


def test_device_barrier_and_graph_capture(ctx):
    for _ in range(3):
        ctx.device_barrier()
    torch.cuda.synchronize()
    # the barrier keeps its round counter on the device, so a captured launch can be replayed
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        ctx.device_barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            ctx.device_barrier()
        for _ in range(3):
            g.replay()
    torch.cuda.synchronize()
    ctx.check()


def test_wait_flag_times_out_without_hanging(ctx):
    flag = ctx.zeros(1, dtype=torch.int32)
    assert ctx.wait_flag(flag, 1, timeout_ms=50) is False      # nothing sets the flag: bounded wait gives up
    flag.fill_(3)
    assert ctx.wait_flag(flag, 2, timeout_ms=50) is True
    x = torch.ones(8, device="cuda") * 2                         # the context is still usable
    assert float(x.sum()) == 16.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.int32, torch.bfloat16, torch.int64, torch.int8])
def test_rma_data_movement(ctx, dtype):
    n = 1000
    src = ctx.zeros(n, dtype=dtype)
    src.copy_(torch.arange(n, device="cuda").to(dtype))
    dst = ctx.zeros(n, dtype=dtype)
    for cm in (None, ".ca", ".cg", ".cv", ".cs"):
        got = ctx.rma.load(src, from_rank=0, cache_modifier=cm)
        assert torch.equal(got, src)
    assert torch.equal(ctx.rma.load(src, from_rank=0, volatile=True), src)
    assert torch.equal(ctx.rma.load(src, from_rank=0, oo=True), src)
    for cm in (None, ".wb", ".cg", ".cs", ".wt"):
        dst.zero_()
        ctx.rma.store(dst, src, to_rank=0, cache_modifier=cm)
        assert torch.equal(dst, src)
    dst.zero_()
    ctx.rma.put(src, dst, to_rank=0)
    assert torch.equal(dst, src)
    dst.zero_()
    ctx.rma.get(src, dst, from_rank=0, oo=True)
    assert torch.equal(dst, src)
    dst.zero_()
    ctx.rma.copy(src, dst, from_rank=0, to_rank=0)
    assert torch.equal(dst, src)
    if dtype != torch.int8:
        ctx.rma.store(dst, 7, to_rank=0)
        assert torch.all(dst == 7)


@pytest.mark.parametrize("sem", ["relaxed", "acquire", "release", "acq_rel"])
@pytest.mark.parametrize("scope", ["cta", "gpu", "sys"])
def test_rma_atomics(ctx, sem, scope):
    t = ctx.full((257,), 5, dtype=torch.int32)
    old = ctx.rma.atomic_add(t, 3, to_rank=0, sem=sem, scope=scope)
    assert torch.all(old == 5) and torch.all(t == 8)
    ctx.rma.atomic_sub(t, 1, to_rank=0, sem=sem, scope=scope)
    assert torch.all(t == 7)
    ctx.rma.atomic_max(t, 9, to_rank=0, sem=sem, scope=scope)
    ctx.rma.atomic_min(t, 8, to_rank=0, sem=sem, scope=scope)
    assert torch.all(t == 8)
    old = ctx.rma.atomic_cas(t, 8, 1, to_rank=0, sem=sem, scope=scope)
    assert torch.all(old == 8) and torch.all(t == 1)
    old = ctx.rma.atomic_cas(t, 5, 2, to_rank=0, sem=sem, scope=scope)
    assert torch.all(old == 1) and torch.all(t == 1)
    old = ctx.rma.atomic_xchg(t, 6, to_rank=0, sem=sem, scope=scope)
    assert torch.all(old == 1) and torch.all(t == 6)
    f = ctx.full((64,), 1.5, dtype=torch.float32)
    ctx.rma.atomic_add(f, 2.25, to_rank=0, sem=sem, scope=scope)
    assert torch.all(f == 3.75)
    h = ctx.full((64,), 1.5, dtype=torch.bfloat16)
    ctx.rma.atomic_add(h, 0.5, to_rank=0, scope="sys" if scope == "sys" else "gpu")
    assert torch.all(h == 2.0)


def test_tracing_records_events(ctx, tmp_path):
    ctx.tracing.enable(max_events=4096)
    try:
        assert int(ctx.get_device_context()[3]) == 1
        t = ctx.zeros(100, dtype=torch.float32)
        ctx.rma.store(t, 1.0, to_rank=0)
        ctx.rma.load(t, from_rank=0)
        torch.cuda.synchronize()
        assert ctx.tracing.num_events() == 200
        ctx.tracing.export(str(tmp_path / "trace.json"), merge=True)
        import json

        doc = json.load(open(tmp_path / "trace.json"))
        names = {e["name"] for e in doc["traceEvents"]}
        assert names == {"store", "load"}
        assert all(e["ph"] in ("X", "i") for e in doc["traceEvents"])
        assert min(e["ts"] for e in doc["traceEvents"]) == 0
    finally:
        ctx.tracing.enabled = False
        ctx._build_device_context()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_collectives_world1(ctx, dtype):
    from iris_b200.ccl import Config

    M, N = 96, 200
    inp = ctx.empty((M, N), dtype=dtype)
    inp.copy_(torch.rand(M, N, device="cuda") * 2 - 1)
    out = ctx.zeros((M, N), dtype=dtype)
    for v in ("one_shot", "two_shot", "atomic", "ring", "spinlock", "auto", "push"):
        out.zero_()
        ctx.ccl.all_reduce(out, inp, config=Config(all_reduce_variant=v))
        assert torch.equal(out, inp), v
    out.zero_()
    ctx.ccl.all_gather(out, inp)
    assert torch.equal(out, inp)
    out.zero_()
    ctx.ccl.all_to_all(out, inp)
    assert torch.equal(out, inp)
    out.zero_()
    ctx.ccl.reduce_scatter(out, inp)
    assert torch.equal(out, inp)
    ctx.check()


def test_fused_ops_world1(ctx):
    dt = torch.bfloat16
    torch.manual_seed(1)
    A = torch.randn(384, 512, device="cuda", dtype=dt)
    B = torch.randn(512, 640, device="cuda", dtype=dt) * 0.05
    ref = A.float() @ B.float()
    for op, kw in (("all_gather_matmul", {"shard_dim": 0}), ("all_gather_matmul", {"shard_dim": 1}), ("matmul_all_gather", {}),
                   ("matmul_all_reduce", {}), ("matmul_reduce_scatter", {"scatter_rows": True}), ("matmul_reduce_scatter", {})):
        C = ctx.zeros((384, 640), dtype=dt)
        ws = None
        for _ in range(3):                       # repeated calls reuse the double-buffered workspace
            ws = getattr(ctx.ops, op)(C, A, B, workspace=ws, **kw)
        assert ws.variant == "fused", op
        assert _rel_err(C, ref) < 1e-2, op
    ctx.check()


@pytest.mark.parametrize("batch,lens,page", [(1, [700], 16), (3, [1, 300, 1025], 64), (2, [4096, 77], 128)])
@pytest.mark.parametrize("heads", [(16, 2), (64, 8), (8, 8)])
def test_flash_decode_matches_reference(ctx, batch, lens, page, heads):
    from iris_b200.models import FlashDecodeLayer, reference_decode

    Hq, Hkv = heads
    dt = torch.bfloat16
    torch.manual_seed(3)
    max_blocks = -(-max(lens) // page)
    nblocks = batch * max_blocks + 3
    kc = torch.randn(nblocks, page, Hkv, 128, device="cuda", dtype=dt)
    vc = torch.randn(nblocks, page, Hkv, 128, device="cuda", dtype=dt)
    perm = torch.randperm(nblocks, device="cuda")[: batch * max_blocks].to(torch.int32).view(batch, max_blocks)
    q = torch.randn(batch, Hq, 128, device="cuda", dtype=dt)
    kv_lens = torch.tensor([lens], device="cuda", dtype=torch.int32)
    layer = FlashDecodeLayer(ctx, Hq, Hkv, 128, max_batch=4)
    for _ in range(2):
        out, lse = layer(q, kc, vc, kv_lens, perm, return_lse=True)
    ro, rlse = reference_decode(q, kc, vc, kv_lens[0], perm)
    assert (out.float() - ro).abs().max().item() < 2e-2
    assert (lse - rlse).abs().max().item() < 2e-2
    ctx.check()


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 1024), (200, 520, 336), (1024, 1024, 7168)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_fp8_block_scaled_gemm_matches_dequantised_product(M, N, K, out_dtype):
    """1 x 128 activation scales, 128 x 128 weight scales, e4m3 operands: the kernel's result against
    the fp32 product of the dequantised operands (what the scales mean)."""
    from iris_b200.ops.gemm_fp8 import dequant_matmul, matmul_fp8, quantize_1x128, quantize_128x128

    torch.manual_seed(11)
    x = torch.randn(M, K, device="cuda") * (1 + 3 * torch.rand(M, 1, device="cuda"))     # rows of different magnitude
    w = torch.randn(N, K, device="cuda") * 0.05
    aq, asc = quantize_1x128(x)
    bq, bsc = quantize_128x128(w)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = matmul_fp8(aq, asc, bq, bsc, out_dtype=out_dtype, status=status)
    ref = dequant_matmul(aq, asc, bq, bsc)
    assert int(status.item()) == 0
    assert (out.float() - ref).abs().max().item() / ref.abs().max().item() < 1e-2
    # and the quantised product stays close to the unquantised one
    assert (out.float() - x @ w.t()).abs().max().item() / ref.abs().max().item() < 8e-2


def _distinct_scale_operands(M, N, K):
    """Operands whose every quantisation block gets a different scale: row magnitudes, K-block
    magnitudes and 128 x 128 weight-block magnitudes all differ by powers of two and more."""
    kb, nb = -(-K // 128), -(-N // 128)
    x = torch.randn(M, K, device="cuda")
    x = x * torch.exp2(torch.randint(-6, 6, (M, 1), device="cuda").float()) * (1 + torch.rand(M, 1, device="cuda"))
    x = x * torch.exp2(torch.randint(-3, 3, (1, kb), device="cuda").float()).repeat_interleave(128, 1)[:, :K]
    w = torch.randn(N, K, device="cuda") * 0.05
    w = w * torch.exp2(torch.randint(-4, 4, (nb, kb), device="cuda").float()).repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    return x, w


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (200, 520, 336)])
def test_fp8_scale_layout_with_distinct_scales_per_block(M, N, K):
    """Pins the 1 x 128 / 128 x 128 scale layout of the software-promotion kernel: every block has its own
    scale, so a scale applied to the wrong row, column block or K block shows up as a large error."""
    from iris_b200.ops.gemm_fp8 import dequant_matmul, matmul_fp8, quantize_1x128, quantize_128x128

    torch.manual_seed(5)
    x, w = _distinct_scale_operands(M, N, K)
    aq, asc = quantize_1x128(x)
    bq, bsc = quantize_128x128(w)
    assert asc.unique().numel() > M // 2 and bsc.unique().numel() >= min(bsc.numel(), 3)
    out = matmul_fp8(aq, asc, bq, bsc)
    ref = dequant_matmul(aq, asc, bq, bsc)
    # row by row: rows differ by up to 2^12 in magnitude, a global maximum would hide the small ones
    err = (out.float() - ref).abs().amax(dim=1) / ref.abs().amax(dim=1).clamp_min(1e-20)
    assert err.max().item() < 1.5e-2


@pytest.mark.parametrize("M,N,K,bn,two_sm", [(128, 224, 128, 0, None), (256, 448, 1024, 0, None), (200, 520, 336, 0, None),
                                             (256, 256, 512, 128, None), (512, 896, 2048, 0, True), (1024, 1024, 7168, 0, None)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_fp8_hardware_block_scaled_gemm(M, N, K, bn, two_sm, out_dtype):
    """tcgen05.mma.kind::mxf8f6f4.block_scale with UE8M0 scales staged in TMEM: power-of-two scales,
    distinct per block, against the fp32 product of the dequantised operands, row by row."""
    from iris_b200.ops.gemm_fp8 import (blockscaled_tile_n, dequant_matmul, matmul_fp8_blockscaled, pack_scales_a, pack_scales_b,
                                        quantize_1x128, quantize_128x128)

    torch.manual_seed(6)
    x, w = _distinct_scale_operands(M, N, K)
    aq, asc = quantize_1x128(x, pow2=True)
    bq, bsc = quantize_128x128(w, pow2=True)
    tile = blockscaled_tile_n(M, N, bn, two_sm)
    out = matmul_fp8_blockscaled(aq, pack_scales_a(asc), bq, pack_scales_b(bsc, N, tile), out_dtype=out_dtype, bn=bn, two_sm=two_sm)
    ref = dequant_matmul(aq, asc, bq, bsc)
    err = (out.float() - ref).abs().amax(dim=1) / ref.abs().amax(dim=1).clamp_min(1e-20)
    assert err.max().item() < 1.5e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,K", [(256, 512), (200, 328), (1, 128)])
def test_activation_quantiser_kernel(M, K, dtype):
    """One-kernel activation quantiser: power-of-two 1 x 128 scales, e4m3 values within half a step of
    x / scale, and scale atoms equal to the PyTorch packing of the scales it reports."""
    from iris_b200.ops.gemm_fp8 import pack_scales_a, quantize_activation

    torch.manual_seed(9)
    x = (torch.randn(M, K, device="cuda") * torch.exp2(torch.randint(-8, 8, (M, 1), device="cuda").float())).to(dtype)
    b = quantize_activation(x)
    s = b.scale
    assert tuple(b.q.shape) == (M, K) and tuple(s.shape) == (M, -(-K // 128))
    assert torch.all(torch.log2(s) == torch.round(torch.log2(s)))
    amax = torch.nn.functional.pad(x.float().abs(), (0, s.shape[1] * 128 - K)).view(M, -1, 128).amax(dim=2).clamp_min(1e-12)
    assert torch.all(amax / s <= 448.0) and torch.all(amax / s > 448.0 / 2 - 1e-3)       # the smallest power of two that fits
    back = b.dequantize()
    step = s.repeat_interleave(128, dim=1)[:, :K] * 32.0                                  # e4m3 spacing at the top binade (256..448)
    assert torch.all((back - x.float()).abs() <= step / 2 + 1e-30)
    assert torch.equal(b.sf(), pack_scales_a(s))
    again = quantize_activation(x, out=b)                                                 # buffers reused
    assert again is b and torch.equal(again.sf(), pack_scales_a(s))


def test_fp8_fused_ops_world1(ctx):
    """The fused ops with block-scaled e4m3 operands (one rank: same kernels, no peers)."""
    from iris_b200.ops import quantize_activation, quantize_weight

    torch.manual_seed(2)
    xs, wt = _distinct_scale_operands(384, 640, 512)
    x, w = quantize_activation(xs), quantize_weight(wt)
    ref = x.dequantize() @ w.dequantize()
    for op, kw in (("all_gather_matmul", {"shard_dim": 0}), ("all_gather_matmul", {"shard_dim": 1}), ("matmul_all_gather", {}),
                   ("matmul_all_reduce", {}), ("matmul_reduce_scatter", {"scatter_rows": True}), ("matmul_reduce_scatter", {})):
        C = ctx.zeros((384, 640), dtype=torch.bfloat16)
        ws = None
        for _ in range(3):
            ws = getattr(ctx.ops, op)(C, x, w, workspace=ws, **kw)
        assert ws.variant == "fused" and ws.bn == 224, op
        err = (C.float() - ref).abs().amax(dim=1) / ref.abs().amax(dim=1).clamp_min(1e-20)
        assert err.max().item() < 1.5e-2, op
    ctx.check()


def test_fused_op_reads_a_bias_updated_in_place(ctx):
    """A 16-bit bias is converted to fp32 for the kernel and the conversion is kept with the cached
    descriptor: an in-place update of the bias (an optimizer step) must reach the next call."""
    dt = torch.bfloat16
    torch.manual_seed(3)
    A = torch.randn(256, 256, device="cuda", dtype=dt)
    B = torch.randn(256, 256, device="cuda", dtype=dt) * 0.05
    bias = torch.randn(256, device="cuda", dtype=dt)
    C = ctx.zeros((256, 256), dtype=dt)
    ws = ctx.ops.matmul_all_reduce(C, A, B, bias=bias)
    ref = A.float() @ B.float()
    assert _rel_err(C, ref + bias.float()[:, None]) < 1e-2
    bias.add_(5.0)
    ctx.ops.matmul_all_reduce(C, A, B, bias=bias, workspace=ws)
    assert _rel_err(C, ref + bias.float()[:, None]) < 1e-2
    ctx.check()


@pytest.mark.parametrize("page,use_tma", [(64, None), (16, None), (64, False), (48, None)])
def test_flash_decode_ignores_positions_past_the_length(ctx, page, use_tma):
    """Cache rows past a sequence's length (same page or unused pages) hold NaN: both tile-fill paths
    (TMA boxes per page, cp.async for page sizes a 64-position tile does not divide into) must mask them."""
    from iris_b200.models import FlashDecodeLayer, reference_decode

    Hq, Hkv, dt = 16, 2, torch.bfloat16
    lens = [page * 3 + 5, 70, 1]
    batch = len(lens)
    torch.manual_seed(5)
    max_blocks = -(-max(lens) // page)
    nblocks = batch * max_blocks + 2
    kc = torch.randn(nblocks, page, Hkv, 128, device="cuda", dtype=dt)
    vc = torch.randn(nblocks, page, Hkv, 128, device="cuda", dtype=dt)
    table = torch.randperm(nblocks, device="cuda")[: batch * max_blocks].to(torch.int32).view(batch, max_blocks)
    used = torch.zeros(nblocks, page, dtype=torch.bool, device="cuda")
    for b, n in enumerate(lens):
        for pos in range(n):
            used[int(table[b, pos // page]), pos % page] = True
    kc[~used] = float("nan")
    vc[~used] = float("nan")
    q = torch.randn(batch, Hq, 128, device="cuda", dtype=dt)
    kv_lens = torch.tensor([lens], device="cuda", dtype=torch.int32)
    layer = FlashDecodeLayer(ctx, Hq, Hkv, 128, max_batch=4, use_tma=use_tma)
    out, lse = layer(q, kc, vc, kv_lens, table, return_lse=True)
    kz, vz = torch.nan_to_num(kc, nan=0.0), torch.nan_to_num(vc, nan=0.0)
    ro, rlse = reference_decode(q, kz, vz, kv_lens[0], table)
    assert torch.isfinite(out.float()).all()
    assert (out.float() - ro).abs().max().item() < 2e-2
    assert (lse - rlse).abs().max().item() < 2e-2
    ctx.check()


@pytest.mark.parametrize("T,E,K", [(64, 8, 2), (200, 16, 4), (128, 32, 8)])
def test_moe_layer_world1(ctx, T, E, K):
    from iris_b200.models import MoELayer, reference_moe

    D, F = 256, 128
    torch.manual_seed(4)
    dt = torch.bfloat16
    wg = (torch.randn(E, D, F, device="cuda") * 0.05).to(dt)
    wu = (torch.randn(E, D, F, device="cuda") * 0.05).to(dt)
    wd = (torch.randn(E, F, D, device="cuda") * 0.05).to(dt)
    layer = MoELayer(ctx, D, F, E, K, max_tokens=T, w_gate=wg, w_up=wu, w_down=wd)
    for it in range(2):
        x = torch.randn(T, D, device="cuda", dtype=dt)
        logits = torch.randn(T, E, device="cuda")
        out = layer(x, logits)
        ref = reference_moe(x, logits, wg, wu, wd, K)
        err = (out.float() - ref).abs().max().item()
        assert err < 3e-2 * max(ref.abs().max().item(), 1.0), (it, err)
    ctx.check()


@pytest.mark.parametrize("T,E,K,D,F", [(64, 8, 2, 256, 128), (200, 16, 4, 512, 256), (128, 4, 2, 1024, 512)])
def test_moe_layer_fp8_world1(ctx, T, E, K, D, F):
    """Block-scaled e4m3 MoE (tokens and hidden activations quantised 1 x 128, weights 128 x 128, scales applied by
    the tensor core) against the fp32 layer evaluated on the SAME quantised weights: what remains is the
    quantisation of the tokens and of the hidden activations."""
    from iris_b200.models import MoELayer, reference_moe
    from iris_b200.ops.gemm_fp8 import dequantize, quantize_128x128

    torch.manual_seed(4)
    dt = torch.bfloat16
    wg = (torch.randn(E, D, F, device="cuda") * 0.05).to(dt)
    wu = (torch.randn(E, D, F, device="cuda") * 0.05).to(dt)
    wd = (torch.randn(E, F, D, device="cuda") * 0.05).to(dt)
    layer = MoELayer(ctx, D, F, E, K, max_tokens=T, w_gate=wg, w_up=wu, w_down=wd, fp8=True)

    def deq(w):      # [E, in, out] -> the values the layer's e4m3 weights stand for
        out = []
        for e in range(E):
            q, s = quantize_128x128(w[e].t().contiguous().float(), pow2=True)       # stored [out, in]
            out.append(dequantize(q, s, 128).t())
        return torch.stack(out)

    wgd, wud, wdd = deq(wg), deq(wu), deq(wd)
    for it in range(2):
        x = torch.randn(T, D, device="cuda", dtype=dt)
        logits = torch.randn(T, E, device="cuda")
        out = layer(x, logits)
        ref = reference_moe(x, logits, wgd, wud, wdd, K)
        err = (out.float() - ref).abs().max().item()
        assert err < 6e-2 * max(ref.abs().max().item(), 1.0), (it, err)
    ctx.check()


def test_router_matches_torch_topk(ctx):
    from iris_b200.models import MoELayer, route

    T, E, K, D, F = 96, 64, 8, 256, 128
    dt = torch.bfloat16
    z = lambda *s: torch.zeros(*s, device="cuda", dtype=dt)  # noqa: E731
    layer = MoELayer(ctx, D, F, E, K, max_tokens=T, w_gate=z(E, D, F), w_up=z(E, D, F), w_down=z(E, F, D))
    torch.manual_seed(9)
    logits = torch.randn(T, E, device="cuda")
    layer(torch.zeros(T, D, device="cuda", dtype=dt), logits)
    torch.cuda.synchronize()
    idx, w = route(logits, K)
    assert torch.equal(layer.topk_idx.long(), idx)
    assert torch.allclose(layer.topk_w, w, atol=1e-5)


@pytest.mark.parametrize("S,Hq,Hkv,causal,tc", [(128, 4, 2, False, None), (200, 8, 2, True, None), (64, 2, 2, True, None),
                                                 (128, 2, 2, True, None), (384, 8, 2, True, None), (512, 4, 4, False, None),
                                                 (384, 8, 2, True, False)])
def test_ring_attention_world1(ctx, S, Hq, Hkv, causal, tc):
    """Multiples of 128 run the tcgen05 attention CTAs, other lengths (or tc=False) the mma.sync ones."""
    from iris_b200.models import RingAttention, reference_attention

    dt = torch.bfloat16
    torch.manual_seed(6)
    q = torch.randn(S, Hq, 128, device="cuda", dtype=dt)
    k = torch.randn(S, Hkv, 128, device="cuda", dtype=dt)
    v = torch.randn(S, Hkv, 128, device="cuda", dtype=dt)
    layer = RingAttention(ctx, S, Hq, Hkv, use_tcgen05=tc)
    for _ in range(2):
        out, lse = layer(q, k, v, causal=causal, return_lse=True)
    ref = reference_attention(q, k, v, causal)
    assert (out.float() - ref).abs().max().item() < 2e-2
    g = Hq // Hkv
    s = torch.einsum("qhd,khd->hqk", q.float(), k.float().repeat_interleave(g, dim=1)) / 128 ** 0.5
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device="cuda"), 1)[None], float("-inf"))
    assert (lse - torch.logsumexp(s, dim=-1).t()).abs().max().item() < 2e-2
    ctx.check()


def test_ring_attention_zigzag_world1(ctx):
    """With one rank the zigzag block [chunk 0 | chunk 1] is the plain sequence: the zigzag tile walk
    must reproduce ordinary causal attention."""
    from iris_b200.models import RingAttention, reference_attention

    S, Hq, Hkv, dt = 512, 4, 2, torch.bfloat16
    torch.manual_seed(8)
    q = torch.randn(S, Hq, 128, device="cuda", dtype=dt)
    k = torch.randn(S, Hkv, 128, device="cuda", dtype=dt)
    v = torch.randn(S, Hkv, 128, device="cuda", dtype=dt)
    layer = RingAttention(ctx, S, Hq, Hkv, layout="zigzag")
    for causal in (True, False):
        out = layer(q, k, v, causal=causal)
        assert (out.float() - reference_attention(q, k, v, causal)).abs().max().item() < 2e-2
    with pytest.raises(ValueError):
        RingAttention(ctx, 384, Hq, Hkv, layout="zigzag")
    ctx.check()


@pytest.fixture(scope="module")
def user_module():
    from iris_b200 import jit

    here = os.path.dirname(os.path.abspath(__file__))
    return jit.compile_file(os.path.join(here, "kernels", "user_kernels.cu"))


def test_user_kernels_functional_and_oo_api(ctx, user_module):
    buf = ctx.zeros(4096, dtype=torch.float32)
    user_module.fn("store_blocks")(ctx, buf, 3000, 2.5, 0)
    torch.cuda.synchronize()
    assert torch.all(buf[:3000] == 2.5) and torch.all(buf[3000:] == 0)      # mask: lanes past n do nothing
    src = ctx.arange(0, 512, dtype=torch.int32)
    out = torch.zeros(512, dtype=torch.int32, device="cuda")
    user_module.fn("masked_load")(ctx.get_device_context(), src, out, 512, 300, 0)   # context built from the int64 tensor
    torch.cuda.synchronize()
    assert torch.equal(out[:300], src[:300]) and torch.all(out[300:] == -7)  # `other` for masked lanes
    counter = ctx.zeros(1, dtype=torch.int32)
    user_module.fn("count")(ctx, counter, 256, 0)
    torch.cuda.synchronize()
    assert int(counter.item()) == 256


@pytest.mark.parametrize("op", [0, 1, 2, 3, 4, 5, 6, 7, 8])
def test_tile_collectives_world1(ctx, user_module, op):
    M, N, bm, bn = 100, 72, 32, 16
    torch.manual_seed(op)
    src = ctx.zeros((M, N), dtype=torch.float32)
    src.copy_(torch.randn(M, N, device="cuda"))
    dst = ctx.zeros((M, N), dtype=torch.float32)
    tiles = -(-M // bm) * -(-N // bn)
    locks = ctx.zeros(tiles, dtype=torch.int32)
    arg = N if op == 6 else 0
    user_module.fn("tile_collective")(ctx, op, src, dst, locks, M, N, M, N, bm, bn, arg, 1)
    torch.cuda.synchronize()
    assert torch.equal(dst, src), op          # with one rank every collective is the identity
    ctx.check()


def test_tensor_parallel_mlp_forward_backward_world1(ctx):
    from iris_b200.models import TensorParallelMLP

    dt = torch.bfloat16
    torch.manual_seed(12)
    M, K, F = 256, 512, 384
    X = torch.randn(M, K, device="cuda")
    W1 = torch.randn(K, F, device="cuda") * 0.1
    W2 = torch.randn(F, K, device="cuda") * 0.1
    G = torch.randn(M, K, device="cuda")
    mlp = TensorParallelMLP(ctx, K, F, activation="silu", dtype=dt, w1=W1.to(dt), w2=W2.to(dt))
    x = X.to(dt).requires_grad_(True)
    y = mlp(x)
    y.backward(G.to(dt))
    assert mlp._ws["ag1"].variant == "fused" and mlp._ws["rs2"].variant == "fused"
    Xr, W1r, W2r = X.to(dt).float().requires_grad_(True), W1.to(dt).float().requires_grad_(True), W2.to(dt).float().requires_grad_(True)
    Yr = torch.nn.functional.silu(Xr @ W1r) @ W2r
    Yr.backward(G.to(dt).float())
    for a, b in ((y.detach(), Yr.detach()), (x.grad, Xr.grad), (mlp.w1.grad, W1r.grad), (mlp.w2.grad, W2r.grad)):
        assert (a.float() - b).abs().max().item() / b.abs().max().item() < 3e-2
    ctx.check()
