"""Host-layer tests that need no GPU: tensor factories, configs, bench harness parsing, logging,
collectives / fused ops / flash decode on the CPU backend (gloo ranks sharing memfd heaps)."""
import logging
import math

import pytest
import torch

from helpers import run_ranks


# ------------------------------------------------------------------ pure python
def test_ccl_config_validation():
    from iris_b200.ccl import Config, ReduceOp

    c = Config()
    assert (c.block_size_m, c.block_size_n, c.comm_sms, c.swizzle_size) == (32, 64, 64, 4)
    assert ReduceOp.SUM == 0
    for bad in (dict(block_size_m=0), dict(comm_sms=-1), dict(all_reduce_variant="nope"), dict(all_gather_variant="x"),
                dict(all_reduce_distribution=2), dict(threads_per_warp=48), dict(swizzle_size=0)):
        with pytest.raises(ValueError):
            Config(**bad)
    # AMD-only knobs are accepted
    Config(num_xcds=8, waves_per_eu=2, threads_per_warp=64, num_warps=8)


def test_fused_config():
    from iris_b200.ops import FusedConfig

    c = FusedConfig()
    assert c.tile_n() == 0 and FusedConfig(block_size_n=224).tile_n() == 224
    with pytest.raises(ValueError):
        FusedConfig(all_reduce_variant="bogus")
    c.validate(8)
    with pytest.raises(ValueError):
        c.validate(0)


def test_bench_axis_parsing_and_registry():
    from iris_b200.bench import State, axis, linear_range, power_of_two, register, registry
    from iris_b200.bench._core import SkipCombination, combinations
    from iris_b200.bench._runner import format_console, format_csv, format_json, parse_axis_values
    from iris_b200.bench import Result

    assert power_of_two(2, 4) == [4, 8, 16] and linear_range(0, 6, 3) == [0, 3, 6]
    assert parse_axis_values("pow2:10:12") == [1024, 2048, 4096]
    assert parse_axis_values("lin:0:64:32") == [0, 32, 64]
    assert parse_axis_values("bf16,fp32") == [torch.bfloat16, torch.float32]
    assert parse_axis_values("1, 2,x") == [1, 2, "x"]
    before = len(registry)

    @register
    @axis("M", [1, 2])
    @axis("N", [3])
    def demo(state, ctx):
        state.set_bytes(10)

    assert len(registry) == before + 1 and [a.name for a in registry[-1].axes] == ["M", "N"]
    combos = list(combinations(registry[-1].axes, {"M": [7, 8, 9]}, {"M": [8]}))
    assert combos == [{"M": 7, "N": 3}, {"M": 9, "N": 3}]
    registry.pop()
    s = State({"M": 4})
    assert s["M"] == 4 and s.get("Q", 1) == 1
    with pytest.raises(SkipCombination):
        s.skip("why")
    r = [Result("b", {"M": 4, "dtype": torch.float16}, 0.5, [], bandwidth_gbps=3.0, tflops=None, roofline_frac=0.5)]
    assert "b" in format_console(r) and "float16" in format_json(r) and "gpu_time_ms" in format_csv(r)


def test_logging_format(capsys):
    import iris_b200 as iris
    from iris_b200.host.logging import IrisFormatter, log_rank, logger

    rec = logging.LogRecord("iris", logging.INFO, "f.py", 1, "hello", None, None)
    rec.iris_rank, rec.iris_num_ranks, rec.iris_module = 1, 4, "mod"
    out = IrisFormatter().format(rec)
    assert "[Iris]" in out and "[1/4]" in out and "[mod]" in out and out.endswith("hello")
    iris.set_logger_level(iris.DEBUG)
    assert logger.level == logging.DEBUG
    iris.set_logger_level(iris.WARNING)
    log_rank(iris.WARNING, "w", 0, 2)


def test_device_symbols_point_to_headers():
    import os

    import iris_b200 as iris

    root = os.path.dirname(os.path.dirname(os.path.abspath(iris.__file__)))
    for sym in (iris.load, iris.store, iris.atomic_cas, iris.DeviceContext, iris.TensorView):
        assert os.path.exists(os.path.join(root, sym.header))
        src = open(os.path.join(root, sym.header)).read()
        assert sym.name in src
    with pytest.raises(RuntimeError):
        iris.load()
    # every symbol of the device namespace names something that exists in its header
    from iris_b200 import device, gluon, mem

    syms = [v for v in vars(device).values() if isinstance(v, device.DeviceSymbol)]
    assert len(syms) >= 26
    for sym in syms:
        assert sym.name in open(os.path.join(root, sym.header)).read(), sym
    # the reference's module paths for the same API
    assert gluon.IrisDeviceCtx is iris.Context and gluon.GluonDeviceTracing is device.Tracing
    assert iris.experimental.gluon_context is gluon and mem.atomic_add is iris.atomic_add and mem.get_cu_id.cuda == "iris::get_cu_id"


def test_owned_tiles_partition():
    from iris_b200.ccl import owned_tiles
    from iris_b200.ops import owned_tile_range

    for dist_mode in (0, 1):
        seen = set()
        for r in range(3):
            for t in owned_tiles(100, 130, 32, 64, 3, r, dist_mode):
                assert t not in seen
                seen.add(t)
        assert len(seen) == 4 * 3
    for total, W in ((10, 4), (3, 8), (16, 8)):
        got = [t for r in range(W) for t in owned_tile_range(total, W, r)]
        assert sorted(got) == list(range(total))


# ------------------------------------------------------------------ CPU backend, world 2 / 3
def _factories(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 26)
    z = ctx.zeros(2, 3, dtype=torch.float32)
    assert z.shape == (2, 3) and torch.all(z == 0) and ctx.is_symmetric(z)
    assert ctx.zeros((4, 5)).shape == (4, 5) and ctx.zeros([2, 2]).shape == (2, 2)
    o = ctx.ones(7, dtype=torch.int32)
    assert torch.all(o == 1) and o.dtype == torch.int32
    f = ctx.full((2, 2), 3.5)
    assert torch.all(f == 3.5) and f.dtype == torch.get_default_dtype()
    assert ctx.full((2,), 3).dtype == torch.int64
    e = ctx.empty(5, 5, dtype=torch.bfloat16)
    assert e.shape == (5, 5) and e.dtype == torch.bfloat16
    zl = ctx.zeros_like(torch.ones(3, 4, dtype=torch.float16))
    assert zl.shape == (3, 4) and zl.dtype == torch.float16 and ctx.is_symmetric(zl)
    r = ctx.rand(100)
    assert 0 <= float(r.min()) and float(r.max()) <= 1
    assert ctx.randn(10, 10).shape == (10, 10)
    ri = ctx.randint(0, 5, (50,))
    assert ri.dtype == torch.int64 and int(ri.min()) >= 0 and int(ri.max()) < 5
    assert ctx.randint(7, (4,)).shape == (4,)
    u = ctx.uniform((20,), -2.0, -1.0)
    assert float(u.max()) <= -1.0 and float(u.min()) >= -2.0
    assert torch.equal(ctx.arange(5), torch.arange(5))
    assert torch.equal(ctx.arange(1, 10, 3), torch.arange(1, 10, 3))
    assert torch.allclose(ctx.arange(0.0, 1.0, 0.25), torch.arange(0.0, 1.0, 0.25))
    assert torch.allclose(ctx.linspace(0, 1, 5), torch.linspace(0, 1, 5))
    # out= must be a heap tensor of the right size and dtype
    out = ctx.empty(6, dtype=torch.float32)
    got = ctx.zeros(2, 3, out=out)
    assert got.data_ptr() == out.data_ptr() and got.shape == (2, 3)
    with pytest.raises(RuntimeError):
        ctx.zeros(2, 3, out=torch.empty(6))
    with pytest.raises(RuntimeError):
        ctx.zeros(2, 2, out=out)
    with pytest.raises(RuntimeError):
        ctx.zeros(2, 3, out=out, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        ctx.zeros(2, device="cuda:0")
    with pytest.raises(ValueError):
        ctx.zeros(2, layout=torch.sparse_coo)
    cl = ctx.zeros(2, 3, 4, 5, memory_format=torch.channels_last)
    assert cl.stride() == torch.zeros(2, 3, 4, 5).to(memory_format=torch.channels_last).stride() and ctx.is_symmetric(cl)
    g = ctx.ones(3, requires_grad=True)
    assert g.requires_grad
    # alignment and exhaustion
    assert ctx.zeros(1).data_ptr() % 1024 == 0
    with pytest.raises(MemoryError):
        ctx.empty(1 << 30, dtype=torch.uint8)
    # broadcast
    assert ctx.broadcast(rank * 10 + 5, src=1) == 15
    t = ctx.broadcast(torch.full((3,), float(rank)), src=0)
    assert torch.all(torch.as_tensor(t) == 0)
    s = ctx.as_symmetric(torch.arange(6))
    assert ctx.is_symmetric(s) and torch.equal(s, torch.arange(6))
    dc = ctx.get_device_context()
    assert int(dc[0]) == rank and int(dc[1]) == world and dc.numel() == 2 + world + 17
    ctx.barrier()


def test_factories_world2():
    run_ranks(_factories, 2)


def _ccl_cpu(rank, world):
    import iris_b200 as iris
    from iris_b200.ccl import Config, owned_tiles

    ctx = iris.iris(1 << 26)
    M, N = 8, 6 * world
    inp = ctx.zeros((M, N), dtype=torch.float32)
    inp.copy_(torch.arange(M * N, dtype=torch.float32).view(M, N) + 1000 * rank)
    out = ctx.zeros((M, N), dtype=torch.float32)
    ctx.barrier()
    ctx.ccl.all_reduce(out, inp)
    exp = sum(torch.arange(M * N, dtype=torch.float32).view(M, N) + 1000 * r for r in range(world))
    assert torch.equal(out, exp)
    ag = ctx.zeros((world * M, N), dtype=torch.float32)
    ctx.ccl.all_gather(ag, inp)
    for r in range(world):
        assert torch.equal(ag[r * M:(r + 1) * M], torch.arange(M * N, dtype=torch.float32).view(M, N) + 1000 * r)
    a2a = ctx.zeros((M, N), dtype=torch.float32)
    ctx.ccl.all_to_all(a2a, inp)
    n = N // world
    for s in range(world):
        src = torch.arange(M * N, dtype=torch.float32).view(M, N) + 1000 * s
        assert torch.equal(a2a[:, s * n:(s + 1) * n], src[:, rank * n:(rank + 1) * n])
    rs = ctx.zeros((M, N), dtype=torch.float32)
    cfg = Config(block_size_m=4, block_size_n=4, all_reduce_distribution=0)
    ctx.ccl.reduce_scatter(rs, inp, config=cfg)
    mask = torch.zeros(M, N, dtype=torch.bool)
    for (r0, r1, c0, c1) in owned_tiles(M, N, 4, 4, world, rank, 0):
        mask[r0:r1, c0:c1] = True
    assert torch.equal(rs[mask], exp[mask]) and torch.all(rs[~mask] == 0)
    with pytest.raises(ValueError):
        ctx.ccl.all_reduce(out, torch.zeros(M, N))
    with pytest.raises(ValueError):
        ctx.ccl.all_gather(out, inp)
    # vectors: gathered end to end; 1-D tensors of other collectives are one row
    vec, cat = ctx.full((5,), float(rank)), ctx.zeros(5 * world)
    ctx.ccl.all_gather(cat, vec)
    assert cat.tolist() == [float(r) for r in range(world) for _ in range(5)]
    vsum = ctx.zeros(5)
    ctx.ccl.all_reduce(vsum, vec)
    assert torch.all(vsum == sum(range(world)))
    with pytest.raises(ValueError, match="do not split"):
        ctx.ccl.reduce_scatter(ctx.zeros((3, 4)), ctx.zeros((2 * world + 1, 4)), config=Config(reduce_scatter_rows=True))
    # fused ops fall back to GEMM + collective on this backend, same results
    A = torch.randn(4, 8)
    B = torch.randn(8, 5)
    C = ctx.zeros((4 * world, 5), dtype=torch.float32)
    ctx.ops.all_gather_matmul(C, A, B, shard_dim=0)
    import torch.distributed as dist

    parts = [torch.empty_like(A) for _ in range(world)]
    dist.all_gather(parts, A)
    assert torch.allclose(C, torch.cat(parts, 0) @ B, atol=1e-5)
    C2 = ctx.zeros((4, 5), dtype=torch.float32)
    ctx.ops.matmul_all_reduce(C2, A, B)
    tot = A @ B
    dist.all_reduce(tot)
    assert torch.allclose(C2, tot, atol=1e-4)
    ctx.barrier()


def test_collectives_cpu_world2():
    run_ranks(_ccl_cpu, 2)


def test_collectives_cpu_world3():
    run_ranks(_ccl_cpu, 3)


def _decode_cpu(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.models import FlashDecodeLayer, merge_partials, reference_decode

    ctx = iris.iris(1 << 26)
    Hq, Hkv, D, page, B = 8, 2, 128, 16, 2
    torch.manual_seed(0)
    q = torch.randn(B, Hq, D)
    torch.manual_seed(10 + rank)
    lens = torch.tensor([20 + rank, 5], dtype=torch.int32)
    kc, vc = torch.randn(8, page, Hkv, D), torch.randn(8, page, Hkv, D)
    table = torch.arange(8, dtype=torch.int32).view(2, 4)
    all_lens = [torch.empty_like(lens) for _ in range(world)]
    dist.all_gather(all_lens, lens)
    layer = FlashDecodeLayer(ctx, Hq, Hkv, D, max_batch=2, dtype=torch.float32)
    out = layer(q, kc, vc, torch.stack(all_lens), table)
    # oracle: attention over the concatenation of all shards
    o, lse = reference_decode(q, kc, vc, lens, table)
    os_, ls_ = [torch.empty_like(o) for _ in range(world)], [torch.empty_like(lse) for _ in range(world)]
    dist.all_gather(os_, o)
    dist.all_gather(ls_, lse)
    assert torch.allclose(out, merge_partials(torch.stack(os_), torch.stack(ls_)), atol=1e-5)
    # arguments are checked before anything could be launched with them
    good = dict(q=q, k_cache=kc, v_cache=vc, global_kv_lens=torch.stack(all_lens), block_table=table)
    for bad in (dict(q=torch.randn(B, Hq - 1, D)), dict(k_cache=torch.randn(8, page, Hkv + 1, D)), dict(v_cache=torch.randn(7, page, Hkv, D)),
                dict(block_table=table.long()), dict(block_table=table[:1]), dict(global_kv_lens=torch.stack(all_lens).long()),
                dict(global_kv_lens=torch.stack(all_lens)[:, :1]), dict(q=torch.randn(3, Hq, D))):
        with pytest.raises(ValueError):
            layer(**{**good, **bad})
    with pytest.raises(TypeError):
        layer(**{**good, "k_cache": kc.double(), "v_cache": vc.double()})
    with pytest.raises(ValueError):
        layer(**good, out=torch.empty(B, Hq, D + 1))
    # value checks belong to debug mode
    ctx.debug_checks = True
    try:
        layer(**good)
        with pytest.raises(ValueError, match="outside the cache"):
            layer(**{**good, "block_table": table + 5})
        long = torch.stack(all_lens).clone()
        long[rank, 0] = 4 * page + 1
        with pytest.raises(ValueError, match="sequence length"):
            layer(**{**good, "global_kv_lens": long})
    finally:
        ctx.debug_checks = False
    ctx.barrier()


def test_flash_decode_cpu_world2():
    run_ranks(_decode_cpu, 2)


def test_reference_decode_equals_dense_attention():
    from iris_b200.models import merge_partials, reference_decode

    torch.manual_seed(1)
    B, Hq, Hkv, D, page = 2, 4, 2, 128, 8
    kc, vc = torch.randn(6, page, Hkv, D), torch.randn(6, page, Hkv, D)
    q = torch.randn(B, Hq, D)
    table = torch.tensor([[0, 1, 2], [3, 4, 5]], dtype=torch.int32)
    lens = torch.tensor([20, 9], dtype=torch.int32)
    o, lse = reference_decode(q, kc, vc, lens, table)
    for b in range(B):
        k = kc[table[b].long()].reshape(-1, Hkv, D)[: lens[b]]
        v = vc[table[b].long()].reshape(-1, Hkv, D)[: lens[b]]
        for h in range(Hq):
            s = (k[:, h // 2] @ q[b, h]) / math.sqrt(D)
            p = torch.softmax(s, 0)
            assert torch.allclose(o[b, h], p @ v[:, h // 2], atol=1e-5)
            assert abs(float(lse[b, h]) - float(torch.logsumexp(s, 0))) < 1e-5
    # splitting a sequence in two shards and merging gives the same answer
    o1, l1 = reference_decode(q, kc, vc, torch.tensor([8, 8], dtype=torch.int32), table)
    o2, l2 = reference_decode(q, kc[:, :, :, :], vc, torch.tensor([0, 0], dtype=torch.int32), table)
    m = merge_partials(torch.stack([o1, o2]), torch.stack([l1, l2]))
    assert torch.allclose(m, o1, atol=1e-6)


def _moe_cpu(rank, world):
    import iris_b200 as iris
    from iris_b200.models import MoELayer, reference_moe

    ctx = iris.iris(1 << 26)
    T, D, F, K = 10, 16, 8, 2
    E = 2 * world
    torch.manual_seed(3)
    wg, wu, wd = torch.randn(E, D, F), torch.randn(E, D, F), torch.randn(E, F, D)
    sl = slice(rank * 2, rank * 2 + 2)
    layer = MoELayer(ctx, D, F, E, K, max_tokens=T, w_gate=wg[sl], w_up=wu[sl], w_down=wd[sl])
    torch.manual_seed(50 + rank)
    x, logits = torch.randn(T, D), torch.randn(T, E)
    out = layer(x, logits)
    assert torch.allclose(out, reference_moe(x, logits, wg, wu, wd, K), atol=1e-4)
    ctx.barrier()


def test_moe_cpu_world2():
    run_ranks(_moe_cpu, 2)


def _moe_cpu_fp8(rank, world):
    """``fp8=True`` on the CPU backend applies the roundings of the e4m3 kernels (tokens and hidden activations in
    1 x 128 blocks, weights in 128 x 128 blocks, power-of-two scales): the result equals a reference built from
    the rounded operands and differs from the unrounded layer by a quantisation error, not by nothing."""
    import iris_b200 as iris
    from iris_b200.models import MoELayer, reference_moe
    from iris_b200.models.moe import route

    if not hasattr(torch, "float8_e4m3fn"):
        return
    ctx = iris.iris(1 << 26)
    T, D, F, K = 12, 256, 128, 2
    E = 2 * world
    torch.manual_seed(5)
    wg, wu, wd = torch.randn(E, D, F) * 0.1, torch.randn(E, D, F) * 0.1, torch.randn(E, F, D) * 0.1
    sl = slice(rank * 2, rank * 2 + 2)
    layer = MoELayer(ctx, D, F, E, K, max_tokens=T, w_gate=wg[sl], w_up=wu[sl], w_down=wd[sl], fp8=True)
    torch.manual_seed(60 + rank)
    x, logits = torch.randn(T, D), torch.randn(T, E)
    out = layer(x, logits)
    fq = MoELayer._cpu_fake_quant
    wq = lambda w: torch.stack([fq(m.t().contiguous(), weight=True).t() for m in w])          # noqa: E731
    xq = fq(x)
    assert not torch.equal(xq, x) and torch.allclose(xq, x, atol=0.3, rtol=0.07)                # e4m3: 3 mantissa bits
    idx, wts = route(logits, K)
    ref = torch.zeros(T, D)
    for t in range(T):
        for k in range(K):
            e = int(idx[t, k])
            h = fq((torch.nn.functional.silu(xq[t:t + 1] @ wq(wg)[e]) * (xq[t:t + 1] @ wq(wu)[e])))
            ref[t] += (h @ wq(wd)[e])[0] * wts[t, k]
    assert torch.allclose(out, ref, atol=1e-3, rtol=1e-3)
    plain = reference_moe(x, logits, wg, wu, wd, K)
    err = (out - plain).abs().max().item() / plain.abs().max().item()
    assert 1e-4 < err < 0.15
    ctx.barrier()


def test_moe_cpu_fp8_mode_applies_the_e4m3_roundings():
    run_ranks(_moe_cpu_fp8, 2)


def test_fuse_gate_up_layout():
    from iris_b200.models import fuse_gate_up

    g = torch.arange(2 * 3 * 256, dtype=torch.float32).view(2, 3, 256)
    u = -g
    f = fuse_gate_up(g, u)
    assert f.shape == (2, 3, 512)
    assert torch.equal(f[:, :, 0:128], g[:, :, 0:128]) and torch.equal(f[:, :, 128:256], u[:, :, 0:128])
    assert torch.equal(f[:, :, 256:384], g[:, :, 128:256]) and torch.equal(f[:, :, 384:512], u[:, :, 128:256])


def _ring_cpu(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.models import RingAttention, reference_attention

    ctx = iris.iris(1 << 26)
    S, Hq, Hkv, D = 12, 4, 2, 128
    torch.manual_seed(rank)
    q, k, v = torch.randn(S, Hq, D), torch.randn(S, Hkv, D), torch.randn(S, Hkv, D)
    ks, vs = [torch.empty_like(k) for _ in range(world)], [torch.empty_like(v) for _ in range(world)]
    dist.all_gather(ks, k)
    dist.all_gather(vs, v)
    layer = RingAttention(ctx, S, Hq, Hkv, dtype=torch.float32)
    for causal in (False, True):
        out = layer(q, k, v, causal=causal)
        ref = reference_attention(q, torch.cat(ks), torch.cat(vs), causal, q_offset=rank * S)
        assert torch.allclose(out, ref, atol=1e-5)
    ctx.barrier()


def test_ring_attention_cpu_world2():
    run_ranks(_ring_cpu, 2)


def test_kernel_artifacts_parse(tmp_path):
    from iris_b200.host import artifacts

    text = """ptxas info    : Compiling entry function '_Z3fooPf' for 'sm_100a'
ptxas info    : Function properties for _Z3fooPf
    32 bytes stack frame, 36 bytes spill stores, 40 bytes spill loads
ptxas info    : Used 255 registers, used 1 barriers, 32 bytes cumulative stack size, 128 bytes smem
ptxas info    : Compiling entry function '_Z3barv' for 'sm_100a'
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Used 18 registers, used 0 barriers
"""
    ks = artifacts.parse_ptxas_log(text)
    assert [k["name"] for k in ks] == ["_Z3fooPf", "_Z3barv"]
    assert ks[0]["registers"] == 255 and ks[0]["spill_stores"] == 36 and ks[0]["smem_bytes"] == 128
    assert ks[1]["registers"] == 18 and ks[1]["spill_loads"] == 0
    meta = artifacts.collect()
    if meta:                                  # a build has run in this tree
        out = artifacts.export(tmp_path)
        assert any((out / name.replace(".cu", "") / "metadata.json").exists() for name in meta)


def test_fp8_block_quantisation_round_trip():
    """1 x 128 and 128 x 128 block scales: shapes, range, and the error of the dequantised product."""
    from iris_b200.ops.gemm_fp8 import FP8_MAX, dequant_matmul, dequantize, quantize_1x128, quantize_128x128

    torch.manual_seed(0)
    x = torch.randn(200, 336) * 3
    w = torch.randn(520, 336) * 0.05
    aq, asc = quantize_1x128(x)
    bq, bsc = quantize_128x128(w)
    assert aq.dtype == torch.float8_e4m3fn and tuple(asc.shape) == (200, 3) and tuple(bsc.shape) == (5, 3)
    assert aq.float().abs().max().item() <= FP8_MAX
    assert (dequantize(aq, asc, 1) - x).abs().max().item() <= x.abs().max().item() * 0.07     # e4m3: 3 mantissa bits
    ref = x @ w.t()
    assert (dequant_matmul(aq, asc, bq, bsc) - ref).abs().max().item() / ref.abs().max().item() < 8e-2


def test_gemm_plan_tile_choice():
    """The plan of the fused GEMMs is pure arithmetic behind the C ABI: large shapes get 256-wide CTA-pair
    tiles, shapes whose rows do not split into whole 256-row tiles per source / owner keep single CTAs."""
    import ctypes as C

    from iris_b200 import _lib

    lib = _lib.kernels()

    def plan(op, M, N, K, W=1, M_local=0, two_sm=0, bn=0):
        d = _lib.IrisGemmDesc()
        d.op, d.M, d.N, d.K, d.dtype, d.M_local, d.two_sm, d.bn = op, M, N, K, 1, M_local, two_sm, bn
        d.ctx.world = W
        out = [C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_int32(), C.c_int32()]
        rc = lib.iris_gemm_workspace(C.byref(d), *[C.byref(o) for o in out])
        return rc, out[3].value, out[4].value, out[0].value, out[2].value

    # 448 pair tiles of width 256 on 74 pairs are 6.05 waves, 512 of width 224 are 6.92: the nearly empty seventh
    # wave of the wide tiles costs more than the narrower tiles do (a part-filled wave counts as half)
    assert plan(_lib.GEMM_LOCAL, 8192, 3584, 8192)[:3] == (0, 224, 1)
    assert plan(_lib.GEMM_LOCAL, 8192, 8192, 3584)[:3] == (0, 256, 1)                # 13.8 against 16.0 waves: wide tiles
    assert plan(_lib.GEMM_LOCAL, 8192, 3584, 8192, two_sm=1)[2] == 0                 # pairs switched off
    assert plan(_lib.GEMM_LOCAL, 128, 8192, 3584)[:3] == (0, 128, 0)                 # few tiles: narrow single-CTA tiles
    rc, bn, pair, inbox, _ = plan(_lib.GEMM_AG_M, 8192, 3584, 8192, W=8, M_local=1024)
    assert (rc, bn, pair) == (0, 256, 1) and inbox == 2 * 8 * 1024 * 8192 * 2       # double-buffered inbox of all shards
    assert plan(_lib.GEMM_AG_M, 8 * 384, 3584, 8192, W=8, M_local=384)[2] == 0       # 384 rows per source: no whole 256-row tiles
    rc, bn, pair, _, staging = plan(_lib.GEMM_REDUCE_SCATTER, 8192, 8192, 3584, W=8)
    assert (rc, bn, pair) == (0, 256, 1) and staging == 2 * 8 * (8 * 32) * 128 * 256 * 2
    assert plan(_lib.GEMM_REDUCE_SCATTER, 1000, 8192, 3584, W=8)[0] != 0             # rows must split into 128-row tiles per rank
    assert plan(_lib.GEMM_RS_TILES, 8192, 8192, 3584, W=8)[2] == 0                   # tile-granular scatter keeps single CTAs


def test_zigzag_positions_cover_the_sequence_and_balance_causal_work():
    from iris_b200.models import reference_attention, zigzag_positions

    W, S = 4, 64
    pos = [zigzag_positions(r, W, S) for r in range(W)]
    assert torch.equal(torch.sort(torch.cat(pos)).values, torch.arange(W * S))
    # every rank sees the same number of (query, key) pairs under a causal mask
    work = [int((torch.cat(pos)[None, :] <= p[:, None]).sum()) for p in pos]
    assert max(work) - min(work) <= S
    # attention with explicit positions equals attention over the sorted sequence
    torch.manual_seed(0)
    q, k, v = torch.randn(W * S, 2, 16), torch.randn(W * S, 2, 16), torch.randn(W * S, 2, 16)
    full = reference_attention(q, k, v, causal=True)
    order = torch.cat(pos)
    for r in range(W):
        mine = reference_attention(q[pos[r]], k[order], v[order], causal=True, q_pos=pos[r], k_pos=order)
        assert torch.allclose(mine, full[pos[r]], atol=1e-5)


def _tp_mlp_check(rank, world, dtype_name, Ml, K, F, tol):
    """Forward and backward of TensorParallelMLP against autograd on the unsharded MLP."""
    import torch

    import iris_b200 as iris
    from iris_b200.models import TensorParallelMLP

    ctx = iris.iris(1 << 30)
    dt = getattr(torch, dtype_name)
    dev = ctx.get_device()
    g = torch.Generator().manual_seed(0)          # the same full tensors on every rank
    Xall = torch.randn(world * Ml, K, generator=g).to(dev)
    W1 = (torch.randn(K, world * F, generator=g) * 0.1).to(dev)
    W2 = (torch.randn(world * F, K, generator=g) * 0.1).to(dev)
    G = torch.randn(world * Ml, K, generator=g).to(dev)
    rows, cols = slice(rank * Ml, (rank + 1) * Ml), slice(rank * F, (rank + 1) * F)
    for act in (None, "silu", "gelu"):
        mlp = TensorParallelMLP(ctx, K, F, activation=act, dtype=dt, w1=W1[:, cols].to(dt).contiguous(), w2=W2[cols].to(dt).contiguous())
        for _ in range(2):                                    # the second step reuses the fused workspaces
            mlp.zero_grad()
            x = Xall[rows].to(dt).clone().requires_grad_(True)
            y = mlp(x)
            y.backward(G[rows].to(dt))
        Xr = Xall.to(dt).float().clone().requires_grad_(True)
        W1r = W1.to(dt).float().clone().requires_grad_(True)
        W2r = W2.to(dt).float().clone().requires_grad_(True)
        hp = Xr @ W1r
        h = hp if act is None else (torch.nn.functional.silu(hp) if act == "silu" else torch.nn.functional.gelu(hp, approximate="tanh"))
        Yr = h @ W2r
        Yr.backward(G.to(dt).float())

        def close(a, b, what):
            err = (a.float() - b).abs().max().item() / max(b.abs().max().item(), 1e-6)
            assert err < tol, (act, what, err)

        close(y.detach(), Yr[rows].detach(), "y")
        close(x.grad, Xr.grad[rows], "dx")
        close(mlp.w1.grad, W1r.grad[:, cols], "dw1")
        close(mlp.w2.grad, W2r.grad[cols], "dw2")
    ctx.check()
    ctx.barrier()


def test_tensor_parallel_mlp_forward_backward_cpu():
    run_ranks(_tp_mlp_check, 2, args=("float32", 8, 16, 12, 1e-4))


def test_launch_records(tmp_path, monkeypatch):
    import json

    import torch

    from iris_b200.host import artifacts

    monkeypatch.delenv("IRIS_KERNEL_ARTIFACTS_DIR", raising=False)
    artifacts.configure(None)
    assert not artifacts.ACTIVE and artifacts.record_launch("ccl", "all_reduce_two_shot", 0, {"M": 8, "N": 8}) is None
    artifacts.configure(tmp_path)
    try:
        assert artifacts.ACTIVE
        params = {"M": 8192, "N": 4096, "dtype": torch.bfloat16, "world": 8, "comm_sms": 64, "use_multicast": True}
        d = artifacts.record_launch("ccl", "all_reduce_nvls", 3, params, source="ccl.cu")
        # <dir>/<algo>/<kernel>/rank_N/<M x N _ dtype _ world>/<sha12>/metadata.json
        rel = d.relative_to(tmp_path).parts
        assert rel[:4] == ("ccl", "all_reduce_nvls", "rank_3", "8192x4096_bfloat16_w8") and len(rel[4]) == 12
        meta = json.loads((d / "metadata.json").read_text())
        assert meta["kernel"] == "all_reduce_nvls" and meta["rank"] == 3 and meta["arch"] == "sm_100a" and meta["source"] == "ccl.cu"
        assert meta["params"]["dtype"] == "torch.bfloat16" and meta["params"]["comm_sms"] == 64
        if (artifacts._build.OBJDIR / "ccl.cu.ptxas.log").exists():
            assert (d / "ptxas.log").exists() and any(k["registers"] for k in meta["compiled"])
        # the same configuration is written once; another configuration or rank gets its own directory
        assert artifacts.record_launch("ccl", "all_reduce_nvls", 3, params, source="ccl.cu") is None
        d2 = artifacts.record_launch("ccl", "all_reduce_nvls", 3, dict(params, comm_sms=148), source="ccl.cu")
        assert d2 is not None and d2 != d and d2.parent == d.parent
        d3 = artifacts.record_launch("ops", "matmul_all_reduce", 0, {"M": 128, "N": 8192, "K": 3584, "dtype": torch.float16, "world": 2})
        assert d3.relative_to(tmp_path).parts[:4] == ("ops", "matmul_all_reduce", "rank_0", "128x8192_float16_w2")
        assert json.loads((d3 / "metadata.json").read_text())["compiled"] == []
    finally:
        artifacts.configure(None)
    assert not artifacts.ACTIVE


def test_launch_paths_write_records(tmp_path, monkeypatch):
    """The GPU launch functions of the collectives and the fused ops, driven with stand-ins for the
    native library: each distinct configuration leaves one record, the launch itself still happens."""
    import os
    import types

    import torch

    from iris_b200 import _lib, ccl, ops
    from iris_b200.host import artifacts

    calls = []
    fake = types.SimpleNamespace(iris_ccl_launch=lambda op, d, s: calls.append(op) or 0, iris_gemm_launch=lambda d, s: calls.append("gemm") or 0)
    monkeypatch.setattr(_lib, "current_stream_ptr", lambda: 0)
    monkeypatch.setattr(_lib, "kernels", lambda: fake)
    artifacts.configure(tmp_path)
    try:
        me = types.SimpleNamespace(ctx=types.SimpleNamespace(cur_rank=1), _lib=lambda: fake)
        d = ccl.IrisCclDesc()
        d.M, d.N, d.dtype, d.variant, d.ctx.world = 64, 128, 1, 5, 4
        ccl.CCL._launch(me, 2, d)
        ccl.CCL._launch(me, 2, d)                      # same configuration: launched again, recorded once
        d.rows_mode = 1
        ccl.CCL._launch(me, 3, d)
        ccl.CCL._launch(me, 0, d)
        g = _lib.IrisGemmDesc()
        g.M, g.N, g.K, g.op = 256, 512, 64, _lib.GEMM_ALL_REDUCE
        ws = ops.FusedWorkspace(operation="matmul_all_reduce", dtype=torch.bfloat16, sync_block=torch.zeros(4, dtype=torch.int32), bn=256)
        ops._launch(types.SimpleNamespace(cur_rank=1, num_ranks=4), g, ws)
    finally:
        artifacts.configure(None)
    assert calls == [2, 2, 3, 0, "gemm"]
    found = sorted(os.path.relpath(root, tmp_path).rsplit(os.sep, 1)[0] for root, _, files in os.walk(tmp_path)
                   if "metadata.json" in files and not os.path.relpath(root, tmp_path).startswith("build"))
    assert found == ["ccl/all_gather/rank_1/64x128_bfloat16_w4", "ccl/all_reduce_nvls/rank_1/64x128_bfloat16_w4",
                     "ccl/reduce_scatter_rows/rank_1/64x128_bfloat16_w4", "ops/matmul_all_reduce/rank_1/256x512_bfloat16_w4"]


def _context_manager(rank, world):
    import iris_b200 as iris

    with iris.iris(1 << 22) as ctx:
        t = ctx.full((8,), float(rank))
        got = ctx.rma.load(t, from_rank=(rank + 1) % world)
        assert torch.all(got == (rank + 1) % world)
        del t
    # the heap is gone; a new context can be created by the same processes
    with iris.iris(1 << 22) as ctx2:
        assert ctx2.get_num_ranks() == world and torch.all(ctx2.zeros(4) == 0)
    with pytest.raises(RuntimeError, match="boom"):
        with iris.iris(1 << 22):
            raise RuntimeError("boom")            # no barrier on the way out: nothing hangs


def test_context_manager_releases_the_heap():
    run_ranks(_context_manager, 2)
