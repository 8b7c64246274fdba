"""Multi-GPU tests: one child process per GPU (nccl), world = min(#GPUs, 4).

Oracles are torch.distributed collectives and fp32/fp64 host arithmetic, as in the reference's
tests/ccl and tests/ops. Skipped on a machine with fewer than two GPUs.
"""
import pytest
import torch

from helpers import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _world():
    """Ranks of the multi-GPU cases: ``IRIS_TEST_WORLD`` when set (the suite is run at 2, 4 and 8),
    else every GPU up to four."""
    import os

    want = int(os.environ.get("IRIS_TEST_WORLD", "0"))
    return min(torch.cuda.device_count(), want if want > 0 else 4)


def _maxerr(a, b):
    return (a.double() - b.double()).abs().max().item()


def _rma(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris

    ctx = iris.iris(1 << 30)
    buf = ctx.zeros(4096, dtype=torch.float32)
    cnt = ctx.zeros(1, dtype=torch.int32)
    ctx.barrier()
    if rank == 0:
        for b in range(4):
            ctx.rma.store(buf[b * 1024:(b + 1) * 1024], 1.0, to_rank=1)
    for p in range(world):
        ctx.rma.atomic_add(cnt, 1, to_rank=p, sem="acq_rel", scope="sys")
    ctx.barrier()
    assert torch.all(buf == (1.0 if rank == 1 else 0.0))
    assert int(cnt.item()) == world
    peer = (rank + 1) % world
    a = ctx.arange(0, 512, dtype=torch.int32)
    a += 1000 * rank
    b = ctx.zeros(512, dtype=torch.int32)
    ctx.barrier()
    for cm in (None, ".cg", ".cv"):
        assert torch.equal(ctx.rma.load(a, from_rank=peer, cache_modifier=cm).cpu(), torch.arange(512, dtype=torch.int32) + 1000 * peer)
    ctx.rma.get(a, b, from_rank=peer)
    assert torch.equal(b.cpu(), torch.arange(512, dtype=torch.int32) + 1000 * peer)
    ctx.barrier()
    b.zero_()
    ctx.barrier()
    ctx.rma.put(a, b, to_rank=peer)
    ctx.barrier()
    assert torch.equal(b.cpu(), torch.arange(512, dtype=torch.int32) + 1000 * ((rank - 1) % world))
    # device barrier orders a remote store before the peer's read, with no host sync in between
    x = ctx.zeros(64, dtype=torch.float32)
    ctx.barrier()
    ctx.rma.store(x, float(rank + 1), to_rank=peer)
    ctx.device_barrier()
    got = x.clone()
    torch.cuda.synchronize()
    assert torch.all(got == float(((rank - 1) % world) + 1))
    ctx.check()
    ctx.barrier()


def test_rma_between_gpus():
    run_ranks(_rma, _world(), backend="nccl")


def _vmem(rank, world):
    """allocator_type="vmem" on real GPUs: physical memory mapped on demand behind a reserved address range,
    every new segment exported to and mapped by every peer, and an allocation made outside the heap with the
    virtual-memory API taken in without a copy (reference: tests/unittests/test_vmem_allocator.py,
    test_vmem_segmented_export_import.py, test_vmem_imported_tensor_rma.py)."""
    import iris_b200 as iris
    from iris_b200.host import platform as hip
    from iris_b200.host.heap import _rt
    from iris_b200.host.tensor_utils import tensor_from_ptr

    ctx = iris.iris(256 << 20, allocator_type="vmem")
    heap, rt = ctx.heap, _rt()
    assert heap.reserve == 256 << 20 and not ctx.has_multicast()
    first = rt.iris_heap_mapped_size(heap._handle)
    a = ctx.zeros(1 << 20, dtype=torch.float32)                    # 4 MB
    b = ctx.zeros(8 << 20, dtype=torch.float32)                    # 32 MB: beyond the 16 MB mapped at first
    assert rt.iris_heap_num_segments(heap._handle) >= 1 and rt.iris_heap_mapped_size(heap._handle) > first
    a.fill_(float(rank + 1))
    b.fill_(float(10 * (rank + 1)))
    ctx.barrier()
    peer = (rank + 1) % world
    assert float(ctx.rma.load(a[-4:], from_rank=peer)[0]) == peer + 1
    assert float(ctx.rma.load(b[-4:], from_rank=peer)[0]) == 10 * (peer + 1)        # the grown segment, read from the peer
    out, inp = ctx.zeros((64, 256), dtype=torch.float32), ctx.full((64, 256), float(rank + 1))
    ctx.ccl.all_reduce(out, inp)                                    # collectives on a heap without a multicast window
    assert torch.all(out == sum(range(1, world + 1)))
    # external VMM allocation -> part of the heap, no copy
    dev = ctx.gpu_id
    gran = hip.get_allocation_granularity(dev)
    h = hip.mem_create(gran, dev)
    va = hip.mem_address_reserve(gran)
    hip.mem_map(va, gran, 0, h)
    hip.mem_set_access(va, gran, dev)
    ext = tensor_from_ptr(va, 4096, torch.int32, ctx.get_device())
    ext.copy_(torch.arange(4096, dtype=torch.int32, device=ctx.get_device()) + 1000 * rank)
    sym = ctx.as_symmetric(ext)
    assert ctx.is_symmetric(sym) and sym.data_ptr() != ext.data_ptr() and torch.equal(sym, ext)
    ext[0] = -7
    torch.cuda.synchronize()
    assert int(sym[0]) == -7                                        # the same memory under a second address
    ctx.barrier()
    got = ctx.rma.load(sym[:8], from_rank=peer).cpu()
    assert int(got[0]) == -7 and int(got[1]) == 1 + 1000 * peer     # and peers reach it like any heap tensor
    ctx.barrier()
    ctx.check()
    del a, b, sym, ext, out, inp
    ctx.close()
    hip.mem_unmap(va, gran)
    hip.mem_address_free(va, gran)
    hip.mem_release(h)


def test_growable_vmem_heap_and_zero_copy_import_between_gpus():
    run_ranks(_vmem, _world(), backend="nccl", env={"IRIS_VMEM_INITIAL": str(16 << 20)}, timeout=300)


def _ccl(rank, world, nvls):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.ccl import Config, owned_tiles

    ctx = iris.iris(2 << 30)
    for dtype, M, N in ((torch.bfloat16, 256, 512), (torch.float32, 128, 192), (torch.float16, 100, 72), (torch.float32, 1024, 2048)):
        g = torch.Generator(device="cuda")
        g.manual_seed(1234 + rank)
        inp = ctx.empty((M, N), dtype=dtype)
        inp.copy_((torch.rand(M, N, device="cuda", generator=g) * 2 - 1).to(dtype))
        gathered = [torch.empty_like(inp) for _ in range(world)]
        dist.all_gather(gathered, inp)
        total = torch.stack([x.double() for x in gathered]).sum(0)
        tol = 1e-5 * world if dtype == torch.float32 else 0.03 * world
        out = ctx.zeros((world * M, N), dtype=dtype)
        for v in ("persistent", "partitioned"):
            out.zero_()
            ctx.barrier()
            ctx.ccl.all_gather(out, inp, config=Config(all_gather_variant=v))
            assert torch.equal(out, torch.cat(gathered, 0)), v
        if N % world == 0:
            o2 = ctx.zeros((M, N), dtype=dtype)
            ctx.barrier()
            ctx.ccl.all_to_all(o2, inp)
            n = N // world
            exp = torch.cat([gathered[s][:, rank * n:(rank + 1) * n] for s in range(world)], 1)
            assert torch.equal(o2, exp)
        for v in ("one_shot", "two_shot", "atomic", "ring", "spinlock", "auto", "nvls", "push"):
            o3 = ctx.zeros((M, N), dtype=dtype)
            ctx.barrier()
            ws = None
            for _ in range(3):
                ws = ctx.ccl.all_reduce(o3, inp, config=Config(all_reduce_variant=v), workspace=ws)
            assert _maxerr(o3, total) <= tol, (v, ws.variant, str(dtype))
        for dmode in (0, 1):
            o4 = ctx.zeros((M, N), dtype=dtype)
            ctx.barrier()
            cfg = Config(all_reduce_distribution=dmode)
            ctx.ccl.reduce_scatter(o4, inp, config=cfg)
            exp = torch.zeros(M, N, dtype=torch.float64, device="cuda")
            for (r0, r1, c0, c1) in owned_tiles(M, N, cfg.block_size_m, cfg.block_size_n, world, rank, dmode):
                exp[r0:r1, c0:c1] = total[r0:r1, c0:c1]
            assert _maxerr(o4, exp) <= tol
        if M % world == 0:
            o5 = ctx.zeros((M // world, N), dtype=dtype)
            ctx.barrier()
            ctx.ccl.reduce_scatter(o5, inp, config=Config(reduce_scatter_rows=True))
            assert _maxerr(o5, total[rank * (M // world):(rank + 1) * (M // world)]) <= tol
    ctx.check()
    ctx.barrier()


@pytest.mark.parametrize("nvls", [False, True])
def test_collectives_match_nccl(nvls):
    run_ranks(_ccl, _world(), args=(nvls,), backend="nccl", env={"IRIS_NVLS": "1" if nvls else "0"})


def _groups(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris

    ctx = iris.iris(1 << 30)
    # consecutive pairs and strided pairs, every collective restricted to the group
    layouts = [[[0, 1], [2, 3]], [[0, 2], [1, 3]]]
    for layout in layouts:
        groups = [dist.new_group(r) for r in layout]
        mine = next(g for g, r in zip(groups, layout) if rank in r)
        members = next(r for r in layout if rank in r)
        inp = ctx.full((64, 128), float(rank + 1), dtype=torch.float32)
        out = ctx.zeros((64, 128), dtype=torch.float32)
        ctx.barrier()
        ctx.ccl.all_reduce(out, inp, group=mine)
        assert torch.all(out == float(sum(m + 1 for m in members)))
        ag = ctx.zeros((128, 128), dtype=torch.float32)
        ctx.barrier()
        ctx.ccl.all_gather(ag, inp, group=mine)
        assert torch.all(ag[:64] == float(members[0] + 1)) and torch.all(ag[64:] == float(members[1] + 1))
        ctx.barrier()
    ctx.check()


def test_process_groups():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    run_ranks(_groups, 4, backend="nccl")


def _ops(rank, world, nvls):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.ops import FusedConfig, owned_tile_range

    ctx = iris.iris(4 << 30)
    W = world
    for dtype, Ml, N, K, kmajor in ((torch.bfloat16, 256, 512, 512, False), (torch.float16, 128, 768, 1024, True),
                                    (torch.bfloat16, 512, 3584, 1024, False)):
        torch.manual_seed(7 + rank)

        def mkB(k, n):
            return (torch.randn(n, k, device="cuda", dtype=dtype) * 0.05).t() if kmajor else torch.randn(k, n, device="cuda", dtype=dtype) * 0.05

        A = torch.randn(Ml, K, device="cuda", dtype=dtype)
        B = mkB(K, N)
        Aall = torch.empty(W * Ml, K, device="cuda", dtype=dtype)
        dist.all_gather_into_tensor(Aall, A)
        ref = Aall.float() @ B.float()
        C = ctx.zeros((W * Ml, N), dtype=dtype)
        ws = None
        for _ in range(3):
            ws = ctx.ops.all_gather_matmul(C, A, B, shard_dim=0, workspace=ws)
        assert ws.variant == "fused"
        assert _maxerr(C, ref) <= 0.02 * ref.abs().max().item()
        if K % (64 * W) == 0:
            A2 = torch.randn(W * Ml, K // W, device="cuda", dtype=dtype)
            bias = torch.randn(W * Ml, device="cuda", dtype=dtype)
            parts = [torch.empty_like(A2) for _ in range(W)]
            dist.all_gather(parts, A2)
            ref2 = torch.cat(parts, 1).float() @ B.float() + bias.float()[:, None]
            C2 = ctx.zeros((W * Ml, N), dtype=dtype)
            ws2 = None
            for _ in range(2):
                ws2 = ctx.ops.all_gather_matmul(C2, A2, B, bias=bias, workspace=ws2)
            assert _maxerr(C2, ref2) <= 0.02 * ref2.abs().max().item()
        loc = (A.float() @ B.float()).to(dtype)
        ref_ag = torch.empty(W * Ml, N, device="cuda", dtype=dtype)
        dist.all_gather_into_tensor(ref_ag, loc)
        C3 = ctx.zeros((W * Ml, N), dtype=dtype)
        ws3 = None
        for _ in range(2):
            ws3 = ctx.ops.matmul_all_gather(C3, A, B, workspace=ws3)
        assert _maxerr(C3, ref_ag) <= 0.02 * ref.abs().max().item()
        # the other overlap patterns of GEMM + all-gather / all-scatter: communication CTAs inside the kernel, and GEMM then collective
        ref_cols = ref_ag.view(W, Ml, N).permute(1, 0, 2).reshape(Ml, W * N)
        for overlap in ("wg_specialized", "bulk_synchronous", "fused"):
            cfg = FusedConfig(overlap=overlap)
            Cr, Cc = ctx.zeros((W * Ml, N), dtype=dtype), ctx.zeros((Ml, W * N), dtype=dtype)
            wr = wc = None
            for _ in range(3):
                wr = ctx.ops.matmul_all_gather(Cr, A, B, workspace=wr, config=cfg)
                wc = ctx.ops.matmul_all_gather(Cc, A, B, workspace=wc, config=cfg, scatter_cols=True)
            assert (wr.variant == "unfused") == (overlap == "bulk_synchronous"), overlap
            if overlap == "wg_specialized":
                assert wr.extra["overlap"] == "wg_specialized" and wr.flags is not None
            assert _maxerr(Cr, ref_ag) <= 0.02 * ref.abs().max().item(), overlap
            assert _maxerr(Cc, ref_cols) <= 0.02 * ref.abs().max().item(), overlap
        M = W * Ml
        A4 = torch.randn(M, K, device="cuda", dtype=dtype)
        B4 = mkB(K, N)
        tot = A4.float() @ B4.float()
        dist.all_reduce(tot)
        tol = 0.03 * tot.abs().max().item()
        C4 = ctx.zeros((M, N), dtype=dtype)
        ws4 = None
        for _ in range(3):
            ws4 = ctx.ops.matmul_all_reduce(C4, A4, B4, workspace=ws4)
        assert _maxerr(C4, tot) <= tol
        # every variant of the all-reduce half, three calls each (the staging is double-buffered by call parity)
        for variant in ("two_shot", "one_shot", "atomic"):
            Cv = ctx.zeros((M, N), dtype=dtype)
            wv = None
            for _ in range(3):
                wv = ctx.ops.matmul_all_reduce(Cv, A4, B4, workspace=wv, config=FusedConfig(all_reduce_variant=variant))
            assert wv.variant == "fused" and wv.extra["all_reduce_variant"] == variant
            # atomic: 16-bit accumulation in memory, one rounding per rank
            assert _maxerr(Cv, tot) <= (tol * (1 + W / 4) if variant == "atomic" else tol), variant
        C5 = ctx.zeros((Ml, N), dtype=dtype)
        ws5 = None
        for _ in range(3):
            ws5 = ctx.ops.matmul_reduce_scatter(C5, A4, B4, scatter_rows=True, workspace=ws5)
        assert _maxerr(C5, tot[rank * Ml:(rank + 1) * Ml]) <= tol
        C6 = ctx.zeros((M, N), dtype=dtype)
        ws6 = None
        for _ in range(2):
            ws6 = ctx.ops.matmul_reduce_scatter(C6, A4, B4, workspace=ws6)
        bn = ws6.bn
        tiles_n = -(-N // bn)
        exp = torch.zeros(M, N, device="cuda")
        for t in owned_tile_range(-(-M // 128) * tiles_n, W, rank):
            tm, tn = divmod(t, tiles_n)
            exp[tm * 128:(tm + 1) * 128, tn * bn:(tn + 1) * bn] = tot[tm * 128:(tm + 1) * 128, tn * bn:(tn + 1) * bn]
        assert _maxerr(C6, exp) <= tol
    ctx.check()
    ctx.barrier()


@pytest.mark.parametrize("nvls", [False, True])
def test_fused_ops_match_reference(nvls):
    run_ranks(_ops, _world(), args=(nvls,), backend="nccl", env={"IRIS_NVLS": "1" if nvls else "0"}, timeout=600)


def _fp8_ops(rank, world, nvls):
    """The fused ops on block-scaled e4m3 operands (scales applied by the tensor core, shards and their
    scale atoms gathered inside the kernel) against fp32 products of the dequantised operands."""
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.ops import quantize_activation, quantize_weight

    ctx = iris.iris(4 << 30)
    W = world
    dt = torch.bfloat16

    def rowerr(c, ref):
        return ((c.float() - ref).abs().amax(dim=1) / ref.abs().amax(dim=1).clamp_min(1e-20)).max().item()

    for Ml, N, K in ((256, 448, 1024), (128, 896, 512 * W)):
        torch.manual_seed(21 + rank)
        x = torch.randn(Ml, K, device="cuda") * torch.exp2(torch.randint(-4, 4, (Ml, 1), device="cuda").float())
        w = torch.randn(N, K, device="cuda") * 0.05 * torch.exp2(torch.randint(-3, 3, (-(-N // 128), -(-K // 128)), device="cuda").float()) \
            .repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
        xq, wq = quantize_activation(x), quantize_weight(w)
        xd, wd = xq.dequantize(), wq.dequantize()
        # all_gather_matmul, rows sharded
        xall = torch.empty(W * Ml, K, device="cuda")
        dist.all_gather_into_tensor(xall, xd)
        ref = xall @ wd
        C = ctx.zeros((W * Ml, N), dtype=dt)
        ws = None
        for _ in range(3):
            ws = ctx.ops.all_gather_matmul(C, xq, wq, shard_dim=0, workspace=ws)
        assert ws.variant == "fused" and ws.bn == 224
        assert rowerr(C, ref) < 1.5e-2
        # all_gather_matmul, K sharded: rank r holds columns [r K/W, (r+1) K/W) of the activations, weights replicated
        torch.manual_seed(99)
        wfull = quantize_weight(torch.randn(N, K, device="cuda") * 0.05)
        torch.manual_seed(21 + rank)
        xs = quantize_activation(torch.randn(W * Ml, K // W, device="cuda"))
        parts = [torch.empty(W * Ml, K // W, device="cuda") for _ in range(W)]
        dist.all_gather(parts, xs.dequantize())
        ref2 = torch.cat(parts, 1) @ wfull.dequantize()
        C2 = ctx.zeros((W * Ml, N), dtype=dt)
        ws2 = None
        for _ in range(2):
            ws2 = ctx.ops.all_gather_matmul(C2, xs, wfull, workspace=ws2)
        assert ws2.variant == "fused" and rowerr(C2, ref2) < 1.5e-2
        # reduce ops: sum over ranks of the local products
        M = W * Ml
        x4 = quantize_activation(torch.randn(M, K, device="cuda"))
        tot = x4.dequantize() @ wd
        dist.all_reduce(tot)
        C4 = ctx.zeros((M, N), dtype=dt)
        C5 = ctx.zeros((Ml, N), dtype=dt)
        w4 = w5 = None
        for _ in range(3):
            w4 = ctx.ops.matmul_all_reduce(C4, x4, wq, workspace=w4)
            w5 = ctx.ops.matmul_reduce_scatter(C5, x4, wq, scatter_rows=True, workspace=w5)
        assert w4.variant == "fused" and w5.variant == "fused"
        tol = 0.03 * tot.abs().max().item()
        assert _maxerr(C4, tot) <= tol and _maxerr(C5, tot[rank * Ml:(rank + 1) * Ml]) <= tol
        # matmul_all_gather
        loc = (xd @ wd).to(dt)
        ref_ag = torch.empty(W * Ml, N, device="cuda", dtype=dt)
        dist.all_gather_into_tensor(ref_ag, loc)
        C3 = ctx.zeros((W * Ml, N), dtype=dt)
        w3 = None
        for _ in range(2):
            w3 = ctx.ops.matmul_all_gather(C3, xq, wq, workspace=w3)
        assert w3.variant == "fused" and rowerr(C3, ref_ag.float()) < 1.5e-2
    ctx.check()
    ctx.barrier()


@pytest.mark.parametrize("nvls", [False, True])
def test_fp8_fused_ops_match_dequantised_reference(nvls):
    run_ranks(_fp8_ops, _world(), args=(nvls,), backend="nccl", env={"IRIS_NVLS": "1" if nvls else "0"}, timeout=600)


def _decode(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.models import FlashDecodeLayer, merge_partials, reference_decode

    ctx = iris.iris(1 << 30)
    Hq, Hkv, D, page, B = 32, 4, 128, 64, 3
    dt = torch.bfloat16
    torch.manual_seed(5)
    q = torch.randn(B, Hq, D, device="cuda", dtype=dt)           # replicated (same seed)
    torch.manual_seed(100 + rank)
    lens = [300 + 37 * rank, 64 * (rank + 1), 1 + rank]
    max_blocks = -(-max(lens) // page)
    kc = torch.randn(B * max_blocks, page, Hkv, D, device="cuda", dtype=dt)
    vc = torch.randn(B * max_blocks, page, Hkv, D, device="cuda", dtype=dt)
    table = torch.arange(B * max_blocks, device="cuda", dtype=torch.int32).view(B, max_blocks)
    my_lens = torch.tensor(lens, device="cuda", dtype=torch.int32)
    all_lens = torch.empty(world, B, device="cuda", dtype=torch.int32)
    dist.all_gather_into_tensor(all_lens, my_lens)
    layer = FlashDecodeLayer(ctx, Hq, Hkv, D, max_batch=4)
    for _ in range(3):
        out = layer(q, kc, vc, all_lens, table)
    o, lse = reference_decode(q, kc, vc, my_lens, table)
    os_ = [torch.empty_like(o) for _ in range(world)]
    ls_ = [torch.empty_like(lse) for _ in range(world)]
    dist.all_gather(os_, o)
    dist.all_gather(ls_, lse)
    ref = merge_partials(torch.stack(os_), torch.stack(ls_))
    assert (out.float() - ref).abs().max().item() < 2e-2
    ctx.check()
    ctx.barrier()


def test_distributed_flash_decode():
    run_ranks(_decode, _world(), backend="nccl")


def _moe(rank, world, fp8=False):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.models import MoELayer, reference_moe

    ctx = iris.iris(1 << 30)
    T, D, F, K = 160, 512, 256, 4
    E = 4 * world
    El = E // world
    dt = torch.bfloat16
    torch.manual_seed(21)                                   # every rank builds the full weight set ...
    wg = (torch.randn(E, D, F, device="cuda") * 0.05).to(dt)
    wu = (torch.randn(E, D, F, device="cuda") * 0.05).to(dt)
    wd = (torch.randn(E, F, D, device="cuda") * 0.05).to(dt)
    sl = slice(rank * El, (rank + 1) * El)                  # ... and keeps its own experts
    layer = MoELayer(ctx, D, F, E, K, max_tokens=T, w_gate=wg[sl].contiguous(), w_up=wu[sl].contiguous(), w_down=wd[sl].contiguous(),
                     fp8=fp8)
    if fp8:
        # the oracle runs on the values the e4m3 weights stand for (same 128 x 128 power-of-two quantiser as the layer):
        # what remains is the quantisation of the tokens and of the hidden activations
        from iris_b200.ops.gemm_fp8 import dequantize, quantize_128x128

        def deq(w):
            out = []
            for e in range(E):
                q, sc = quantize_128x128(w[e].t().contiguous().float(), pow2=True)
                out.append(dequantize(q, sc, 128).t())
            return torch.stack(out)

        wg, wu, wd = deq(wg), deq(wu), deq(wd)
    for it in range(3):
        torch.manual_seed(100 * it + rank)
        x = torch.randn(T, D, device="cuda", dtype=dt)
        logits = torch.randn(T, E, device="cuda")
        out = layer(x, logits)
        ref = reference_moe(x, logits, wg, wu, wd, K)
        err = (out.float() - ref).abs().max().item()
        # e4m3 tokens, weights and hidden activations: a few per cent of the largest output
        assert err < (6e-2 if fp8 else 3e-2) * max(ref.abs().max().item(), 1.0), (it, err, ref.abs().max().item())
    ctx.check()
    ctx.barrier()


@pytest.mark.parametrize("fp8", [False, True])
def test_expert_sharded_moe(fp8):
    run_ranks(_moe, _world(), args=(fp8,), backend="nccl", timeout=600)


def _ring(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.models import RingAttention, reference_attention

    ctx = iris.iris(1 << 30)
    Hq, Hkv, D = 8, 2, 128
    dt = torch.bfloat16
    torch.manual_seed(30 + rank)
    for S in (192, 256):          # 192: mma.sync attention CTAs, 256: tcgen05 attention CTAs
        q = torch.randn(S, Hq, D, device="cuda", dtype=dt)
        k = torch.randn(S, Hkv, D, device="cuda", dtype=dt)
        v = torch.randn(S, Hkv, D, device="cuda", dtype=dt)
        ks = torch.empty(world * S, Hkv, D, device="cuda", dtype=dt)
        vs = torch.empty(world * S, Hkv, D, device="cuda", dtype=dt)
        dist.all_gather_into_tensor(ks, k)
        dist.all_gather_into_tensor(vs, v)
        layer = RingAttention(ctx, S, Hq, Hkv)
        for causal in (False, True):
            for _ in range(3):
                out = layer(q, k, v, causal=causal)
            ref = reference_attention(q, ks, vs, causal, q_offset=rank * S)
            assert (out.float() - ref).abs().max().item() < 2e-2, (S, causal)
        ctx.check()
    ctx.barrier()


def test_ring_attention_between_gpus():
    run_ranks(_ring, _world(), backend="nccl")


def _ring_zigzag(rank, world):
    """Zigzag layout: rank r holds chunks r and 2W-1-r of the sequence; the causal result must equal
    attention over the whole sequence with the tokens' global positions."""
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.models import RingAttention, reference_attention, zigzag_positions

    ctx = iris.iris(1 << 30)
    S, Hq, Hkv, D = 512, 8, 2, 128
    dt = torch.bfloat16
    torch.manual_seed(40 + rank)
    q = torch.randn(S, Hq, D, device="cuda", dtype=dt)
    k = torch.randn(S, Hkv, D, device="cuda", dtype=dt)
    v = torch.randn(S, Hkv, D, device="cuda", dtype=dt)
    ks = torch.empty(world * S, Hkv, D, device="cuda", dtype=dt)
    vs = torch.empty(world * S, Hkv, D, device="cuda", dtype=dt)
    dist.all_gather_into_tensor(ks, k)
    dist.all_gather_into_tensor(vs, v)
    q_pos = zigzag_positions(rank, world, S, device="cuda")
    k_pos = torch.cat([zigzag_positions(r, world, S, device="cuda") for r in range(world)])
    layer = RingAttention(ctx, S, Hq, Hkv, layout="zigzag")
    for causal in (True, False):
        for _ in range(2):
            out = layer(q, k, v, causal=causal)
        ref = reference_attention(q, ks, vs, causal, q_pos=q_pos, k_pos=k_pos)
        assert (out.float() - ref).abs().max().item() < 2e-2, causal
    ctx.check()
    ctx.barrier()


def test_ring_attention_zigzag_layout_between_gpus():
    run_ranks(_ring_zigzag, _world(), backend="nccl")


def _tiles(rank, world):
    import os

    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200 import jit

    ctx = iris.iris(1 << 28)
    here = os.path.dirname(os.path.abspath(__file__))
    mod = jit.compile_file(os.path.join(here, "kernels", "user_kernels.cu"))
    call = mod.fn("tile_collective")
    M, N, bm, bn = 96, 64 * world, 32, 32
    g = torch.Generator(device="cuda")
    g.manual_seed(77 + rank)
    src = ctx.zeros((M, N), dtype=torch.float32)
    src.copy_(torch.randn(M, N, device="cuda", generator=g))
    parts = [torch.empty_like(src) for _ in range(world)]
    dist.all_gather(parts, src)
    total = torch.stack(parts).sum(0)
    tiles_n = N // bn
    tiles = (M // bm) * tiles_n
    ready = 0
    for op in (0, 1, 2, 3, 7, 8):                   # the reductions (8 = ring order)
        dst = ctx.zeros((M, N), dtype=torch.float32)
        locks = ctx.zeros(tiles, dtype=torch.int32)
        ctx.barrier()
        ready = 1
        call(ctx, op, src, dst, locks, M, N, M, N, bm, bn, 0, ready)
        ctx.barrier()
        if op in (0, 1, 2, 3, 8):
            if op == 3 or op == 2 or op in (0, 1, 8):
                assert torch.allclose(dst, total, atol=1e-4), op
        else:                                       # reduce_scatter: contiguous tile blocks, last rank takes the rest
            per = max(tiles // world, 1)
            lo = min(rank * per, tiles)
            hi = tiles if rank == world - 1 else min(lo + per, tiles)
            exp = torch.zeros_like(total)
            for t in range(lo, hi):
                tm, tn = divmod(t, tiles_n)
                exp[tm * bm:(tm + 1) * bm, tn * bn:(tn + 1) * bn] = total[tm * bm:(tm + 1) * bm, tn * bn:(tn + 1) * bn]
            assert torch.allclose(dst, exp, atol=1e-4)
    # all_gather along rows, gather from the next rank, all_to_all of column chunks
    ag = ctx.zeros((world * M, N), dtype=torch.float32)
    locks = ctx.zeros(tiles, dtype=torch.int32)
    ctx.barrier()
    call(ctx, 4, src, ag, locks, M, N, world * M, N, bm, bn, 0, 1)
    ctx.barrier()
    assert torch.equal(ag, torch.cat(parts))
    got = ctx.zeros((M, N), dtype=torch.float32)
    nxt = (rank + 1) % world
    call(ctx, 5, src, got, locks, M, N, M, N, bm, bn, nxt, 1)
    torch.cuda.synchronize()
    assert torch.equal(got, parts[nxt])
    a2a = ctx.zeros((M, N), dtype=torch.float32)
    ctx.barrier()
    n = N // world
    call(ctx, 6, src, a2a, locks, M, N, M, N, bm, bn, n, 1)
    ctx.barrier()
    exp = torch.cat([parts[s][:, rank * n:(rank + 1) * n] for s in range(world)], 1)
    assert torch.equal(a2a, exp)
    ctx.check()
    ctx.barrier()


def test_tile_collectives_between_gpus():
    run_ranks(_tiles, _world(), backend="nccl")


def _graph(rank, world):
    """A tensor-parallel MLP step (all_gather_matmul, matmul_reduce_scatter, all_reduce of a checksum)
    captured ONCE in a CUDA graph and replayed with new inputs: the kernels keep their call counters on
    the device and double-buffer their workspaces by call parity, so a replay needs no host-side state."""
    import torch.distributed as dist

    import iris_b200 as iris

    ctx = iris.iris(2 << 30)
    dt = torch.bfloat16
    M_local, K, F = 256, 512, 768
    torch.manual_seed(70 + rank)
    X = torch.randn(M_local, K, device="cuda", dtype=dt)
    W1 = torch.randn(K, F, device="cuda", dtype=dt) * 0.05
    W2 = torch.randn(F, K, device="cuda", dtype=dt) * 0.05
    H = torch.empty(world * M_local, F, device="cuda", dtype=dt)
    Y = ctx.zeros((M_local, K), dtype=dt)
    S = ctx.zeros((M_local, K), dtype=dt)
    ws1 = ctx.ops.all_gather_matmul(H, X, W1, shard_dim=0)
    ws2 = ctx.ops.matmul_reduce_scatter(Y, H, W2, scatter_rows=True)
    ws3 = ctx.ccl.all_reduce(S, Y)
    assert ws1.variant == "fused" and ws2.variant == "fused"

    def step():
        ctx.ops.all_gather_matmul(H, X, W1, shard_dim=0, workspace=ws1, async_op=True)
        ctx.ops.matmul_reduce_scatter(Y, H, W2, scatter_rows=True, workspace=ws2, async_op=True)
        ctx.ccl.all_reduce(S, Y, workspace=ws3, async_op=True)

    def reference():
        xs = [torch.empty_like(X) for _ in range(world)]
        dist.all_gather(xs, X)
        h = (torch.cat(xs).float() @ W1.float()).to(dt)
        y = h.float() @ W2.float()
        dist.all_reduce(y)                                   # sum over ranks of the partial products
        y_mine = y[rank * M_local:(rank + 1) * M_local].to(dt).float()
        s = y_mine.clone()
        dist.all_reduce(s)
        return y_mine, s

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        step()                                               # an odd number of eager calls before the capture
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):     # other threads (NCCL watchdog) keep running
            step()
        for it in range(4):
            X.copy_(torch.randn(M_local, K, device="cuda", dtype=dt))
            g.replay()
            stream.synchronize()
            y_ref, s_ref = reference()
            tol = 3e-2 * max(1.0, y_ref.abs().max().item())
            assert _maxerr(Y.float(), y_ref) < tol, it
            assert _maxerr(S.float(), s_ref) < world * tol, it
        step()                                               # eager calls still line up after replays
        stream.synchronize()
    ctx.check()
    ctx.barrier()


def test_fused_step_replays_from_a_cuda_graph():
    run_ranks(_graph, _world(), backend="nccl", timeout=600)


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


def test_tensor_parallel_mlp_forward_backward_between_gpus():
    """bf16, 256 rows per rank: the four matrix products of a training step run on the fused kernels."""
    run_ranks(_tp_mlp_check, _world(), args=("bfloat16", 256, 512, 384, 3e-2), backend="nccl", timeout=600)
