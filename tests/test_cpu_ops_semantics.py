"""Layouts and argument checks of the fused ops, on gloo ranks (no GPU).

On the CPU backend every op runs as GEMM + collective, the path that shapes and dtypes outside the
fused kernels' range also take on a GPU; what is checked here is what the op MEANS: which rank
holds which block of the operands and of the result, where the bias goes, what the workspaces and
the module-level forms accept. The reference checks the same layouts against torch.matmul + a
collective in tests/ops/test_all_gather_matmul.py, test_matmul_all_gather.py,
test_matmul_all_reduce.py and test_matmul_reduce_scatter.py (the last one tile by tile because of
its ownership rule).
"""
import pytest
import torch

from helpers import run_ranks


def _gather(t):
    import torch.distributed as dist

    parts = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, t.contiguous())
    return parts


def _ops(rank, world):
    import iris_b200 as iris
    from iris_b200 import ops
    from iris_b200.ops import FusedConfig, FusedWorkspace, owned_tile_range

    ctx = iris.iris(1 << 27)
    g = torch.Generator().manual_seed(100 + rank)
    tol = dict(atol=1e-4, rtol=1e-4)

    # ---- all_gather_matmul, A sharded along K (the reference layout) and along M
    M, Kl, N = 12, 5, 7
    A = torch.randn(M, Kl, generator=g)
    B = torch.randn(Kl * world, N, generator=torch.Generator().manual_seed(1))       # replicated
    bias = torch.randn(M, generator=torch.Generator().manual_seed(2))
    want = torch.cat(_gather(A), dim=1) @ B
    out = ctx.zeros((M, N))
    ws = ctx.ops.all_gather_matmul(out, A, B)
    assert isinstance(ws, FusedWorkspace) and ws.operation == "all_gather_matmul" and ws.variant == "unfused"
    assert torch.allclose(out, want, **tol)
    ctx.ops.all_gather_matmul(out, A, B, bias=bias, workspace=ws)
    assert torch.allclose(out, want + bias[:, None], **tol)                           # the bias is per output ROW
    plain = torch.zeros(M, N)                                                         # the output need not be on the heap
    ops.all_gather_matmul(ctx, plain, A, B)                                           # module-level form: context first
    assert torch.allclose(plain, want, **tol)
    Ml = 4
    Am = torch.randn(Ml, Kl * world, generator=g)
    out_m = ctx.zeros((Ml * world, N))
    ctx.ops.all_gather_matmul(out_m, Am, B, shard_dim=0)
    assert torch.allclose(out_m, torch.cat(_gather(Am), dim=0) @ B, **tol)
    with pytest.raises(ValueError):
        ops._agm_desc(ctx, torch.zeros(M, N + 1), A, B, None, FusedConfig(), 1)
    with pytest.raises(ValueError):
        ops._agm_desc(ctx, torch.zeros(M, N), A, torch.zeros(Kl * world + 1, N), None, FusedConfig(), 1)
    with pytest.raises(ValueError):
        ops._agm_desc(ctx, torch.zeros(Ml * world, N), Am, torch.zeros(Kl * world + 1, N), None, FusedConfig(), 0)

    # ---- matmul_all_gather: row blocks (reference) and column blocks (GEMM + all-scatter)
    Ar = torch.randn(Ml, 9, generator=g)
    Br = torch.randn(9, N, generator=torch.Generator().manual_seed(3))
    rows = ctx.zeros((Ml * world, N))
    ws = ctx.ops.matmul_all_gather(rows, Ar, Br)
    assert ws.operation == "matmul_all_gather"
    assert torch.allclose(rows, torch.cat([a @ Br for a in _gather(Ar)], dim=0), **tol)
    Bc = torch.randn(9, N, generator=g)                                               # this rank's column block of B
    cols = ctx.zeros((Ml, N * world))
    Arep = torch.randn(Ml, 9, generator=torch.Generator().manual_seed(4))             # replicated activations
    ctx.ops.matmul_all_gather(cols, Arep, Bc, scatter_cols=True)
    assert torch.allclose(cols, Arep @ torch.cat(_gather(Bc), dim=1), **tol)
    off_heap = torch.zeros(Ml, N * world)
    ctx.ops.matmul_all_gather(off_heap, Arep, Bc, scatter_cols=True)
    assert torch.allclose(off_heap, cols)
    with pytest.raises(ValueError):
        ctx.ops.matmul_all_gather(ctx.zeros((Ml, N)), Ar, Br)

    # ---- matmul_all_reduce: every rank gets the sum; a bias enters once
    Ap = torch.randn(M, 6, generator=g)
    Bp = torch.randn(6, N, generator=g)
    total = sum(a @ b for a, b in zip(_gather(Ap), _gather(Bp)))
    summed = ctx.zeros((M, N))
    ws = ctx.ops.matmul_all_reduce(summed, Ap, Bp)
    assert torch.allclose(summed, total, **tol)
    ctx.ops.matmul_all_reduce(summed, Ap, Bp, bias=bias, workspace=ws)
    assert torch.allclose(summed, total + bias[:, None], **tol)
    off = torch.zeros(M, N)
    ops.matmul_all_reduce(ctx, off, Ap, Bp)
    assert torch.allclose(off, total, **tol)
    with pytest.raises(ValueError):
        ctx.ops.matmul_all_reduce(ctx.zeros((M + 1, N)), Ap, Bp)

    # ---- matmul_reduce_scatter: row blocks, and the reference's tile ownership
    Mr = 4 * world
    Aq = torch.randn(Mr, 6, generator=g)
    Bq = torch.randn(6, N, generator=g)
    total = sum(a @ b for a, b in zip(_gather(Aq), _gather(Bq)))
    mine = torch.zeros(Mr // world, N)
    ctx.ops.matmul_reduce_scatter(mine, Aq, Bq, scatter_rows=True)
    assert torch.allclose(mine, total[rank * 4:(rank + 1) * 4], **tol)
    # tile layout: output keeps the full shape, only owned 128 x bn tiles are written
    Mt, Nt = 256, 300
    At = torch.randn(Mt, 6, generator=g)
    Bt = torch.randn(6, Nt, generator=g)
    total = sum(a @ b for a, b in zip(_gather(At), _gather(Bt)))
    full = torch.full((Mt, Nt), -7.0)
    ws = ctx.ops.matmul_reduce_scatter(full, At, Bt)
    bn = ws.bn
    tiles_n = -(-Nt // bn)
    owned = owned_tile_range(2 * tiles_n, world, rank)
    mask = torch.zeros(Mt, Nt, dtype=torch.bool)
    for t in owned:
        tm, tn = divmod(t, tiles_n)
        mask[tm * 128:(tm + 1) * 128, tn * bn:(tn + 1) * bn] = True
    assert mask.any() and torch.allclose(full[mask], total[mask], **tol) and torch.all(full[~mask] == -7.0)
    with pytest.raises(ValueError):
        ctx.ops.matmul_reduce_scatter(torch.zeros(Mr, N), Aq, Bq, scatter_rows=True)
    with pytest.raises(ValueError):
        ctx.ops.matmul_reduce_scatter(torch.zeros(Mr // world, N), Aq, Bq)

    # ---- operands the kernels would take on trust are checked first
    for call in (lambda: ctx.ops.matmul_all_reduce(summed, Ap, torch.zeros(7, N)),            # inner dimensions differ
                 lambda: ctx.ops.matmul_all_gather(rows, Ar, torch.zeros(8, N)),
                 lambda: ctx.ops.matmul_reduce_scatter(mine, Aq, torch.zeros(5, N), scatter_rows=True),
                 lambda: ctx.ops.all_gather_matmul(out, A, torch.zeros(Kl * world + 1, N)),
                 lambda: ctx.ops.all_gather_matmul(out, A, B, shard_dim=2),
                 lambda: ctx.ops.matmul_all_reduce(summed, Ap, Bp, bias=torch.zeros(M + 1)),      # one bias entry per output row
                 lambda: ctx.ops.all_gather_matmul(out_m, Am, B, shard_dim=0, bias=torch.zeros(Ml)),
                 lambda: ctx.ops.matmul_all_reduce(summed, Ap[0], Bp)):                           # a vector is not a matrix
        with pytest.raises(ValueError):
            call()
    with pytest.raises(TypeError):
        ctx.ops.matmul_all_reduce(summed, Ap, Bp.double())
    if world > 1:
        with pytest.raises(ValueError, match="do not split"):
            ctx.ops.matmul_reduce_scatter(torch.zeros(1, N), torch.zeros(world + 1, 6), Bq, scatter_rows=True)

    # ---- repeated calls, with or without the returned workspace, leave the heap where it is
    def one_round():
        ctx.ops.all_gather_matmul(out, A, B)
        ctx.ops.all_gather_matmul(out_m, Am, B, shard_dim=0)
        ctx.ops.matmul_all_gather(rows, Ar, Br)
        ctx.ops.matmul_all_gather(off_heap, Arep, Bc, scatter_cols=True)
        ctx.ops.matmul_all_reduce(off, Ap, Bp)
        ctx.ops.matmul_reduce_scatter(mine, Aq, Bq, scatter_rows=True)
        ctx.ops.matmul_reduce_scatter(full, At, Bt)

    one_round()
    level = ctx.heap_mark()
    for _ in range(3):
        one_round()
    assert ctx.heap_mark() == level
    assert torch.allclose(off, sum(a @ b for a, b in zip(_gather(Ap), _gather(Bp))), **tol)       # and still compute the same thing

    # ---- preambles return reusable workspaces; config is validated
    for fn, args in ((ops.all_gather_matmul_preamble, (ctx, A, B)), (ops.matmul_all_gather_preamble, (ctx, Ar, Br)),
                     (ops.matmul_all_reduce_preamble, (ctx, summed, Ap, Bp)), (ops.matmul_reduce_scatter_preamble, (ctx, mine, Aq, Bq))):
        w = fn(*args)
        assert isinstance(w, FusedWorkspace) and w.prepared and w.world_size == world
    cfg = FusedConfig()
    # the reference's field names are kept; the tile defaults are the tcgen05 ones (128 rows, width chosen per problem)
    for name in ("block_size_m", "block_size_n", "block_size_k", "group_size_m", "num_sms", "num_xcds", "chunk_size",
                 "all_reduce_variant", "all_reduce_num_rings"):
        assert hasattr(cfg, name), name
    assert cfg.block_size_m == 128 and cfg.tile_n() == 0 and cfg.all_reduce_variant == "auto"
    assert FusedConfig(block_size_n=224).tile_n() == 224 and FusedConfig(block_size_n=64).tile_n() == 0
    cfg.validate(world)
    with pytest.raises(ValueError):
        FusedConfig(all_reduce_variant="tree")
    with pytest.raises(ValueError):
        FusedConfig(block_size_m=0)
    ctx.barrier()


def test_fused_op_layouts_world2():
    run_ranks(_ops, 2)


def test_fused_op_layouts_world3():
    run_ranks(_ops, 3)


def test_owned_tile_range_partitions_the_tiles():
    from iris_b200.ops import owned_tile_range

    for tiles in (1, 2, 7, 8, 64, 65):
        for world in (1, 2, 3, 8):
            got = [t for r in range(world) for t in owned_tile_range(tiles, world, r)]
            assert sorted(got) == list(range(tiles)) or tiles < world
            if tiles >= world:
                assert got == list(range(tiles))                      # contiguous blocks in rank order
                sizes = [len(owned_tile_range(tiles, world, r)) for r in range(world)]
                assert sizes[:-1] == [tiles // world] * (world - 1) and sizes[-1] == tiles - (world - 1) * (tiles // world)


def _fp8_ops(rank, world):
    """Block-scaled e4m3 operands through the four fused ops (dequantised on the CPU backend): each op
    means what its 16-bit form means on the dequantised matrices."""
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.ops import BlockScaled, pack_scales_a, pack_scales_b, quantize_activation, quantize_weight

    if not hasattr(torch, "float8_e4m3fn"):
        return
    ctx = iris.iris(1 << 27)
    g = torch.Generator().manual_seed(7 + rank)
    M, K, N = 32, 256, 24
    x = quantize_activation(torch.randn(M, K, generator=g) * 3)
    w = quantize_weight(torch.randn(N, K, generator=g) * 0.1)            # [N, K], used as the [K, N] matrix
    assert x.shape == (M, K) and w.shape == (K, N) and x.kind == "activation" and w.kind == "weight"
    assert torch.all(torch.log2(x.scale) == torch.round(torch.log2(x.scale)))                  # powers of two
    assert x.sf().shape == (1, 2, 512) and w.sf(224).shape == (1, 2, 2, 512) and w.sf(128).shape == (1, 2, 1, 512)
    # the atom layout: row r of a 128-row tile at byte (r % 32) * 16 + (r // 32) * 4, four equal bytes per block
    e = (torch.log2(x.scale) + 127).to(torch.uint8)
    for r, kb in ((0, 0), (17, 1), (31, 0)):
        off = (r % 32) * 16 + (r // 32) * 4
        assert torch.all(x.sf()[0, kb, off:off + 4] == e[r, kb])
    xd, wd = x.dequantize(), w.dequantize()
    tol = dict(atol=2e-2, rtol=2e-2)
    parts_x = [torch.empty_like(xd) for _ in range(world)]
    dist.all_gather(parts_x, xd)
    # all_gather_matmul, rows sharded: every rank multiplies the gathered activations by ITS weight
    out = ctx.zeros((M * world, N), dtype=torch.bfloat16)
    ws = ctx.ops.all_gather_matmul(out, x, w, shard_dim=0)
    assert ws.variant == "unfused"
    assert torch.allclose(out.float(), torch.cat(parts_x, 0) @ wd, **tol)
    # matmul_all_reduce / matmul_reduce_scatter: sum over ranks of the local products
    local = xd @ wd
    total = local.clone()
    dist.all_reduce(total)
    out2 = ctx.zeros((M, N), dtype=torch.bfloat16)
    ctx.ops.matmul_all_reduce(out2, x, w)
    assert torch.allclose(out2.float(), total, atol=0.2, rtol=3e-2)
    out3 = ctx.zeros((M // world, N), dtype=torch.bfloat16)
    ctx.ops.matmul_reduce_scatter(out3, x, w, scatter_rows=True)
    assert torch.allclose(out3.float(), total[rank * (M // world):(rank + 1) * (M // world)], atol=0.2, rtol=3e-2)
    # matmul_all_gather: every rank's product, stacked by rank
    out4 = ctx.zeros((M * world, N), dtype=torch.bfloat16)
    ctx.ops.matmul_all_gather(out4, x, w)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local)
    assert torch.allclose(out4.float(), torch.cat(parts, 0), **tol)
    with pytest.raises((TypeError, ValueError)):
        BlockScaled(x.q, x.scale[:, :1], "activation")


def test_fp8_block_scaled_operands_through_the_fused_ops():
    run_ranks(_fp8_ops, 2)
