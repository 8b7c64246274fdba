"""The parallelism package on gloo ranks (no GPU): layouts, tensor-parallel linears, gradient
buckets, sequence sharding and the Ulysses exchange, expert-parallel tables.

Oracles are plain PyTorch on the gathered, unsharded problem. The reference tests the same
strategies only through its collectives on hand-built groups (tests/ccl/test_process_groups.py) and
its MoE example's tables against its own torch reference (tests/examples/test_expert_sharded_moe.py).
"""
import pytest
import torch

from helpers import run_ranks


# ----------------------------------------------------------------------------- layout (pure arithmetic)
def test_layout_arithmetic():
    from iris_b200.parallel import ParallelLayout

    L = ParallelLayout({"tp": 2, "cp": 2, "dp": 2}, world_size=8, rank=5)
    assert L.coords() == {"tp": 1, "cp": 0, "dp": 1}
    assert L.ranks("tp") == [4, 5] and L.ranks("cp") == [5, 7] and L.ranks("dp") == [1, 5]
    assert L.stride("tp") == 1 and L.stride("cp") == 2 and L.stride("dp") == 4
    assert L.rank_of(tp=0) == 4 and L.rank_of(cp=1, dp=0) == 3
    for name in ("tp", "cp", "dp"):
        groups = L.all_groups(name)
        assert sorted(r for g in groups for r in g) == list(range(8))       # a partition
        for g in groups:                                                    # evenly strided, as kernels require
            assert all(b - a == L.stride(name) for a, b in zip(g, g[1:]))
        for r in range(8):
            assert r in L.ranks(name, r) and L.ranks(name, r)[L.coord(name, r)] == r
    for r in range(8):
        assert L.rank_of(**L.coords(r)) == r
    with pytest.raises(ValueError):
        ParallelLayout({"tp": 3}, world_size=8, rank=0)
    with pytest.raises(ValueError):
        ParallelLayout({"tp": 0, "dp": 8}, world_size=8, rank=0)
    with pytest.raises(KeyError):
        L.ranks("pp")
    with pytest.raises(ValueError):
        L.rank_of(tp=2)
    with pytest.raises(RuntimeError):
        L.group("tp")                                                        # not built yet
    assert ParallelLayout({"tp": 8}, world_size=8, rank=0).group("tp") is None   # the whole job: default group


def _layout_groups(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.parallel import ParallelLayout

    ctx = iris.iris(1 << 24)
    L = ParallelLayout({"tp": 2, "dp": 2}).build_groups()
    assert L.world_size == world and L.rank == rank
    for name in ("tp", "dp"):
        g = L.group(name)
        assert dist.get_process_group_ranks(g) == L.ranks(name)
        inp = ctx.full((4, 8), float(rank + 1))
        out = ctx.zeros((4, 8))
        ctx.ccl.all_reduce(out, inp, group=g)
        assert torch.all(out == sum(r + 1 for r in L.ranks(name))), name
    ctx.barrier()


def test_layout_groups_drive_collectives_world4():
    run_ranks(_layout_groups, 4)


# ----------------------------------------------------------------------------- tensor parallel
def _tp_linears(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.parallel import ColumnParallelLinear, RowParallelLinear

    ctx = iris.iris(1 << 26)
    dt = torch.float32
    Ml, K, F = 6, 16, 8            # rows per rank, hidden, ffn per rank
    M = Ml * world
    g = torch.Generator().manual_seed(7)
    X = torch.randn(M, K, generator=g)
    W1 = torch.randn(K, F * world, generator=g) * 0.3
    b1 = torch.randn(F * world, generator=g)
    W2 = torch.randn(F * world, K, generator=g) * 0.3
    b2 = torch.randn(K, generator=g)
    w1_r, b1_r = W1[:, rank * F:(rank + 1) * F], b1[rank * F:(rank + 1) * F]
    w2_r = W2[rank * F:(rank + 1) * F]
    x_r = X[rank * Ml:(rank + 1) * Ml].contiguous()
    H = X @ W1 + b1
    Y = H @ W2 + b2

    # sequence-parallel pair: rows in, rows out
    col = ColumnParallelLinear(ctx, K, F, sequence_parallel=True, dtype=dt, weight=w1_r, bias_value=b1_r)
    row = RowParallelLinear(ctx, F, K, sequence_parallel=True, dtype=dt, weight=w2_r, bias_value=b2)
    h = col(x_r)
    assert h.shape == (M, F) and torch.allclose(h, H[:, rank * F:(rank + 1) * F], atol=1e-4)
    y = row(h)
    assert y.shape == (Ml, K) and torch.allclose(y, Y[rank * Ml:(rank + 1) * Ml], atol=1e-3)
    # a second call reuses workspaces and buffers: same answer, same storage
    p = y.data_ptr()
    y2 = row(col(x_r))
    assert y2.data_ptr() == p and torch.allclose(y2, Y[rank * Ml:(rank + 1) * Ml], atol=1e-3)

    # replicated activations: local GEMM, then all-reduce
    col2 = ColumnParallelLinear(ctx, K, F, sequence_parallel=False, dtype=dt, weight=w1_r, bias_value=b1_r)
    row2 = RowParallelLinear(ctx, F, K, sequence_parallel=False, dtype=dt, weight=w2_r, bias_value=b2)
    h2 = col2(X)
    assert torch.allclose(h2, H[:, rank * F:(rank + 1) * F], atol=1e-4)
    y3 = row2(h2)
    assert y3.shape == (M, K) and torch.allclose(y3, Y, atol=1e-3)

    # gathered outputs, from both input forms
    for sp, inp in ((False, X), (True, x_r)):
        colg = ColumnParallelLinear(ctx, K, F, sequence_parallel=sp, gather_output=True, dtype=dt, weight=w1_r, bias_value=b1_r)
        hg = colg(inp)
        assert hg.shape == (M, F * world) and torch.allclose(hg, H, atol=1e-4), sp
    nob = ColumnParallelLinear(ctx, K, F, sequence_parallel=False, gather_output=True, dtype=dt, weight=w1_r)
    assert torch.allclose(nob(X), X @ W1, atol=1e-4)

    # random init is reproducible from the seed and differs between seeds
    a = ColumnParallelLinear(ctx, K, F, dtype=dt, seed=3)
    b = ColumnParallelLinear(ctx, K, F, dtype=dt, seed=3)
    c = ColumnParallelLinear(ctx, K, F, dtype=dt, seed=4)
    assert torch.equal(a.weight, b.weight) and not torch.equal(a.weight, c.weight) and a.bias is None
    with pytest.raises(ValueError):
        col(torch.zeros(Ml, K + 1))
    with pytest.raises(TypeError):
        col(torch.zeros(Ml, K, dtype=torch.float64))
    with pytest.raises(ValueError):
        ColumnParallelLinear(ctx, K, F, dtype=dt, weight=torch.zeros(K, F + 1))
    if world > 1:
        with pytest.raises(ValueError):
            row(torch.zeros(M + 1, F))
    dist.barrier()
    ctx.barrier()


def test_tensor_parallel_linears_world2():
    run_ranks(_tp_linears, 2)


def test_tensor_parallel_linears_world3():
    run_ranks(_tp_linears, 3)


# ----------------------------------------------------------------------------- data parallel
def _dp(rank, world, use_hooks, with_groups):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.parallel import GradientBuckets, ParallelLayout

    ctx = iris.iris(1 << 26)
    group, members = None, list(range(world))
    if with_groups:
        L = ParallelLayout({"tp": 2, "dp": world // 2}).build_groups()
        group, members = L.group("dp"), L.ranks("dp")
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(12, 40), torch.nn.Tanh(), torch.nn.Linear(40, 9), torch.nn.Tanh(),
                                torch.nn.Linear(9, 3))
    frozen = torch.nn.Linear(3, 3)
    for p in frozen.parameters():
        p.requires_grad_(False)
    unused = torch.nn.Parameter(torch.ones(5))
    params = list(model.parameters()) + list(frozen.parameters()) + [unused]
    # tiny buckets so that several exist; the unused parameter rides along as zeros
    buckets = GradientBuckets(ctx, params, bucket_bytes=1024, group=group)
    assert len(buckets.buckets) >= 3 and buckets.nbytes() > 0
    assert sum(len(b.params) for b in buckets.buckets) == len([p for p in params if p.requires_grad])
    if use_hooks:
        buckets.attach()

    def batch(r, step):
        g = torch.Generator().manual_seed(100 * step + r)
        return torch.randn(8, 12, generator=g), torch.randn(8, 3, generator=g)

    for step in range(3):
        for p in params:
            p.grad = None
        x, t = batch(rank, step)
        loss = ((frozen(model(x)) - t) ** 2).mean()
        loss.backward()
        if use_hooks:
            buckets.finish()
        else:
            buckets.all_reduce()
        # oracle: the same model on every member's batch, gradients averaged
        want = None
        for r in members:
            ref = [p.detach().clone().requires_grad_(True) for p in model.parameters()]
            xr, tr = batch(r, step)
            h = xr
            for i in range(0, len(ref), 2):
                h = h @ ref[i].t() + ref[i + 1]
                if i + 2 < len(ref):
                    h = torch.tanh(h)
            ((frozen(h) - tr) ** 2).mean().backward()
            grads = [p.grad for p in ref]
            want = grads if want is None else [a + b for a, b in zip(want, grads)]
        for p, w in zip(model.parameters(), want):
            assert torch.allclose(p.grad, w / len(members), atol=1e-6), step
        assert torch.all(unused.grad == 0)
        with torch.no_grad():
            for p in model.parameters():
                p -= 0.1 * p.grad
    # replicas stayed identical inside the group
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    parts = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(parts, flat)
    for r in members:
        assert torch.equal(parts[r], flat)
    buckets.detach()
    sums = GradientBuckets(ctx, list(model.parameters()), group=group, average=False)
    for p in model.parameters():
        p.grad = torch.full_like(p, float(rank + 1))
    sums.all_reduce()
    for p in model.parameters():
        assert torch.all(p.grad == sum(r + 1 for r in members))
    with pytest.raises(ValueError):
        GradientBuckets(ctx, list(frozen.parameters()))
    ctx.barrier()


def test_gradient_buckets_world2():
    run_ranks(_dp, 2, args=(False, False))


def test_gradient_buckets_with_hooks_world3():
    run_ranks(_dp, 3, args=(True, False))


def test_gradient_buckets_inside_strided_groups_world4():
    run_ranks(_dp, 4, args=(True, True))


# ----------------------------------------------------------------------------- sequence parallel
def test_sequence_sharding_round_trip():
    from iris_b200.parallel import sequence_positions, shard_sequence, unshard_sequence

    x = torch.arange(48 * 3).view(48, 3)
    for world in (1, 2, 3, 4):
        for layout in ("contiguous", "zigzag"):
            pieces = [shard_sequence(x, r, world, layout) for r in range(world)]
            assert all(p.shape == (48 // world, 3) and p.is_contiguous() for p in pieces)
            assert torch.equal(unshard_sequence(pieces, layout), x)
            pos = torch.cat([sequence_positions(r, world, 48 // world, layout) for r in range(world)])
            assert sorted(pos.tolist()) == list(range(48))
            for r in range(world):
                assert torch.equal(pieces[r][:, 0], 3 * sequence_positions(r, world, 48 // world, layout))
    # the zigzag layout gives every rank the same number of (query, key) pairs under a causal mask
    S, W = 64, 4
    work = [int((sequence_positions(r, W, S // W, "zigzag") + 1).sum()) for r in range(W)]
    assert len(set(work)) == 1
    work_c = [int((sequence_positions(r, W, S // W, "contiguous") + 1).sum()) for r in range(W)]
    assert work_c[-1] > 3 * work_c[0]
    y = torch.arange(2 * 12 * 5).view(2, 12, 5)
    assert torch.equal(unshard_sequence([shard_sequence(y, r, 3, "zigzag", dim=1) for r in range(3)], "zigzag", dim=1), y)
    with pytest.raises(ValueError):
        shard_sequence(x, 0, 5)
    with pytest.raises(ValueError):
        shard_sequence(torch.zeros(6, 2), 0, 2, "zigzag")
    with pytest.raises(ValueError):
        sequence_positions(0, 2, 4, "spiral")
    with pytest.raises(TypeError):
        unshard_sequence(x)


def _ulysses(rank, world):
    import iris_b200 as iris
    from iris_b200.models import reference_attention
    from iris_b200.parallel import UlyssesExchange, shard_sequence

    ctx = iris.iris(1 << 26)
    S, H, D = 8 * world, 2 * world, 4
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(S, H, D, generator=g) for _ in range(3))
    ex = UlyssesExchange(ctx)
    mine = [shard_sequence(t, rank, world) for t in (q, k, v)]
    heads = [ex.to_heads(t).clone() for t in mine]
    Hl = H // world
    for full, got in zip((q, k, v), heads):
        assert got.shape == (S, Hl, D) and torch.equal(got, full[:, rank * Hl:(rank + 1) * Hl])
    # attention on full sequences of my heads, then back to my tokens for all heads
    o_heads = reference_attention(*heads, causal=True).to(q.dtype)
    o_mine = ex.to_sequence(o_heads)
    want = reference_attention(q, k, v, causal=True).to(q.dtype)
    assert o_mine.shape == (S // world, H, D)
    assert torch.allclose(o_mine, want[rank * (S // world):(rank + 1) * (S // world)], atol=1e-5)
    # the round trip is the identity, repeatedly (staging buffers are reused)
    for _ in range(2):
        assert torch.equal(ex.to_sequence(ex.to_heads(mine[0])), mine[0])
    with pytest.raises(ValueError):
        ex.to_heads(torch.zeros(4, H + 1, D))
    with pytest.raises(ValueError):
        ex.to_sequence(torch.zeros(S + 1, Hl, D))
    ctx.barrier()


def test_ulysses_exchange_world2():
    run_ranks(_ulysses, 2)


def test_ulysses_exchange_world4():
    run_ranks(_ulysses, 4)


# ----------------------------------------------------------------------------- expert parallel
def test_expert_assignment_tables():
    from iris_b200.parallel import expert_assignment, uniform_expert_dict

    for W, E in ((2, 8), (4, 64), (3, 96), (8, 256), (2, 40)):
        a = expert_assignment(W, E)
        assert a.expt_bitmask.shape == (W, (E + 31) // 32) and a.expt_bitmask.dtype == torch.int32
        assert a.expt_boolmask.shape == (W, E) and a.expt_map.shape == (W, E) and a.expt_map.dtype == torch.int32
        assert a.n_expts_per_shard == [E // W] * W
        for e in range(E):
            owner = e // (E // W)
            assert a.owner_of(e) == owner
            for s in range(W):
                bit = (int(a.expt_bitmask[s, e >> 5]) >> (e & 31)) & 1
                assert bit == int(s == owner) == int(a.expt_boolmask[s, e])
                assert int(a.expt_map[s, e]) == (e - owner * (E // W) if s == owner else -1)
    # an arbitrary ownership: local ids follow increasing global id
    a = expert_assignment(2, 6, {0: [5, 0, 3], 1: [1, 2, 4]})
    assert a.expt_map.tolist() == [[0, -1, -1, 1, -1, 2], [-1, 0, 1, -1, 2, -1]]
    assert a.expt_bitmask.tolist() == [[0b101001], [0b010110]]
    assert uniform_expert_dict(2, 4) == {0: [0, 1], 1: [2, 3]}
    for bad in ({0: [0, 1], 1: [1, 2]}, {0: [0, 1, 2]}, {0: [0, 1, 2], 1: []}, {0: [0, 1], 2: [2]}, {0: [0, 1], 1: [2, 3]}):
        with pytest.raises(ValueError):
            expert_assignment(2, 3, bad)
    with pytest.raises(ValueError):
        uniform_expert_dict(3, 8)


def test_dispatch_tables_and_ragged_slices():
    from iris_b200.parallel import dispatch_tables, expert_assignment, ragged_slices, topk_routing

    torch.manual_seed(5)
    T, E, k, W = 37, 8, 3, 2
    logits = torch.randn(T, E)
    res = topk_routing(logits, k)
    assert res.indx.dtype == torch.int16 and res.vals.shape == (T, k)
    assert torch.allclose(res.vals.sum(-1), torch.ones(T), atol=1e-6)
    tv, ti = torch.topk(logits, k, dim=1)
    assert torch.equal(res.indx.long(), ti) and torch.allclose(res.vals, torch.softmax(tv, -1))
    raw = topk_routing(logits, k, apply_softmax=False)
    assert torch.equal(raw.vals, tv)
    md = res.mask_metadata
    flat = ti.reshape(-1)
    assert md.col_sum.tolist() == [int((flat == e).sum()) for e in range(E)] and int(md.col_sum.sum()) == T * k
    # expert-sorted order: experts ascend, slots of one expert keep their original order
    experts_sorted = flat[md.col_sorted_indx.long()]
    assert torch.all(experts_sorted[1:] >= experts_sorted[:-1])
    for e in range(E):
        slots = md.col_sorted_indx[experts_sorted == e]
        assert torch.all(slots[1:] > slots[:-1])
    # the two tables are inverse permutations
    assert torch.equal(md.row_sorted_indx[md.col_sorted_indx.long()].long(), torch.arange(T * k))
    assert torch.equal(md.col_sorted_indx[md.row_sorted_indx.long()].long(), torch.arange(T * k))
    # invalid slots drop out
    idx = ti.clone()
    idx[::5, 0] = -1
    md2 = dispatch_tables(idx, E)
    n_valid = int((idx >= 0).sum())
    assert int(md2.col_sum.sum()) == n_valid
    assert torch.all(md2.col_sorted_indx[n_valid:] == -1) and torch.all(md2.col_sorted_indx[:n_valid] >= 0)
    assert torch.all(md2.row_sorted_indx[(idx.reshape(-1) < 0)] == -1)
    assert sorted(md2.row_sorted_indx[idx.reshape(-1) >= 0].tolist()) == list(range(n_valid))
    # ragged view: global, then per rank with global offsets
    glob = ragged_slices(md.col_sum)
    assert glob.n_slices == E and glob.slice_offs[0] == 0 and int(glob.slice_offs[-1]) == T * k
    assert torch.equal(glob.slice_offs[1:] - glob.slice_offs[:-1], glob.slice_sizes)
    a = expert_assignment(W, E)
    covered = 0
    for r in range(W):
        loc = ragged_slices(md.col_sum, a.expt_map[r])
        mine = [e for e in range(E) if a.expt_boolmask[r, e]]
        assert loc.n_slices == len(mine) and loc.slice_sizes.tolist() == [int(md.col_sum[e]) for e in mine]
        assert loc.slice_offs[:-1].tolist() == [int(glob.slice_offs[e]) for e in mine]
        assert int(loc.slice_offs[-1]) == int(glob.slice_offs[mine[-1] + 1])
        covered += int(loc.slice_sizes.sum())
    assert covered == T * k
    odd = expert_assignment(2, 6, {0: [5, 0, 3], 1: [1, 2, 4]})
    cs = torch.tensor([4, 1, 0, 2, 7, 3], dtype=torch.int32)
    loc = ragged_slices(cs, odd.expt_map[0])
    assert loc.slice_sizes.tolist() == [4, 2, 3] and loc.slice_offs.tolist() == [0, 5, 14, 17]
    assert ragged_slices(cs, torch.full((6,), -1, dtype=torch.int32)).n_slices == 0


# ----------------------------------------------------------------------------- point to point
def _p2p(rank, world):
    import iris_b200 as iris
    from iris_b200.parallel import P2PChannel

    ctx = iris.iris(1 << 24)
    ch = P2PChannel(ctx, (4, 3), dtype=torch.float32, depth=2, timeout_ms=3000)
    nxt, prv = (rank + 1) % world, (rank - 1) % world

    def msg(src, n):
        return torch.full((4, 3), 100.0 * src + n)

    # a pipeline: every rank sends five messages to its successor and takes five from its predecessor;
    # with two slots the sender has to wait for acknowledgements, and messages arrive in order
    for n in range(1, 6):
        assert ch.send(msg(rank, n), nxt) == n
        got = ch.recv(prv)
        assert torch.equal(got, msg(prv, n)), (n, got[0, 0])
    # receive into a buffer of the caller; availability can be asked without waiting
    ch.send(msg(rank, 6), nxt)
    ctx.barrier()
    assert ch.pending(prv)
    buf = torch.empty(4, 3)
    assert ch.recv(prv, out=buf) is buf and torch.equal(buf, msg(prv, 6))
    assert not ch.pending(prv)
    ctx.barrier()
    # nobody sends: the wait is bounded
    quick = P2PChannel(ctx, (2,), depth=1, timeout_ms=200)
    with pytest.raises(TimeoutError, match="has not reached"):
        quick.recv(prv)
    ctx.barrier()
    # one slot and a receiver that does not take the message: the second send gives up, the first stays intact
    quick.send(torch.tensor([1.0, 2.0]), nxt)
    with pytest.raises(TimeoutError, match="has not taken"):
        quick.send(torch.tensor([3.0, 4.0]), nxt)
    ctx.barrier()
    assert torch.equal(quick.recv(prv), torch.tensor([1.0, 2.0]))
    ctx.barrier()
    quick.send(torch.tensor([3.0, 4.0]), nxt)                    # acknowledged now: goes through
    assert torch.equal(quick.recv(prv), torch.tensor([3.0, 4.0]))
    for bad in (lambda: ch.send(torch.zeros(4, 4), nxt), lambda: ch.send(torch.zeros(4, 3, dtype=torch.float64), nxt),
                lambda: ch.send(msg(0, 0), rank), lambda: ch.recv(rank), lambda: ch.recv(world)):
        with pytest.raises(ValueError):
            bad()
    with pytest.raises(ValueError):
        P2PChannel(ctx, (1,), depth=0)
    ctx.check()
    ctx.barrier()


def test_point_to_point_channel_world2():
    run_ranks(_p2p, 2)


def test_point_to_point_channel_world3():
    run_ranks(_p2p, 3)
