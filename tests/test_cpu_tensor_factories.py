"""torch parity of the heap's tensor factories over dtypes, shapes and options (gloo, no GPU).

The reference keeps one file per factory (tests/unittests/test_zeros.py, test_ones.py, test_full.py,
test_empty.py, test_zeros_like.py, test_rand.py, test_randn.py, test_randint.py, test_arange.py,
test_linspace.py): shape / dtype / ``out=`` / device errors / memory_format parity with torch and
heap membership of every result. Here one rank walks the same table; a second scenario checks that
two ranks that allocate in the same order get the same offsets.
"""
import itertools

import pytest
import torch

from helpers import run_ranks

FLOATS = [torch.float16, torch.bfloat16, torch.float32, torch.float64]
INTS = [torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64]
SHAPES = [(1,), (7,), (3, 5), (2, 3, 4), (2, 3, 4, 5), (0,), (4, 0, 2), ()]


def _same_meta(a, b):
    assert a.shape == b.shape, (a.shape, b.shape)
    assert a.dtype == b.dtype, (a.dtype, b.dtype)
    assert a.stride() == b.stride() or a.numel() == 0, (a.stride(), b.stride())
    assert a.layout == b.layout


def _parity(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 27)
    on_heap = ctx.is_symmetric

    # ---- zeros / ones / full / empty: value, metadata, heap membership, the three size spellings
    for dt, shape in itertools.product(FLOATS + INTS + [torch.bool], SHAPES):
        for name, ref in (("zeros", torch.zeros), ("ones", torch.ones)):
            got = getattr(ctx, name)(shape, dtype=dt)
            want = ref(shape, dtype=dt)
            _same_meta(got, want)
            assert torch.equal(got, want) and on_heap(got), (name, dt, shape)
            if len(shape) > 0:
                assert torch.equal(getattr(ctx, name)(*shape, dtype=dt), want)
                assert torch.equal(getattr(ctx, name)(list(shape), dtype=dt), want)
        e = ctx.empty(shape, dtype=dt)
        _same_meta(e, torch.empty(shape, dtype=dt))
        assert on_heap(e)
        fv = True if dt == torch.bool else 3
        f = ctx.full(shape, fv, dtype=dt)
        _same_meta(f, torch.full(shape, fv, dtype=dt))
        assert torch.equal(f, torch.full(shape, fv, dtype=dt)) and on_heap(f)
    # default dtypes follow torch
    assert ctx.zeros(3).dtype == torch.get_default_dtype()
    assert ctx.full((2,), 1.5).dtype == torch.full((2,), 1.5).dtype
    assert ctx.full((2,), 7).dtype == torch.full((2,), 7).dtype
    assert ctx.full((2,), True).dtype == torch.full((2,), True).dtype
    torch.set_default_dtype(torch.float64)
    try:
        assert ctx.zeros(3).dtype == torch.float64 and ctx.rand(3).dtype == torch.float64
        assert ctx.arange(0.0, 1.0, 0.5).dtype == torch.float64 and ctx.linspace(0, 1, 3).dtype == torch.float64
    finally:
        torch.set_default_dtype(torch.float32)

    # ---- zeros_like: dtype / shape inheritance, overrides, formats; input may live anywhere
    for dt, shape in itertools.product([torch.float16, torch.float32, torch.int32], SHAPES):
        src = torch.ones(shape, dtype=dt)
        zl = ctx.zeros_like(src)
        _same_meta(zl, torch.zeros_like(src))
        assert torch.equal(zl, torch.zeros_like(src)) and on_heap(zl)
        assert ctx.zeros_like(src, dtype=torch.float64).dtype == torch.float64
    heap_src = ctx.ones(2, 3)
    assert on_heap(ctx.zeros_like(heap_src)) and ctx.zeros_like(heap_src).data_ptr() != heap_src.data_ptr()
    cl_src = torch.ones(2, 3, 4, 5).to(memory_format=torch.channels_last)
    assert ctx.zeros_like(cl_src).stride() == torch.zeros_like(cl_src).stride()
    assert ctx.zeros_like(cl_src, memory_format=torch.contiguous_format).is_contiguous()
    assert ctx.zeros_like(torch.ones(2, 2), requires_grad=True).requires_grad

    # ---- memory formats
    for name in ("zeros", "ones", "empty", "rand", "randn"):
        t4 = getattr(ctx, name)(2, 3, 4, 5, memory_format=torch.channels_last)
        assert t4.stride() == torch.empty(2, 3, 4, 5).to(memory_format=torch.channels_last).stride(), name
        assert t4.is_contiguous(memory_format=torch.channels_last) and on_heap(t4)
        t5 = getattr(ctx, name)(2, 3, 4, 5, 6, memory_format=torch.channels_last_3d)
        assert t5.stride() == torch.empty(2, 3, 4, 5, 6).to(memory_format=torch.channels_last_3d).stride(), name
        assert on_heap(t5)
        # a format that does not fit the rank of the tensor is ignored
        assert getattr(ctx, name)(2, 3, memory_format=torch.channels_last).is_contiguous()
    ones_cl = ctx.ones(2, 3, 4, 5, memory_format=torch.channels_last)
    assert torch.equal(ones_cl, torch.ones(2, 3, 4, 5))

    # ---- random factories: ranges, dtypes, generators
    for dt in FLOATS:
        r = ctx.rand(64, 8, dtype=dt)
        assert r.dtype == dt and r.shape == (64, 8) and float(r.min()) >= 0 and float(r.max()) <= 1 and on_heap(r)
        n = ctx.randn(64, 8, dtype=dt)
        assert n.dtype == dt and torch.isfinite(n.float()).all() and on_heap(n)
    big = ctx.randn(20000)
    assert abs(float(big.mean())) < 0.05 and abs(float(big.std()) - 1) < 0.05
    g1, g2 = torch.Generator().manual_seed(1234), torch.Generator().manual_seed(1234)
    assert torch.equal(ctx.rand(33, generator=g1), ctx.rand(33, generator=g2))
    g1, g2 = torch.Generator().manual_seed(5), torch.Generator().manual_seed(5)
    assert torch.equal(ctx.randn(33, generator=g1), ctx.randn(33, generator=g2))
    g1, g2 = torch.Generator().manual_seed(9), torch.Generator().manual_seed(9)
    assert torch.equal(ctx.randint(0, 100, (33,), generator=g1), ctx.randint(0, 100, (33,), generator=g2))
    for dt in INTS:
        ri = ctx.randint(2, 9, (200,), dtype=dt)
        assert ri.dtype == dt and int(ri.min()) >= 2 and int(ri.max()) < 9 and on_heap(ri)
    assert ctx.randint(5, (3, 4)).shape == (3, 4) and int(ctx.randint(5, (100,)).max()) < 5
    assert ctx.randint(-4, 0, (100,)).max() < 0
    u = ctx.uniform((500,), 2.0, 3.0)
    assert u.dtype == torch.float32 and float(u.min()) >= 2 and float(u.max()) <= 3 and on_heap(u)
    assert ctx.uniform((4,), dtype=torch.float64).dtype == torch.float64

    # ---- arange / linspace
    for args in ((5,), (2, 9), (1, 10, 3), (10, 1, -2), (0.0, 1.0, 0.125), (-3, 3), (0, 7, 2)):
        got, want = ctx.arange(*args), torch.arange(*args)
        _same_meta(got, want)
        assert torch.equal(got, want) and on_heap(got), args
    for dt in FLOATS + [torch.int32, torch.int64]:
        got, want = ctx.arange(0, 20, 2, dtype=dt), torch.arange(0, 20, 2, dtype=dt)
        assert got.dtype == dt and torch.equal(got, want), dt
    for bad in ((5, 5), (5, 1), (1, 5, -1)):
        with pytest.raises(ValueError):
            ctx.arange(*bad)
    with pytest.raises(ValueError):
        ctx.arange(0, 5, 0)
    for start, end, steps in ((0, 1, 5), (-1, 1, 11), (3, 3, 4), (0, 10, 1), (5, -5, 6), (0, 1, 0)):
        got, want = ctx.linspace(start, end, steps), torch.linspace(start, end, steps)
        _same_meta(got, want)
        assert torch.allclose(got, want) and on_heap(got), (start, end, steps)
    for dt in FLOATS:
        tol = 1e-2 if dt in (torch.float16, torch.bfloat16) else 1e-6
        assert torch.allclose(ctx.linspace(0, 1, 9, dtype=dt).float(), torch.linspace(0, 1, 9).float(), atol=tol)
    assert torch.equal(ctx.linspace(0, 8, 5, dtype=torch.int32), torch.tensor([0, 2, 4, 6, 8], dtype=torch.int32))
    assert torch.allclose(ctx.linspace(torch.tensor(1.0), torch.tensor(2.0), 3), torch.linspace(1, 2, 3))
    with pytest.raises(ValueError):
        ctx.linspace(0, 1, -1)

    # ---- out=
    for name in ("zeros", "ones", "rand", "randn", "empty"):
        out = ctx.full((12,), 9.0)
        got = getattr(ctx, name)(3, 4, out=out)
        assert got.data_ptr() == out.data_ptr() and got.shape == (3, 4), name
        if name == "zeros":
            assert torch.all(out == 0)
        if name == "ones":
            assert torch.all(out == 1)
        if name == "empty":
            assert torch.all(out == 9)
    out = ctx.empty(5, dtype=torch.int64)
    assert ctx.arange(5, out=out).data_ptr() == out.data_ptr() and torch.equal(out, torch.arange(5))
    out = ctx.empty(4)
    assert ctx.linspace(0, 3, 4, out=out).data_ptr() == out.data_ptr() and torch.equal(out, torch.tensor([0., 1., 2., 3.]))
    out = ctx.empty(6, dtype=torch.int32)
    assert torch.all(ctx.full((2, 3), 4, out=out, dtype=torch.int32) == 4) and torch.all(out == 4)
    out = ctx.empty(6, dtype=torch.int64)
    assert ctx.randint(0, 3, (6,), out=out).data_ptr() == out.data_ptr() and int(out.max()) < 3
    good = ctx.empty(6)
    for kwargs in (dict(out=torch.empty(6)), dict(out=ctx.empty(5)), dict(out=good, dtype=torch.float64)):
        for name in ("zeros", "ones", "empty", "rand", "randn"):
            with pytest.raises(RuntimeError):
                getattr(ctx, name)(2, 3, **kwargs)
        with pytest.raises(RuntimeError):
            ctx.full((2, 3), 1.0, **kwargs)

    # ---- device / layout / pin_memory / requires_grad
    for name in ("zeros", "ones", "empty", "rand", "randn"):
        assert getattr(ctx, name)(2, device="cpu").device.type == "cpu"
        assert getattr(ctx, name)(2, device=torch.device("cpu")).device.type == "cpu"
        assert getattr(ctx, name)(2, device=None).device == ctx.get_device() or ctx.get_device().index is None
        with pytest.raises(RuntimeError):
            getattr(ctx, name)(2, device="cuda")
        with pytest.raises(RuntimeError):
            getattr(ctx, name)(2, device="cuda:1")
        with pytest.raises(ValueError):
            getattr(ctx, name)(2, layout=torch.sparse_coo)
        assert getattr(ctx, name)(2, requires_grad=True).requires_grad
        assert not getattr(ctx, name)(2).requires_grad
    for fn, args in ((ctx.full, ((2,), 1.0)), (ctx.arange, (4,)), (ctx.linspace, (0, 1, 4))):
        with pytest.raises(RuntimeError):
            fn(*args, device="cuda:0")
        with pytest.raises(ValueError):
            fn(*args, layout=torch.sparse_coo)
    with pytest.raises(RuntimeError):
        ctx.zeros_like(torch.ones(2), device="cuda")
    with pytest.raises(RuntimeError):
        ctx.empty(4, pin_memory=True)
    g = ctx.arange(0.0, 4.0, 1.0, requires_grad=True)
    (g * 2).sum().backward()
    assert torch.all(g.grad == 2)

    # ---- heap membership
    base = ctx.zeros(8, 8)
    assert on_heap(base[2:4]) and on_heap(base.t()) and on_heap(base.view(-1)[5:])
    assert not on_heap(torch.zeros(8, 8)) and not on_heap(base.clone())
    assert on_heap(ctx.zeros(0))  # an empty tensor still counts as a heap tensor
    nc = torch.arange(24).reshape(4, 6).t()
    sym = ctx.as_symmetric(nc)
    assert on_heap(sym) and torch.equal(sym, nc)
    again = ctx.as_symmetric(sym)
    assert on_heap(again) and torch.equal(again, nc)
    ctx.barrier()


def test_factory_parity_with_torch():
    run_ranks(_parity, 1, timeout=600.0)


def _offsets(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 26)
    base = int(ctx.get_heap_bases()[rank])
    seq = []
    for i, (n, dt) in enumerate([(1, torch.int8), (1000, torch.float32), (3, torch.float64), (0, torch.int32),
                                 (1025, torch.uint8), (64, torch.bfloat16)]):
        t = ctx.zeros(n, dtype=dt) if i % 2 == 0 else ctx.empty(n, dtype=dt)
        if n == 0:
            continue  # an empty tensor has no address to compare
        seq.append(t.data_ptr() - base)
        assert t.data_ptr() % 1024 == 0
    # each allocation starts at a 1024-byte boundary after the end of the previous one
    assert all(b > a for a, b in zip(seq, seq[1:]))
    assert seq[2] - seq[1] == 4096 and seq[4] - seq[3] == 2048
    mine = torch.tensor(seq, dtype=torch.int64)
    others = [torch.zeros_like(mine) for _ in range(world)]
    import torch.distributed as dist

    dist.all_gather(others, mine)
    for o in others:
        assert torch.equal(o, mine), "ranks that allocate in the same order must see the same offsets"
    ctx.verify_symmetry()
    # mark / release returns the space; the next allocation lands where the released one was
    mark = ctx.heap_mark()
    a = ctx.zeros(4096)
    off_a = a.data_ptr() - base
    del a
    ctx.heap_release(mark)
    b = ctx.zeros(16)
    assert b.data_ptr() - base == off_a
    ctx.barrier()


def test_offsets_are_symmetric_world2():
    run_ranks(_offsets, 2)
