"""Collectives restricted to process groups, four gloo ranks (no GPU).

Mirrors the reference's tests/ccl/test_process_groups.py (needs >= 4 ranks): consecutive groups
[0,1] [2,3] and strided groups [0,2] [1,3], every collective inside the caller's group, the two
groups running at the same time with different data; a group whose ranks are not evenly strided is
rejected (iris/host/distributed/helpers.py:281-299).
"""
import pytest
import torch

from helpers import run_ranks


def _data(rank, M, N, dtype):
    return (torch.arange(M * N, dtype=torch.float32).view(M, N) % 5 + 10 * (rank + 1)).to(dtype)


def _groups(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.ccl import Config, owned_tiles
    from iris_b200.host.distributed import extract_group_info

    ctx = iris.iris(1 << 26)
    layouts = {"consecutive": [[0, 1], [2, 3]], "strided": [[0, 2], [1, 3]], "all": [[0, 1, 2, 3]], "single": [[0], [1], [2], [3]]}
    for label, layout in layouts.items():
        groups = [dist.new_group(r) for r in layout]  # every rank creates every group, in the same order
        members = next(r for r in layout if rank in r)
        mine = groups[layout.index(members)]
        W = len(members)
        me = members.index(rank)
        info = extract_group_info(mine, rank, world)
        stride = members[1] - members[0] if W > 1 else 1
        assert info == (me, rank, W, members[0], stride), (label, info)
        for dtype in (torch.float32, torch.float16, torch.bfloat16, torch.int32):
            M, N = 8, 4 * W
            inp = ctx.zeros((M, N), dtype=dtype)
            inp.copy_(_data(rank, M, N, dtype))
            total = sum(_data(r, M, N, torch.float32) for r in members).to(dtype)
            # all_reduce: only the group's members contribute
            out = ctx.zeros((M, N), dtype=dtype)
            ctx.barrier()
            ctx.ccl.all_reduce(out, inp, group=mine)
            assert torch.equal(out, total), (label, dtype, "all_reduce")
            for variant in ("one_shot", "two_shot", "atomic", "ring", "spinlock"):
                if variant == "atomic" and dtype not in (torch.float32, torch.int32):
                    continue
                out.zero_()
                ctx.barrier()
                ctx.ccl.all_reduce(out, inp, group=mine, config=Config(all_reduce_variant=variant, block_size_m=4, block_size_n=W * 2))
                assert torch.equal(out, total), (label, dtype, variant)
            # all_gather: rows ordered by rank inside the group
            ag = ctx.zeros((W * M, N), dtype=dtype)
            ctx.barrier()
            ctx.ccl.all_gather(ag, inp, group=mine)
            for i, r in enumerate(members):
                assert torch.equal(ag[i * M:(i + 1) * M], _data(r, M, N, dtype)), (label, dtype, "all_gather", r)
            # all_to_all: column chunk d of member s lands in column chunk s of member d
            a2a = ctx.zeros((M, N), dtype=dtype)
            ctx.barrier()
            ctx.ccl.all_to_all(a2a, inp, group=mine)
            n = N // W
            for i, r in enumerate(members):
                assert torch.equal(a2a[:, i * n:(i + 1) * n], _data(r, M, N, dtype)[:, me * n:(me + 1) * n]), (label, dtype, "a2a")
            # reduce_scatter: the full-shape output holds only the tiles this member owns
            for dist_mode in (0, 1):
                rs = ctx.zeros((M, N), dtype=dtype)
                ctx.barrier()
                ctx.ccl.reduce_scatter(rs, inp, group=mine, config=Config(block_size_m=4, block_size_n=4, all_reduce_distribution=dist_mode))
                mask = torch.zeros(M, N, dtype=torch.bool)
                for (r0, r1, c0, c1) in owned_tiles(M, N, 4, 4, W, me, dist_mode):
                    mask[r0:r1, c0:c1] = True
                assert torch.equal(rs[mask], total[mask]) and torch.all(rs[~mask] == 0), (label, dtype, "reduce_scatter", dist_mode)
            ctx.barrier()
        # barriers inside the group, host and device style, repeated (the flag block is reused)
        for _ in range(3):
            ctx.barrier(group=mine)
            ctx.device_barrier(group=mine)
        ctx.check()
        ctx.barrier()
    # visibility through a group barrier: a store before it is seen by the partner after it
    pair = [[0, 1], [2, 3]]
    gs = [dist.new_group(r) for r in pair]
    members = next(r for r in pair if rank in r)
    g = gs[pair.index(members)]
    partner = members[1 - members.index(rank)]
    cell = ctx.zeros(4, dtype=torch.int32)
    ctx.barrier()
    for it in range(1, 6):
        ctx.rma.store(cell, it * 10 + rank, to_rank=partner)
        ctx.device_barrier(group=g)
        assert torch.all(cell == it * 10 + partner), (it, cell)
        ctx.device_barrier(group=g)
    # uneven strides are refused, and so is a group the caller is not part of
    uneven = dist.new_group([0, 1, 3])
    a, b = ctx.zeros((4, 4)), ctx.zeros((4, 4))
    if rank in (0, 1, 3):
        with pytest.raises(RuntimeError):
            extract_group_info(uneven, rank, world)
        with pytest.raises(RuntimeError):
            ctx.ccl.all_reduce(a, b, group=uneven)
    else:
        with pytest.raises(RuntimeError):
            extract_group_info(uneven, rank, world)
    ctx.barrier()


def test_every_collective_inside_consecutive_and_strided_groups():
    run_ranks(_groups, 4, timeout=900.0)
