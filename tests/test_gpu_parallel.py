"""The parallelism package, the timing helper and the launch records on real GPUs.

Single-GPU cases run in this process (world 1); the multi-GPU cases start one child per GPU (nccl,
world = min(#GPUs, 4)) and are skipped with fewer than two GPUs. Oracles are the unsharded fp32
computations, as in tests/test_cpu_parallel.py, which runs the same layers on gloo ranks.
"""
import json
import os

import pytest
import torch

from helpers import free_port, run_ranks

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import torch.distributed as dist

    torch.cuda.set_device(0)
    if not dist.is_initialized():
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(free_port())
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    import iris_b200 as iris

    c = iris.iris(1 << 30)
    yield c
    c.barrier()


def _rel(a, ref):
    return (a.float() - ref.float()).abs().max().item() / max(ref.float().abs().max().item(), 1e-6)


def _mlp_case(ctx, rank, world, sequence_parallel):
    from iris_b200.parallel import ColumnParallelLinear, RowParallelLinear

    dt, dev = torch.bfloat16, ctx.get_device()
    Ml, K, F = 256, 512, 384
    M = Ml * world
    g = torch.Generator().manual_seed(3)
    X = (torch.randn(M, K, generator=g) * 0.5).to(dt)
    W1 = (torch.randn(K, F * world, generator=g) * 0.05).to(dt)
    W2 = (torch.randn(F * world, K, generator=g) * 0.05).to(dt)
    b2 = torch.randn(K, generator=g).to(dt)
    up = ColumnParallelLinear(ctx, K, F, sequence_parallel=sequence_parallel, dtype=dt, weight=W1[:, rank * F:(rank + 1) * F].contiguous())
    down = RowParallelLinear(ctx, F, K, sequence_parallel=sequence_parallel, dtype=dt, weight=W2[rank * F:(rank + 1) * F].contiguous(),
                             bias_value=b2)
    x = (X[rank * Ml:(rank + 1) * Ml] if sequence_parallel else X).to(dev).contiguous()
    H = X.float() @ W1.float()
    Y = torch.nn.functional.silu(H).to(dt).float() @ W2.float() + b2.float()
    for _ in range(2):                                   # the second pass reuses workspaces and buffers
        h = up(x)
        y = down(torch.nn.functional.silu(h.float()).to(dt))
    torch.cuda.synchronize()
    assert _rel(h.cpu(), H[:, rank * F:(rank + 1) * F]) < 2e-2
    want = Y[rank * Ml:(rank + 1) * Ml] if sequence_parallel else Y
    assert y.shape == want.shape and _rel(y.cpu(), want) < 3e-2
    ctx.check()


@pytest.mark.parametrize("sequence_parallel", [True, False])
def test_tensor_parallel_linears_world1(ctx, sequence_parallel):
    _mlp_case(ctx, 0, 1, sequence_parallel)


def test_gradient_buckets_and_ulysses_world1(ctx):
    from iris_b200.parallel import GradientBuckets, UlyssesExchange

    dev = ctx.get_device()
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(), torch.nn.Linear(256, 16)).to(dev)
    buckets = GradientBuckets(ctx, model.parameters(), bucket_bytes=32 << 10).attach()
    model(torch.randn(32, 64, device=dev)).square().mean().backward()
    before = [p.grad.clone() for p in model.parameters()]
    buckets.finish()
    torch.cuda.synchronize()
    for p, b in zip(model.parameters(), before):
        assert torch.allclose(p.grad, b, atol=1e-6)       # the average over one replica is the gradient itself
    buckets.detach()
    ex = UlyssesExchange(ctx)
    x = torch.randn(128, 8, 64, device=dev, dtype=torch.bfloat16)
    assert torch.equal(ex.to_heads(x), x) and torch.equal(ex.to_sequence(x), x)
    ctx.check()


def test_time_max_over_ranks_and_launch_records(ctx, tmp_path):
    from iris_b200.host import artifacts
    from iris_b200.utils import time_max_over_ranks

    inp = ctx.full((256, 4096), 1.0, dtype=torch.bfloat16)
    out = ctx.zeros((256, 4096), dtype=torch.bfloat16)
    artifacts.configure(tmp_path)
    try:
        ws = ctx.ccl.all_reduce(out, inp)
        res = time_max_over_ranks(lambda: ctx.ccl.all_reduce(out, inp, workspace=ws, async_op=True), ctx, n_warmup=3, n_repeat=5)
    finally:
        artifacts.configure(None)
    assert res["ms"] > 0 and res["ms"] == res["ms_this_rank"] == res["ms_min_over_ranks"] and torch.all(out == 1)
    records = [os.path.join(root, "metadata.json") for root, _, files in os.walk(tmp_path / "ccl") if "metadata.json" in files]
    assert len(records) == 1                                  # one configuration, recorded once however often it ran
    meta = json.load(open(records[0]))
    assert meta["params"]["M"] == 256 and meta["params"]["N"] == 4096 and meta["kernel"].startswith("all_reduce")
    if (artifacts._build.OBJDIR / "ccl.cu.ptxas.log").exists():          # the compile report travels with the build directory
        assert any(k["registers"] for k in meta["compiled"])


def _world():
    """Ranks of the multi-GPU cases: ``IRIS_TEST_WORLD`` when set (the suite is run at 2, 4 and 8),
    else every GPU up to four."""
    import os

    want = int(os.environ.get("IRIS_TEST_WORLD", "0"))
    return min(torch.cuda.device_count(), want if want > 0 else 4)


def _multi(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.models import reference_attention
    from iris_b200.parallel import GradientBuckets, P2PChannel, UlyssesExchange, shard_sequence

    ctx = iris.iris(1 << 30)
    dev = ctx.get_device()
    for sp in (True, False):
        _mlp_case(ctx, rank, world, sp)
    # gradient buckets: replicas with different batches end up with the same averaged gradients
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(), torch.nn.Linear(256, 16)).to(dev)
    buckets = GradientBuckets(ctx, model.parameters(), bucket_bytes=32 << 10).attach()
    for step in range(2):
        model.zero_grad(set_to_none=True)
        data = torch.randn(32, 64, generator=torch.Generator().manual_seed(10 * step + rank)).to(dev)
        model(data).square().mean().backward()
        local = [p.grad.detach().clone() for p in model.parameters()]
        buckets.finish()
        for p, gl in zip(model.parameters(), local):
            want = gl.clone()
            dist.all_reduce(want)
            assert torch.allclose(p.grad, want / world, atol=1e-5, rtol=1e-4), step
    buckets.detach()
    # Ulysses: heads for tokens and back, attention in between
    S, H, D = 64 * world, 2 * world, 64
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(S, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
    ex = UlyssesExchange(ctx)
    heads = [ex.to_heads(shard_sequence(t, rank, world).to(dev)).clone() for t in (q, k, v)]
    Hl = H // world
    for full, got in zip((q, k, v), heads):
        assert torch.equal(got.cpu(), full[:, rank * Hl:(rank + 1) * Hl])
    o = ex.to_sequence(reference_attention(*heads, causal=True).to(torch.bfloat16))
    want = reference_attention(q, k, v, causal=True).to(torch.bfloat16)[rank * (S // world):(rank + 1) * (S // world)]
    assert _rel(o.cpu(), want) < 2e-2
    # point-to-point ring: more messages than slots, so acknowledgements are exercised too
    ch = P2PChannel(ctx, (8, 16), dtype=torch.float32, depth=2, timeout_ms=3000)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    for n in range(1, 6):
        ch.send(torch.full((8, 16), 100.0 * rank + n, device=dev), nxt)
        got = ch.recv(prv)
        assert torch.all(got == 100.0 * prv + n), (n, float(got[0, 0]))
    ctx.check()
    ctx.barrier()


@pytest.mark.multigpu
def test_parallel_package_between_gpus():
    run_ranks(_multi, _world(), backend="nccl", timeout=600)
