"""The GPU code paths of the Python layer, walked without a GPU.

On a machine without CUDA the collectives and fused ops take their host fallbacks, so the code that
builds kernel descriptors, sizes workspaces and picks variants would never run in the CPU suite. Here
two gloo ranks create a normal CPU-backend context and then pretend to be on the GPU path: the
kernel library's planning entry point (pure host code) is called for real, the launch entry points
are replaced by recorders, and stream / synchronise calls by no-ops. Nothing is computed; what is
checked is what each call WOULD launch: operation codes, shapes, leading dimensions, pointers,
workspace buffers, variant choice by message size, descriptor reuse on repeated calls. The reference
has no equivalent (its launch code only ever runs on GPUs).
"""

import torch

from helpers import run_ranks


class _Recorder:
    """Stands in front of the real library: planning goes through, launches are recorded."""

    def __init__(self, real, ccl_desc_type, gemm_desc_type):
        self._real = real
        self.ccl, self.gemm = [], []
        self._ccl_t, self._gemm_t = ccl_desc_type, gemm_desc_type
        self.iris_gemm_workspace = real.iris_gemm_workspace
        self.iris_gemm_sf_inbox_bytes = real.iris_gemm_sf_inbox_bytes

        def ccl_launch(op, d, stream):
            self.ccl.append((op, self._ccl_t.from_buffer_copy(d._obj)))
            return 0

        def gemm_launch(d, stream):
            self.gemm.append(self._gemm_t.from_buffer_copy(d._obj))
            return 0

        self.iris_ccl_launch, self.iris_gemm_launch = ccl_launch, gemm_launch
        self.models = []

        def model_entry(name, module, desc_name):
            def call(d, stream):
                import importlib

                desc_t = getattr(importlib.import_module(module), desc_name)
                self.models.append((name, desc_t.from_buffer_copy(d._obj)))
                return 0

            return call

        self.iris_flash_decode = model_entry("decode", "iris_b200.models.flash_decode", "IrisDecodeDesc")
        self.iris_moe_forward = model_entry("moe", "iris_b200.models.moe", "IrisMoeDesc")
        self.iris_ring_attention = model_entry("ring", "iris_b200.models.ring_attention", "IrisRingAttnDesc")


def _pretend_gpu(ctx):
    """Route ``ctx`` through the GPU branches with recorded launches; returns the recorder."""
    from iris_b200 import _lib, ccl

    rec = _Recorder(_lib.kernels(), ccl.IrisCclDesc, _lib.IrisGemmDesc)
    _lib.kernels = lambda: rec
    _lib.current_stream_ptr = lambda: 0
    torch.cuda.synchronize = lambda *a, **k: None
    ctx.is_cpu = False
    ctx.device_barrier = lambda group=None: None          # a kernel launch of its own on a GPU; not part of this walk
    ctx.get_cu_count = lambda: 148
    return rec


def _dry_run(rank, world):
    import iris_b200 as iris
    from iris_b200 import _lib, ops
    from iris_b200.ops import FusedConfig
    from iris_b200.ccl import Config
    from iris_b200.parallel import ColumnParallelLinear, GradientBuckets, RowParallelLinear, UlyssesExchange

    ctx = iris.iris(1 << 28)
    rec = _pretend_gpu(ctx)
    dt = torch.bfloat16
    W = world

    # ---- collectives: descriptors and variant choice
    inp, out = ctx.zeros((64, 512), dtype=dt), ctx.zeros((64, 512), dtype=dt)          # 64 KB
    ctx.ccl.all_reduce(out, inp)
    op, d = rec.ccl[-1]
    assert op == 2 and (d.M, d.N) == (64, 512) and d.dtype == _lib.DTYPE_CODE[dt] and d.ctx.world == W and d.ctx.rank == rank
    assert d.inp == inp.data_ptr() and d.out == out.data_ptr() and d.ld_in == 512 and d.ld_out == 512
    big_in, big_out = ctx.zeros((1024, 4096), dtype=dt), ctx.zeros((1024, 4096), dtype=dt)      # 8 MB
    ws = ctx.ccl.all_reduce(big_out, big_in)
    if W > 1:
        assert d.variant == 6 and d.ring_buf and d.flags                               # small message: one-shot push, own workspace
        assert rec.ccl[-1][1].variant == 3 and ws.variant == "two_shot"                # no multicast window here: two-shot
        for name, code in (("one_shot", 2), ("two_shot", 3), ("atomic", 0), ("ring", 1), ("spinlock", 4)):
            w2 = ctx.ccl.all_reduce(big_out, big_in, config=Config(all_reduce_variant=name))
            assert rec.ccl[-1][1].variant == code and w2.variant == name
            if name == "ring":
                assert rec.ccl[-1][1].ring_buf == w2.ring_buffer.data_ptr() and rec.ccl[-1][1].flags == w2.flags.data_ptr()
    else:
        assert d.variant == 2 and ws.variant == "one_shot"                             # one rank: every variant is a copy
    if W > 1:
        # other tensors of the same shape: the ring variant's heap buffers are not allocated again
        ring_a = ctx.ccl.all_reduce(big_out, big_in, config=Config(all_reduce_variant="ring"))
        other_in, other_out = ctx.zeros((1024, 4096), dtype=dt), ctx.zeros((1024, 4096), dtype=dt)
        level = ctx.heap_mark()
        ring_b = ctx.ccl.all_reduce(other_out, other_in, config=Config(all_reduce_variant="ring"))
        assert ring_b is ring_a and ctx.heap_mark() == level and rec.ccl[-1][1].ring_buf == ring_a.ring_buffer.data_ptr()
        assert rec.ccl[-1][1].inp == other_in.data_ptr()
        # ring -> two_shot -> ring on the SAME tensors: each variant keeps its own descriptor, so the
        # two-shot call runs on the context's sync block (not on the ring workspace's) with its own CTA count
        ctx.ccl.all_reduce(big_out, big_in, config=Config(all_reduce_variant="ring"))
        ring_d = bytes(rec.ccl[-1][1])
        ctx.ccl.all_reduce(big_out, big_in, config=Config(all_reduce_variant="two_shot"))
        two = rec.ccl[-1][1]
        assert two.variant == 3 and two.sync_block != ring_a.sync_block.data_ptr() and not two.ring_buf
        assert two.sync_block == ctx.sync_block(("ccl", ctx._group_key(None))).data_ptr() and two.comm_sms == Config().comm_sms
        ctx.ccl.all_reduce(big_out, big_in, config=Config(all_reduce_variant="ring"))
        assert bytes(rec.ccl[-1][1]) == ring_d
    n_before = len(rec.ccl)
    ctx.ccl.all_reduce(big_out, big_in, workspace=ws, async_op=True)
    ctx.ccl.all_reduce(big_out, big_in, workspace=ws, async_op=True)                   # replayed from the call cache
    assert len(rec.ccl) == n_before + 2 and bytes(rec.ccl[-1][1]) == bytes(rec.ccl[-2][1])
    ag = ctx.zeros((W * 64, 512), dtype=dt)
    ctx.ccl.all_gather(ag, inp)
    op, d = rec.ccl[-1]
    assert op == 0 and (d.M, d.N) == (64, 512) and d.out == ag.data_ptr()
    a2a_in, a2a_out = ctx.zeros((64, 128 * W), dtype=dt), ctx.zeros((64, 128 * W), dtype=dt)
    ctx.ccl.all_to_all(a2a_out, a2a_in)
    assert rec.ccl[-1][0] == 1
    rs_out = ctx.zeros((64 // W, 512), dtype=dt)
    ctx.ccl.reduce_scatter(rs_out, inp, config=Config(reduce_scatter_rows=True))
    op, d = rec.ccl[-1]
    assert op == 3 and d.rows_mode == 1 and d.out == rs_out.data_ptr()
    ctx.ccl.reduce_scatter(out, inp, config=Config(block_size_m=32, block_size_n=64, all_reduce_distribution=1))
    op, d = rec.ccl[-1]
    assert op == 3 and d.rows_mode == 0 and (d.block_m, d.block_n, d.distribution) == (32, 64, 1)

    # ---- fused ops: operation codes, shapes, workspaces
    Ml, K, N = 256, 512, 384
    A = torch.zeros(Ml, K, dtype=dt)
    B = torch.zeros(K, N, dtype=dt)
    Cfull = torch.zeros(Ml * W, N, dtype=dt)
    ws1 = ctx.ops.all_gather_matmul(Cfull, A, B, shard_dim=0)
    g = rec.gemm[-1]
    assert ws1.variant == "fused" and g.op == _lib.GEMM_AG_M and (g.M, g.N, g.K, g.M_local) == (Ml * W, N, K, Ml)
    assert g.A == A.data_ptr() and g.C == Cfull.data_ptr() and (g.lda, g.ldc) == (K, N) and g.b_kmajor == 0
    assert g.sync_block == ws1.sync_block.data_ptr() and g.bn == ws1.bn and g.bn in (128, 224, 256) and g.ctx.world == W
    if W > 1:
        assert g.inbox == ws1.inbox.data_ptr() and g.flags == ws1.flags.data_ptr()
    Bt = torch.zeros(N, K, dtype=dt).t()                                             # a K-major weight view: no copy
    ctx.ops.all_gather_matmul(Cfull, A, Bt, shard_dim=0)
    assert rec.gemm[-1].b_kmajor == 1 and rec.gemm[-1].B == Bt.data_ptr()
    n_before = len(rec.gemm)
    ctx.ops.all_gather_matmul(Cfull, A, B, shard_dim=0, workspace=ws1, async_op=True)
    ctx.ops.all_gather_matmul(Cfull, A, B, shard_dim=0, workspace=ws1, async_op=True)
    assert len(rec.gemm) == n_before + 2 and bytes(rec.gemm[-1]) == bytes(rec.gemm[-2])
    # a caller that never hands the workspace back gets the same one again: no heap growth per call
    first = ctx.ops.all_gather_matmul(Cfull, A, B, shard_dim=0)
    level = ctx.heap_mark()
    for _ in range(3):
        assert ctx.ops.all_gather_matmul(Cfull, A, B, shard_dim=0) is first
    assert ctx.heap_mark() == level
    Ak = torch.zeros(Ml, K // W, dtype=dt)
    Ck = torch.zeros(Ml, N, dtype=dt)
    ctx.ops.all_gather_matmul(Ck, Ak, B)                                             # the reference layout: K sharded
    g = rec.gemm[-1]
    assert g.op == _lib.GEMM_AG_K and g.K_local == K // W and g.K == K
    H = torch.zeros(Ml * W, N, dtype=dt)
    W2 = torch.zeros(N, K, dtype=dt)
    Y = torch.zeros(Ml, K, dtype=dt)
    ws2 = ctx.ops.matmul_reduce_scatter(Y, H, W2, scatter_rows=True)
    g = rec.gemm[-1]
    assert ws2.variant == "fused" and g.op == _lib.GEMM_REDUCE_SCATTER and (g.M, g.N, g.K) == (Ml * W, K, N)
    if W > 1:
        assert g.staging == ws2.staging.data_ptr() and g.flags == ws2.flags.data_ptr()
    Yt = ctx.zeros((Ml * W, K), dtype=dt)
    ctx.ops.matmul_reduce_scatter(Yt, H, W2)                                         # tile ownership, full-shape output
    assert rec.gemm[-1].op == _lib.GEMM_RS_TILES
    bias = torch.ones(Ml * W)
    ws3 = ctx.ops.matmul_all_reduce(Yt, H, W2, bias=bias)
    g = rec.gemm[-1]
    # the default variant is "auto": a small output takes the one-shot kernel, a large one the two-shot kernel
    small = Ml * W * K * 2 <= ops.ONE_SHOT_MAX_BYTES
    assert ws3.variant == "fused" and g.op == (_lib.GEMM_AR_ONE_SHOT if small else _lib.GEMM_ALL_REDUCE) and g.C == Yt.data_ptr()
    assert bool(g.bias_row) == (rank == 0)                                           # the bias enters the sum once
    for name, code in (("two_shot", _lib.GEMM_ALL_REDUCE), ("one_shot", _lib.GEMM_AR_ONE_SHOT), ("atomic", _lib.GEMM_AR_ATOMIC)):
        wv = ctx.ops.matmul_all_reduce(Yt, H, W2, config=FusedConfig(all_reduce_variant=name))
        assert rec.gemm[-1].op == code and wv.extra["all_reduce_variant"] == name and rec.gemm[-1].staging == (wv.staging.data_ptr() if wv.staging is not None else None)
    for name in ("ring", "spinlock"):                                                # no fused kernel: refused, not ignored
        try:
            ctx.ops.matmul_all_reduce(Yt, H, W2, config=FusedConfig(all_reduce_variant=name))
            raise AssertionError("expected a ValueError")
        except ValueError:
            pass
    off_heap = torch.zeros(Ml * W, K, dtype=dt)
    n_before = len(rec.gemm)
    ctx.ops.matmul_all_reduce(off_heap, H, W2)                                       # output not on the heap: GEMM + collective
    assert all(x.op == _lib.GEMM_LOCAL for x in rec.gemm[n_before:]) and rec.ccl[-1][0] == 2
    rows = ctx.zeros((Ml * W, N), dtype=dt)
    ctx.ops.matmul_all_gather(rows, A, B)
    assert rec.gemm[-1].op == _lib.GEMM_ALL_GATHER
    cols = ctx.zeros((Ml, N * W), dtype=dt)
    ctx.ops.matmul_all_gather(cols, A, B, scatter_cols=True)
    assert rec.gemm[-1].op == _lib.GEMM_ALL_SCATTER and rec.gemm[-1].ldc == N * W
    # fp32 operands are outside the kernels' range: library GEMM + collective, no fused launch
    n_before = len(rec.gemm)
    wsf = ctx.ops.matmul_all_reduce(ctx.zeros((8, 8)), torch.zeros(8, 4), torch.zeros(4, 8))
    assert wsf.variant == "unfused" and len(rec.gemm) == n_before

    # ---- the local GEMM entry point
    import pytest

    from iris_b200.ops.gemm import matmul

    col_bias, row_bias = torch.ones(N, dtype=dt), torch.ones(Ml, dtype=dt)
    Cl = matmul(A, B, bias=col_bias)
    g = rec.gemm[-1]
    assert g.op == _lib.GEMM_LOCAL and (g.M, g.N, g.K) == (Ml, N, K) and g.C == Cl.data_ptr() and g.bias_col and not g.bias_row
    matmul(A, B, bias=row_bias, bias_dim=0, out=Cl, two_sm=True)
    assert rec.gemm[-1].bias_row and not rec.gemm[-1].bias_col and rec.gemm[-1].two_sm == 2 and rec.gemm[-1].C == Cl.data_ptr()
    n_before = len(rec.gemm)
    for bad in (lambda: matmul(A, torch.zeros(K + 1, N, dtype=dt)), lambda: matmul(A, B, out=torch.zeros(Ml, N + 1, dtype=dt)),
                lambda: matmul(A, B, bias=row_bias), lambda: matmul(A, B, bias=col_bias, bias_dim=0)):
        with pytest.raises(ValueError):
            bad()
    with pytest.raises(TypeError):
        matmul(A.float(), B.float())
    assert len(rec.gemm) == n_before                      # nothing was launched with the rejected arguments

    # ---- the layers of iris_b200.parallel on the same path
    up = ColumnParallelLinear(ctx, K, N, dtype=dt, seed=1)
    down = RowParallelLinear(ctx, N, K, dtype=dt, seed=2, bias=True)
    n_before = len(rec.gemm)
    y = down(up(torch.zeros(Ml, K, dtype=dt)))
    assert y.shape == (Ml, K) and [x.op for x in rec.gemm[n_before:]] == [_lib.GEMM_AG_M, _lib.GEMM_REDUCE_SCATTER]
    down2 = RowParallelLinear(ctx, N, K, dtype=dt, seed=2, sequence_parallel=False)
    y2 = down2(torch.zeros(Ml * W, N, dtype=dt))
    assert ctx.is_symmetric(y2) and rec.gemm[-1].op in (_lib.GEMM_ALL_REDUCE, _lib.GEMM_AR_ONE_SHOT) and rec.gemm[-1].C == y2.data_ptr()
    model = torch.nn.Linear(32, 16)
    model(torch.ones(4, 32)).sum().backward()
    buckets = GradientBuckets(ctx, model.parameters())
    n_before = len(rec.ccl)
    buckets.all_reduce()
    launched = rec.ccl[n_before:]
    assert len(launched) == len(buckets.buckets) == 1 and launched[0][0] == 2 and launched[0][1].N == 4096
    assert launched[0][1].dtype == _lib.DTYPE_CODE[torch.float32] and launched[0][1].inp == buckets.buckets[0].inp.data_ptr()
    ex = UlyssesExchange(ctx)
    n_before = len(rec.ccl)
    heads = ex.to_heads(torch.zeros(16, 2 * W, 8, dtype=dt))
    assert heads.shape == (16 * W, 2, 8) and rec.ccl[-1][0] == 1 and len(rec.ccl) == n_before + 1
    assert (rec.ccl[-1][1].M, rec.ccl[-1][1].N) == (16, 2 * 8)                        # N is the width of one rank's chunk
    # ---- rewinding the heap drops what was allocated after the mark, including cached workspaces
    mark = ctx.heap_mark()
    t_in, t_out = ctx.zeros((8, 256), dtype=dt), ctx.zeros((8, 256), dtype=dt)
    ctx.ccl._push_ws = None
    ctx.ccl.all_reduce(t_out, t_in)                                                  # allocates the push workspace after the mark
    if W > 1:
        assert ctx.ccl._push_ws is not None and ctx.heap.offset_of(ctx.ccl._push_ws[0]) >= mark
    late = ctx.ops.matmul_all_reduce(ctx.zeros((Ml * W, 256), dtype=dt), torch.zeros(Ml * W, 128, dtype=dt), torch.zeros(128, 256, dtype=dt))
    assert late.variant == "fused" and late in ctx._ops_workspaces.values() and first in ctx._ops_workspaces.values()
    ctx.heap_release(mark)
    assert ctx.heap_mark() == mark and ctx.ccl._push_ws is None and not ctx.ccl._desc_cache
    # workspaces kept for callers that pass none: the one allocated after the mark is gone, earlier ones stay
    assert late not in ctx._ops_workspaces.values() and first in ctx._ops_workspaces.values()
    old_push = rec.ccl[-1][1].ring_buf
    t_in2, t_out2 = ctx.zeros((8, 256), dtype=dt), ctx.zeros((8, 256), dtype=dt)
    filler = ctx.zeros(4096, dtype=torch.int32)                                      # shifts what is allocated next
    assert t_in2.data_ptr() == t_in.data_ptr() and t_out2.data_ptr() == t_out.data_ptr()      # the space is handed out again
    ctx.ccl.all_reduce(t_out2, t_in2)
    if W > 1:
        # same tensors' addresses as before the release, but the call is not replayed from the cache:
        # its descriptor names the workspace allocated now, not the released one
        assert rec.ccl[-1][1].ring_buf == ctx.ccl._push_ws[0].data_ptr() != old_push and filler.data_ptr() < rec.ccl[-1][1].ring_buf
    import torch.distributed as dist

    dist.barrier()


def test_gpu_paths_of_collectives_fused_ops_and_layers_world2():
    run_ranks(_dry_run, 2)


def test_gpu_paths_world1():
    run_ranks(_dry_run, 1)


def _groups_dry_run(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.parallel import ParallelLayout

    ctx = iris.iris(1 << 26)
    rec = _pretend_gpu(ctx)
    layout = ParallelLayout({"tp": 2, "dp": 2}).build_groups()
    bases = [int(b) for b in ctx.heap.bases_host()]
    inp, out = ctx.zeros((32, 256), dtype=torch.bfloat16), ctx.zeros((32, 256), dtype=torch.bfloat16)
    for name in ("tp", "dp"):
        members = layout.ranks(name)
        ctx.ccl.all_reduce(out, inp, group=layout.group(name))
        op, d = rec.ccl[-1]
        # inside a group ranks are renumbered, only the members' heaps are listed, in group order, and the
        # multicast window (which spans all ranks) is not used
        assert op == 2 and d.ctx.world == 2 and d.ctx.rank == members.index(rank)
        assert [d.ctx.bases[i] for i in range(2)] == [bases[m] for m in members]
        assert d.ctx.mc_base == 0 and d.use_mc == 0 and d.variant in (2, 3)            # no push / NVLS inside groups
    # each group has its own sync block, distinct from the one of the whole job
    ctx.ccl.all_reduce(out, inp)
    blocks = {rec.ccl[-3][1].sync_block, rec.ccl[-2][1].sync_block, rec.ccl[-1][1].sync_block}
    assert len(blocks) == 3 and rec.ccl[-1][1].ctx.world == world
    dist.barrier()


def test_gpu_paths_of_group_collectives_world4():
    run_ranks(_groups_dry_run, 4)


def _models_dry_run(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200 import _lib
    from iris_b200.models import FlashDecodeLayer, MoELayer, RingAttention

    ctx = iris.iris(1 << 28)
    rec = _pretend_gpu(ctx)
    dt, W = torch.bfloat16, world

    # ---- flash decode: sizes, pointers and the split count reach the descriptor
    Hq, Hkv, D, page, B, blocks = 16, 2, 128, 64, 3, 5
    dec = FlashDecodeLayer(ctx, Hq, Hkv, D, max_batch=4)
    q = torch.zeros(B, Hq, D, dtype=dt)
    kc, vc = torch.zeros(B * blocks, page, Hkv, D, dtype=dt), torch.zeros(B * blocks, page, Hkv, D, dtype=dt)
    table = torch.arange(B * blocks, dtype=torch.int32).view(B, blocks)
    lens = torch.full((W, B), 300, dtype=torch.int32)
    out, lse = dec(q, kc, vc, lens, table, return_lse=True)
    name, d = rec.models[-1]
    assert name == "decode" and (d.B, d.Bmax, d.Hq, d.Hkv, d.D, d.page, d.max_blocks) == (B, 4, Hq, Hkv, D, page, blocks)
    assert d.q == q.data_ptr() and d.k_cache == kc.data_ptr() and d.block_table == table.data_ptr() and d.out == out.data_ptr()
    assert d.out_lse == lse.data_ptr() and d.gathered == dec.gathered.data_ptr() and d.flags == dec.signal_flags.data_ptr()
    assert d.exchange == 1 and d.num_blocks == B * blocks and 1 <= d.splits <= 2 and d.ctx.world == W      # 320 positions: two splits at most
    assert out.shape == (B, Hq, D) and lse.shape == (B, Hq) and d.dtype == _lib.DTYPE_CODE[dt]
    FlashDecodeLayer(ctx, Hq, Hkv, D, max_batch=4, use_tma=False)(q, kc, vc, lens, table)
    assert rec.models[-1][1].num_blocks == 0                                      # the cp.async tile fill was asked for
    n_before = len(rec.models)
    import pytest

    with pytest.raises(ValueError):
        dec(q, kc, vc, lens, table.long())
    with pytest.raises(ValueError):
        dec(q.transpose(0, 1).contiguous().transpose(0, 1), kc, vc, lens, table)     # not contiguous
    assert len(rec.models) == n_before

    # ---- ring attention
    S, Hq2, Hkv2 = 256, 4, 2
    ring = RingAttention(ctx, S, Hq2, Hkv2, layout="zigzag")
    qa, ka, va = torch.zeros(S, Hq2, 128, dtype=dt), torch.zeros(S, Hkv2, 128, dtype=dt), torch.zeros(S, Hkv2, 128, dtype=dt)
    o = ring(qa, ka, va, causal=True)
    name, d = rec.models[-1]
    assert name == "ring" and (d.S, d.Hq, d.Hkv, d.D, d.causal) == (S, Hq2, Hkv2, 128, 1) and d.options & 2 and not d.options & 1
    assert d.q == qa.data_ptr() and d.out == o.data_ptr() and d.kv_buf == ring.kv_buf.data_ptr() and d.flags == ring.flags.data_ptr()
    RingAttention(ctx, S, Hq2, Hkv2, use_tcgen05=False)(qa, ka, va)
    assert rec.models[-1][1].options == 1 and rec.models[-1][1].causal == 0
    for bad in (lambda: ring(qa[:128], ka[:128], va[:128]), lambda: ring(qa, ka, va, out=torch.zeros(S, Hq2, 64, dtype=dt)),
                lambda: ring(qa, ka, va[:, :1])):
        with pytest.raises(ValueError):
            bad()
    with pytest.raises(TypeError):
        ring(qa.float(), ka.float(), va.float())

    # ---- MoE
    hidden, ffn, E, topk, T = 256, 128, 2 * W, 2, 64
    El = E // W
    moe = MoELayer(ctx, hidden, ffn, E, topk, T, w_gate=torch.zeros(El, hidden, ffn, dtype=dt), w_up=torch.zeros(El, hidden, ffn, dtype=dt),
                   w_down=torch.zeros(El, ffn, hidden, dtype=dt))
    x, logits = torch.zeros(T, hidden, dtype=dt), torch.zeros(T, E)
    y = moe(x, logits)
    name, d = rec.models[-1]
    assert name == "moe" and (d.T, d.K, d.E, d.El, d.D, d.F) == (T, topk, E, El, hidden, ffn) and d.weights_kmajor == 1
    assert d.x == x.data_ptr() and d.out == y.data_ptr() and d.inbox == moe.inbox.data_ptr() and d.comb == moe.comb.data_ptr()
    assert d.w13 == moe.w13.data_ptr() and d.w2 == moe.w2.data_ptr() and d.capacity == moe.capacity and d.ctx.world == W
    # the fused gate / up weight is K-major: [local experts, 2 ffn, hidden]; the down weight [local experts, hidden, ffn]
    assert tuple(moe.w13.shape) == (El, 2 * ffn, hidden) and tuple(moe.w2.shape) == (El, hidden, ffn)
    for bad in (lambda: moe(torch.zeros(T + 1, hidden, dtype=dt), torch.zeros(T + 1, E)), lambda: moe(x, torch.zeros(T, E + 1)),
                lambda: moe(x, logits, out=torch.zeros(T, hidden + 1, dtype=dt))):
        with pytest.raises(ValueError):
            bad()
    with pytest.raises(TypeError):
        moe(x.float(), logits)
    dist.barrier()


def test_gpu_paths_of_the_model_layers_world2():
    run_ranks(_models_dry_run, 2)
