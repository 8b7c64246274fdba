"""Fused GEMM + collective operations (reference: iris/ops/__init__.py:37-178).

Each op is ONE sm_100a kernel (``csrc/kernels/gemm_ops.cu``): tcgen05/TMEM tiles fed by TMA, with
the collective carried out by the same kernel through peer stores, NVLS multimem stores and
per-tile flags on the symmetric heap.

=========================  =====================================================================
``all_gather_matmul``      ``C = gather(A_sharded) @ B``; A sharded along K (reference layout,
                           ``shard_dim=1``) or along rows (``shard_dim=0``, tensor-parallel MLP)
``matmul_all_gather``      ``C[r*M:(r+1)*M] = A_r @ B`` gathered on every rank
``matmul_all_reduce``      ``C = sum_r A_r @ B_r`` on every rank
``matmul_reduce_scatter``  ``sum_r A_r @ B_r`` with each rank keeping its tiles (reference layout:
                           full-shape output, owned tiles only) or its row block (``scatter_rows``)
=========================  =====================================================================

Module-level functions take the context first (``iris_b200.ops.matmul_all_reduce(ctx, C, A, B)``);
``ctx.ops.<op>(C, A, B, ...)`` binds it. Every op returns its ``FusedWorkspace``; pass it back to
skip the (collective) allocation of buffers on later calls. Inputs that the tensor-core kernel
cannot take (fp32, shapes that do not tile) go through the unfused path: GEMM, then the
collective of ``ctx.ccl``.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from ..host import artifacts as _artifacts
from .config import FusedConfig
from .gemm import fill_desc, matmul
from .gemm_fp8 import (BlockScaled, dequant_matmul, matmul_fp8, matmul_fp8_blockscaled, pack_scales_a, pack_scales_b,
                       quantize_1x128, quantize_128x128, quantize_activation, quantize_weight)
from .workspace import FusedWorkspace

__all__ = [
    "FusedConfig", "FusedWorkspace", "OpsNamespace", "matmul", "matmul_fp8", "quantize_1x128", "quantize_128x128", "dequant_matmul",
    "BlockScaled", "quantize_activation", "quantize_weight", "matmul_fp8_blockscaled", "pack_scales_a", "pack_scales_b",
    "matmul_all_reduce", "matmul_all_reduce_preamble", "all_gather_matmul", "all_gather_matmul_preamble",
    "matmul_all_gather", "matmul_all_gather_preamble", "matmul_reduce_scatter", "matmul_reduce_scatter_preamble",
]

_FUSED_DTYPES = (torch.bfloat16, torch.float16)
_DEFAULT_CONFIG = FusedConfig()      # what config=None means; never mutated


def _is_fp8(*tensors) -> bool:
    return all(isinstance(t, BlockScaled) for t in tensors)


def _fusable(ctx, *tensors) -> bool:
    if ctx.is_cpu:
        return False
    if _is_fp8(*tensors):
        return tensors[0].kind == "activation" and tensors[-1].kind == "weight"
    return all((not isinstance(t, BlockScaled)) and t.dtype in _FUSED_DTYPES and t.dim() == 2 for t in tensors)


def _fp8_tile(config) -> int:
    return 128 if config.tile_n() == 128 else 224


def _lower_fp8(A, B, dtype):
    """Block-scaled operands as plain matrices of ``dtype`` (the path of the CPU backend and of shapes
    the tensor-core kernel cannot take): dequantised, then handled like 16-bit inputs."""
    if isinstance(A, BlockScaled):
        A = A.dequantize().to(dtype)
    if isinstance(B, BlockScaled):
        B = B.dequantize().to(dtype)
    return A, B


def _base_desc(ctx, op, M, N, K, A, B, out, config, bias_row=None, bias_col=None) -> tuple:
    d = _lib.IrisGemmDesc()
    d.op = op
    d.M, d.N, d.K = M, N, K
    if _is_fp8(A, B):
        # e4m3 operands, scales applied by the tensor core; the output tensor gives the 16-bit result format
        if out.dtype not in _FUSED_DTYPES or out.stride(1) != 1:
            raise TypeError("the output of an fp8 op is a row-major fp16 or bf16 tensor")
        tile = _fp8_tile(config)
        d.dtype, d.in_dtype, d.b_kmajor, d.bn = _lib.DTYPE_CODE[out.dtype], _lib.DTYPE_CODE[torch.float8_e4m3fn], 1, tile
        d.A, d.lda = A.q.data_ptr(), A.q.stride(0)
        d.B, d.ldb = B.q.data_ptr(), B.q.stride(0)
        d.C, d.ldc = out.data_ptr(), out.stride(0)
        sa, sb = A.sf(), B.sf(tile)
        d.sf_a, d.sf_b = sa.data_ptr(), sb.data_ptr()
        d.bias_row = bias_row.data_ptr() if bias_row is not None else None
        d.bias_col = bias_col.data_ptr() if bias_col is not None else None
        keep = (A.q, B.q, sa, sb)
    else:
        keep = fill_desc(d, A, B, out, bias_row=bias_row, bias_col=bias_col, bn=config.tile_n())
    d.group_m = config.group_size_m
    d.comm_ctas = config.comm_sms
    d.two_sm = 0 if config.two_sm is None else (2 if config.two_sm else 1)
    d.use_mc = 1 if (config.use_multicast and ctx.has_multicast()) else 0
    d.overlap = 1 if config.overlap in ("wg_specialized", "producer_consumer") else 0
    d.ctx = ctx.ctx_struct()
    return d, keep


def _plan(d) -> tuple:
    inbox, flags, staging, bn, pair = C.c_uint64(0), C.c_uint64(0), C.c_uint64(0), C.c_int32(0), C.c_int32(0)
    rc = _lib.kernels().iris_gemm_workspace(C.byref(d), C.byref(inbox), C.byref(flags), C.byref(staging), C.byref(bn),
                                            C.byref(pair))
    return rc, inbox.value, flags.value, staging.value, bn.value, pair.value


def _make_workspace(ctx, operation, shape, dtype, variant, d) -> FusedWorkspace | None:
    """Allocate the op's heap buffers (collective). None when the kernel cannot take the shape."""
    rc, inbox, flags, staging, bn, pair = _plan(d)
    if rc != 0:
        return None
    ws = FusedWorkspace(operation=operation, shape=tuple(shape), dtype=dtype, world_size=ctx.num_ranks, variant=variant, bn=bn)
    ws.sync_block = ctx.zeros(80, dtype=torch.int32)
    if inbox:
        ws.inbox = ctx.heap.allocate(inbox, torch.uint8)
    if flags:
        ws.flags = ctx.zeros(flags // 4, dtype=torch.int32)
        ws.locks = ws.flags
    if staging:
        ws.staging = ctx.heap.allocate(staging, torch.uint8)
        ws.aux_buffer = ws.staging
    sf_inbox = int(_lib.kernels().iris_gemm_sf_inbox_bytes(C.byref(d)))
    if sf_inbox:        # fp8 all-gather: the gathered shards' scale atoms
        ws.extra["sf_inbox"] = ctx.heap.allocate(sf_inbox, torch.uint8)
    ws.prepared = True
    # arrival counters count communication CTAs: the number used at creation is part of the workspace
    ws.extra["comm_ctas"] = d.comm_ctas
    # the staging layout depends on the tile (width, single CTA or CTA pair): pinned with the buffers
    ws.extra["two_sm"] = 2 if pair else 1
    ctx.barrier()
    return ws


def _auto_workspace(ctx, operation, key, dtype, config, make, extra=None):
    """Workspace of a call that did not bring a matching one: created once per (operation, shapes,
    dtype, tile configuration) and kept on the context, so a loop that calls an op without passing
    the returned workspace back does not allocate heap memory (and run a barrier) on every call."""
    cache = ctx.__dict__.setdefault("_ops_workspaces", {})
    ck = (operation, tuple(key), dtype, config.tile_n(), config.two_sm, config.comm_sms, config.use_multicast, config.overlap, extra)
    ws = cache.get(ck)
    if ws is None:
        ws = cache[ck] = make()
    return ws


def _scratch(ctx, ws, tag, shape, dtype):
    """A heap buffer of the unfused path, allocated on first use (collectively) and kept in the
    workspace: the fallback must not consume heap memory on every call either."""
    bufs = ws.extra.setdefault("scratch", {})
    key = (tag, tuple(shape), dtype)
    buf = bufs.get(key)
    if buf is None:
        buf = bufs[key] = ctx.empty(tuple(shape), dtype=dtype)
    return buf


def _on_heap(ctx, ws, tag, t):
    """``t`` itself when it is a contiguous heap tensor, else its copy in a kept heap buffer."""
    if ctx.is_symmetric(t) and t.is_contiguous():
        return t
    buf = _scratch(ctx, ws, tag, t.shape, t.dtype)
    buf.copy_(t)
    return buf


def _cached_desc(ws, key, build):
    """Descriptor of a repeated call (same buffers): built once, then reused from the workspace."""
    cache = ws.extra.setdefault("desc", {})
    hit = cache.get(key)
    if hit is None:
        if len(cache) > 64:
            cache.clear()
        hit = cache[key] = build()
    return hit


def _with_bias(bias, build):
    """Run ``build(bias_fp32)`` and keep the converted bias, and the tensor it came from, next to the
    descriptor it is baked into."""
    b32 = _bias32(bias)
    d, keep = build(b32)
    return d, (keep, b32, bias)


def _refresh_bias(keep) -> None:
    """The kernels read an fp32 bias. For a 16-bit bias that is a converted copy kept with the cached
    descriptor; the source may have been updated in place since (an optimizer step, load_state_dict), so
    the copy is rewritten on every call: one small kernel on the launching stream."""
    _, b32, bias = keep
    if b32 is not None and b32.data_ptr() != bias.data_ptr():
        b32.copy_(bias)


def _ptr_key(*tensors):
    return tuple(None if t is None else (t.key() if isinstance(t, BlockScaled) else (t.data_ptr(), t.stride(0))) for t in tensors)


def _launch(ctx, d, ws) -> None:
    d.sync_block = ws.sync_block.data_ptr()
    d.inbox = ws.inbox.data_ptr() if ws.inbox is not None else None
    d.flags = ws.flags.data_ptr() if ws.flags is not None else None
    d.staging = ws.staging.data_ptr() if ws.staging is not None else None
    d.bn = ws.bn
    sfi = ws.extra.get("sf_inbox")
    d.sf_inbox = sfi.data_ptr() if sfi is not None else None
    d.comm_ctas = ws.extra.get("comm_ctas", d.comm_ctas)
    d.two_sm = ws.extra.get("two_sm", d.two_sm)
    tl = ws.extra.get("timeline")
    d.timeline = tl.data_ptr() if tl is not None else None
    if _artifacts.ACTIVE:
        _artifacts.record_launch("ops", ws.operation, ctx.cur_rank,
                                 {"M": d.M, "N": d.N, "K": d.K, "dtype": ws.dtype, "world": ctx.num_ranks, "op_code": d.op, "tile_n": d.bn,
                                  "cta_pairs": d.two_sm == 2, "comm_ctas": d.comm_ctas, "group_m": d.group_m, "use_multicast": bool(d.use_mc),
                                  "timeline": tl is not None}, source="gemm_ops.cu")
    _lib.check(_lib.kernels().iris_gemm_launch(C.byref(d), C.c_void_p(_lib.current_stream_ptr())), f"{ws.operation} launch", kernels=1)


def _local_matmul(A, B, bias=None, bias_dim=1):
    if A.is_cuda and A.dtype in _FUSED_DTYPES and A.stride(-1) == 1:
        return matmul(A, B, bias=bias, bias_dim=bias_dim)
    out = A @ B
    if bias is not None:
        out = out + (bias[:, None] if bias_dim == 0 else bias[None, :])
    return out


def _check_operands(name, A, B, bias=None, bias_len=None):
    """Shapes the kernels take on trust: the inner dimensions must agree and a bias has one entry per
    output row (the reference's convention, iris/ops/all_gather_matmul.py:146-150)."""
    if A.dim() != 2 or B.dim() != 2:
        raise ValueError(f"{name}: A and B must be matrices, got {tuple(A.shape)} and {tuple(B.shape)}")
    if A.dtype != B.dtype:
        raise TypeError(f"{name}: A is {A.dtype}, B is {B.dtype}")
    if bias is not None and bias_len is not None and (bias.dim() != 1 or bias.numel() != bias_len):
        raise ValueError(f"{name}: bias must have {bias_len} entries (one per output row), got {tuple(bias.shape)}")


def _bias32(bias):
    return bias.float().contiguous() if bias is not None else None


def _finish(ctx, async_op):
    if not async_op:
        ctx.barrier()


# ----------------------------------------------------------------------------- all_gather_matmul
def _agm_desc(ctx, out, A_sharded, B, bias, config, shard_dim):
    W = ctx.num_ranks
    if shard_dim == 1:
        M, K_local = A_sharded.shape
        K, N = B.shape
        if K != K_local * W:
            raise ValueError(f"all_gather_matmul: B has K={K} but A_sharded supplies {K_local} x {W} ranks")
        if tuple(out.shape) != (M, N):
            raise ValueError(f"all_gather_matmul: output must be {(M, N)}, got {tuple(out.shape)}")
        d, keep = _base_desc(ctx, _lib.GEMM_AG_K, M, N, K, A_sharded, B, out, config, bias_row=bias)
        d.K_local = K_local
    else:
        M_local, K = A_sharded.shape
        K2, N = B.shape
        if K != K2:
            raise ValueError(f"all_gather_matmul: A has K={K}, B has K={K2}")
        if tuple(out.shape) != (M_local * W, N):
            raise ValueError(f"all_gather_matmul: output must be {(M_local * W, N)}, got {tuple(out.shape)}")
        d, keep = _base_desc(ctx, _lib.GEMM_AG_M, M_local * W, N, K, A_sharded, B, out, config, bias_row=bias)
        d.M_local = M_local
    return d, keep


def all_gather_matmul_preamble(shmem, A_sharded, B, config=None, shard_dim=1):
    """Allocate the workspace of ``all_gather_matmul`` (collective)."""
    config = config or _DEFAULT_CONFIG
    if not _fusable(shmem, A_sharded, B):
        return FusedWorkspace(operation="all_gather_matmul", variant="unfused", world_size=shmem.num_ranks, prepared=True)
    W = shmem.num_ranks
    shape = (A_sharded.shape[0], B.shape[1]) if shard_dim == 1 else (A_sharded.shape[0] * W, B.shape[1])
    out = torch.empty(shape, dtype=torch.bfloat16 if isinstance(A_sharded, BlockScaled) else A_sharded.dtype, device=A_sharded.device)
    d, _ = _agm_desc(shmem, out, A_sharded, B, None, config, shard_dim)
    key = tuple(A_sharded.shape) + tuple(B.shape) + (shard_dim,)
    ws = _make_workspace(shmem, "all_gather_matmul", key, A_sharded.dtype, "fused", d)
    if ws is None:
        return FusedWorkspace(operation="all_gather_matmul", variant="unfused", world_size=W, prepared=True)
    return ws


def all_gather_matmul(shmem, output_tensor, A_sharded, B, bias=None, async_op=False, config=None, workspace=None,
                      shard_dim=1):
    """``output = gather(A_sharded) @ B (+ bias[:, None])``.

    ``shard_dim=1`` (reference layout, iris/ops/all_gather_matmul.py:202-204): ``A_sharded`` is
    ``(M, K/W)``, rank r holding columns ``[r*K/W, (r+1)*K/W)``. ``shard_dim=0``: ``A_sharded`` is
    ``(M/W, K)``, rank r holding rows ``[r*M/W, (r+1)*M/W)`` and the output is ``(M, N)``.
    """
    config = config or _DEFAULT_CONFIG
    W = shmem.num_ranks
    if shard_dim not in (0, 1):
        raise ValueError("shard_dim is 0 (rows sharded) or 1 (K sharded)")
    _check_operands("all_gather_matmul", A_sharded, B, bias, A_sharded.shape[0] * (W if shard_dim == 0 else 1))
    if B.shape[0] != A_sharded.shape[1] * (W if shard_dim == 1 else 1):
        raise ValueError(f"all_gather_matmul: gathered A has K = {A_sharded.shape[1] * (W if shard_dim == 1 else 1)}, B has {B.shape[0]} rows")
    key = tuple(A_sharded.shape) + tuple(B.shape) + (shard_dim,)
    ws = workspace
    if ws is None or not (ws.variant == "unfused" or ws.matches("all_gather_matmul", key, A_sharded.dtype, W, "fused")):
        ws = _auto_workspace(shmem, "all_gather_matmul", key, A_sharded.dtype, config,
                             lambda: all_gather_matmul_preamble(shmem, A_sharded, B, config, shard_dim), extra=B.stride(-1) == 1)
    if ws.variant == "unfused":
        A_sharded, B = _lower_fp8(A_sharded, B, output_tensor.dtype)
        gathered = _unfused_gather(shmem, ws, A_sharded, shard_dim)
        output_tensor.copy_(_local_matmul(gathered, B, bias, bias_dim=0))
    else:
        d, keep = _cached_desc(ws, _ptr_key(output_tensor, A_sharded, B, bias) + (id(shmem._ctx_epoch),),
                               lambda: _with_bias(bias, lambda b32: _agm_desc(shmem, output_tensor, A_sharded, B, b32, config, shard_dim)))
        _refresh_bias(keep)
        _launch(shmem, d, ws)
    _finish(shmem, async_op)
    return ws


def _unfused_gather(ctx, ws, A_sharded, shard_dim):
    W = ctx.num_ranks
    src = _on_heap(ctx, ws, "gather_src", A_sharded)
    dst = _scratch(ctx, ws, "gather_dst", (W * A_sharded.shape[0], A_sharded.shape[1]), A_sharded.dtype)
    ctx.ccl.all_gather(dst, src, async_op=False)
    if shard_dim == 0:
        return dst
    M, Kl = A_sharded.shape
    return dst.view(W, M, Kl).permute(1, 0, 2).reshape(M, W * Kl)


# ----------------------------------------------------------------------------- matmul_all_gather
def matmul_all_gather_preamble(shmem, A, B, config=None, scatter_cols=False):
    config = config or _DEFAULT_CONFIG
    if not _fusable(shmem, A, B) or config.overlap == "bulk_synchronous":
        return FusedWorkspace(operation="matmul_all_gather", variant="unfused", world_size=shmem.num_ranks, prepared=True)
    W = shmem.num_ranks
    M, K = A.shape
    N = B.shape[1]
    out = torch.empty((M * W, N) if not scatter_cols else (M, N * W), dtype=torch.bfloat16 if isinstance(A, BlockScaled) else A.dtype, device=A.device)
    op = _lib.GEMM_ALL_SCATTER if scatter_cols else _lib.GEMM_ALL_GATHER
    d, _ = _base_desc(shmem, op, M, N, K, A, B, out, config)
    ws = _make_workspace(shmem, "matmul_all_gather", tuple(A.shape) + tuple(B.shape) + (scatter_cols,), A.dtype, "fused", d)
    if ws is not None:
        ws.extra["overlap"] = "wg_specialized" if d.overlap else "fused"
    return ws or FusedWorkspace(operation="matmul_all_gather", variant="unfused", world_size=W, prepared=True)


def matmul_all_gather(shmem, output_tensor, A, B, bias=None, async_op=False, config=None, workspace=None,
                      scatter_cols=False):
    """``output[r*M:(r+1)*M] = A_r @ B`` on every rank (reference: iris/ops/matmul_all_gather.py:173-196).

    With ``scatter_cols`` the local result is ``(M, N_local)`` and lands in columns
    ``[r*N_local, (r+1)*N_local)`` of every rank's ``(M, W*N_local)`` output: the "GEMM +
    all-scatter" layout of the reference's examples/07_gemm_all_scatter.

    ``config.overlap`` selects the overlap pattern (``FusedConfig``): ``"fused"`` (default),
    ``"wg_specialized"`` (communication CTAs inside the kernel; ``"producer_consumer"`` is accepted as a
    synonym: its two-kernel form, two kernels that wait on one another on one GPU, is not built) or
    ``"bulk_synchronous"`` (GEMM, then ``ctx.ccl.all_gather``).
    """
    config = config or _DEFAULT_CONFIG
    W = shmem.num_ranks
    M, K = A.shape
    N = B.shape[1]
    want = (M, N * W) if scatter_cols else (M * W, N)
    _check_operands("matmul_all_gather", A, B, bias, M)
    if B.shape[0] != K:
        raise ValueError(f"matmul_all_gather: A has K = {K}, B has {B.shape[0]} rows")
    if tuple(output_tensor.shape) != want:
        raise ValueError(f"matmul_all_gather: output must be {want}, got {tuple(output_tensor.shape)}")
    key = tuple(A.shape) + tuple(B.shape) + (scatter_cols,)
    ws = workspace
    want_overlap = "wg_specialized" if config.overlap in ("wg_specialized", "producer_consumer") else config.overlap
    if ws is not None and ws.variant == "fused" and ws.extra.get("overlap", "fused") != want_overlap:
        ws = None            # the flags of the workgroup-specialised form belong to its own workspace
    if ws is not None and (ws.variant == "unfused") != (config.overlap == "bulk_synchronous") and _fusable(shmem, A, B):
        ws = None
    if ws is None or not (ws.variant == "unfused" or ws.matches("matmul_all_gather", key, A.dtype, W, "fused")):
        ws = _auto_workspace(shmem, "matmul_all_gather", key, A.dtype, config,
                             lambda: matmul_all_gather_preamble(shmem, A, B, config, scatter_cols), extra=B.stride(-1) == 1)
    if ws.variant == "unfused" or not shmem.is_symmetric(output_tensor):
        A, B = _lower_fp8(A, B, output_tensor.dtype)
        local = _local_matmul(A, B, bias, bias_dim=0)
        part = _on_heap(shmem, ws, "part", local)
        if scatter_cols:
            tmp = _scratch(shmem, ws, "stacked", (W * M, N), A.dtype)
            shmem.ccl.all_gather(tmp, part)
            output_tensor.copy_(tmp.view(W, M, N).permute(1, 0, 2).reshape(M, W * N))
        else:
            dst = output_tensor if shmem.is_symmetric(output_tensor) else _scratch(shmem, ws, "out", want, A.dtype)
            shmem.ccl.all_gather(dst, part)
            if dst is not output_tensor:
                output_tensor.copy_(dst)
    else:
        op = _lib.GEMM_ALL_SCATTER if scatter_cols else _lib.GEMM_ALL_GATHER
        d, keep = _cached_desc(ws, _ptr_key(output_tensor, A, B, bias) + (id(shmem._ctx_epoch),),
                               lambda: _with_bias(bias, lambda b32: _base_desc(shmem, op, M, N, K, A, B, output_tensor, config, bias_row=b32)))
        _refresh_bias(keep)
        _launch(shmem, d, ws)
    _finish(shmem, async_op)
    return ws


# ----------------------------------------------------------------------------- matmul_all_reduce
# Variants (reference: iris/ops/matmul_all_reduce.py:120-144, FusedConfig.all_reduce_variant):
#   two_shot  every tile has an owner rank; the others push their partial tile to it, the owner adds them to
#             its own accumulators and sends the finished tile to every rank (the default for large outputs)
#   one_shot  every rank sends its partial tiles to ALL ranks and sums the W partials itself: one NVLink
#             traversal and no second hop, W times the traffic; for small outputs (latency bound)
#   atomic    every rank adds its partial tiles into every rank's pre-zeroed output with remote atomics
#             (in the switch with NVLS); 16-bit accumulation in memory, summation order not fixed
#   auto      one_shot while the output is at most ONE_SHOT_MAX_BYTES, else two_shot
# spinlock and ring have no fused kernel here and are refused (ctx.ccl.all_reduce has both).
ONE_SHOT_MAX_BYTES = 4 << 20
_AR_OPS = {"two_shot": _lib.GEMM_ALL_REDUCE, "one_shot": _lib.GEMM_AR_ONE_SHOT, "atomic": _lib.GEMM_AR_ATOMIC}


def _ar_variant(config, M: int, N: int) -> str:
    v = config.all_reduce_variant
    if v == "auto":
        return "one_shot" if M * N * 2 <= ONE_SHOT_MAX_BYTES else "two_shot"
    if v not in _AR_OPS:
        raise ValueError(f"matmul_all_reduce has no fused kernel for all_reduce_variant={v!r}; use two_shot, one_shot, atomic or auto "
                         "(ctx.ccl.all_reduce implements ring and spinlock for a GEMM + collective pair)")
    return v


def matmul_all_reduce_preamble(shmem, C_out, A, B, config=None):
    config = config or _DEFAULT_CONFIG
    M, K = A.shape
    N = B.shape[1]
    variant = _ar_variant(config, M, N)
    if not _fusable(shmem, A, B) or not shmem.is_symmetric(C_out):
        return FusedWorkspace(operation="matmul_all_reduce", variant="unfused", world_size=shmem.num_ranks, prepared=True)
    d, _ = _base_desc(shmem, _AR_OPS[variant], M, N, K, A, B, C_out, config)
    ws = _make_workspace(shmem, "matmul_all_reduce", tuple(A.shape) + tuple(B.shape) + (variant,), A.dtype, "fused", d)
    if ws is not None:
        ws.extra["all_reduce_variant"] = variant
    return ws or FusedWorkspace(operation="matmul_all_reduce", variant="unfused", world_size=shmem.num_ranks, prepared=True)


def matmul_all_reduce(shmem, output_tensor, A, B, bias=None, async_op=False, config=None, workspace=None):
    """``output = sum over ranks of (A_r @ B_r)`` (+ bias) on every rank
    (reference: iris/ops/matmul_all_reduce.py:222-372). The bias, if any, is added once.
    ``config.all_reduce_variant`` picks the algorithm (see the table above this function)."""
    config = config or _DEFAULT_CONFIG
    W = shmem.num_ranks
    M, K = A.shape
    N = B.shape[1]
    _check_operands("matmul_all_reduce", A, B, bias, M)
    if B.shape[0] != K:
        raise ValueError(f"matmul_all_reduce: A has K = {K}, B has {B.shape[0]} rows")
    if tuple(output_tensor.shape) != (M, N):
        raise ValueError(f"matmul_all_reduce: output must be {(M, N)}, got {tuple(output_tensor.shape)}")
    variant = _ar_variant(config, M, N)
    key = tuple(A.shape) + tuple(B.shape) + (variant,)
    ws = workspace
    if ws is None or not (ws.variant == "unfused" or ws.matches("matmul_all_reduce", key, A.dtype, W, "fused")):
        ws = _auto_workspace(shmem, "matmul_all_reduce", key, A.dtype, config,
                             lambda: matmul_all_reduce_preamble(shmem, output_tensor, A, B, config),
                             extra=(B.stride(-1) == 1, shmem.is_symmetric(output_tensor)))
    # a bias must enter the sum exactly once: rank 0 adds it to its partial product
    b = bias if (bias is not None and shmem.cur_rank == 0) else None
    if ws.variant == "unfused":
        A, B = _lower_fp8(A, B, output_tensor.dtype)
        part = _on_heap(shmem, ws, "part", _local_matmul(A, B, b, bias_dim=0))
        dst = output_tensor if shmem.is_symmetric(output_tensor) else _scratch(shmem, ws, "out", (M, N), A.dtype)
        shmem.ccl.all_reduce(dst, part)
        if dst is not output_tensor:
            output_tensor.copy_(dst)
    else:
        if variant == "atomic":
            # every rank's output starts at zero before any rank adds to it (as the reference's preamble does)
            output_tensor.zero_()
            shmem.barrier()
        d, keep = _cached_desc(ws, _ptr_key(output_tensor, A, B, b) + (id(shmem._ctx_epoch), variant),
                               lambda: _with_bias(b, lambda b32: _base_desc(shmem, _AR_OPS[variant], M, N, K, A, B, output_tensor, config, bias_row=b32)))
        _refresh_bias(keep)
        _launch(shmem, d, ws)
    _finish(shmem, async_op)
    return ws


# ----------------------------------------------------------------------------- matmul_reduce_scatter
def matmul_reduce_scatter_preamble(shmem, C_out, A, B, config=None, scatter_rows=False):
    config = config or _DEFAULT_CONFIG
    if not _fusable(shmem, A, B):
        return FusedWorkspace(operation="matmul_reduce_scatter", variant="unfused", world_size=shmem.num_ranks, prepared=True)
    M, K = A.shape
    N = B.shape[1]
    op = _lib.GEMM_REDUCE_SCATTER if scatter_rows else _lib.GEMM_RS_TILES
    d, _ = _base_desc(shmem, op, M, N, K, A, B, C_out, config)
    ws = _make_workspace(shmem, "matmul_reduce_scatter", tuple(A.shape) + tuple(B.shape) + (scatter_rows,), A.dtype, "fused", d)
    return ws or FusedWorkspace(operation="matmul_reduce_scatter", variant="unfused", world_size=shmem.num_ranks, prepared=True)


def owned_tile_range(num_tiles: int, world: int, rank: int) -> range:
    """Tiles (row-major ids) owned by ``rank`` in the reference layout of matmul_reduce_scatter:
    contiguous blocks of ``num_tiles // world``, the last rank also taking the remainder
    (iris/mem/triton/context.py:967-979)."""
    per = max(num_tiles // world, 1)
    lo = min(rank * per, num_tiles)
    hi = num_tiles if rank == world - 1 else min(lo + per, num_tiles)
    return range(lo, hi)


def matmul_reduce_scatter(shmem, output_tensor, A, B, bias=None, async_op=False, config=None, workspace=None,
                          scatter_rows=False):
    """``sum over ranks of (A_r @ B_r)``, scattered.

    Default (reference layout, iris/ops/matmul_reduce_scatter.py:191-294): ``output`` is ``(M, N)``
    and this rank writes only the 128 x ``ws.bn`` tiles in ``owned_tile_range``; the rest of
    ``output`` is left untouched. ``scatter_rows=True``: ``output`` is ``(M/W, N)``, this rank's row
    block of the sum (the tensor-parallel layout).
    """
    config = config or _DEFAULT_CONFIG
    W = shmem.num_ranks
    M, K = A.shape
    N = B.shape[1]
    want = (M // W, N) if scatter_rows else (M, N)
    _check_operands("matmul_reduce_scatter", A, B, bias, M)
    if B.shape[0] != K:
        raise ValueError(f"matmul_reduce_scatter: A has K = {K}, B has {B.shape[0]} rows")
    if scatter_rows and M % W:
        raise ValueError(f"matmul_reduce_scatter: {M} rows do not split over {W} ranks")
    if tuple(output_tensor.shape) != want:
        raise ValueError(f"matmul_reduce_scatter: output must be {want}, got {tuple(output_tensor.shape)}")
    key = tuple(A.shape) + tuple(B.shape) + (scatter_rows,)
    ws = workspace
    if ws is None or not (ws.variant == "unfused" or ws.matches("matmul_reduce_scatter", key, A.dtype, W, "fused")):
        ws = _auto_workspace(shmem, "matmul_reduce_scatter", key, A.dtype, config,
                             lambda: matmul_reduce_scatter_preamble(shmem, output_tensor, A, B, config, scatter_rows), extra=B.stride(-1) == 1)
    b = bias if (bias is not None and shmem.cur_rank == 0) else None
    if ws.variant == "unfused":
        from ..ccl import Config

        A, B = _lower_fp8(A, B, output_tensor.dtype)
        part = _on_heap(shmem, ws, "part", _local_matmul(A, B, b, bias_dim=0))
        if scatter_rows:
            dst = _scratch(shmem, ws, "out", want, A.dtype)
            shmem.ccl.reduce_scatter(dst, part, config=Config(reduce_scatter_rows=True))
            output_tensor.copy_(dst)
        else:
            full = _scratch(shmem, ws, "full", (M, N), A.dtype)
            shmem.ccl.all_reduce(full, part)
            bn = ws.bn or 256
            tiles_n = -(-N // bn)
            for t in owned_tile_range(-(-M // 128) * tiles_n, W, shmem.cur_rank):
                tm, tn = divmod(t, tiles_n)
                output_tensor[tm * 128:(tm + 1) * 128, tn * bn:(tn + 1) * bn] = full[tm * 128:(tm + 1) * 128, tn * bn:(tn + 1) * bn]
            ws.bn = bn
    else:
        op = _lib.GEMM_REDUCE_SCATTER if scatter_rows else _lib.GEMM_RS_TILES
        d, keep = _cached_desc(ws, _ptr_key(output_tensor, A, B, b) + (id(shmem._ctx_epoch),),
                               lambda: _with_bias(b, lambda b32: _base_desc(shmem, op, M, N, K, A, B, output_tensor, config, bias_row=b32)))
        _refresh_bias(keep)
        _launch(shmem, d, ws)
    _finish(shmem, async_op)
    return ws


class OpsNamespace:
    """``ctx.ops``: the module-level functions with the context bound."""

    def __init__(self, ctx):
        self._ctx = ctx

    def matmul(self, A, B, bias=None, out=None):
        return matmul(A, B, bias=bias, out=out)

    def matmul_all_reduce(self, output_tensor, A, B, bias=None, async_op=False, config=None, workspace=None):
        return matmul_all_reduce(self._ctx, output_tensor, A, B, bias, async_op, config, workspace)

    def all_gather_matmul(self, output_tensor, A_sharded, B, bias=None, async_op=False, config=None, workspace=None,
                          shard_dim=1):
        return all_gather_matmul(self._ctx, output_tensor, A_sharded, B, bias, async_op, config, workspace, shard_dim)

    def matmul_all_gather(self, output_tensor, A, B, bias=None, async_op=False, config=None, workspace=None,
                          scatter_cols=False):
        return matmul_all_gather(self._ctx, output_tensor, A, B, bias, async_op, config, workspace, scatter_cols)

    def matmul_reduce_scatter(self, output_tensor, A, B, bias=None, async_op=False, config=None, workspace=None,
                              scatter_rows=False):
        return matmul_reduce_scatter(self._ctx, output_tensor, A, B, bias, async_op, config, workspace, scatter_rows)
