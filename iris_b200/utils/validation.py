"""Result checks shared by examples and benchmarks: compare against plain PyTorch, report the first
mismatch through the context's rank-prefixed logger, return a bool.

Same helpers as the reference's examples/common/validation.py:7-165 (``validate_gemm``,
``validate_all_scatter``, ``validate_all_reduce``, ``validate_reduce_scatter``), plus the row
layout of an all-gather. Oracles are computed in fp32 from the ranks' inputs gathered with
``torch.distributed``; every function is collective where it needs other ranks' data.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _report(ctx, what: str, got: torch.Tensor, want: torch.Tensor, atol: float, rtol: float = 0.0) -> bool:
    got32, want32 = got.float(), want.float()
    close = torch.isclose(got32, want32, atol=atol, rtol=rtol)
    if bool(close.all()):
        return True
    bad = torch.nonzero(~close)
    first = tuple(bad[0].tolist())
    ctx.error(f"{what}: {bad.shape[0]} of {got.numel()} elements differ (atol {atol}); max abs difference "
              f"{(got32 - want32).abs().max().item():.6g}; first at {first}: got {got32[first].item():.6g}, "
              f"expected {want32[first].item():.6g}")
    return False


def _gather(t: torch.Tensor, group=None) -> list:
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return [t]
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return parts


def validate_gemm(A, B, C, ctx, atol: float = 1.0, bias=None) -> bool:
    """``C == A @ B`` (+ bias per column) on this rank."""
    want = A.float() @ B.float()
    if bias is not None:
        want = want + bias.float()
    return _report(ctx, "gemm", C, want, atol)


def validate_all_scatter(local_tensor, global_tensor, ctx, atol: float = 1.0, group=None) -> bool:
    """Rank r's ``(M, N)`` tensor must sit in columns ``[r N, (r+1) N)`` of every rank's ``(M, W N)``."""
    parts = _gather(local_tensor, group)
    return _report(ctx, "all_scatter", global_tensor, torch.cat([p.float() for p in parts], dim=1), atol)


def validate_all_gather(local_tensor, global_tensor, ctx, atol: float = 0.0, group=None) -> bool:
    """Rank r's ``(M, N)`` tensor must sit in rows ``[r M, (r+1) M)`` of every rank's ``(W M, N)``."""
    parts = _gather(local_tensor, group)
    return _report(ctx, "all_gather", global_tensor, torch.cat([p.float() for p in parts], dim=0), atol)


def validate_all_reduce(local_tensor, global_tensor, ctx, atol: float = 1.0, group=None) -> bool:
    """``global_tensor`` must be the sum over ranks of ``local_tensor``."""
    parts = _gather(local_tensor, group)
    return _report(ctx, "all_reduce", global_tensor, torch.stack([p.double() for p in parts]).sum(0).float(), atol)


def validate_reduce_scatter(local_tensor, output_tensor, ctx, tp_group=None, atol: float = 1.0) -> bool:
    """``output_tensor`` (``(M / W, N)``) must be this rank's row block of the sum over ranks."""
    parts = _gather(local_tensor, tp_group)
    total = torch.stack([p.double() for p in parts]).sum(0).float()
    world = len(parts)
    me = dist.get_rank(tp_group) if dist.is_initialized() else 0
    rows = total.shape[0] // world
    return _report(ctx, "reduce_scatter", output_tensor, total[me * rows:(me + 1) * rows], atol)
