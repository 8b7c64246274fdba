"""Sequence / context parallelism: how a sequence is cut across ranks, and the head <-> sequence swap.

The reference shards only the KV cache of its flash-decode example by sequence
(examples/13_flash_decode) and offers ``ccl.all_to_all`` as the closest primitive to a Ulysses
exchange; it has no ring attention. Here:

* ``shard_sequence`` / ``unshard_sequence`` cut a ``[S, ...]`` tensor into the per-rank pieces that
  ``RingAttention`` expects, in the ``"contiguous"`` layout (rank r holds tokens
  ``[r S/W, (r+1) S/W)``) or the ``"zigzag"`` layout (chunks r and 2W-1-r of 2W, which balances the
  work of a causal mask), and put gathered pieces back into sequence order.
* ``sequence_positions`` gives the global token index of every local row, for rotary embeddings
  and masks.
* ``UlyssesExchange`` turns a sequence-sharded ``[S/W, H, D]`` tensor into a head-sharded
  ``[S, H/W, D]`` one and back with one ``ccl.all_to_all`` each way, so that an ordinary
  single-GPU attention kernel can run on full sequences of a subset of heads.
"""
from __future__ import annotations

import torch

from ..models.ring_attention import zigzag_positions

LAYOUTS = ("contiguous", "zigzag")


def sequence_positions(rank: int, world: int, seq_per_rank: int, layout: str = "contiguous", device=None) -> torch.Tensor:
    """Global positions (int64 ``[seq_per_rank]``) of the tokens rank ``rank`` holds."""
    if layout == "contiguous":
        return rank * seq_per_rank + torch.arange(seq_per_rank, device=device)
    if layout == "zigzag":
        if seq_per_rank % 2:
            raise ValueError("the zigzag layout needs an even number of tokens per rank")
        return zigzag_positions(rank, world, seq_per_rank, device=device)
    raise ValueError(f"layout must be one of {LAYOUTS}, got {layout!r}")


def shard_sequence(x: torch.Tensor, rank: int, world: int, layout: str = "contiguous", dim: int = 0) -> torch.Tensor:
    """Rank ``rank``'s piece of ``x`` along ``dim`` (a copy, contiguous)."""
    S = x.shape[dim]
    if S % world or (layout == "zigzag" and S % (2 * world)):
        raise ValueError(f"{S} tokens do not split over {world} ranks in the {layout} layout")
    pos = sequence_positions(rank, world, S // world, layout, device=x.device)
    return x.index_select(dim, pos).contiguous()


def unshard_sequence(pieces, layout: str = "contiguous", dim: int = 0) -> torch.Tensor:
    """Inverse of ``shard_sequence``: ``pieces[r]`` is rank r's piece (or one tensor with the pieces
    stacked along ``dim`` in rank order, as an all-gather leaves them)."""
    if isinstance(pieces, torch.Tensor):
        raise TypeError("pass the list of per-rank pieces; use tensor.chunk(world, dim) on a gathered tensor")
    world = len(pieces)
    cat = torch.cat(list(pieces), dim=dim)
    if layout == "contiguous":
        return cat
    per = pieces[0].shape[dim]
    pos = torch.cat([sequence_positions(r, world, per, layout, device=cat.device) for r in range(world)])
    out = torch.empty_like(cat)
    out.index_copy_(dim, pos, cat)
    return out


class UlyssesExchange:
    """Head <-> sequence swap of DeepSpeed-Ulysses style sequence parallelism over ``ccl.all_to_all``.

    ``to_heads(x)``: ``x [S/W, H, D]`` (this rank's tokens, all heads) -> ``[S, H/W, D]`` (all tokens
    in rank order, heads ``[r H/W, (r+1) H/W)``). ``to_sequence(y)`` is the inverse. Both directions
    stage through two heap buffers per shape, allocated on first use (collectively).
    """

    def __init__(self, ctx, group=None):
        self.ctx, self.group = ctx, group
        self.world = ctx.ctx_struct(group).world
        self._bufs: dict = {}

    def _staging(self, rows: int, cols: int, dtype):
        key = (rows, cols, dtype)
        if key not in self._bufs:
            self._bufs[key] = (self.ctx.empty((rows, cols), dtype=dtype), self.ctx.empty((rows, cols), dtype=dtype))
        return self._bufs[key]

    def to_heads(self, x: torch.Tensor) -> torch.Tensor:
        W = self.world
        Sl, H, D = x.shape
        if H % W:
            raise ValueError(f"{H} heads do not split over {W} ranks")
        Hl = H // W
        src, dst = self._staging(Sl, H * D, x.dtype)
        src.copy_(x.reshape(Sl, H * D))           # column chunk d = the heads rank d will own
        self.ctx.ccl.all_to_all(dst, src, group=self.group)
        # column chunk s of dst = rank s's tokens for my heads
        return dst.view(Sl, W, Hl, D).permute(1, 0, 2, 3).reshape(W * Sl, Hl, D)

    def to_sequence(self, y: torch.Tensor) -> torch.Tensor:
        W = self.world
        S, Hl, D = y.shape
        if S % W:
            raise ValueError(f"{S} tokens do not split over {W} ranks")
        Sl = S // W
        src, dst = self._staging(Sl, W * Hl * D, y.dtype)
        # column chunk d = the tokens rank d owns, for my heads
        src.view(Sl, W, Hl * D).copy_(y.reshape(W, Sl, Hl * D).permute(1, 0, 2))
        self.ctx.ccl.all_to_all(dst, src, group=self.group)
        # column chunk s of dst = heads of rank s for my tokens: heads come back in global order
        return dst.view(Sl, W * Hl, D).clone()
