"""Expert parallelism: which rank owns which expert, and the index tables of dispatch and combine.

``MoELayer`` computes all of this on the device inside its router kernel. The functions here give
the same tables on the host, in the layouts the reference's MoE example publishes
(examples/31_expert_sharded_moe/expert_assignment.py:16-73, topk.py:22-121,
ragged_metadata.py:35-78), for code that consumes them directly, for tests and for tools:

``expert_assignment``    ``expt_bitmask int32[W, ceil(E/32)]`` (bit j of word j//32 set iff the rank
                         owns expert j), ``expt_boolmask bool[W, E]``, ``expt_map int32[W, E]``
                         (local expert id, -1 when the expert lives elsewhere).
``topk_routing``         top-k of the logits, softmax over the selected k, indices as int16.
``dispatch_tables``      ``col_sum int32[E]`` tokens per expert; ``col_sorted_indx`` maps a position
                         of the expert-sorted order to the flat ``(token, k)`` slot it came from;
                         ``row_sorted_indx`` is its inverse (the dispatch row of a slot). Slots
                         whose expert index is negative are invalid and map to -1.
``ragged_slices``        per-expert row counts and offsets of the expert-sorted buffer; the local
                         view keeps the GLOBAL offsets, because the dispatch buffer is indexed by
                         global expert-sorted row.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Sequence

import torch


@dataclass
class ExpertAssignment:
    expt_bitmask: torch.Tensor      # int32 [W, ceil(E / 32)]
    expt_boolmask: torch.Tensor     # bool  [W, E]
    expt_map: torch.Tensor          # int32 [W, E], local id or -1
    n_expts_per_shard: list

    def owner_of(self, expert: int) -> int:
        return int(torch.nonzero(self.expt_boolmask[:, expert])[0])


def uniform_expert_dict(n_shards: int, n_experts: int) -> dict:
    """Contiguous blocks: shard i owns experts ``[i E/W, (i+1) E/W)``."""
    if n_experts % n_shards:
        raise ValueError(f"{n_experts} experts do not split evenly over {n_shards} shards")
    per = n_experts // n_shards
    return {i: list(range(i * per, (i + 1) * per)) for i in range(n_shards)}


def expert_assignment(n_shards: int, n_experts: int, owners: Mapping[int, Sequence[int]] | None = None, device="cpu") -> ExpertAssignment:
    """Ownership tables from ``{shard: [experts]}`` (default: contiguous blocks). Every expert must
    have exactly one owner and every shard at least one expert."""
    owners = uniform_expert_dict(n_shards, n_experts) if owners is None else owners
    owner = torch.full((n_experts,), -1, dtype=torch.int64)
    for shard, experts in owners.items():
        if not 0 <= shard < n_shards:
            raise ValueError(f"shard {shard} out of range [0, {n_shards})")
        if len(experts) == 0:
            raise ValueError(f"shard {shard} has no experts")
        for e in experts:
            if not 0 <= e < n_experts:
                raise ValueError(f"expert id {e} out of range [0, {n_experts})")
            if owner[e] != -1:
                raise ValueError("each expert must be owned by exactly one shard")
            owner[e] = shard
    if bool((owner < 0).any()):
        raise ValueError("each expert must be owned by exactly one shard")
    boolmask = owner[None, :] == torch.arange(n_shards)[:, None]
    if not bool(boolmask.any(dim=1).all()):
        raise ValueError("every shard must own at least one expert")
    # local id = rank of the expert among its owner's experts, in increasing global id
    local = (torch.cumsum(boolmask.to(torch.int32), dim=1) - 1).to(torch.int32)
    expt_map = torch.where(boolmask, local, torch.full_like(local, -1))
    words = (n_experts + 31) // 32
    padded = torch.zeros(n_shards, words * 32, dtype=torch.int64)
    padded[:, :n_experts] = boolmask
    weights = 1 << torch.arange(32, dtype=torch.int64)
    packed = (padded.view(n_shards, words, 32) * weights).sum(-1)          # 0 .. 2^32 - 1
    bitmask = torch.where(packed >= 2**31, packed - 2**32, packed).to(torch.int32)
    return ExpertAssignment(bitmask.to(device), boolmask.to(device), expt_map.to(device),
                            [int(boolmask[s].sum()) for s in range(n_shards)])


@dataclass
class DispatchTables:
    col_sum: torch.Tensor           # int32 [E]
    col_sorted_indx: torch.Tensor   # int32 [T * k]
    row_sorted_indx: torch.Tensor   # int32 [T * k]


@dataclass
class TopkResult:
    vals: torch.Tensor              # [T, k], dtype of the logits
    indx: torch.Tensor              # int16 [T, k]
    mask_metadata: DispatchTables


def dispatch_tables(indx: torch.Tensor, n_experts: int) -> DispatchTables:
    flat = indx.reshape(-1).to(torch.int64)
    n = flat.numel()
    valid = flat >= 0
    n_valid = int(valid.sum())
    col_sum = torch.bincount(flat[valid], minlength=n_experts).to(torch.int32)
    keys = torch.where(valid, flat, torch.full_like(flat, n_experts))      # invalid slots sort last
    order = torch.argsort(keys, stable=True)
    col_sorted = torch.full((n,), -1, dtype=torch.int32, device=indx.device)
    row_sorted = torch.full((n,), -1, dtype=torch.int32, device=indx.device)
    col_sorted[:n_valid] = order[:n_valid].to(torch.int32)
    row_sorted[order[:n_valid]] = torch.arange(n_valid, dtype=torch.int32, device=indx.device)
    return DispatchTables(col_sum, col_sorted, row_sorted)


def topk_routing(logits: torch.Tensor, k: int, apply_softmax: bool = True) -> TopkResult:
    vals, indx = torch.topk(logits.float(), k, dim=1, sorted=True)
    vals = torch.softmax(vals, dim=-1) if apply_softmax else vals
    return TopkResult(vals.to(logits.dtype), indx.to(torch.int16), dispatch_tables(indx, logits.shape[1]))


@dataclass
class RaggedSlices:
    slice_sizes: torch.Tensor       # int32 [n]
    slice_offs: torch.Tensor        # int32 [n + 1]

    @property
    def n_slices(self) -> int:
        return self.slice_sizes.shape[0]


def ragged_slices(col_sum: torch.Tensor, expt_map_row: torch.Tensor | None = None) -> RaggedSlices:
    """Row ranges of the expert-sorted buffer. With ``expt_map_row`` (one rank's row of ``expt_map``)
    only that rank's experts are listed, in local order, each with its global start; the last entry
    of ``slice_offs`` is the end of the last local expert."""
    sizes = col_sum.to(torch.int32)
    offs = torch.zeros(sizes.numel() + 1, dtype=torch.int32, device=sizes.device)
    offs[1:] = torch.cumsum(sizes, dim=0)
    if expt_map_row is None:
        return RaggedSlices(sizes, offs)
    mine = torch.nonzero(expt_map_row >= 0).flatten()
    if mine.numel() == 0:
        return RaggedSlices(sizes[:0], offs[:1].clone().zero_())
    order = torch.argsort(expt_map_row[mine])                 # local id 0, 1, ...
    mine = mine[order]
    local_sizes = sizes[mine]
    local_offs = torch.cat([offs[mine], (offs[mine[-1]] + local_sizes[-1]).reshape(1)])
    return RaggedSlices(local_sizes, local_offs)
