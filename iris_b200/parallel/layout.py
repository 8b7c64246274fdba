"""Named parallel dimensions over the ranks of one job, and the process groups they induce.

The reference has no layout object: its tests build consecutive groups ``[0,1] [2,3]`` (tensor
parallel) and strided groups ``[0,2] [1,3]`` (data parallel) by hand with ``dist.new_group``
(tests/ccl/test_process_groups.py:49-77) and its kernels address the members of a group as
``rank_start + i * rank_stride`` (iris/host/distributed/helpers.py:234-301), which is why a group
must be an arithmetic progression of global ranks. ``ParallelLayout`` produces exactly such groups:
ranks are numbered with the FIRST dimension varying fastest, so the group along dimension ``d``
has stride ``prod(sizes of the dimensions before d)``.

    layout = ParallelLayout({"tp": 4, "dp": 2})          # 8 ranks: tp inside a node half, dp across
    layout.build_groups()                                  # collective: every rank, same order
    ctx.ccl.all_reduce(out, inp, group=layout.group("tp"))

Put the dimension that communicates most first: its members are neighbouring ranks.
"""
from __future__ import annotations

import math
from typing import Mapping


class ParallelLayout:
    """``ParallelLayout({"tp": 4, "dp": 2})``: ranks numbered with the first dimension fastest; groups
    along a dimension are arithmetic progressions of global ranks (see the module docstring)."""

    def __init__(self, dims: Mapping[str, int], world_size: int | None = None, rank: int | None = None):
        if not dims:
            raise ValueError("at least one dimension is needed")
        self.names = list(dims)
        self.sizes = [int(dims[n]) for n in self.names]
        if any(s < 1 for s in self.sizes):
            raise ValueError(f"dimension sizes must be positive, got {dict(dims)}")
        total = math.prod(self.sizes)
        if world_size is None or rank is None:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                world_size = dist.get_world_size() if world_size is None else world_size
                rank = dist.get_rank() if rank is None else rank
            else:
                world_size = total if world_size is None else world_size
                rank = 0 if rank is None else rank
        if total != world_size:
            raise ValueError(f"dimensions {dict(dims)} describe {total} ranks, the job has {world_size}")
        if not 0 <= rank < world_size:
            raise ValueError(f"rank {rank} out of range")
        self.world_size, self.rank = world_size, rank
        self._strides = [math.prod(self.sizes[:i]) for i in range(len(self.sizes))]
        self._groups: dict[str, object] = {}

    # ------------------------------------------------------------------ pure arithmetic
    def size(self, name: str) -> int:
        return self.sizes[self._index(name)]

    def stride(self, name: str) -> int:
        """Distance in global ranks between neighbours along ``name``."""
        return self._strides[self._index(name)]

    def _index(self, name: str) -> int:
        try:
            return self.names.index(name)
        except ValueError:
            raise KeyError(f"no dimension {name!r}; dimensions are {self.names}") from None

    def coords(self, rank: int | None = None) -> dict[str, int]:
        """Position of ``rank`` (default: this rank) along every dimension."""
        r = self.rank if rank is None else rank
        return {n: (r // st) % sz for n, sz, st in zip(self.names, self.sizes, self._strides)}

    def coord(self, name: str, rank: int | None = None) -> int:
        return self.coords(rank)[name]

    def rank_of(self, **coords: int) -> int:
        """Global rank at the given coordinates (dimensions left out keep this rank's position)."""
        c = self.coords()
        for k, v in coords.items():
            if not 0 <= v < self.size(k):
                raise ValueError(f"{k}={v} outside [0, {self.size(k)})")
            c[k] = v
        return sum(c[n] * st for n, st in zip(self.names, self._strides))

    def ranks(self, name: str, rank: int | None = None) -> list[int]:
        """Global ranks of the group along ``name`` that contains ``rank``: an arithmetic progression."""
        i = self._index(name)
        r = self.rank if rank is None else rank
        first = r - ((r // self._strides[i]) % self.sizes[i]) * self._strides[i]
        return [first + k * self._strides[i] for k in range(self.sizes[i])]

    def all_groups(self, name: str) -> list[list[int]]:
        """Every group along ``name``, ordered by first member: a partition of the ranks."""
        seen, out = set(), []
        for r in range(self.world_size):
            if r not in seen:
                g = self.ranks(name, r)
                seen.update(g)
                out.append(g)
        return out

    # ------------------------------------------------------------------ process groups
    def build_groups(self, names=None, backend=None) -> "ParallelLayout":
        """Create the process groups of the given dimensions (default: all). Collective: every rank
        creates every group, in the same order, as ``torch.distributed.new_group`` requires."""
        import torch.distributed as dist

        for n in (self.names if names is None else list(names)):
            if n in self._groups:
                continue
            mine = None
            for members in self.all_groups(n):
                g = dist.new_group(members, backend=backend)
                if self.rank in members:
                    mine = g
            self._groups[n] = mine
        return self

    def group(self, name: str):
        """This rank's process group along ``name`` (``build_groups`` first). A dimension that spans
        the whole job returns ``None``, i.e. the default group, which keeps the NVLS paths usable."""
        self._index(name)
        if self.size(name) == self.world_size:
            return None
        if name not in self._groups:
            raise RuntimeError(f"group {name!r} has not been built; call build_groups() on every rank first")
        return self._groups[name]

    def __repr__(self) -> str:
        dims = ", ".join(f"{n}={s}" for n, s in zip(self.names, self.sizes))
        return f"ParallelLayout({dims}; rank {self.rank} at {self.coords()})"
