"""Data parallelism: gradients summed across replicas through buckets on the symmetric heap.

The reference has data parallelism only as strided process groups for its collectives
(iris/host/distributed/helpers.py:281-299, tests/ccl/test_process_groups.py:57-77); what a training
loop does with them is left to the user. ``GradientBuckets`` is that missing piece: parameters are
packed, in order, into a few large heap buffers; a step's gradients are copied in, each bucket is
summed with ``ctx.ccl.all_reduce`` (NVLS or two-shot for buckets of this size, chosen by the
collective itself) and the averages are copied back into ``param.grad``.

    buckets = GradientBuckets(ctx, model.parameters(), group=layout.group("dp"))
    buckets.attach()            # optional: start a bucket's all-reduce as soon as its gradients exist
    loss.backward()
    buckets.finish()            # wait, average, write back   (or buckets.all_reduce() without attach)

Buckets are sized for launch latency and overlap, not for link count: through NVSwitch a collective
costs the same whichever peers take part, so a few tens of megabytes per bucket amortise the launch
while leaving several buckets to overlap with the rest of the backward pass. Every rank must build
the buckets from the same parameter list (they are heap allocations), and with ``attach()`` every
rank must run the same autograd graph: the collectives are launched in the order in which buckets
fill up, and kernels that wait for one another have to be queued in the same order on every rank
(a rank that differs runs into the bounded waits and ``ctx.check()`` reports it).
"""
from __future__ import annotations

import torch

_COLS = 4096   # bucket row length in elements: 16-byte vectors for every dtype, whole rows per CTA


class _Bucket:
    def __init__(self, ctx, dtype, params, numel):
        rows = -(-numel // _COLS)
        self.dtype, self.params, self.numel = dtype, params, numel
        self.inp = ctx.zeros((rows, _COLS), dtype=dtype)
        self.out = ctx.zeros((rows, _COLS), dtype=dtype)
        self.slices = []
        off = 0
        for p in params:
            self.slices.append((off, off + p.numel()))
            off += p.numel()
        self.pending = len(params)
        self.launched = False
        self.workspace = None


class GradientBuckets:
    """Heap buckets over ``params`` (those that require a gradient), summed or averaged across
    ``group`` by ``all_reduce()`` after backward, or by ``attach()`` + ``finish()`` during it."""

    def __init__(self, ctx, params, bucket_bytes: int = 64 << 20, group=None, average: bool = True, reduce_dtype=None):
        self.ctx, self.group, self.average = ctx, group, average
        self.world = ctx.ctx_struct(group).world
        plist = [p for p in params if p.requires_grad]
        if not plist:
            raise ValueError("no parameter requires a gradient")
        self.buckets: list[_Bucket] = []
        self._where: dict[int, tuple[_Bucket, int]] = {}
        # gradients become available roughly in reverse order of the parameters: fill buckets from
        # the back so that the first bucket to complete is also the first one created
        cur, cur_dtype, cur_n = [], None, 0
        for p in reversed(plist):
            dt = reduce_dtype or p.dtype
            size = p.numel() * torch.empty((), dtype=dt).element_size()
            if cur and (dt != cur_dtype or (cur_n * torch.empty((), dtype=cur_dtype).element_size() + size) > bucket_bytes):
                self._close(cur, cur_dtype, cur_n)
                cur, cur_n = [], 0
            cur.append(p)
            cur_dtype = dt
            cur_n += p.numel()
        self._close(cur, cur_dtype, cur_n)
        self._hooks = []

    def _close(self, params, dtype, numel):
        b = _Bucket(self.ctx, dtype, params, numel)
        for i, p in enumerate(params):
            self._where[id(p)] = (b, i)
        self.buckets.append(b)

    # ------------------------------------------------------------------ one bucket
    def _copy_in(self, b: _Bucket) -> None:
        flat = b.inp.view(-1)
        for p, (lo, hi) in zip(b.params, b.slices):
            if p.grad is None:
                flat[lo:hi].zero_()      # a parameter that took no part in this step adds nothing
            else:
                flat[lo:hi].copy_(p.grad.reshape(-1))

    def _launch(self, b: _Bucket) -> None:
        self._copy_in(b)
        b.workspace = self.ctx.ccl.all_reduce(b.out, b.inp, group=self.group, async_op=True, workspace=b.workspace)
        b.launched = True

    def _copy_out(self, b: _Bucket) -> None:
        flat = b.out.view(-1)
        scale = 1.0 / self.world if self.average else None
        for p, (lo, hi) in zip(b.params, b.slices):
            g = flat[lo:hi].view(p.shape)
            if p.grad is None:
                p.grad = torch.empty_like(p)
            if scale is None:
                p.grad.copy_(g)
            else:
                torch.mul(g, scale, out=p.grad) if p.grad.dtype == g.dtype else p.grad.copy_(g.float() * scale)

    # ------------------------------------------------------------------ whole step
    def all_reduce(self) -> None:
        """Sum (or average) every gradient across the group, after ``backward()`` has finished."""
        for b in self.buckets:
            if not b.launched:
                self._launch(b)
        self.finish()

    def attach(self) -> "GradientBuckets":
        """Install hooks that launch a bucket's all-reduce when the last of its gradients has been
        accumulated, so that communication overlaps the rest of the backward pass."""
        if self._hooks:
            return self
        for b in self.buckets:
            for p in b.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))
        return self

    def detach(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []

    def _on_grad(self, p) -> None:
        b, _ = self._where[id(p)]
        b.pending -= 1
        if b.pending == 0 and not b.launched:
            self._launch(b)

    def finish(self) -> None:
        """Launch what the hooks did not (parameters without a gradient this step), wait until every
        rank's reductions are done, write the results back and re-arm the buckets."""
        for b in self.buckets:
            if not b.launched:
                self._launch(b)
        # peers read this rank's input buckets while they reduce: nobody may refill them (the next
        # step) before every rank is past this point
        self.ctx.device_barrier(group=self.group)
        for b in self.buckets:
            self._copy_out(b)
            b.pending, b.launched = len(b.params), False

    def nbytes(self) -> int:
        return sum(2 * b.inp.numel() * b.inp.element_size() for b in self.buckets)
