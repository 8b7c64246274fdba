"""Tensor-parallel linear layers on the fused GEMM + collective kernels.

The reference stops at the four fused ops (iris/ops/*.py) and leaves their composition to the
caller; its own docstrings name the patterns (column-parallel GEMM + all-gather, row-parallel GEMM +
all-reduce / reduce-scatter, all-gather + GEMM). These modules are those patterns with the weight
shard attached:

``ColumnParallelLinear``  weight ``(in, out / W)`` per rank.
    sequence_parallel=True   x is this rank's ``(M / W, in)`` rows; ``y = all_gather(x) @ W_r`` in one
                             kernel (``all_gather_matmul``), result ``(M, out / W)``.
    sequence_parallel=False  x is the replicated ``(M, in)``; ``y = x @ W_r`` is a local GEMM.
    gather_output=True       additionally gathers the column blocks: ``(M, out)`` on every rank
                             (``matmul_all_gather`` with the all-scatter layout).

``RowParallelLinear``     weight ``(in / W, out)`` per rank, x is ``(M, in / W)``.
    sequence_parallel=True   ``y = reduce_scatter(x @ W_r)``: this rank's ``(M / W, out)`` rows
                             (``matmul_reduce_scatter``).
    sequence_parallel=False  ``y = all_reduce(x @ W_r)``: ``(M, out)`` on every rank
                             (``matmul_all_reduce``).

Forward only (inference); ``TensorParallelMLP`` is the trainable pairing of the two with its own
backward. Shapes or dtypes the fused kernels do not take run as GEMM + collective inside
``iris_b200.ops``. Workspaces and output buffers are kept per input shape, so a layer called in a
loop allocates nothing after its first call with a shape; every rank must call with the same shapes
in the same order (the buffers are heap allocations). The tensor a layer returns is one of those
buffers: it is overwritten by the layer's next call with the same shape, so copy it to keep it.
"""
from __future__ import annotations

import torch

from ..models.tp_mlp import TensorParallelMLP  # noqa: F401  (re-exported)


def _init_weight(rows: int, cols: int, dtype, device, seed: int | None):
    g = None
    if seed is not None:
        g = torch.Generator(device="cpu").manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * (1.0 / max(rows, 1)) ** 0.5
    return w.to(dtype).to(device)


class _TPLinearBase(torch.nn.Module):
    def __init__(self, ctx, weight: torch.Tensor, bias: torch.Tensor | None):
        super().__init__()
        self.ctx = ctx
        self.weight = torch.nn.Parameter(weight, requires_grad=False)
        self.bias = torch.nn.Parameter(bias, requires_grad=False) if bias is not None else None
        self._ws: dict = {}
        self._out: dict = {}

    def _buffer(self, tag: str, shape, dtype, on_heap: bool) -> torch.Tensor:
        key = (tag, tuple(shape), dtype)
        buf = self._out.get(key)
        if buf is None:
            buf = self.ctx.empty(tuple(shape), dtype=dtype) if on_heap else torch.empty(tuple(shape), dtype=dtype, device=self.ctx.get_device())
            self._out[key] = buf
        return buf

    def _check(self, x: torch.Tensor, cols: int) -> None:
        if x.dim() != 2 or x.shape[1] != cols:
            raise ValueError(f"{type(self).__name__}: input must be (rows, {cols}), got {tuple(x.shape)}")
        if x.dtype != self.weight.dtype:
            raise TypeError(f"{type(self).__name__}: input dtype {x.dtype} differs from the weight's {self.weight.dtype}")


class ColumnParallelLinear(_TPLinearBase):
    """``y = x @ W[:, r-th column block]`` with this rank's ``(in, out / W)`` weight; all-gather of
    sequence-parallel input fused into the GEMM, optional gather of the output columns."""

    def __init__(self, ctx, in_features: int, out_features_local: int, bias: bool = False, sequence_parallel: bool = True,
                 gather_output: bool = False, dtype=torch.bfloat16, weight: torch.Tensor | None = None,
                 bias_value: torch.Tensor | None = None, seed: int | None = None):
        dev = ctx.get_device()
        w = weight.detach().clone().to(dev) if weight is not None else _init_weight(in_features, out_features_local, dtype, dev, seed)
        if tuple(w.shape) != (in_features, out_features_local):
            raise ValueError(f"weight must be {(in_features, out_features_local)}, got {tuple(w.shape)}")
        b = None
        if bias or bias_value is not None:
            b = bias_value.detach().clone().to(dev) if bias_value is not None else torch.zeros(out_features_local, dtype=w.dtype, device=dev)
        super().__init__(ctx, w, b)
        self.in_features, self.out_features_local = in_features, out_features_local
        self.sequence_parallel, self.gather_output = sequence_parallel, gather_output

    def _full_bias(self) -> torch.Tensor:
        """Every rank's bias block side by side (gathered once, on the first call that needs it)."""
        full = self._out.get("full_bias")
        if full is None:
            import torch.distributed as dist

            parts = [torch.empty_like(self.bias.data) for _ in range(self.ctx.get_num_ranks())]
            dist.all_gather(parts, self.bias.data.contiguous())
            full = self._out["full_bias"] = torch.cat(parts)
        return full

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ctx, W = self.ctx, self.ctx.get_num_ranks()
        self._check(x, self.in_features)
        rows = x.shape[0] * W if self.sequence_parallel else x.shape[0]
        n = self.out_features_local
        if self.gather_output and not self.sequence_parallel:
            # GEMM whose epilogue writes this rank's column block into every rank's output
            out = self._buffer("gathered", (rows, W * n), x.dtype, on_heap=True)
            self._ws["mag"] = ctx.ops.matmul_all_gather(out, x, self.weight, scatter_cols=True, workspace=self._ws.get("mag"))
            if self.bias is not None:
                out += self._full_bias()
            return out
        if self.sequence_parallel:
            y = self._buffer("agm", (rows, n), x.dtype, on_heap=False)
            self._ws["agm"] = ctx.ops.all_gather_matmul(y, x, self.weight, shard_dim=0, workspace=self._ws.get("agm"), async_op=True)
            if self.bias is not None:
                y += self.bias
        else:
            from ..ops import _local_matmul

            y = _local_matmul(x, self.weight, self.bias, bias_dim=1)
        if not self.gather_output:
            return y
        # sequence-parallel input and gathered output: exchange the column blocks afterwards
        # (y already carries this rank's bias)
        part = self._buffer("part", (rows, n), x.dtype, on_heap=True)
        part.copy_(y)
        stacked = self._buffer("stacked", (W * rows, n), x.dtype, on_heap=True)
        ctx.ccl.all_gather(stacked, part)
        return stacked.view(W, rows, n).permute(1, 0, 2).reshape(rows, W * n)


class RowParallelLinear(_TPLinearBase):
    """``y = sum over ranks of x_r @ W[r-th row block]`` with this rank's ``(in / W, out)`` weight;
    the sum is a reduce-scatter (sequence parallel) or an all-reduce fused into the GEMM."""

    def __init__(self, ctx, in_features_local: int, out_features: int, bias: bool = False, sequence_parallel: bool = True,
                 dtype=torch.bfloat16, weight: torch.Tensor | None = None, bias_value: torch.Tensor | None = None,
                 seed: int | None = None):
        dev = ctx.get_device()
        w = weight.detach().clone().to(dev) if weight is not None else _init_weight(in_features_local, out_features, dtype, dev, seed)
        if tuple(w.shape) != (in_features_local, out_features):
            raise ValueError(f"weight must be {(in_features_local, out_features)}, got {tuple(w.shape)}")
        b = None
        if bias or bias_value is not None:
            b = bias_value.detach().clone().to(dev) if bias_value is not None else torch.zeros(out_features, dtype=w.dtype, device=dev)
        super().__init__(ctx, w, b)
        self.in_features_local, self.out_features = in_features_local, out_features
        self.sequence_parallel = sequence_parallel

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ctx, W = self.ctx, self.ctx.get_num_ranks()
        self._check(x, self.in_features_local)
        M = x.shape[0]
        if self.sequence_parallel:
            if M % W:
                raise ValueError(f"RowParallelLinear: {M} rows do not split over {W} ranks")
            y = self._buffer("rs", (M // W, self.out_features), x.dtype, on_heap=False)
            self._ws["rs"] = ctx.ops.matmul_reduce_scatter(y, x, self.weight, scatter_rows=True, workspace=self._ws.get("rs"),
                                                           async_op=True)
        else:
            y = self._buffer("ar", (M, self.out_features), x.dtype, on_heap=True)
            self._ws["ar"] = ctx.ops.matmul_all_reduce(y, x, self.weight, workspace=self._ws.get("ar"), async_op=True)
        if self.bias is not None:
            y += self.bias     # the same on every rank, added after the sum
        return y
