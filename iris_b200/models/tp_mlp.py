"""Tensor-parallel MLP with sequence-parallel activations, forward and backward on the fused ops.

Rank r holds ``M / W`` rows of the activations (sequence parallel), a column block ``W1[:, r]`` of
the up projection and the matching row block ``W2[r, :]`` of the down projection:

    forward     H  = act(all_gather(X) @ W1_r)              all_gather_matmul       (one kernel)
                Y  = reduce_scatter(H @ W2_r)                matmul_reduce_scatter   (one kernel)
    backward    dH = all_gather(dY) @ W2_r^T                 all_gather_matmul
                dX = reduce_scatter((dH * act') @ W1_r^T)    matmul_reduce_scatter
                dW1 = all_gather(X)^T @ (dH * act'),  dW2 = H^T @ all_gather(dY)
                                                             ccl.all_gather + torch.matmul (plain library GEMMs)

The reference wraps its GEMM examples in a ``torch.autograd.Function`` the same way
(examples/07_gemm_all_scatter/matmul_wrapper.py); it has no backward through its fused ops.
Shapes the fused kernels do not take (rows per rank not a multiple of 128, fp32) go through the
unfused path of ``iris_b200.ops`` automatically.
"""
from __future__ import annotations

import torch

_ACTS = {
    None: (lambda x: x, lambda x: torch.ones_like(x)),
    "silu": (torch.nn.functional.silu, lambda x: torch.sigmoid(x) * (1 + x * (1 - torch.sigmoid(x)))),
    "gelu": (lambda x: torch.nn.functional.gelu(x, approximate="tanh"), None),
}


def _act_grad(name, x):
    if name == "gelu":      # derivative of the tanh approximation through autograd on a detached copy
        with torch.enable_grad():
            xx = x.detach().float().requires_grad_(True)
            y = torch.nn.functional.gelu(xx, approximate="tanh")
            (g,) = torch.autograd.grad(y.sum(), xx)
        return g.to(x.dtype)
    return _ACTS[name][1](x.float()).to(x.dtype)


class _TPMLPFunction(torch.autograd.Function):
    @staticmethod
    def forward(fctx, x, w1, w2, layer):
        ctx, W = layer.ctx, layer.ctx.get_num_ranks()
        M_local, K = x.shape
        F = w1.shape[1]
        xd, w1d, w2d = x.detach(), w1.detach(), w2.detach()
        h_pre = torch.empty(W * M_local, F, dtype=x.dtype, device=x.device)
        layer._ws["ag1"] = ctx.ops.all_gather_matmul(h_pre, xd, w1d, shard_dim=0, workspace=layer._ws.get("ag1"), async_op=True)
        h = _ACTS[layer.activation][0](h_pre) if layer.activation else h_pre
        y = torch.empty(M_local, K, dtype=x.dtype, device=x.device)
        layer._ws["rs1"] = ctx.ops.matmul_reduce_scatter(y, h, w2d, scatter_rows=True, workspace=layer._ws.get("rs1"), async_op=True)
        fctx.layer = layer
        fctx.save_for_backward(xd, w1d, w2d, h_pre)
        return y

    @staticmethod
    def backward(fctx, dy):
        layer = fctx.layer
        ctx, W = layer.ctx, layer.ctx.get_num_ranks()
        x, w1, w2, h_pre = fctx.saved_tensors
        dy = dy.contiguous()
        M_local, K = x.shape
        F = w1.shape[1]
        # dH = all_gather(dY) @ W2^T (W2^T is the K-major view the kernel takes without a copy)
        dh = torch.empty(W * M_local, F, dtype=x.dtype, device=x.device)
        layer._ws["ag2"] = ctx.ops.all_gather_matmul(dh, dy, w2.t(), shard_dim=0, workspace=layer._ws.get("ag2"), async_op=True)
        if layer.activation:
            dh = dh * _act_grad(layer.activation, h_pre)
        # dX = reduce_scatter(dH @ W1^T)
        dx = torch.empty(M_local, K, dtype=x.dtype, device=x.device)
        layer._ws["rs2"] = ctx.ops.matmul_reduce_scatter(dx, dh, w1.t(), scatter_rows=True, workspace=layer._ws.get("rs2"), async_op=True)
        # weight gradients: gathered activations, then plain library GEMMs
        if W > 1:
            x_loc, dy_loc, x_all, dy_all = layer._gather_buffers(M_local, K, x.dtype)
            x_loc.copy_(x)
            dy_loc.copy_(dy)
            ctx.ccl.all_gather(x_all, x_loc, async_op=True)
            ctx.ccl.all_gather(dy_all, dy_loc, async_op=True)
        else:
            x_all, dy_all = x, dy
        h = _ACTS[layer.activation][0](h_pre) if layer.activation else h_pre
        dw1 = x_all.t() @ dh
        dw2 = h.t() @ dy_all
        return dx, dw1, dw2, None


class TensorParallelMLP(torch.nn.Module):
    """``y = reduce_scatter(act(all_gather(x) @ W1_r) @ W2_r)`` with ``x``, ``y`` of shape ``(M / W, hidden)``.

    ``w1`` is this rank's ``(hidden, ffn / W)`` block, ``w2`` its ``(ffn / W, hidden)`` block (random
    init when omitted). The workspaces of the four fused ops and the heap buffers of the backward
    pass's all-gathers are created on first use (collectively) and reused by later steps.
    """

    def __init__(self, ctx, hidden: int, ffn_local: int, activation: str | None = "silu", dtype=torch.bfloat16, w1=None,
                 w2=None):
        super().__init__()
        if activation not in _ACTS:
            raise ValueError(f"unknown activation {activation!r}")
        self.ctx, self.activation = ctx, activation
        dev = ctx.get_device()
        self.w1 = torch.nn.Parameter((torch.randn(hidden, ffn_local, device=dev) * 0.02).to(dtype) if w1 is None else w1.detach().clone())
        self.w2 = torch.nn.Parameter((torch.randn(ffn_local, hidden, device=dev) * 0.02).to(dtype) if w2 is None else w2.detach().clone())
        self._ws: dict = {}
        self._bufs: dict = {}

    def _gather_buffers(self, M_local: int, K: int, dtype):
        """Heap tensors of the backward pass's two all-gathers, allocated once per shape (collective)."""
        key = (M_local, K, dtype)
        if key not in self._bufs:
            W = self.ctx.get_num_ranks()
            self._bufs[key] = (self.ctx.empty((M_local, K), dtype=dtype), self.ctx.empty((M_local, K), dtype=dtype),
                               self.ctx.empty((W * M_local, K), dtype=dtype), self.ctx.empty((W * M_local, K), dtype=dtype))
        return self._bufs[key]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _TPMLPFunction.apply(x, self.w1, self.w2, self)
