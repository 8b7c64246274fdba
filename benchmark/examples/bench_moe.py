#!/usr/bin/env python3
"""Expert-sharded MoE layer throughput (reference: benchmark/examples/bench_moe.py).

Default point: 4096 tokens per rank, hidden 7168, 32 experts per rank, top-8, SwiGLU FFN 2048,
bf16 weights. FLOPs counted: 2 * pairs * (hidden * 2 * ffn + ffn * hidden) per rank.

``impl=nccl`` is the stock PyTorch form of the same layer: ``torch.topk`` routing, NCCL
``all_to_all_single`` dispatch (split sizes read back on the host, as the reference's pipeline does,
examples/31_expert_sharded_moe/moe.py:262), a loop of cuBLAS GEMMs over the local experts, NCCL
``all_to_all_single`` back and a weighted ``index_add_``."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402
from iris_b200.models import MoELayer  # noqa: E402

PEAK_TFLOPS = 1383.6


def moe_nccl(x, logits, wg, wu, wd, K, W, rank):
    """One forward pass of the expert-sharded layer with NCCL all-to-all and per-expert cuBLAS GEMMs."""
    T, D = x.shape
    El = wg.shape[0]
    vals, idx = torch.topk(logits, K, dim=1)
    wts = torch.softmax(vals, dim=1)
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)                   # pairs by expert, hence by owner rank
    tok = order // K
    send = x[tok]
    e_sorted = flat_e[order]
    send_counts = torch.bincount(e_sorted // El, minlength=W)
    recv_counts = torch.empty_like(send_counts)
    if W > 1:
        dist.all_to_all_single(recv_counts, send_counts)
    else:
        recv_counts.copy_(send_counts)
    sc, rc = send_counts.tolist(), recv_counts.tolist()          # host round trip: NCCL needs the split sizes
    recv = torch.empty(sum(rc), D, device=x.device, dtype=x.dtype)
    recv_e = torch.empty(sum(rc), device=x.device, dtype=e_sorted.dtype)
    if W > 1:
        dist.all_to_all_single(recv, send, rc, sc)
        dist.all_to_all_single(recv_e, e_sorted, rc, sc)
    else:
        recv.copy_(send)
        recv_e.copy_(e_sorted)
    local_e = recv_e - rank * El
    order2 = torch.argsort(local_e, stable=True)
    xs = recv[order2]
    per = torch.bincount(local_e, minlength=El).tolist()
    ys = torch.empty_like(xs)
    r0 = 0
    for j, n in enumerate(per):
        if n:
            xe = xs[r0:r0 + n]
            h = torch.nn.functional.silu(xe @ wg[j]) * (xe @ wu[j])
            ys[r0:r0 + n] = h @ wd[j]
        r0 += n
    back = torch.empty_like(ys)
    back[order2] = ys
    ret = torch.empty_like(send)
    if W > 1:
        dist.all_to_all_single(ret, back, sc, rc)
    else:
        ret.copy_(back)
    out = torch.zeros(T, D, device=x.device, dtype=torch.float32)
    out.index_add_(0, tok, ret.float() * wts.reshape(-1)[order][:, None])
    return out.to(x.dtype)


@bench.register
@bench.axis("num_ranks", [1, 2, 4, 8])
@bench.axis("impl", ["iris", "iris_fp8", "nccl"])
@bench.axis("tokens", [4096])
@bench.axis("hidden", [7168])
@bench.axis("ffn", [2048])
@bench.axis("experts_per_rank", [32])
@bench.axis("top_k", [8])
def moe_layer(state, ctx):
    W = ctx.get_num_ranks()
    T, D, F, El, K = state["tokens"], state["hidden"], state["ffn"], state["experts_per_rank"], state["top_k"]
    E = El * W
    dev = ctx.get_device()
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32          # gloo ranks: the layer's host path, fp32
    wg = (torch.randn(El, D, F, device=dev) * 0.02).to(dt)
    wu = (torch.randn(El, D, F, device=dev) * 0.02).to(dt)
    wd = (torch.randn(El, F, D, device=dev) * 0.02).to(dt)
    layer = MoELayer(ctx, D, F, E, K, max_tokens=T, w_gate=wg, w_up=wu, w_down=wd, capacity_factor=2.0, fp8=state["impl"] == "iris_fp8")
    x = torch.randn(T, D, device=dev, dtype=dt)
    logits = torch.randn(T, E, device=dev)
    out = torch.empty_like(x)
    flops = 2 * T * K * (D * 2 * F + F * D)
    state.set_flops(flops)
    # roofline: the FLOPs at the measured bf16 tensor throughput (fp8 rows: at twice that)
    state.set_roofline_us(flops / (PEAK_TFLOPS * 1e6 * (2 if state["impl"] == "iris_fp8" else 1)))
    state.set_repeat(min(state.n_repeat, 20))            # long kernels: fewer repeats than the default, never more than asked for
    state.set_warmup(min(state.n_warmup, 5))
    rank = ctx.get_rank()
    if state["impl"] == "nccl":
        state.exec(lambda: out.copy_(moe_nccl(x, logits, wg, wu, wd, K, W, rank)))
        return
    # deviation of the layer from the stock PyTorch form above on the same inputs (a counter: benchmarks report, tests
    # assert; bf16 gives a few 1e-3, the e4m3 mode a few 1e-2). Every rank runs the same collectives here.
    got = layer(x, logits, out=out)
    ref = moe_nccl(x, logits, wg, wu, wd, K, W, rank).float()
    err = (got.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-12)
    state.add_counter("max_rel_err_vs_unfused", round(err, 6))
    state.exec(lambda: layer(x, logits, out=out))


if __name__ == "__main__":
    bench.main()
