#!/usr/bin/env python3
"""Distributed flash-decode throughput (reference: benchmark/examples/bench_flash_decode.py).

64 query heads, 8 KV heads, head_dim 128, bf16; the total KV length is split evenly over the ranks.
Bytes counted are the K and V bytes each rank must read (the roofline is those bytes over the
measured HBM bandwidth).

``impl=nccl`` is the reference's baseline (examples/benchmark/reference/flash_decode_rccl/
flash_decode_layer_rccl.py:100-130): the same local split-K decode, then ``all_gather_into_tensor`` of
the partial (o, lse) over NCCL and a log-sum-exp merge, instead of the in-kernel exchange."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402
from iris_b200.models import FlashDecodeLayer  # noqa: E402

HBM_GBPS = 6553.0


@bench.register
@bench.axis("num_ranks", [1, 2, 4, 8])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("batch", [1, 8, 32, 64])
@bench.axis("total_kv", [32768, 131072, 524288])
def flash_decode(state, ctx):
    W, B, total = ctx.get_num_ranks(), state["batch"], state["total_kv"]
    Hq, Hkv, D, page = 64, 8, 128, 64
    L = total // max(W, 8) if W < 8 else total // W     # per-rank shard of the 8-way split
    nb = -(-L // page)
    need = 2 * B * nb * page * Hkv * D * 2
    if need > 60 << 30:
        state.skip("KV shard does not fit the benchmark's memory budget")
    dev = ctx.get_device()
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32          # gloo ranks: the layer's host path, fp32
    kc = torch.randn(B * nb, page, Hkv, D, device=dev, dtype=dt)
    vc = torch.randn(B * nb, page, Hkv, D, device=dev, dtype=dt)
    table = torch.arange(B * nb, device=dev, dtype=torch.int32).view(B, nb)
    lens = torch.full((W, B), L, device=dev, dtype=torch.int32)
    q = torch.randn(B, Hq, D, device=dev, dtype=dt)
    if W > 1:
        dist.broadcast(q, 0)                      # the query is replicated, the KV cache is what is sharded
    layer = FlashDecodeLayer(ctx, Hq, Hkv, D, max_batch=B)
    out = torch.empty(B, Hq, D, device=dev, dtype=dt)
    kv_bytes = 2 * B * L * Hkv * D * 2
    state.set_bytes(kv_bytes)
    state.set_roofline_us(kv_bytes / (HBM_GBPS * 1e3))
    state.set_repeat(min(state.n_repeat, 30))            # fewer repeats than the default, never more than asked for
    if state["impl"] == "nccl":
        po = torch.empty(B, Hq, D, device=dev, dtype=dt)
        g_o = torch.empty(W, B, Hq, D, device=dev, dtype=dt)
        g_l = torch.empty(W, B, Hq, device=dev, dtype=torch.float32)

        def base():
            _, pl = layer(q, kc, vc, lens, table, out=po, local_only=True)
            if W > 1:
                dist.all_gather_into_tensor(g_o, po)
                dist.all_gather_into_tensor(g_l, pl)
                out.copy_(FlashDecodeLayer.merge_partials(g_o, g_l))
            else:
                out.copy_(po)

        state.exec(base)
        return
    # deviation of batch entry 0 from fp32 attention over the keys of all ranks (a counter: benchmarks report, tests
    # assert; bf16 gives a few 1e-3). Every rank runs the same collectives here.
    got = layer(q, kc, vc, lens, table, out=out)
    got = got[0] if isinstance(got, tuple) else got
    k0 = kc[table[0].long()].reshape(-1, Hkv, D)[:L].contiguous()
    v0 = vc[table[0].long()].reshape(-1, Hkv, D)[:L].contiguous()
    ks, vs = [torch.empty_like(k0) for _ in range(W)], [torch.empty_like(v0) for _ in range(W)]
    if W > 1:
        dist.all_gather(ks, k0)
        dist.all_gather(vs, v0)
    else:
        ks, vs = [k0], [v0]
    qf = q[0].float().view(Hkv, Hq // Hkv, D)
    sc = torch.einsum("hgd,khd->hgk", qf, torch.cat(ks).float()) / D ** 0.5
    ref = torch.einsum("hgk,khd->hgd", torch.softmax(sc, dim=-1), torch.cat(vs).float()).reshape(Hq, D)
    state.add_counter("max_rel_err", round((got[0].float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-12), 6))
    del ks, vs, sc, ref, k0, v0
    state.exec(lambda: layer(q, kc, vc, lens, table, out=out))


if __name__ == "__main__":
    bench.main()
