#!/usr/bin/env python3
"""Expert-sharded mixture of experts: every rank holds E / W experts and T tokens; tokens are routed
(top-k), dispatched to the ranks of their experts, run through the SwiGLU expert FFN and combined
back, weighted by the router (reference: examples/31_expert_sharded_moe). Validated against the
unsharded fp32 computation.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/moe.py
"""
import torch

from _common import finish, init

if __name__ == "__main__":
    ctx = init(1 << 30)
    from iris_b200.models import MoELayer, reference_moe

    W, r = ctx.get_num_ranks(), ctx.get_rank()
    dev = ctx.get_device()
    dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
    T, D, F, E, K = 96, 256, 128, 8 * W, 2
    El = E // W
    torch.manual_seed(5)                                   # all experts' weights, same on every rank
    wg = (torch.randn(E, D, F) * 0.05).to(dt).to(dev)
    wu = (torch.randn(E, D, F) * 0.05).to(dt).to(dev)
    wd = (torch.randn(E, F, D) * 0.05).to(dt).to(dev)
    mine = slice(r * El, (r + 1) * El)
    layer = MoELayer(ctx, D, F, E, K, max_tokens=T, w_gate=wg[mine].contiguous(), w_up=wu[mine].contiguous(),
                     w_down=wd[mine].contiguous())
    torch.manual_seed(50 + r)
    x = torch.randn(T, D, device=dev, dtype=dt)
    logits = torch.randn(T, E, device=dev)
    out = layer(x, logits)
    ref = reference_moe(x, logits, wg, wu, wd, K)
    err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
    assert err < 3e-2, err
    ctx.check()
    ctx.info(f"MoE layer validated (relative error {err:.1e})")
    finish(ctx)
