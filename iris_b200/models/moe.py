"""Expert-sharded mixture-of-experts layer (expert parallelism over the ranks of the heap).

Every rank holds ``num_experts / W`` experts (SwiGLU FFN: gate/up ``[hidden, ffn]``, down
``[ffn, hidden]``) and ``T`` tokens. ``forward(x, router_logits)`` routes each token to its top-k
experts (softmax over the selected k logits), moves the token rows to the experts' owners, runs
the expert FFNs as grouped GEMMs and returns the weighted sum of the k expert outputs in token
order. On a GPU the whole pass is the launch sequence of ``csrc/kernels/moe.cu`` on the current
stream, with the dispatch fused into the first grouped GEMM and the combine fused into the second
one's epilogue; the reference pipeline with its host barriers and Python-side metadata is
examples/31_expert_sharded_moe/moe.py:195-328. Weights are bf16, or (``fp8=True``) e4m3 with
128 x 128 power-of-two block scales: then the tokens are quantised to e4m3 with 1 x 128 scales before
the dispatch (half the bytes on the wire), both grouped GEMMs run on the tensor core's block-scaled
path, and the SwiGLU epilogue re-quantises the hidden activations for the down projection; the
combine and the output stay bf16. ``reference_moe`` is the unsharded fp32 PyTorch statement of the layer.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib


class IrisMoeDesc(C.Structure):
    _fields_ = [
        ("ctx", _lib.IrisCtx),
        ("T", C.c_int32), ("K", C.c_int32), ("E", C.c_int32), ("El", C.c_int32), ("D", C.c_int32), ("F", C.c_int32),
        ("capacity", C.c_int32), ("comm_ctas", C.c_int32),
        ("x", C.c_void_p), ("logits", C.c_void_p), ("w13", C.c_void_p), ("w2", C.c_void_p), ("out", C.c_void_p),
        ("inbox", C.c_void_p), ("H", C.c_void_p), ("comb", C.c_void_p),
        ("sync_meta", C.c_void_p), ("sync_gemm2", C.c_void_p),
        ("topk_idx", C.c_void_p), ("topk_w", C.c_void_p),
        ("counts_local", C.c_void_p), ("counts_all", C.c_void_p), ("cursor", C.c_void_p), ("list_off", C.c_void_p),
        ("sorted_pairs", C.c_void_p), ("my_off", C.c_void_p),
        ("expert_rows", C.c_void_p), ("expert_row0", C.c_void_p), ("tile_prefix", C.c_void_p), ("expected_cum", C.c_void_p),
        ("arrived", C.c_void_p), ("inbox_meta", C.c_void_p),
        ("weights_kmajor", C.c_int32),
        ("fp8", C.c_int32), ("sf_ld1", C.c_int32), ("sf_ld2", C.c_int32),
        ("x_sf", C.c_void_p), ("inbox_sf", C.c_void_p), ("H_sf", C.c_void_p), ("w13_sf", C.c_void_p), ("w2_sf", C.c_void_p),
    ]


def route(logits: torch.Tensor, top_k: int):
    """Top-k of the logits and softmax over the selected k (reference: topk.py:93-121)."""
    vals, idx = torch.topk(logits.float(), top_k, dim=-1)
    return idx, torch.softmax(vals, dim=-1)


def reference_moe(x, logits, w_gate, w_up, w_down, top_k: int):
    """Unsharded fp32 MoE: ``w_*`` hold ALL experts, ``[E, hidden, ffn]`` / ``[E, ffn, hidden]``."""
    idx, w = route(logits, top_k)
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(w_gate.shape[0]):
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xf[tok]
        g, u = h @ w_gate[e].float(), h @ w_up[e].float()
        y = (torch.nn.functional.silu(g) * u) @ w_down[e].float()
        out.index_add_(0, tok, y * w[tok, slot][:, None])
    return out


def fuse_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``[El, D, F]`` x 2 -> ``[El, D, 2F]`` whose 256-column blocks are ``[gate 128 | up 128]``: the
    layout the SwiGLU epilogue expects (it pairs column c with column c + 128 of a tile)."""
    El, D, F = w_gate.shape
    g = w_gate.reshape(El, D, F // 128, 1, 128)
    u = w_up.reshape(El, D, F // 128, 1, 128)
    return torch.cat([g, u], dim=3).reshape(El, D, 2 * F).contiguous()


class MoELayer:
    def __init__(self, ctx, hidden: int, ffn: int, num_experts: int, top_k: int, max_tokens: int,
                 w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, capacity_factor: float | None = None,
                 comm_sms: int = 16, fp8: bool = False):
        W = ctx.get_num_ranks()
        if num_experts % W:
            raise ValueError("num_experts must be a multiple of the number of ranks")
        El = num_experts // W
        if tuple(w_gate.shape) != (El, hidden, ffn) or tuple(w_up.shape) != (El, hidden, ffn) or tuple(w_down.shape) != (El, ffn, hidden):
            raise ValueError("expected local expert weights [E/W, hidden, ffn] (gate, up) and [E/W, ffn, hidden] (down)")
        self.ctx, self.D, self.F, self.E, self.El, self.K, self.T = ctx, hidden, ffn, num_experts, El, top_k, max_tokens
        self.comm_sms = comm_sms
        self.fp8 = bool(fp8)
        self.w_gate, self.w_up, self.w_down = w_gate, w_up, w_down
        if ctx.is_cpu:
            return
        if hidden % 256 or ffn % 128:
            raise ValueError("the fused kernels need hidden % 256 == 0 and ffn % 128 == 0")
        dev = ctx.get_device()
        # each expert's weight is kept transposed (K contiguous): the layout the tensor cores read fastest
        self.w13 = fuse_gate_up(w_gate.to(torch.bfloat16), w_up.to(torch.bfloat16)).transpose(1, 2).contiguous()   # [El, 2F, D]
        self.w2 = w_down.to(torch.bfloat16).transpose(1, 2).contiguous()                                          # [El, D, F]
        pairs = max_tokens * top_k
        cap = W * pairs if capacity_factor is None else min(W * pairs, int(capacity_factor * pairs))
        self.capacity = max(128, -(-cap // 128) * 128)
        i32 = torch.int32
        if self.fp8:
            self._init_fp8(dev)
        else:
            self.inbox = ctx.heap.allocate(self.capacity * hidden, torch.bfloat16).view(self.capacity, hidden)
        self.inbox_meta = ctx.zeros(self.capacity, dtype=torch.int64)
        self.comb = ctx.heap.allocate(pairs * hidden, torch.bfloat16).view(pairs, hidden)
        self.counts_all = ctx.zeros((W, num_experts), dtype=i32)
        self.arrived = ctx.zeros(El, dtype=i32)
        self.sync_meta = ctx.zeros(80, dtype=i32)
        self.sync_gemm2 = ctx.zeros(80, dtype=i32)
        if not self.fp8:
            self.H = torch.zeros(self.capacity, ffn, dtype=torch.bfloat16, device=dev)
        self.topk_idx = torch.zeros(max_tokens, top_k, dtype=i32, device=dev)
        self.topk_w = torch.zeros(max_tokens, top_k, dtype=torch.float32, device=dev)
        z = lambda n: torch.zeros(n, dtype=i32, device=dev)  # noqa: E731
        self.counts_local, self.cursor, self.list_off, self.my_off = z(num_experts), z(num_experts), z(num_experts + 1), z(num_experts)
        self.sorted_pairs = z(pairs)
        self.expert_rows, self.expert_row0, self.tile_prefix, self.expected_cum = z(El), z(El + 1), z(El + 1), z(El)
        ctx.barrier()

    def _init_fp8(self, dev) -> None:
        """Quantise the expert weights (e4m3, 128 x 128 power-of-two block scales, scale atoms packed for the
        tile widths of the two grouped GEMMs: 256 for gate|up, 224 for down) and allocate the e4m3 buffers."""
        from ..ops.gemm_fp8 import pack_scales_b, quantize_128x128

        ctx, El, D, F = self.ctx, self.El, self.D, self.F
        if D % 128 or F % 128:
            raise ValueError("the fp8 MoE needs hidden and ffn to be multiples of 128")
        q13, s13 = quantize_128x128(self.w13.reshape(El * 2 * F, D).float(), pow2=True)
        self.w13_q = q13.view(El, 2 * F, D)
        self.w13_scale = s13                                                     # [El * 2F / 128, D / 128]
        self.w13_sf = pack_scales_b(s13, El * 2 * F, 256)                        # experts start on tile boundaries (2F % 256 == 0)
        q2, s2 = quantize_128x128(self.w2.reshape(El * D, F).float(), pow2=True)
        self.w2_q = q2.view(El, D, F)
        self.w2_scale = s2                                                       # [El * D / 128, F / 128]
        per = D // 128
        self.w2_sf = torch.stack([pack_scales_b(s2[j * per:(j + 1) * per], D, 224) for j in range(El)]).contiguous()
        self.sf_ld1 = -(-(D // 128) // 16) * 16
        self.sf_ld2 = -(-(F // 128) // 16) * 16
        u8 = torch.uint8
        self.inbox = ctx.heap.allocate(self.capacity * D, u8).view(self.capacity, D)
        self.inbox_sf = ctx.heap.allocate(self.capacity * self.sf_ld1, u8).view(self.capacity, self.sf_ld1)
        self.inbox_sf.fill_(127)
        self.H = torch.zeros(self.capacity, F, dtype=u8, device=dev)
        self.H_sf = torch.full((self.capacity, self.sf_ld2), 127, dtype=u8, device=dev)
        self.xq = torch.zeros(self.T, D, dtype=u8, device=dev)
        self.x_sf = torch.full((self.T, self.sf_ld1), 127, dtype=u8, device=dev)
        del self.w13, self.w2

    def _quantise_tokens(self, x) -> None:
        lib = _lib.kernels()
        if not getattr(lib, "_iris_quant_rows_typed", False):
            lib.iris_quantize_1x128_pow2_rows.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                                          C.c_int32, C.c_int32, C.c_void_p]
            lib.iris_quantize_1x128_pow2_rows.restype = C.c_int
            lib._iris_quant_rows_typed = True
        _lib.check(lib.iris_quantize_1x128_pow2_rows(C.c_void_p(x.data_ptr()), x.stride(0), _lib.DTYPE_CODE[x.dtype], C.c_void_p(self.xq.data_ptr()),
                                                     self.xq.stride(0), C.c_void_p(self.x_sf.data_ptr()), self.sf_ld1, x.shape[0], self.D,
                                                     C.c_void_p(_lib.current_stream_ptr())), "token quantiser launch", kernels=1)

    def _lib(self):
        lib = _lib.kernels()
        if not getattr(lib, "_iris_moe_typed", False):
            lib.iris_moe_forward.argtypes = [C.POINTER(IrisMoeDesc), C.c_void_p]
            lib.iris_moe_forward.restype = C.c_int
            lib._iris_moe_typed = True
        return lib

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        ctx = self.ctx
        T = x.shape[0]
        if T > self.T or x.shape[1] != self.D or tuple(router_logits.shape) != (T, self.E):
            raise ValueError("x must be [T <= max_tokens, hidden] and router_logits [T, num_experts]")
        if ctx.is_cpu:
            return self._forward_cpu(x, router_logits)
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise TypeError("the fused MoE takes contiguous bf16 tokens")
        logits = router_logits.float().contiguous()
        if out is None:
            out = torch.empty_like(x)
        elif out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous() or out.device != x.device:
            raise ValueError("out must be a contiguous tensor of x's shape, dtype and device")
        d = IrisMoeDesc()
        d.ctx = ctx.ctx_struct()
        d.T, d.K, d.E, d.El, d.D, d.F, d.capacity, d.comm_ctas = T, self.K, self.E, self.El, self.D, self.F, self.capacity, self.comm_sms
        if self.fp8:
            self._quantise_tokens(x)
            d.fp8, d.sf_ld1, d.sf_ld2 = 1, self.sf_ld1, self.sf_ld2
            d.x, d.w13, d.w2 = self.xq.data_ptr(), self.w13_q.data_ptr(), self.w2_q.data_ptr()
            d.x_sf, d.inbox_sf, d.H_sf = self.x_sf.data_ptr(), self.inbox_sf.data_ptr(), self.H_sf.data_ptr()
            d.w13_sf, d.w2_sf = self.w13_sf.data_ptr(), self.w2_sf.data_ptr()
        else:
            d.x, d.w13, d.w2 = x.data_ptr(), self.w13.data_ptr(), self.w2.data_ptr()
        d.logits, d.out = logits.data_ptr(), out.data_ptr()
        d.inbox, d.H, d.comb = self.inbox.data_ptr(), self.H.data_ptr(), self.comb.data_ptr()
        d.sync_meta, d.sync_gemm2 = self.sync_meta.data_ptr(), self.sync_gemm2.data_ptr()
        for name in ("topk_idx", "topk_w", "counts_local", "counts_all", "cursor", "list_off", "sorted_pairs", "my_off",
                     "expert_rows", "expert_row0", "tile_prefix", "expected_cum", "arrived", "inbox_meta"):
            setattr(d, name, getattr(self, name).data_ptr())
        d.weights_kmajor = 1
        _lib.check(self._lib().iris_moe_forward(C.byref(d), C.c_void_p(_lib.current_stream_ptr())), "MoE forward launch", kernels=7)
        self._keep = logits
        return out

    __call__ = forward

    @staticmethod
    def _cpu_fake_quant(t: torch.Tensor, weight: bool = False) -> torch.Tensor:
        """Round ``t`` the way the e4m3 path stores it: rows in 1 x 128 blocks (activations) or 128 x 128 blocks
        (a weight given as [out, in]), power-of-two scales."""
        from ..ops.gemm_fp8 import dequantize, quantize_1x128, quantize_128x128

        q, sc = (quantize_128x128 if weight else quantize_1x128)(t.float(), pow2=True)
        return dequantize(q, sc, 128 if weight else 1)

    def _forward_cpu(self, x, logits):
        """CPU backend: gather every rank's tokens, apply the local experts, sum over ranks."""
        ctx = self.ctx
        W, me, T = ctx.get_num_ranks(), ctx.get_rank(), x.shape[0]
        bufs = self.__dict__.setdefault("_cpu_bufs", {})
        if T not in bufs:            # heap buffers of this path, once per token count (collective)
            f32 = torch.float32
            bufs[T] = (ctx.zeros((T, self.D), dtype=f32), ctx.zeros((T, self.E), dtype=f32), ctx.zeros((W * T, self.D), dtype=f32),
                       ctx.zeros((W * T, self.E), dtype=f32), ctx.zeros((W * T, self.D), dtype=f32), ctx.zeros((W * T, self.D), dtype=f32))
        x_loc, l_loc, xs, ls, part, tot = bufs[T]
        x_loc.copy_(x)
        l_loc.copy_(logits)
        ctx.ccl.all_gather(xs, x_loc)
        ctx.ccl.all_gather(ls, l_loc)
        idx, w = route(ls, self.K)
        part.zero_()
        # fp8 mode: the same roundings as the e4m3 kernels (tokens and hidden activations in 1 x 128 blocks,
        # weights in 128 x 128 blocks, power-of-two scales), applied here as quantise + dequantise in fp32
        q8 = self._cpu_fake_quant if self.fp8 and hasattr(torch, "float8_e4m3fn") else (lambda t, weight=False: t)
        xs_q = q8(xs)
        for j in range(self.El):
            e = me * self.El + j
            tok, slot = torch.nonzero(idx == e, as_tuple=True)
            if tok.numel() == 0:
                continue
            h = xs_q[tok]
            wg, wu, wd = (q8(m.float().t().contiguous(), weight=True).t() for m in (self.w_gate[j], self.w_up[j], self.w_down[j]))
            hid = q8(torch.nn.functional.silu(h @ wg) * (h @ wu))
            part.index_add_(0, tok, (hid @ wd) * w[tok, slot][:, None])
        ctx.ccl.all_reduce(tot, part)
        return tot[me * T:(me + 1) * T].to(x.dtype)
