"""Ring attention: attention over a sequence that is split across the ranks (context parallelism).

Every rank holds ``S`` consecutive tokens of the sequence: queries ``[S, Hq, D]`` and keys/values
``[S, Hkv, D]``. ``RingAttention.forward(q, k, v, causal)`` returns this rank's ``[S, Hq, D]``
output of attention over the WHOLE sequence. One kernel per call: communication CTAs pass the K/V
blocks round the ring with bulk copies and per-block arrival counters on the heap, attention CTAs
consume the blocks as they arrive. When ``S`` is a multiple of 128 the attention CTAs run on
tcgen05 with TMEM accumulators and TMA-fed tiles (``csrc/kernels/ring_attention_tc.cu``), otherwise
on ``mma.sync`` (``csrc/kernels/ring_attention.cu``). The reference has no
counterpart; ``reference_attention`` is the plain fp32 PyTorch statement used by the tests.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from .. import _lib


class IrisRingAttnDesc(C.Structure):
    _fields_ = [
        ("ctx", _lib.IrisCtx),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("kv_buf", C.c_void_p), ("flags", C.c_void_p), ("state", C.c_void_p),
        ("out", C.c_void_p), ("lse", C.c_void_p),
        ("S", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32), ("causal", C.c_int32),
        ("n_comm", C.c_int32), ("dtype", C.c_int32), ("options", C.c_int32),
        ("sm_scale", C.c_float),
    ]


def zigzag_positions(rank: int, world: int, seq_per_rank: int, device=None) -> torch.Tensor:
    """Global positions of rank ``rank``'s tokens in the zigzag layout: the sequence of
    ``world * seq_per_rank`` tokens is cut into ``2 * world`` chunks and the rank holds chunk ``rank``
    followed by chunk ``2 * world - 1 - rank`` (balanced work under a causal mask)."""
    half = seq_per_rank // 2
    a = torch.arange(half, device=device)
    return torch.cat([rank * half + a, (2 * world - 1 - rank) * half + a])


def reference_attention(q, k, v, causal: bool = False, q_offset: int = 0, sm_scale: float | None = None, q_pos=None,
                        k_pos=None):
    """fp32 attention of ``q [Sq, Hq, D]`` over ``k, v [Sk, Hkv, D]``; query i sits at position
    ``q_offset + i`` of the key sequence when ``causal`` (or at ``q_pos[i]``, key j at ``k_pos[j]``,
    when the positions are given)."""
    Sq, Hq, D = q.shape
    Sk, Hkv, _ = k.shape
    sm_scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
    g = Hq // Hkv
    kf = k.float().repeat_interleave(g, dim=1)
    vf = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * sm_scale
    if causal:
        qi = (torch.arange(Sq, device=q.device) + q_offset if q_pos is None else q_pos.to(q.device))[:, None]
        ki = (torch.arange(Sk, device=q.device) if k_pos is None else k_pos.to(q.device))[None, :]
        s = s.masked_fill((ki > qi)[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vf)


class RingAttention:
    def __init__(self, ctx, seq_per_rank: int, num_q_heads: int, num_kv_heads: int, head_dim: int = 128,
                 sm_scale: float | None = None, comm_sms: int = 8, dtype=torch.bfloat16, use_tcgen05: bool | None = None,
                 layout: str = "contiguous"):
        if head_dim != 128:
            raise ValueError("the ring-attention kernel is specialised for head_dim 128")
        if num_q_heads % num_kv_heads:
            raise ValueError("num_q_heads must be a multiple of num_kv_heads")
        self.ctx, self.S, self.Hq, self.Hkv, self.D = ctx, seq_per_rank, num_q_heads, num_kv_heads, head_dim
        self.sm_scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(head_dim)
        self.comm_sms, self.dtype = comm_sms, dtype
        # None: tcgen05 attention CTAs whenever seq_per_rank is a multiple of 128; False: the mma.sync CTAs
        self.use_tcgen05 = use_tcgen05
        # "contiguous": rank r holds tokens [r*S, (r+1)*S); "zigzag": chunks r and 2W-1-r of 2W chunks
        # (see zigzag_positions), which balances causal attention over the ranks
        if layout not in ("contiguous", "zigzag"):
            raise ValueError(f"unknown layout {layout!r}")
        if layout == "zigzag" and (seq_per_rank % 256 or use_tcgen05 is False) and not ctx.is_cpu:
            raise ValueError("the zigzag layout needs seq_per_rank to be a multiple of 256 and the tcgen05 attention CTAs")
        self.layout = layout
        W = ctx.get_num_ranks()
        esize = 2 if not ctx.is_cpu else torch.empty((), dtype=dtype).element_size()
        # ring buffer [parity][origin rank][K | V][S, Hkv, D] and its arrival counters, on the heap
        self.kv_buf = ctx.heap.allocate(2 * W * 2 * seq_per_rank * num_kv_heads * head_dim * esize, torch.uint8)
        self.flags = ctx.zeros(2 * W, dtype=torch.int32)
        self.state = ctx.zeros(2, dtype=torch.int32)
        ctx.barrier()

    def _lib(self):
        lib = _lib.kernels()
        if not getattr(lib, "_iris_ring_typed", False):
            lib.iris_ring_attention.argtypes = [C.POINTER(IrisRingAttnDesc), C.c_void_p]
            lib.iris_ring_attention.restype = C.c_int
            lib._iris_ring_typed = True
        return lib

    def forward(self, q, k, v, causal: bool = False, out=None, return_lse: bool = False):
        ctx = self.ctx
        if tuple(q.shape) != (self.S, self.Hq, self.D) or tuple(k.shape) != (self.S, self.Hkv, self.D) or k.shape != v.shape:
            raise ValueError("expected q [S, Hq, D] and k, v [S, Hkv, D] with the layer's sizes")
        if ctx.is_cpu:
            return self._forward_cpu(q, k, v, causal)
        if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
            raise TypeError("ring attention takes fp16 or bf16 tensors of one dtype")
        if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
            raise ValueError("ring attention takes contiguous tensors")
        if out is None:
            out = torch.empty_like(q)
        elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous() or out.device != q.device:
            raise ValueError("out must be a contiguous tensor of q's shape, dtype and device")
        lse = torch.empty((self.S, self.Hq), dtype=torch.float32, device=q.device) if return_lse else None
        d = IrisRingAttnDesc()
        d.ctx = ctx.ctx_struct()
        d.q, d.k, d.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
        d.kv_buf, d.flags, d.state = self.kv_buf.data_ptr(), self.flags.data_ptr(), self.state.data_ptr()
        d.out = out.data_ptr()
        d.lse = lse.data_ptr() if lse is not None else None
        d.S, d.Hq, d.Hkv, d.D, d.causal, d.n_comm = self.S, self.Hq, self.Hkv, self.D, int(causal), self.comm_sms
        d.dtype = _lib.DTYPE_CODE[q.dtype]
        d.sm_scale = self.sm_scale
        d.options = (1 if self.use_tcgen05 is False else 0) | (2 if self.layout == "zigzag" else 0)
        _lib.check(self._lib().iris_ring_attention(C.byref(d), C.c_void_p(_lib.current_stream_ptr())), "ring attention launch", kernels=1)
        return (out, lse) if return_lse else out

    __call__ = forward

    def _forward_cpu(self, q, k, v, causal):
        """CPU backend: gather all K/V blocks through the heap, attend in PyTorch."""
        ctx = self.ctx
        W, me = ctx.get_num_ranks(), ctx.get_rank()
        if "_cpu_bufs" not in self.__dict__:          # heap buffers of this path, allocated once (collective)
            f32, cols = torch.float32, self.Hkv * self.D
            self._cpu_bufs = (ctx.zeros((self.S, cols), dtype=f32), ctx.zeros((self.S, cols), dtype=f32),
                              ctx.zeros((W * self.S, cols), dtype=f32), ctx.zeros((W * self.S, cols), dtype=f32))
        k_loc, v_loc, ks, vs = self._cpu_bufs
        k_loc.copy_(k.reshape(self.S, -1))
        v_loc.copy_(v.reshape(self.S, -1))
        ctx.ccl.all_gather(ks, k_loc)
        ctx.ccl.all_gather(vs, v_loc)
        q_pos = k_pos = None
        if self.layout == "zigzag":
            q_pos = zigzag_positions(me, W, self.S)
            k_pos = torch.cat([zigzag_positions(r, W, self.S) for r in range(W)])
        o = reference_attention(q, ks.view(W * self.S, self.Hkv, self.D), vs.view(W * self.S, self.Hkv, self.D), causal,
                                q_offset=me * self.S, sm_scale=self.sm_scale, q_pos=q_pos, k_pos=k_pos)
        return o.to(q.dtype)
