"""Distributed flash-decode layer: one query token per sequence, KV cache sharded along the
sequence across ranks (reference: examples/13_flash_decode/flash_decode_fused_layer.py:38-148).

``FlashDecodeLayer.forward(q, k_cache, v_cache, global_kv_lens, block_table)``

* ``q``             ``[B, Hq, D]`` (replicated on every rank)
* ``k_cache``/``v_cache``  this rank's paged shard ``[num_blocks, page, Hkv, D]``
* ``global_kv_lens`` ``int32 [W, B]``: KV length held by every rank for every sequence
* ``block_table``   ``int32 [B, max_blocks]``: page ids of this rank's shard

Two kernel launches on the current stream (``csrc/kernels/flash_decode.cu``): the split-K pass
over the local shard, then combine + exchange of the partial ``(o, lse)`` by remote stores with
per-(source, batch, head) flags + final merge. No host synchronisation, no flag reset between
calls. ``reference_decode`` is the plain fp32 PyTorch statement of the same computation.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from .. import _lib


class IrisDecodeDesc(C.Structure):
    _fields_ = [
        ("ctx", _lib.IrisCtx),
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("block_table", C.c_void_p), ("kv_lens", C.c_void_p),
        ("partial", C.c_void_p),
        ("gathered", C.c_void_p), ("flags", C.c_void_p), ("state", C.c_void_p),
        ("out", C.c_void_p), ("out_lse", C.c_void_p),
        ("B", C.c_int32), ("Bmax", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
        ("page", C.c_int32), ("max_blocks", C.c_int32), ("splits", C.c_int32),
        ("sm_scale", C.c_float), ("soft_cap", C.c_float),
        ("dtype", C.c_int32),
        ("exchange", C.c_int32),
        ("num_blocks", C.c_int32),
    ]


def reference_decode(q, k_cache, v_cache, kv_lens, block_table, sm_scale=None, soft_cap=0.0):
    """fp32 paged GQA decode over ONE shard: returns ``(o [B,Hq,D] fp32, lse [B,Hq] natural log)``."""
    B, Hq, D = q.shape
    _, page, Hkv, _ = k_cache.shape
    group = Hq // Hkv
    sm_scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
    o = torch.zeros(B, Hq, D, dtype=torch.float32, device=q.device)
    lse = torch.full((B, Hq), float("-inf"), dtype=torch.float32, device=q.device)
    for b in range(B):
        n = int(kv_lens[b])
        if n == 0:
            continue
        nblk = -(-n // page)
        blocks = block_table[b, :nblk].long()
        k = k_cache[blocks].reshape(-1, Hkv, D)[:n].float()
        v = v_cache[blocks].reshape(-1, Hkv, D)[:n].float()
        qb = q[b].float().view(Hkv, group, D)
        s = torch.einsum("hgd,nhd->hgn", qb, k) * sm_scale
        if soft_cap > 0:
            s = soft_cap * torch.tanh(s / soft_cap)
        lse_b = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - lse_b[..., None])
        o[b] = torch.einsum("hgn,nhd->hgd", p, v).reshape(Hq, D)
        lse[b] = lse_b.reshape(Hq)
    return o, lse


def merge_partials(o_parts, lse_parts):
    """Merge per-shard ``(o, lse)`` (leading dim = shard) into the attention over all shards."""
    m = torch.max(lse_parts, dim=0).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(lse_parts - m)
    w = torch.where(torch.isnan(w), torch.zeros_like(w), w)
    den = w.sum(0).clamp_min(1e-38)
    return (w[..., None] * o_parts).sum(0) / den[..., None]


class FlashDecodeLayer:
    def __init__(self, ctx, num_q_heads: int, num_kv_heads: int, head_dim: int = 128, max_batch: int = 64,
                 sm_scale: float | None = None, soft_cap: float = 0.0, max_splits: int = 64, dtype=torch.bfloat16,
                 use_tma: bool | None = None):
        if head_dim != 128:
            raise ValueError("the decode kernel is specialised for head_dim 128")
        if num_q_heads % num_kv_heads:
            raise ValueError("num_q_heads must be a multiple of num_kv_heads")
        self.ctx = ctx
        self.Hq, self.Hkv, self.D = num_q_heads, num_kv_heads, head_dim
        self.max_batch, self.max_splits = max_batch, max_splits
        self.sm_scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(head_dim)
        self.soft_cap = float(soft_cap)
        self.dtype = dtype
        self.use_tma = use_tma      # None: TMA tile fill whenever the page size allows it; False: cp.async fill
        W = ctx.get_num_ranks()
        dev = ctx.get_device()
        # exchange buffers on the heap: [2][W][Bmax][Hq][D+1] fp32 and [2][W][Bmax][Hq] int32
        self.gathered = ctx.zeros((2, W, max_batch, num_q_heads, head_dim + 1), dtype=torch.float32)
        self.signal_flags = ctx.zeros((2, W, max_batch, num_q_heads), dtype=torch.int32)
        self.state = ctx.zeros(2, dtype=torch.int32)
        self.partial = torch.empty((max_batch, num_q_heads, max_splits, head_dim + 1), dtype=torch.float32, device=dev)
        ctx.barrier()

    def _lib(self):
        lib = _lib.kernels()
        if not getattr(lib, "_iris_decode_typed", False):
            lib.iris_flash_decode.argtypes = [C.POINTER(IrisDecodeDesc), C.c_void_p]
            lib.iris_flash_decode.restype = C.c_int
            lib._iris_decode_typed = True
        return lib

    def num_splits(self, batch: int, max_len: int) -> int:
        sms = max(self.ctx.get_cu_count(), 1)
        per_seq = self.Hkv * -(-(self.Hq // self.Hkv) // 16)
        want = -(-4 * sms // max(batch * per_seq, 1))          # ~2 waves of 2 CTAs per SM
        by_len = max(1, -(-max_len // 256))                     # at least 256 positions per split
        return max(1, min(self.max_splits, want, by_len))

    def forward(self, q, k_cache, v_cache, global_kv_lens, block_table, out=None, return_lse: bool = False,
                local_only: bool = False):
        """Decode one token per sequence. ``local_only=True`` stops after this rank's own KV shard and
        returns its partial ``(out, lse)`` without talking to any peer (what the NCCL baseline gathers and
        merges itself, reference: examples/benchmark/reference/flash_decode_rccl/flash_decode_layer_rccl.py:100-130)."""
        ctx = self.ctx
        B = q.shape[0]
        if B > self.max_batch:
            raise ValueError(f"batch {B} exceeds max_batch {self.max_batch}")
        self._validate(q, k_cache, v_cache, global_kv_lens, block_table, out)
        kv_lens = global_kv_lens[ctx.get_rank()].contiguous()
        page = k_cache.shape[1]
        if ctx.is_cpu:
            if local_only:
                raise NotImplementedError("local_only decode is a GPU path")
            return self._forward_cpu(q, k_cache, v_cache, kv_lens, block_table)
        if out is None:
            out = torch.empty((B, self.Hq, self.D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, self.Hq), dtype=torch.float32, device=q.device) if (return_lse or local_only) else None
        d = IrisDecodeDesc()
        d.ctx = ctx.ctx_struct()
        d.q, d.k_cache, d.v_cache = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
        d.block_table, d.kv_lens = block_table.data_ptr(), kv_lens.data_ptr()
        d.partial = self.partial.data_ptr()
        d.gathered, d.flags, d.state = self.gathered.data_ptr(), self.signal_flags.data_ptr(), self.state.data_ptr()
        d.out = out.data_ptr()
        d.out_lse = lse.data_ptr() if lse is not None else None
        d.B, d.Bmax, d.Hq, d.Hkv, d.D = B, self.max_batch, self.Hq, self.Hkv, self.D
        d.page, d.max_blocks = page, block_table.shape[1]
        d.splits = self.num_splits(B, block_table.shape[1] * page)
        d.sm_scale, d.soft_cap = self.sm_scale, self.soft_cap
        d.dtype = _lib.DTYPE_CODE[q.dtype]
        d.exchange = 2 if local_only else 1
        d.num_blocks = 0 if self.use_tma is False else k_cache.shape[0]     # > 0 lets the kernel fill its tiles by TMA
        if not (q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous() and block_table.is_contiguous()):
            raise ValueError("flash decode takes contiguous q, caches and block table")
        _lib.check(self._lib().iris_flash_decode(C.byref(d), C.c_void_p(_lib.current_stream_ptr())), "flash decode launch", kernels=2)
        return (out, lse) if (return_lse or local_only) else out

    __call__ = forward

    def _validate(self, q, k_cache, v_cache, global_kv_lens, block_table, out) -> None:
        """Shapes and dtypes before anything is launched: the kernel indexes the caches through the
        block table and trusts the sizes it is given. In debug mode (``IRIS_DEBUG=1``) the VALUES are
        checked too (block numbers inside the cache, lengths inside the table), at the cost of a
        device synchronisation."""
        W, B = self.ctx.get_num_ranks(), q.shape[0]
        if tuple(q.shape) != (B, self.Hq, self.D):
            raise ValueError(f"q must be [batch, {self.Hq}, {self.D}], got {tuple(q.shape)}")
        if k_cache.dim() != 4 or tuple(k_cache.shape[2:]) != (self.Hkv, self.D) or k_cache.shape != v_cache.shape:
            raise ValueError(f"k_cache and v_cache must both be [blocks, page, {self.Hkv}, {self.D}], got "
                             f"{tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
        if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
            raise TypeError("q and the caches must have one dtype")
        if block_table.dim() != 2 or block_table.shape[0] != B or block_table.dtype != torch.int32:
            raise ValueError(f"block_table must be int32 [batch = {B}, blocks], got {block_table.dtype} {tuple(block_table.shape)}")
        if global_kv_lens.dim() != 2 or tuple(global_kv_lens.shape) != (W, B) or global_kv_lens.dtype != torch.int32:
            raise ValueError(f"global_kv_lens must be int32 [ranks = {W}, batch = {B}], got {global_kv_lens.dtype} "
                             f"{tuple(global_kv_lens.shape)}")
        if out is not None and (tuple(out.shape) != (B, self.Hq, self.D) or out.dtype != q.dtype or not out.is_contiguous()):
            raise ValueError("out must be a contiguous tensor of q's shape and dtype")
        if self.ctx.debug_checks:
            blocks, page = k_cache.shape[0], k_cache.shape[1]
            mine = global_kv_lens[self.ctx.get_rank()]
            if int(mine.min()) < 0 or int(mine.max()) > block_table.shape[1] * page:
                raise ValueError(f"a sequence length lies outside [0, {block_table.shape[1] * page}] (blocks per sequence x page)")
            used = -(-mine.to(torch.int64) // page)
            cols = torch.arange(block_table.shape[1], device=block_table.device)[None, :]
            live = block_table[cols < used[:, None].to(block_table.device)]
            if live.numel() and (int(live.min()) < 0 or int(live.max()) >= blocks):
                raise ValueError(f"block_table names a block outside the cache of {blocks} blocks")

    @staticmethod
    def merge_partials(outs: torch.Tensor, lses: torch.Tensor) -> torch.Tensor:
        """Log-sum-exp merge of per-shard results: ``outs [W, B, Hq, D]``, ``lses [W, B, Hq]`` -> ``[B, Hq, D]``."""
        w = torch.softmax(lses.float(), dim=0)
        w = torch.nan_to_num(w, nan=0.0)                       # a sequence no shard holds: every lse is -inf
        return (w[..., None] * outs.float()).sum(0).to(outs.dtype)

    def _forward_cpu(self, q, k_cache, v_cache, kv_lens, block_table):
        """CPU backend: same exchange layout through the shared-memory heap, math in PyTorch."""
        ctx = self.ctx
        W, me = ctx.get_num_ranks(), ctx.get_rank()
        B = q.shape[0]
        o, lse = reference_decode(q, k_cache, v_cache, kv_lens, block_table, self.sm_scale, self.soft_cap)
        ctx.device_barrier()
        for r in range(W):
            slot = ctx.heap.peer_view(self.gathered, r)[0, me, :B]
            slot[..., : self.D] = o
            slot[..., self.D] = lse
        ctx.device_barrier()
        parts = self.gathered[0, :, :B]
        return merge_partials(parts[..., : self.D], parts[..., self.D]).to(q.dtype)
