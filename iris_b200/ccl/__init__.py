"""Collectives on the symmetric heap: ``ctx.ccl.all_reduce / all_gather / all_to_all /
reduce_scatter`` (reference: iris/host/iris.py:1120-1318 and iris/ccl/*.py).

On a GPU every call is ONE kernel of ``csrc/kernels/ccl.cu`` on the current stream; the kernel
synchronises with its peers on the device, so a call neither needs nor performs a host barrier
(``async_op`` is accepted for compatibility; without it the call ends with ``ctx.barrier()`` as the
reference does). On the CPU backend the same data movement is carried out through peer mappings
of the shared-memory heaps, for tests of the host logic and of the layouts.

Tensors must live on the heap and be 2-D (1-D tensors are treated as one row).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import _lib
from ..host import artifacts as _artifacts
from .config import Config
from .utils import ReduceOp

__all__ = ["Config", "ReduceOp", "CCL", "AllReduceWorkspace"]

_AR_CODE = {"atomic": 0, "ring": 1, "one_shot": 2, "two_shot": 3, "spinlock": 4, "nvls": 5, "push": 6}
PUSH_CAP_KB = 512          # largest message of the one-shot push path (bytes / 1024)


class IrisCclDesc(C.Structure):
    _fields_ = [
        ("ctx", _lib.IrisCtx),
        ("sync_block", C.c_void_p),
        ("inp", C.c_void_p),
        ("out", C.c_void_p),
        ("M", C.c_int32), ("N", C.c_int32),
        ("ld_in", C.c_int64), ("ld_out", C.c_int64),
        ("dtype", C.c_int32),
        ("variant", C.c_int32),
        ("use_mc", C.c_int32),
        ("comm_sms", C.c_int32),
        ("block_m", C.c_int32), ("block_n", C.c_int32), ("distribution", C.c_int32), ("swizzle", C.c_int32),
        ("ring_buf", C.c_void_p),
        ("flags", C.c_void_p),
        ("rows_mode", C.c_int32),
        ("reserved", C.c_int32),
    ]


@dataclass
class AllReduceWorkspace:
    """Buffers an all-reduce variant needs beyond its tensors (ring slots, locks)."""

    variant: str = "two_shot"
    shape: tuple = ()
    dtype: torch.dtype | None = None
    ring_buffer: torch.Tensor | None = None
    flags: torch.Tensor | None = None
    sync_block: torch.Tensor | None = None
    ring_ctas: int = 32
    prepared: bool = False


def _as_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 1:
        return t.view(1, -1)
    if t.dim() != 2:
        raise ValueError(f"collectives take 1-D or 2-D tensors, got {t.dim()}-D")
    return t


class CCL:
    def __init__(self, ctx):
        self.ctx = ctx
        self._desc_cache: dict = {}
        self._ws_cache: dict = {}   # all-reduce workspaces for calls that pass none
        self._fast: dict = {}       # whole calls that ran before: key -> (op code, descriptor copy, return value)
        self._push_ws = None

    # ------------------------------------------------------------------ plumbing
    def _lib(self):
        lib = _lib.kernels()
        if not getattr(lib, "_iris_ccl_typed", False):
            lib.iris_ccl_launch.argtypes = [C.c_int, C.POINTER(IrisCclDesc), C.c_void_p]
            lib.iris_ccl_launch.restype = C.c_int
            lib._iris_ccl_typed = True
        return lib

    def _check(self, out: torch.Tensor, inp: torch.Tensor):
        ctx = self.ctx
        if not ctx.is_symmetric(out) or not ctx.is_symmetric(inp):
            raise ValueError("collective tensors must be allocated on the symmetric heap (ctx.zeros, ctx.empty, ...)")
        if out.dtype != inp.dtype:
            raise ValueError(f"dtype mismatch: output {out.dtype}, input {inp.dtype}")
        if inp.stride(-1) != 1 or out.stride(-1) != 1:
            raise ValueError("collective tensors must be row-major (unit stride in the last dimension)")
        if inp.dtype not in _lib.DTYPE_CODE:
            raise TypeError(f"dtype {inp.dtype} is not supported by the collectives")

    def _desc(self, out, inp, group, config, sync_key="ccl", op="") -> IrisCclDesc:
        ctx = self.ctx
        # descriptors are cached per (buffers, shape, config): a repeated call costs one lookup
        key = (out.data_ptr(), inp.data_ptr(), tuple(out.shape), tuple(inp.shape), out.stride(0), inp.stride(0), inp.dtype,
               ctx._group_key(group), config.use_multicast, config.comm_sms, config.block_size_m, config.block_size_n,
               config.all_reduce_distribution, config.swizzle_size, id(ctx._ctx_epoch), op, config.reduce_scatter_rows)
        hit = self._desc_cache.get(key)
        if hit is not None:
            return hit
        if len(self._desc_cache) > 4096:
            self._desc_cache.clear()
        d = IrisCclDesc()
        self._desc_cache[key] = d
        d.ctx = ctx.ctx_struct(group)
        d.sync_block = ctx.sync_block((sync_key, ctx._group_key(group))).data_ptr()
        d.inp, d.out = inp.data_ptr(), out.data_ptr()
        d.ld_in, d.ld_out = inp.stride(0), out.stride(0)
        d.dtype = _lib.DTYPE_CODE[inp.dtype]
        d.use_mc = 1 if (config.use_multicast and group is None and ctx.has_multicast()) else 0
        d.comm_sms = config.comm_sms
        d.block_m, d.block_n = config.block_size_m, config.block_size_n
        d.distribution, d.swizzle = config.all_reduce_distribution, config.swizzle_size
        return d

    def _launch(self, op: int, d: IrisCclDesc):
        if _artifacts.ACTIVE:
            name = ("all_gather", "all_to_all", "all_reduce", "reduce_scatter")[op]
            variant = {v: k for k, v in _AR_CODE.items()}.get(d.variant, "") if op == 2 else ("rows" if d.rows_mode else "tiles") if op == 3 else ""
            _artifacts.record_launch("ccl", name + ("_" + variant if variant else ""), self.ctx.cur_rank,
                                     {"M": d.M, "N": d.N, "dtype": {v: k for k, v in _lib.DTYPE_CODE.items()}.get(d.dtype, d.dtype),
                                      "world": d.ctx.world, "comm_sms": d.comm_sms, "use_multicast": bool(d.use_mc), "block_m": d.block_m,
                                      "block_n": d.block_n, "distribution": d.distribution}, source="ccl.cu")
        _lib.check(self._lib().iris_ccl_launch(op, C.byref(d), C.c_void_p(_lib.current_stream_ptr())), "collective launch", kernels=1)

    # A repeated call (same buffers, shapes, group and configuration) skips validation and
    # descriptor set-up: one tuple, one dictionary lookup, one launch.
    def _fast_key(self, tag, out, inp, group, config, extra=None):
        return (tag, out.data_ptr(), inp.data_ptr(), out.shape, inp.shape, out.stride(), inp.stride(), out.dtype, inp.dtype,
                None if group is None else id(group), None if config is None else tuple(vars(config).values()),
                id(self.ctx._ctx_epoch), extra)

    def _remember(self, key, op: int, d: IrisCclDesc, ret=None):
        if len(self._fast) > 4096:
            self._fast.clear()
        self._fast[key] = (op, IrisCclDesc.from_buffer_copy(d), ret)     # a copy: cached descriptors are rewritten per call

    def _replay(self, hit, async_op, group):
        self._launch(hit[0], hit[1])
        if not async_op:
            self.ctx.barrier(group=group)
        return hit[2]

    def _finish(self, async_op: bool, group):
        if not async_op:
            self.ctx.barrier(group=group)

    def _world(self, group):
        return self.ctx.ctx_struct(group).world, self.ctx.ctx_struct(group).rank

    # ------------------------------------------------------------------ all_gather
    def all_gather(self, output_tensor, input_tensor, group=None, async_op=False, config=None):
        """``output[(r*M):(r+1)*M, :] = input of rank r`` for every rank r of the group."""
        key = self._fast_key("ag", output_tensor, input_tensor, group, config)
        hit = self._fast.get(key)
        if hit is not None:
            return self._replay(hit, async_op, group)
        config = config or Config()
        W, me = self._world(group)
        if output_tensor.dim() == 1 and input_tensor.dim() == 1 and output_tensor.numel() == W * input_tensor.numel():
            # vectors: rank r's n elements land at [r n, (r+1) n), i.e. row r of a (W, n) matrix
            out, inp = output_tensor.view(W, -1), input_tensor.view(1, -1)
        else:
            out, inp = _as_2d(output_tensor), _as_2d(input_tensor)
        self._check(out, inp)
        M, N = inp.shape
        if tuple(out.shape) != (W * M, N):
            raise ValueError(f"all_gather: output must be {(W * M, N)}, got {tuple(out.shape)}")
        if self.ctx.is_cpu:
            self._cpu_entry(group)
            for r in range(W):
                self._peer(out, r, group)[me * M:(me + 1) * M].copy_(inp)
            self._cpu_exit(group)
        else:
            d = self._desc(out, inp, group, config, op="ag")
            d.M, d.N = M, N
            d.variant = 1 if config.all_gather_variant == "partitioned" else 0
            self._launch(0, d)
            self._remember(key, 0, d)
        self._finish(async_op, group)

    # ------------------------------------------------------------------ all_to_all
    def all_to_all(self, output_tensor, input_tensor, group=None, async_op=False, config=None):
        """Column chunk d of rank s's input lands in column chunk s of rank d's output."""
        key = self._fast_key("a2a", output_tensor, input_tensor, group, config)
        hit = self._fast.get(key)
        if hit is not None:
            return self._replay(hit, async_op, group)
        config = config or Config()
        out, inp = _as_2d(output_tensor), _as_2d(input_tensor)
        self._check(out, inp)
        W, me = self._world(group)
        M, NW = inp.shape
        if NW % W or tuple(out.shape) != (M, NW):
            raise ValueError(f"all_to_all: tensors must be (M, N*{W}) and of equal shape, got {tuple(inp.shape)} / {tuple(out.shape)}")
        N = NW // W
        if self.ctx.is_cpu:
            self._cpu_entry(group)
            for r in range(W):
                self._peer(out, r, group)[:, me * N:(me + 1) * N].copy_(inp[:, r * N:(r + 1) * N])
            self._cpu_exit(group)
        else:
            d = self._desc(out, inp, group, config, op="a2a")
            d.M, d.N = M, N
            self._launch(1, d)
            self._remember(key, 1, d)
        self._finish(async_op, group)

    # ------------------------------------------------------------------ all_reduce
    def _pick_all_reduce(self, config: Config, nbytes: int, group, dtype) -> str:
        v = config.all_reduce_variant
        if self.ctx.ctx_struct(group).world == 1:
            return "one_shot"       # nothing to exchange: every variant is a copy
        nvls_ok = config.use_multicast and group is None and self.ctx.has_multicast() and dtype != torch.int32
        if v == "nvls" and not nvls_ok:
            return "two_shot"
        if v == "push" and (nbytes > PUSH_CAP_KB * 1024 or group is not None):
            return "two_shot"
        if v != "auto":
            return v
        # Every rank pulling everything (one_shot) is one round trip but W x the traffic: best while
        # the message is latency bound. Beyond that the owner-reduces schemes win, in the switch
        # when NVLS is available.
        if nbytes <= PUSH_CAP_KB * 1024 and group is None:
            return "push"           # one NVLink traversal, no barrier rounds
        if nbytes <= 256 * 1024:
            return "one_shot"
        if self.ctx.ctx_struct(group).world == 2 and nbytes >= (8 << 20):
            return "two_shot"       # with one peer the switch has nothing to reduce: pulling on all SMs is faster
        return "nvls" if nvls_ok else "two_shot"

    def all_reduce_preamble(self, output_tensor, input_tensor, config=None, workspace=None, group=None):
        """Allocate what the chosen variant needs (collective when it allocates). Returns the workspace."""
        config = config or Config()
        out = _as_2d(output_tensor)
        variant = self._pick_all_reduce(config, out.numel() * out.element_size(), group, out.dtype)
        ws = workspace
        if ws is None or ws.variant != variant or ws.shape != tuple(out.shape) or ws.dtype != out.dtype:
            # calls that bring no matching workspace share one per (variant, shape, dtype, group, CTA count):
            # the ring and spin-lock variants own heap buffers, which must not be allocated per call
            ck = (variant, tuple(out.shape), out.dtype, self.ctx._group_key(group), config.comm_sms)
            kept = self._ws_cache.get(ck)
            if kept is not None:
                kept.prepared = True
                return kept
            ws = self._ws_cache[ck] = AllReduceWorkspace(variant=variant, shape=tuple(out.shape), dtype=out.dtype)
            ctx = self.ctx
            if not ctx.is_cpu:
                W = ctx.ctx_struct(group).world
                if variant == "ring":
                    ws.ring_ctas = min(config.comm_sms, 64)
                    units = -(-out.numel() // W)
                    ws.ring_buffer = ctx.heap.allocate(2 * (W - 1) * (units + 16) * out.element_size() + 64, torch.uint8)
                    ws.flags = ctx.zeros(2 * (W - 1) * ws.ring_ctas, dtype=torch.int32)
                    ws.sync_block = ctx.zeros(80, dtype=torch.int32)
                    ctx.barrier()
                elif variant == "push":
                    if self._push_ws is None:
                        cap = PUSH_CAP_KB * 1024
                        self._push_ws = (ctx.heap.allocate(2 * W * cap, torch.uint8), ctx.zeros(2 * W * 32, dtype=torch.int32),
                                         ctx.zeros(80, dtype=torch.int32))
                        ctx.barrier()
                    ws.ring_buffer, ws.flags, ws.sync_block = self._push_ws
                elif variant == "spinlock":
                    nseg = -(-out.numel() // 256) + 1
                    ws.flags = ctx.zeros(2 * nseg, dtype=torch.int32)
                    ctx.barrier()
        ws.prepared = True
        return ws

    def all_reduce(self, output_tensor, input_tensor, op=None, group=None, async_op=False, config=None, workspace=None):
        """``output = sum over ranks of input`` on every rank (fp32 accumulation). Returns the workspace."""
        if op is not None and op != ReduceOp.SUM:
            raise ValueError("only ReduceOp.SUM is supported")
        key = self._fast_key("ar", output_tensor, input_tensor, group, config, None if workspace is None else id(workspace))
        hit = self._fast.get(key)
        if hit is not None:
            return self._replay(hit, async_op, group)
        config = config or Config()
        if config.use_gluon:
            raise ValueError("use_gluon has no meaning on this backend")
        out, inp = _as_2d(output_tensor), _as_2d(input_tensor)
        self._check(out, inp)
        if out.shape != inp.shape:
            raise ValueError("all_reduce: input and output must have the same shape")
        if out.data_ptr() == inp.data_ptr():
            raise ValueError("all_reduce is out of place: peers read the input while outputs are written")
        ws = self.all_reduce_preamble(out, inp, config, workspace, group)
        W, me = self._world(group)
        if self.ctx.is_cpu:
            self._cpu_entry(group)
            acc = torch.zeros(inp.shape, dtype=torch.float32 if inp.dtype.is_floating_point else torch.int64)
            for r in range(W):
                acc += self._peer(inp, r, group).to(acc.dtype)
            out.copy_(acc.to(out.dtype))
            self._cpu_exit(group)
        else:
            # one descriptor per resolved variant: the ring, push and spin-lock variants point it at their own
            # sync block, buffers and CTA count, which must not leak into another variant's call on the same tensors
            d = self._desc(out, inp, group, config, op="ar:" + ws.variant)
            d.M, d.N = inp.shape
            d.variant = _AR_CODE[ws.variant]
            if ws.variant == "ring":
                d.sync_block = ws.sync_block.data_ptr()
                d.ring_buf = ws.ring_buffer.data_ptr()
                d.flags = ws.flags.data_ptr()
                d.comm_sms = ws.ring_ctas
            elif ws.variant == "push":
                d.sync_block = ws.sync_block.data_ptr()
                d.ring_buf = ws.ring_buffer.data_ptr()
                d.flags = ws.flags.data_ptr()
                d.block_m = PUSH_CAP_KB
            elif ws.variant == "spinlock":
                d.flags = ws.flags.data_ptr()
            self._launch(2, d)
            self._remember(key, 2, d, ws)
        ws.prepared = False
        self._finish(async_op, group)
        return ws

    # ------------------------------------------------------------------ reduce_scatter
    def reduce_scatter(self, output_tensor, input_tensor, op=None, group=None, async_op=False, config=None):
        """Sum over ranks, each rank keeping a part.

        Default (reference semantics, iris/ccl/reduce_scatter.py:52-56): ``output`` has the full
        ``(M, N)`` shape and this rank writes only the ``block_size_m x block_size_n`` tiles it owns
        (``all_reduce_distribution`` 1: contiguous blocks of tiles, 0: every W-th tile).
        With ``config.reduce_scatter_rows`` the output is ``(M/W, N)``: this rank's row block.
        """
        if op is not None and op != ReduceOp.SUM:
            raise ValueError("only ReduceOp.SUM is supported")
        key = self._fast_key("rs", output_tensor, input_tensor, group, config)
        hit = self._fast.get(key)
        if hit is not None:
            return self._replay(hit, async_op, group)
        config = config or Config()
        out, inp = _as_2d(output_tensor), _as_2d(input_tensor)
        self._check(out, inp)
        W, me = self._world(group)
        M, N = inp.shape
        rows = config.reduce_scatter_rows
        if rows:
            if M % W:
                raise ValueError(f"reduce_scatter(rows): {M} rows do not split over {W} ranks")
            if tuple(out.shape) != (M // W, N):
                raise ValueError(f"reduce_scatter(rows): output must be {(M // W, N)}, got {tuple(out.shape)}")
        elif out.shape != inp.shape:
            raise ValueError("reduce_scatter: output must have the input's shape (only owned tiles are written)")
        if self.ctx.is_cpu:
            self._cpu_entry(group)
            acc = torch.zeros(inp.shape, dtype=torch.float32 if inp.dtype.is_floating_point else torch.int64)
            for r in range(W):
                acc += self._peer(inp, r, group).to(acc.dtype)
            if rows:
                out.copy_(acc[me * (M // W):(me + 1) * (M // W)].to(out.dtype))
            else:
                for (r0, r1, c0, c1) in owned_tiles(M, N, config.block_size_m, config.block_size_n, W, me, config.all_reduce_distribution):
                    out[r0:r1, c0:c1].copy_(acc[r0:r1, c0:c1].to(out.dtype))
            self._cpu_exit(group)
        else:
            d = self._desc(out, inp, group, config, op="rs")
            d.M, d.N = M, N
            d.rows_mode = 1 if rows else 0
            self._launch(3, d)
            self._remember(key, 3, d)
        self._finish(async_op, group)

    # ------------------------------------------------------------------ CPU backend helpers
    def _peer(self, t: torch.Tensor, r_in_group: int, group):
        ctx = self.ctx
        from ..host.distributed import extract_group_info

        _, _, _, start, stride = extract_group_info(group, ctx.cur_rank, ctx.num_ranks)
        return ctx.heap.peer_view(t, start + r_in_group * stride)

    def _cpu_entry(self, group):
        self.ctx.device_barrier(group)

    def _cpu_exit(self, group):
        self.ctx.device_barrier(group)


def owned_tiles(M, N, bm, bn, world, rank, distribution):
    """``(r0, r1, c0, c1)`` of every tile ``rank`` owns in a reduce_scatter of an (M, N) tensor."""
    tiles_m, tiles_n = -(-M // bm), -(-N // bn)
    total = tiles_m * tiles_n
    per = -(-total // world)
    if distribution == 0:
        ids = range(rank, total, world)
    else:
        ids = range(rank * per, min(total, (rank + 1) * per))
    out = []
    for t in ids:
        tm, tn = divmod(t, tiles_n)
        out.append((tm * bm, min(M, (tm + 1) * bm), tn * bn, min(N, (tn + 1) * bn)))
    return out
