"""One-sided operations on heap tensors, callable from the host.

``ctx.rma.store(dst, value, to_rank)``, ``load``, ``get``, ``put``, ``copy`` and the atomics apply
the device RMA functions of ``include/iris/rma.cuh`` elementwise over a (contiguous) tensor: on a
GPU through the generic kernels of ``csrc/kernels/rma_kernels.cu`` on the current stream, on the
CPU backend through the same header compiled for the host. Pointers follow the device API's
convention: a tensor argument always names memory of THIS rank's heap; the rank arguments say on
which rank the access happens (reference semantics: iris/mem/triton/ops.py).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from .heap import _rt

OPS = {"load": 0, "store": 1, "copy": 2, "get": 3, "put": 4, "atomic_add": 5, "atomic_sub": 6, "atomic_and": 7,
       "atomic_or": 8, "atomic_xor": 9, "atomic_min": 10, "atomic_max": 11, "atomic_xchg": 12, "atomic_cas": 13}
SEM = {"relaxed": 0, "acquire": 1, "release": 2, "acq_rel": 3}
SCOPE = {"cta": 0, "gpu": 1, "sys": 2}
CACHE = {None: 0, "": 0, ".ca": 1, ".cg": 2, ".cs": 3, ".cv": 4, ".wb": 5, ".wt": 6}
_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2, torch.int32: 3, torch.int8: 4, torch.int64: 6,
       torch.float64: 7, torch.uint8: 8, torch.int16: 9}
for _name, _code in (("float8_e4m3fn", 5), ("uint32", 10), ("uint64", 11)):
    if hasattr(torch, _name):
        _DT[getattr(torch, _name)] = _code


class HostRMA:
    def __init__(self, ctx):
        self.ctx = ctx

    def _lib(self):
        lib = _lib.kernels()
        if not getattr(lib, "_iris_rma_typed", False):
            vp = C.c_void_p
            lib.iris_rma_launch.argtypes = [C.POINTER(_lib.IrisCtx)] + [C.c_int] * 8 + [vp, vp, vp, C.c_double, C.c_longlong,
                                                                                         C.c_longlong, C.c_ulonglong, C.c_int, C.c_int, vp]
            lib.iris_rma_launch.restype = C.c_int
            lib._iris_rma_typed = True
        return lib

    def _run(self, op: str, a: torch.Tensor, b=None, result=None, value=None, cmp=None, from_rank=None, to_rank=None,
             sem="acq_rel", scope="sys", cache_ld=None, cache_st=None, volatile=False, oo=False):
        ctx = self.ctx
        if not a.is_contiguous() or (b is not None and not b.is_contiguous()):
            raise ValueError("host RMA works on contiguous tensors")
        if a.dtype not in _DT:
            raise TypeError(f"dtype {a.dtype} is not supported by host RMA")
        if sem not in SEM or scope not in SCOPE:
            raise ValueError("sem must be one of relaxed/acquire/release/acq_rel, scope one of cta/gpu/sys")
        if cache_ld not in CACHE or cache_st not in CACHE:
            raise ValueError(f"unknown cache modifier {cache_ld!r}/{cache_st!r}")
        from_rank = ctx.cur_rank if from_rank is None else from_rank
        to_rank = ctx.cur_rank if to_rank is None else to_rank
        for r in (from_rank, to_rank):
            if not 0 <= r < ctx.num_ranks:
                raise ValueError(f"rank {r} out of range")
        # A tensor whose address is translated to another rank must lie on the heap: the same
        # offset has to exist there. (A device kernel would otherwise touch unmapped memory.)
        me = ctx.cur_rank
        translated = {"load": [(a, from_rank)], "store": [(a, to_rank)], "get": [(a, from_rank)], "put": [(b, to_rank)],
                      "copy": [(a, from_rank), (b, to_rank)]}.get(op, [(a, to_rank)])
        for t, r in translated:
            if r != me and not ctx.is_symmetric(t):
                raise ValueError(f"host RMA {op}: the tensor accessed on rank {r} is not on the symmetric heap")
        fval, ival, icmp = 0.0, 0, 0
        if value is not None:
            if a.dtype in (torch.float16, torch.bfloat16):
                ival = int(torch.tensor(value, dtype=a.dtype).view(torch.int16).item()) & 0xFFFF
            elif a.dtype.is_floating_point:
                fval = float(value)
            else:
                ival = int(value)
        if cmp is not None:
            if a.dtype.is_floating_point:
                fval = float(cmp)  # cas on floats compares the scalar given as `cmp`
            icmp = int(cmp) if not a.dtype.is_floating_point else 0
        n = a.numel()
        pa = a.data_ptr()
        pb = b.data_ptr() if b is not None else 0
        pr = result.data_ptr() if result is not None else 0
        if ctx.is_cpu:
            bases = ctx.heap.bases_host()
            arr = (C.c_uint64 * ctx.num_ranks)(*[int(x) for x in bases])
            rc = _rt().iris_cpu_rma(OPS[op], _DT[a.dtype], SEM[sem], pa, pb, pr, fval, ival, icmp, n, from_rank, to_rank,
                                    ctx.cur_rank, arr)
        else:
            c = ctx.ctx_struct()
            rc = self._lib().iris_rma_launch(C.byref(c), OPS[op], _DT[a.dtype], SEM[sem], SCOPE[scope], CACHE[cache_ld],
                                             CACHE[cache_st], int(volatile), int(oo), pa or None, pb or None, pr or None,
                                             fval, ival, icmp, n, from_rank, to_rank, C.c_void_p(_lib.current_stream_ptr()))
        if rc != 0:
            raise RuntimeError(f"host RMA {op} on {a.dtype} failed with code {rc}")
        return result

    # ---- data movement
    def load(self, src: torch.Tensor, from_rank: int, cache_modifier=None, volatile=False, oo=False) -> torch.Tensor:
        """Return ``src`` as stored on ``from_rank`` (a new local tensor)."""
        out = torch.empty_like(src)
        return self._run("load", src, result=out, from_rank=from_rank, cache_ld=cache_modifier, volatile=volatile, oo=oo)

    def store(self, dst: torch.Tensor, value, to_rank: int, cache_modifier=None, oo=False) -> None:
        """Write ``value`` (scalar or tensor of dst's shape) into ``dst`` on ``to_rank``."""
        if isinstance(value, torch.Tensor):
            self._run("store", dst, b=value.to(dst.dtype).contiguous(), to_rank=to_rank, cache_st=cache_modifier, oo=oo)
        else:
            self._run("store", dst, value=value, to_rank=to_rank, cache_st=cache_modifier, oo=oo)

    def get(self, from_tensor: torch.Tensor, to_tensor: torch.Tensor, from_rank: int, oo=False) -> None:
        """Copy ``from_tensor`` as stored on ``from_rank`` into my ``to_tensor``."""
        self._run("get", from_tensor, b=to_tensor, from_rank=from_rank, to_rank=self.ctx.cur_rank, oo=oo)

    def put(self, from_tensor: torch.Tensor, to_tensor: torch.Tensor, to_rank: int, oo=False) -> None:
        """Copy my ``from_tensor`` into ``to_tensor`` on ``to_rank``."""
        self._run("put", from_tensor, b=to_tensor, from_rank=self.ctx.cur_rank, to_rank=to_rank, oo=oo)

    def copy(self, src: torch.Tensor, dst: torch.Tensor, from_rank: int, to_rank: int, oo=False) -> None:
        """Copy ``src`` on ``from_rank`` to ``dst`` on ``to_rank``; this rank must be one of the two."""
        if self.ctx.cur_rank not in (from_rank, to_rank):
            raise ValueError("copy: the calling rank must be the source or the destination")
        self._run("copy", src, b=dst, from_rank=from_rank, to_rank=to_rank, oo=oo)

    # ---- atomics (return the previous values)
    def _atomic(self, op, t, value, to_rank, sem, scope, cmp=None):
        out = torch.empty_like(t)
        if isinstance(value, torch.Tensor):
            return self._run(op, t, b=value.to(t.dtype).contiguous(), result=out, to_rank=to_rank, sem=sem, scope=scope, cmp=cmp)
        return self._run(op, t, result=out, value=value, to_rank=to_rank, sem=sem, scope=scope, cmp=cmp)

    def atomic_add(self, t, value, to_rank, sem="acq_rel", scope="sys"):
        return self._atomic("atomic_add", t, value, to_rank, sem, scope)

    def atomic_sub(self, t, value, to_rank, sem="acq_rel", scope="sys"):
        return self._atomic("atomic_sub", t, value, to_rank, sem, scope)

    def atomic_and(self, t, value, to_rank, sem="acq_rel", scope="sys"):
        return self._atomic("atomic_and", t, value, to_rank, sem, scope)

    def atomic_or(self, t, value, to_rank, sem="acq_rel", scope="sys"):
        return self._atomic("atomic_or", t, value, to_rank, sem, scope)

    def atomic_xor(self, t, value, to_rank, sem="acq_rel", scope="sys"):
        return self._atomic("atomic_xor", t, value, to_rank, sem, scope)

    def atomic_min(self, t, value, to_rank, sem="acq_rel", scope="sys"):
        return self._atomic("atomic_min", t, value, to_rank, sem, scope)

    def atomic_max(self, t, value, to_rank, sem="acq_rel", scope="sys"):
        return self._atomic("atomic_max", t, value, to_rank, sem, scope)

    def atomic_xchg(self, t, value, to_rank, sem="acq_rel", scope="sys"):
        return self._atomic("atomic_xchg", t, value, to_rank, sem, scope)

    def atomic_cas(self, t, cmp, value, to_rank, sem="acq_rel", scope="sys"):
        if t.dtype.is_floating_point:
            raise TypeError("atomic_cas from the host compares integers (flags and locks); view the tensor as int32/int64")
        return self._atomic("atomic_cas", t, value, to_rank, sem, scope, cmp=cmp)
