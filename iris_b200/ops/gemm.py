"""Local GEMM on the hand-written sm_100a kernel (TMA + tcgen05 + TMEM).

``matmul(A, B, bias=None, out=None)`` computes ``A @ B`` for 16-bit inputs with fp32 accumulation.
``B`` may be a row-major ``(K, N)`` tensor (the layout the reference's benchmarks use,
benchmark/ops/bench_all_gather_matmul.py:26) or the transposed view of an ``(N, K)`` weight
(``W.t()``, nn.Linear layout); both run without a copy. This is the stand-in for the tritonblas
main loop the reference's fused ops are built on (iris/ops/matmul_all_reduce.py:95-105).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib


def b_layout(B: torch.Tensor):
    """Return (data tensor, b_kmajor, ldb) for a logical (K, N) matrix B, copying only if needed."""
    if B.dim() != 2:
        raise ValueError("B must be 2-D")
    if B.stride(1) == 1 and B.stride(0) >= B.shape[1]:
        return B, 0, B.stride(0)
    if B.stride(0) == 1 and B.stride(1) >= B.shape[0]:
        return B, 1, B.stride(1)
    Bc = B.contiguous()
    return Bc, 0, Bc.stride(0)


def fill_desc(desc: _lib.IrisGemmDesc, A: torch.Tensor, B: torch.Tensor, out: torch.Tensor, bias_row=None,
              bias_col=None, bn: int = 0):
    if A.dtype not in (torch.bfloat16, torch.float16) or B.dtype != A.dtype or out.dtype != A.dtype:
        raise TypeError("the sm_100a GEMM takes fp16 or bf16 operands of one dtype")
    if A.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("A and the output must be row-major")
    Bd, kmajor, ldb = b_layout(B)
    desc.dtype = _lib.DTYPE_CODE[A.dtype]
    desc.b_kmajor = kmajor
    desc.bn = bn
    desc.A = A.data_ptr()
    desc.lda = A.stride(0)
    desc.B = Bd.data_ptr()
    desc.ldb = ldb
    desc.C = out.data_ptr()
    desc.ldc = out.stride(0)
    desc.bias_row = bias_row.data_ptr() if bias_row is not None else None
    desc.bias_col = bias_col.data_ptr() if bias_col is not None else None
    return Bd


def matmul(A: torch.Tensor, B: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
           bias_dim: int = 1, bn: int = 0, two_sm: bool | None = None) -> torch.Tensor:
    """``out = A @ B (+ bias)``; ``bias_dim=0`` adds ``bias[m]`` to every row m, ``1`` adds ``bias[n]``.

    ``two_sm`` selects the variant in which the two CTAs of a cluster share one 256-row tile
    (``tcgen05.mma.cta_group::2``): ``True`` whenever the shape allows, ``False`` never, ``None``
    lets the plan pick by wave count.

    Block-scaled e4m3 operands (``BlockScaled`` activation and weight, see ``gemm_fp8``) go to the
    hardware-scaled kernel; the result is bf16 unless ``out`` says otherwise."""
    from .gemm_fp8 import BlockScaled, blockscaled_tile_n, matmul_fp8_blockscaled

    if isinstance(A, BlockScaled) or isinstance(B, BlockScaled):
        if not (isinstance(A, BlockScaled) and isinstance(B, BlockScaled) and A.kind == "activation" and B.kind == "weight"):
            raise TypeError("an fp8 product takes a BlockScaled activation and a BlockScaled weight")
        if bias is not None:
            raise ValueError("the block-scaled local GEMM takes no bias")
        tile = blockscaled_tile_n(A.shape[0], B.shape[1], bn, two_sm)
        return matmul_fp8_blockscaled(A.q, A.sf(), B.q, B.sf(tile), out=out, bn=bn, two_sm=two_sm)
    M, K = A.shape
    K2, N = B.shape
    if K != K2:
        raise ValueError(f"shape mismatch {tuple(A.shape)} @ {tuple(B.shape)}")
    if out is None:
        out = torch.empty((M, N), dtype=A.dtype, device=A.device)
    elif tuple(out.shape) != (M, N) or out.device != A.device:
        raise ValueError(f"out must be {(M, N)} on {A.device}, got {tuple(out.shape)} on {out.device}")
    if bias is not None and (bias_dim not in (0, 1) or bias.dim() != 1 or bias.numel() != (M if bias_dim == 0 else N)):
        raise ValueError(f"bias must have {M if bias_dim == 0 else N} entries for bias_dim={bias_dim}, got {tuple(bias.shape)}")
    desc = _lib.IrisGemmDesc()
    desc.op = _lib.GEMM_LOCAL
    desc.M, desc.N, desc.K = M, N, K
    b32 = bias.float().contiguous() if bias is not None else None
    keep = fill_desc(desc, A, B, out, bias_row=b32 if bias_dim == 0 else None, bias_col=b32 if bias_dim == 1 else None, bn=bn)
    desc.ctx.world = 1
    desc.two_sm = 0 if two_sm is None else (2 if two_sm else 1)
    _lib.check(_lib.kernels().iris_gemm_launch(C.byref(desc), _lib.current_stream_ptr()), "gemm launch", kernels=1)
    del keep
    return out
