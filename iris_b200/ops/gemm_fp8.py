"""Block-scaled fp8 (e4m3) GEMM on the hand-written sm_100a kernel (``csrc/kernels/gemm_fp8.cu``).

Scale layout of block-quantised transformer weights: activations carry one fp32 scale per row and
128-wide K block (``1 x 128``), weights one per ``128 x 128`` block. ``matmul_fp8`` computes

    C[m, n] = sum_kb  sa[m, kb] * sb[n // 128, kb] * sum_{k in block kb} A[m, k] * B[n, k]

with fp32 accumulation and a 16-bit result. The reference has no fp8 path; the 16-bit GEMM its
fused ops are built on is iris/ops/matmul_all_reduce.py:95-105.

``quantize_1x128`` / ``quantize_128x128`` produce the operands from 16/32-bit tensors and
``dequant_matmul`` is the plain PyTorch fp32 statement of the same product (used by the tests).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


class IrisFp8GemmDesc(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("scale_a", C.c_void_p), ("scale_b", C.c_void_p), ("C", C.c_void_p),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("out_dtype", C.c_int32),
        ("status", C.c_void_p),
    ]


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def quantize_1x128(x: torch.Tensor):
    """Row-wise quantisation of ``x [M, K]`` in K blocks of 128: returns ``(x_fp8 [M, K], scale [M, ceil(K/128)])``."""
    M, K = x.shape
    kb = _ceil_div(K, 128)
    xp = torch.zeros(M, kb * 128, dtype=torch.float32, device=x.device)
    xp[:, :K] = x.float()
    blocks = xp.view(M, kb, 128)
    amax = blocks.abs().amax(dim=2).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (blocks / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).to(FP8).view(M, kb * 128)[:, :K].contiguous()
    return q, scale.contiguous()


def quantize_128x128(w: torch.Tensor):
    """Block quantisation of a weight ``w [N, K]`` in 128 x 128 blocks: ``(w_fp8 [N, K], scale [ceil(N/128), ceil(K/128)])``."""
    N, K = w.shape
    nb, kb = _ceil_div(N, 128), _ceil_div(K, 128)
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, 128, kb, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(FP8).view(nb * 128, kb * 128)[:N, :K].contiguous()
    return q, scale.contiguous()


def dequantize(q: torch.Tensor, scale: torch.Tensor, block_rows: int) -> torch.Tensor:
    """fp32 tensor from fp8 values and their block scales (``block_rows`` 1 for activations, 128 for weights)."""
    R, K = q.shape
    s = scale.repeat_interleave(128, dim=1)[:, :K]
    if block_rows > 1:
        s = s.repeat_interleave(block_rows, dim=0)[:R]
    return q.float() * s


def dequant_matmul(a_q, a_scale, b_q, b_scale) -> torch.Tensor:
    """fp32 reference: ``dequantize(A) @ dequantize(B).T``."""
    return dequantize(a_q, a_scale, 1) @ dequantize(b_q, b_scale, 128).t()


def _typed(lib):
    if not getattr(lib, "_iris_fp8_typed", False):
        lib.iris_gemm_fp8_launch.argtypes = [C.POINTER(IrisFp8GemmDesc), C.c_void_p]
        lib.iris_gemm_fp8_launch.restype = C.c_int
        lib._iris_fp8_typed = True
    return lib


def matmul_fp8(a_q: torch.Tensor, a_scale: torch.Tensor, b_q: torch.Tensor, b_scale: torch.Tensor,
               out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16, status=None) -> torch.Tensor:
    """``out[M, N] = (a_q * a_scale) @ (b_q * b_scale).T``; ``a_q [M, K]``, ``b_q [N, K]`` e4m3, scales fp32."""
    if a_q.dtype != FP8 or b_q.dtype != FP8:
        raise TypeError("matmul_fp8 takes float8_e4m3fn operands")
    M, K = a_q.shape
    N, K2 = b_q.shape
    if K != K2:
        raise ValueError(f"shape mismatch: A has K={K}, B has K={K2}")
    kb, nb = _ceil_div(K, 128), _ceil_div(N, 128)
    if tuple(a_scale.shape) != (M, kb) or tuple(b_scale.shape) != (nb, kb):
        raise ValueError(f"scales must be {(M, kb)} and {(nb, kb)}, got {tuple(a_scale.shape)} and {tuple(b_scale.shape)}")
    if a_scale.dtype != torch.float32 or b_scale.dtype != torch.float32:
        raise TypeError("scales are fp32")
    if a_q.stride(1) != 1 or b_q.stride(1) != 1 or not a_scale.is_contiguous() or not b_scale.is_contiguous():
        raise ValueError("operands must be row-major, scales contiguous")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a_q.device)
    if out.dtype not in (torch.bfloat16, torch.float16) or out.stride(1) != 1 or tuple(out.shape) != (M, N):
        raise ValueError("the output must be a row-major (M, N) bf16 or fp16 tensor")
    d = IrisFp8GemmDesc()
    d.A, d.B = a_q.data_ptr(), b_q.data_ptr()
    d.scale_a, d.scale_b = a_scale.data_ptr(), b_scale.data_ptr()
    d.C = out.data_ptr()
    d.lda, d.ldb, d.ldc = a_q.stride(0), b_q.stride(0), out.stride(0)
    d.M, d.N, d.K = M, N, K
    d.out_dtype = _lib.DTYPE_CODE[out.dtype]
    d.status = status.data_ptr() if status is not None else None
    _lib.check(_typed(_lib.kernels()).iris_gemm_fp8_launch(C.byref(d), C.c_void_p(_lib.current_stream_ptr())), "fp8 gemm launch", kernels=1)
    return out
