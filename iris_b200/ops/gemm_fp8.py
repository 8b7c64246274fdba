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


def _round_up_pow2(scale: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= ``scale`` (what a UE8M0 scale byte can express exactly)."""
    return torch.exp2(torch.ceil(torch.log2(scale)))


def quantize_1x128(x: torch.Tensor, pow2: bool = False):
    """Row-wise quantisation of ``x [M, K]`` in K blocks of 128: returns ``(x_fp8 [M, K], scale [M, ceil(K/128)])``.

    ``pow2=True`` rounds every scale up to a power of two, which is what the tensor core's own block
    scaling takes (``matmul_fp8_blockscaled`` and the fp8 forms of the fused ops)."""
    M, K = x.shape
    kb = _ceil_div(K, 128)
    xp = torch.zeros(M, kb * 128, dtype=torch.float32, device=x.device)
    xp[:, :K] = x.float()
    blocks = xp.view(M, kb, 128)
    amax = blocks.abs().amax(dim=2).clamp_min(1e-12)
    scale = amax / FP8_MAX
    if pow2:
        scale = _round_up_pow2(scale)
    q = (blocks / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).to(FP8).view(M, kb * 128)[:, :K].contiguous()
    return q, scale.contiguous()


def quantize_128x128(w: torch.Tensor, pow2: bool = False):
    """Block quantisation of a weight ``w [N, K]`` in 128 x 128 blocks: ``(w_fp8 [N, K], scale [ceil(N/128), ceil(K/128)])``.
    ``pow2=True``: scales rounded up to powers of two (see ``quantize_1x128``)."""
    N, K = w.shape
    nb, kb = _ceil_div(N, 128), _ceil_div(K, 128)
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, 128, kb, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / FP8_MAX
    if pow2:
        scale = _round_up_pow2(scale)
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


# ----------------------------------------------------------------------------- hardware block scaling
# tcgen05.mma.kind::mxf8f6f4.block_scale multiplies every 32 elements of K of a row by a UE8M0 byte
# (2 ** (byte - 127)) read from TMEM. The kernels fetch those bytes in 512-byte "atoms" covering 128
# rows and one 128-wide K block: row r of the atom sits at byte (r % 32) * 16 + (r // 32) * 4, and its
# four bytes are the four 32-element groups of the block. A 1 x 128 / 128 x 128 quantiser has one scale
# per 128 elements, so the four bytes are equal.
def _ue8m0(scale: torch.Tensor) -> torch.Tensor:
    """Exponent bytes of power-of-two fp32 scales."""
    e = torch.round(torch.log2(scale.float())) + 127.0
    return e.clamp_(0, 254).to(torch.uint8)


def _atoms(rows_exp: torch.Tensor) -> torch.Tensor:
    """``rows_exp [..., 128, KB]`` (bytes of 128 consecutive rows) -> ``[..., KB, 512]`` atoms."""
    lead = rows_exp.shape[:-2]
    kb = rows_exp.shape[-1]
    v = rows_exp.reshape(*lead, 4, 32, kb)                    # row = a * 32 + b
    n = len(lead)
    v = v.permute(*range(n), n + 2, n + 1, n)                 # [..., KB, b, a]
    return v.unsqueeze(-1).expand(*v.shape, 4).reshape(*lead, kb, 512).contiguous()


def pack_scales_a(scale: torch.Tensor) -> torch.Tensor:
    """Activation scales ``[M, KB]`` (powers of two) -> uint8 ``[ceil(M/128), KB, 512]`` atoms."""
    M, kb = scale.shape
    mt = _ceil_div(M, 128)
    e = torch.full((mt * 128, kb), 127, dtype=torch.uint8, device=scale.device)
    e[:M] = _ue8m0(scale)
    return _atoms(e.view(mt, 128, kb))


def pack_scales_b(scale: torch.Tensor, N: int, bn: int) -> torch.Tensor:
    """Weight scales ``[ceil(N/128), KB]`` (powers of two) -> uint8 ``[ceil(N/bn), KB, ceil(bn/128), 512]``:
    the atoms of each ``bn``-wide column tile, rows counted from the tile's first column (a 224-wide tile
    does not start on a 128 boundary, so the packing depends on the tile width the kernel uses)."""
    nb, kb = scale.shape
    tiles, atoms = _ceil_div(N, bn), _ceil_div(bn, 128)
    row_e = _ue8m0(scale).repeat_interleave(128, dim=0)                              # per weight row
    local = torch.arange(atoms * 128, device=scale.device)
    idx = torch.arange(tiles, device=scale.device)[:, None] * bn + local[None, :]     # [tiles, atoms*128]
    valid = (local[None, :] < bn) & (idx < N)
    e = row_e[idx.clamp_max(row_e.shape[0] - 1)]                                      # [tiles, atoms*128, KB]
    e = torch.where(valid[..., None], e, torch.full_like(e, 127))
    return _atoms(e.view(tiles, atoms, 128, kb)).permute(0, 2, 1, 3).contiguous()     # [tiles, KB, atoms, 512]


def blockscaled_tile_n(M: int, N: int, bn: int = 0, two_sm: bool | None = None) -> int:
    """Tile width the block-scaled kernel uses for this problem (224 unless 128 is asked for): the width
    ``pack_scales_b`` must be given."""
    return 128 if bn == 128 else 224


def matmul_fp8_blockscaled(a_q: torch.Tensor, sf_a: torch.Tensor, b_q: torch.Tensor, sf_b: torch.Tensor,
                           out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16, bn: int = 0,
                           two_sm: bool | None = None) -> torch.Tensor:
    """``out[M, N] = (a_q * 2**sa) @ (b_q * 2**sb).T`` with the scaling done by the tensor core.

    ``a_q [M, K]`` and ``b_q [N, K]`` are e4m3; ``sf_a = pack_scales_a(scale_a)`` and
    ``sf_b = pack_scales_b(scale_b, N, blockscaled_tile_n(M, N, bn))`` carry power-of-two scales."""
    if a_q.dtype != FP8 or b_q.dtype != FP8:
        raise TypeError("matmul_fp8_blockscaled takes float8_e4m3fn operands")
    M, K = a_q.shape
    N, K2 = b_q.shape
    if K != K2 or K % 16:
        raise ValueError(f"A has K={K}, B has K={K2}; K must be a multiple of 16")
    tile = blockscaled_tile_n(M, N, bn, two_sm)
    kb = _ceil_div(K, 128)
    if tuple(sf_a.shape) != (_ceil_div(M, 128), kb, 512) or tuple(sf_b.shape) != (_ceil_div(N, tile), kb, _ceil_div(tile, 128), 512):
        raise ValueError("scale atoms do not match the operands and the tile width (see pack_scales_a / pack_scales_b)")
    if sf_a.dtype != torch.uint8 or sf_b.dtype != torch.uint8 or not sf_a.is_contiguous() or not sf_b.is_contiguous():
        raise TypeError("scale atoms are contiguous uint8 tensors")
    if a_q.stride(1) != 1 or b_q.stride(1) != 1:
        raise ValueError("operands must be row-major")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a_q.device)
    if out.dtype not in (torch.bfloat16, torch.float16) or out.stride(1) != 1 or tuple(out.shape) != (M, N):
        raise ValueError("the output must be a row-major (M, N) bf16 or fp16 tensor")
    d = _lib.IrisGemmDesc()
    d.op = _lib.GEMM_LOCAL
    d.M, d.N, d.K = M, N, K
    d.dtype = _lib.DTYPE_CODE[out.dtype]
    d.in_dtype = _lib.DTYPE_CODE[FP8]
    d.b_kmajor = 1
    d.bn = tile
    d.two_sm = 0 if two_sm is None else (2 if two_sm else 1)
    d.A, d.lda = a_q.data_ptr(), a_q.stride(0)
    d.B, d.ldb = b_q.data_ptr(), b_q.stride(0)
    d.C, d.ldc = out.data_ptr(), out.stride(0)
    d.sf_a, d.sf_b = sf_a.data_ptr(), sf_b.data_ptr()
    _lib.check(_lib.kernels().iris_gemm_launch(C.byref(d), C.c_void_p(_lib.current_stream_ptr())), "block-scaled fp8 gemm launch", kernels=1)
    return out


class BlockScaled:
    """An e4m3 matrix with power-of-two block scales, as the fp8 forms of ``matmul`` and of the fused
    ops take it.

    ``kind="activation"``: ``q [M, K]`` with one scale per row and 128-wide K block (``scale [M, KB]``);
    ``kind="weight"``: ``q [N, K]`` (the nn.Linear layout) with one scale per 128 x 128 block
    (``scale [ceil(N/128), KB]``). In a product ``A @ B`` a weight stands for the ``[K, N]`` matrix
    ``q.t()``. The scale atoms the kernels read are packed on first use and kept (for a weight: per
    tile width)."""

    def __init__(self, q: torch.Tensor, scale: torch.Tensor, kind: str):
        if kind not in ("activation", "weight"):
            raise ValueError("kind is 'activation' or 'weight'")
        if q.dtype != FP8 or q.dim() != 2 or q.stride(1) != 1:
            raise TypeError("q must be a row-major float8_e4m3fn matrix")
        R, K = q.shape
        want = (R, _ceil_div(K, 128)) if kind == "activation" else (_ceil_div(R, 128), _ceil_div(K, 128))
        if tuple(scale.shape) != want or scale.dtype != torch.float32:
            raise ValueError(f"scale must be fp32 of shape {want}, got {tuple(scale.shape)} {scale.dtype}")
        self.q, self.scale, self.kind = q, scale, kind
        self._sf: dict = {}

    @property
    def shape(self):
        """Shape of the matrix in a product: ``[M, K]`` for an activation, ``[K, N]`` for a weight."""
        return tuple(self.q.shape) if self.kind == "activation" else (self.q.shape[1], self.q.shape[0])

    @property
    def dtype(self):
        return FP8

    @property
    def device(self):
        return self.q.device

    def dim(self) -> int:
        return 2

    def stride(self, i: int = None):
        """Strides of the matrix in a product (a weight is the transposed view of its storage)."""
        st = tuple(self.q.stride()) if self.kind == "activation" else (self.q.stride(1), self.q.stride(0))
        return st if i is None else st[i]

    def data_ptr(self) -> int:
        return self.q.data_ptr()

    def key(self) -> tuple:
        """What identifies this operand's buffers in a cached kernel descriptor."""
        return (self.q.data_ptr(), self.q.stride(0), self.scale.data_ptr(), self.kind)

    def sf(self, tile_n: int = 0) -> torch.Tensor:
        """Packed scale atoms (``pack_scales_a``; for a weight ``pack_scales_b`` for ``tile_n``-wide tiles)."""
        key = 0 if self.kind == "activation" else tile_n
        hit = self._sf.get(key)
        if hit is None:
            hit = pack_scales_a(self.scale) if self.kind == "activation" else pack_scales_b(self.scale, self.q.shape[0], tile_n)
            self._sf[key] = hit
        return hit

    def set_sf(self, sf: torch.Tensor, tile_n: int = 0) -> "BlockScaled":
        """Install atoms packed elsewhere (e.g. on the symmetric heap)."""
        self._sf[0 if self.kind == "activation" else tile_n] = sf
        return self

    def dequantize(self) -> torch.Tensor:
        """fp32 matrix of the product: ``[M, K]`` (activation) or ``[K, N]`` (weight)."""
        d = dequantize(self.q, self.scale, 1 if self.kind == "activation" else 128)
        return d if self.kind == "activation" else d.t()


def quantize_activation(x: torch.Tensor, out: BlockScaled | None = None) -> BlockScaled:
    """``x [M, K]`` -> e4m3 with power-of-two 1 x 128 scales.

    On a GPU this is one kernel (``csrc/kernels/quantize.cu``) that writes the values, the fp32 scales
    and the packed scale atoms; pass a previous result as ``out`` to reuse its buffers (same shape)."""
    if x.dim() != 2:
        raise ValueError("quantize_activation takes a matrix")
    if not x.is_cuda or x.dtype not in (torch.float32, torch.bfloat16, torch.float16) or x.stride(1) != 1:
        q, s = quantize_1x128(x, pow2=True)
        return BlockScaled(q, s, "activation")
    M, K = x.shape
    kb, mt = _ceil_div(K, 128), _ceil_div(M, 128)
    if out is not None and tuple(out.q.shape) == (M, K) and out.q.device == x.device and 0 in out._sf:
        q, scale, atoms = out.q, out.scale, out._sf[0]
    else:
        q = torch.empty((M, K), dtype=FP8, device=x.device)
        scale = torch.empty((M, kb), dtype=torch.float32, device=x.device)
        atoms = torch.full((mt, kb, 512), 127, dtype=torch.uint8, device=x.device)   # rows past M: scale 1
        out = BlockScaled(q, scale, "activation").set_sf(atoms)
    lib = _lib.kernels()
    if not getattr(lib, "_iris_quant_typed", False):
        lib.iris_quantize_1x128_pow2.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                                 C.c_int32, C.c_int32, C.c_void_p]
        lib.iris_quantize_1x128_pow2.restype = C.c_int
        lib._iris_quant_typed = True
    _lib.check(lib.iris_quantize_1x128_pow2(C.c_void_p(x.data_ptr()), x.stride(0), _lib.DTYPE_CODE[x.dtype], C.c_void_p(q.data_ptr()),
                                            q.stride(0), C.c_void_p(scale.data_ptr()), C.c_void_p(atoms.data_ptr()), M, K,
                                            C.c_void_p(_lib.current_stream_ptr())), "activation quantiser launch", kernels=1)
    return out


def quantize_weight(w: torch.Tensor) -> BlockScaled:
    """``w [N, K]`` (nn.Linear layout) -> e4m3 with power-of-two 128 x 128 scales."""
    q, s = quantize_128x128(w, pow2=True)
    return BlockScaled(q, s, "weight")


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
