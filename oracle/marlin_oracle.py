"""CPU oracle for the Marlin weight-only GEMM / fused-MoE path.

TEST INFRASTRUCTURE ONLY.  This module restates, in vectorised torch/numpy, the
CPU semantics that the reference project's own test-suite uses to judge its
CUDA kernels.  It is imported only by the tests, by the smoke check and by the
CPU-baseline / reference legs of the benchmark - never by the product package,
which has no CPU fallback.

Parity status: PINNED.  Every function here is checked bit-for-bit (integer
work) or value-for-value (floating point) against outputs of the reference's
own Python helpers, stored as fixtures under ``tests/golden`` by
``tests/golden/make_golden.py`` (which imports the reference), and against the
literal known-answer inputs of the reference's tests.

Reference files restated (paths inside the reference project):
  tests/quant_utils.py:125-240      packed "native" weight layout
  tests/helpers.py:401-445,548-562  GPTQ / AWQ raw packers
  tests/helpers.py:641-698          integer quantisers
  tests/helpers.py:742-911          e2m1 / nvfp4 / mxfp4 / fp8 quantisers
  tests/helpers.py:1094-1184,1576-1641  dequantisers
  tests/helpers.py:1749-1760        dense reference (fp32 matmul)
  tests/helpers.py:2039-2060        MoE reference
  tests/test_marlin_moe.py:111-133,194-213  routing / align oracles
"""
from __future__ import annotations

import math

import numpy as np
import torch

# ---------------------------------------------------------------------------
# scalar type ids (vllm/scalar_type.py:26-43)
# ---------------------------------------------------------------------------


def scalar_type_id(exponent: int, mantissa: int, signed: bool, bias: int = 0,
                   finite_only: bool = False, nan_repr: int = 1) -> int:
    """58-bit packed id: exponent(8) | mantissa(8) | signed(1) | bias(32) | finite(1) | nan(8)."""
    val, off = 0, 0
    for member, width in ((exponent, 8), (mantissa, 8), (int(signed), 1), (bias, 32),
                          (int(finite_only), 1), (nan_repr, 8)):
        val |= (int(member) & ((1 << width) - 1)) << off
        off += width
    return val


TYPE_U4 = scalar_type_id(0, 4, False, 0)
TYPE_U4B8 = scalar_type_id(0, 4, False, 8)
TYPE_U8 = scalar_type_id(0, 8, False, 0)
TYPE_U8B128 = scalar_type_id(0, 8, False, 128)
TYPE_FE2M1 = scalar_type_id(2, 1, True, 0, True, 0)
TYPE_FE4M3 = scalar_type_id(4, 3, True, 0, True, 2)

_ORDER = {4: (0, 2, 4, 6, 1, 3, 5, 7), 8: (0, 2, 1, 3)}

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
               -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def macro_n(size_n: int) -> int:
    """Width of one packed column group (csrc/quantization/marlin/sm70_marlin_common.cuh:295-308)."""
    if size_n % 256 == 0:
        return 256
    if size_n % 128 == 0:
        return 128
    if size_n % 64 == 0:
        return 64
    raise ValueError(f"size_n must be a multiple of 64, got {size_n}")


# ---------------------------------------------------------------------------
# raw checkpoint packers
# ---------------------------------------------------------------------------


def gptq_pack(q: torch.Tensor, bits: int) -> torch.Tensor:
    """[K, N] ints -> int32 [K/pf, N]; value (k, n) sits in word [k // pf, n] at bit (k % pf) * bits
    (tests/helpers.py:401-426)."""
    pf = 32 // bits
    k, n = q.shape
    a = q.to(torch.int64).reshape(k // pf, pf, n)
    shifts = (torch.arange(pf, dtype=torch.int64) * bits).reshape(1, pf, 1)
    word = (a << shifts).sum(dim=1) & 0xFFFFFFFF
    return _to_i32(word)


def awq_pack(q: torch.Tensor, bits: int) -> torch.Tensor:
    """[K, N] ints -> int32 [K, N/pf] with the AWQ interleave inside each word
    (tests/helpers.py:429-445,548-562)."""
    pf = 32 // bits
    k, n = q.shape
    order = torch.tensor(_ORDER[bits], dtype=torch.long)
    a = q.to(torch.int64).reshape(k, n // pf, pf)[:, :, order]
    shifts = (torch.arange(pf, dtype=torch.int64) * bits).reshape(1, 1, pf)
    word = (a << shifts).sum(dim=2) & 0xFFFFFFFF
    return _to_i32(word)


def _to_i32(word: torch.Tensor) -> torch.Tensor:
    word = torch.where(word >= (1 << 31), word - (1 << 32), word)
    return word.to(torch.int32).contiguous()


# ---------------------------------------------------------------------------
# packed weight layout
# ---------------------------------------------------------------------------


def marlin_pack(q: torch.Tensor, bits: int) -> torch.Tensor:
    """[K, N] ints -> int32 [K/16, N*16/pf] in the reference's packed layout.

    Row kt = k // 16.  Inside a row, columns are cut into groups of macro_n(N); a group holds, for
    lk = k % 16 and nv = (n % 64) // pf, the g = macro_n / 64 words of its g 64-wide tiles side by
    side: index = group * g * W + (lk * (64 / pf) + nv) * g + tile_in_group with W = 1024 / pf.
    Inside a word the pf consecutive-n values are stored in the order of ``_ORDER``
    (tests/quant_utils.py:125-240)."""
    pf = 32 // bits
    k, n = q.shape
    if k % 16 or n % 64:
        raise ValueError(f"need K % 16 == 0 and N % 64 == 0, got {(k, n)}")
    g = macro_n(n) // 64
    order = torch.tensor(_ORDER[bits], dtype=torch.long)
    a = q.to(torch.int64).reshape(k // 16, 16, n // (64 * g), g, 64 // pf, pf)[..., order]
    shifts = (torch.arange(pf, dtype=torch.int64) * bits).reshape(1, 1, 1, 1, 1, pf)
    word = (a << shifts).sum(dim=-1) & 0xFFFFFFFF          # [kt, lk, grp, sub, nv]
    word = word.permute(0, 2, 1, 4, 3).reshape(k // 16, n * 16 // pf)
    return _to_i32(word)


def marlin_unpack(packed: torch.Tensor, size_k: int, size_n: int, bits: int) -> torch.Tensor:
    """Inverse of :func:`marlin_pack` -> int32 [K, N] (tests/helpers.py:1657-1723)."""
    pf = 32 // bits
    g = macro_n(size_n) // 64
    w = packed.to(torch.int64) & 0xFFFFFFFF
    w = w.reshape(size_k // 16, size_n // (64 * g), 16, 64 // pf, g)   # [kt, grp, lk, nv, sub]
    shifts = (torch.arange(pf, dtype=torch.int64) * bits)
    vals = (w.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)             # position-major
    inv = torch.empty(pf, dtype=torch.long)
    inv[torch.tensor(_ORDER[bits])] = torch.arange(pf)
    vals = vals[..., inv]                                              # logical n % pf
    vals = vals.permute(0, 2, 1, 4, 3, 5).reshape(size_k, size_n)
    return vals.to(torch.int32).contiguous()


def stream_layout_pack(q: torch.Tensor, bits: int) -> torch.Tensor:
    """[K, N] ints -> int32 [K/16, N*16/pf]: the same codes as :func:`marlin_pack` in the streaming
    layout of the B200 library (no counterpart in the reference; the statement of the layout is
    ``marlin_v100_b200/csrc/stream_layout.cuh``).  Word order [column group of 256][k // 64][n % 256 // 16]
    then, 4-bit: [n % 8][k % 16 // 4][k % 64 // 16], nibble = (k % 2) * 4 + (k % 4 // 2) * 2 + (n % 16 // 8);
    8-bit: [k % 64 // 32][n % 8][k % 16 // 4][k % 32 // 16][k % 4 // 2], byte = (n % 16 // 8) * 2 + k % 2."""
    pf = 32 // bits
    k, n = q.shape
    if k % 128 or n % 256:
        raise ValueError(f"need K % 128 == 0 and N % 256 == 0, got {(k, n)}")
    a = q.to(torch.int64)
    if bits == 4:
        # k = kb*64 + j*16 + t*4 + e2*2 + e1 ; n = grp*256 + slab*16 + hi*8 + g8
        a = a.reshape(k // 64, 4, 4, 2, 2, n // 256, 16, 2, 8)       # kb j t e2 e1 grp slab hi g8
        a = a.permute(5, 0, 6, 8, 2, 1, 4, 3, 7)                      # grp kb slab g8 t j | e1 e2 hi
    else:
        a = a.reshape(k // 64, 2, 2, 4, 2, 2, n // 256, 16, 2, 8)    # kb jh jl t y e1 grp slab hi g8
        a = a.permute(6, 0, 7, 1, 9, 3, 2, 4, 8, 5)                   # grp kb slab jh g8 t jl y | hi e1
    a = a.reshape(-1, pf)
    shifts = (torch.arange(pf, dtype=torch.int64) * bits).reshape(1, pf)
    word = (a << shifts).sum(dim=-1) & 0xFFFFFFFF
    return _to_i32(word).reshape(k // 16, n * 16 // pf)


def stream_layout_unpack(packed: torch.Tensor, size_k: int, size_n: int, bits: int) -> torch.Tensor:
    """Inverse of :func:`stream_layout_pack` -> int32 [K, N]."""
    pf = 32 // bits
    w = (packed.to(torch.int64) & 0xFFFFFFFF).reshape(-1, 1)
    shifts = (torch.arange(pf, dtype=torch.int64) * bits).reshape(1, pf)
    v = (w >> shifts) & ((1 << bits) - 1)
    k, n = size_k, size_n
    if bits == 4:
        v = v.reshape(n // 256, k // 64, 16, 8, 4, 4, 2, 2, 2)       # grp kb slab g8 t j e1 e2 hi
        v = v.permute(1, 5, 4, 7, 6, 0, 2, 8, 3)                      # kb j t e2 e1 grp slab hi g8
    else:
        v = v.reshape(n // 256, k // 64, 16, 2, 8, 4, 2, 2, 2, 2)    # grp kb slab jh g8 t jl y hi e1
        v = v.permute(1, 3, 6, 5, 7, 9, 0, 2, 8, 4)                   # kb jh jl t y e1 grp slab hi g8
    return v.reshape(k, n).to(torch.int32).contiguous()


def gptq_marlin_repack(b_q_weight: torch.Tensor, perm: torch.Tensor | None, size_k: int,
                       size_n: int, bits: int) -> torch.Tensor:
    """Oracle of the repack op: unpack GPTQ words, gather rows by ``perm`` (act-order), re-pack
    (csrc/quantization/marlin/gptq_marlin_repack.cu:399-469)."""
    pf = 32 // bits
    w = b_q_weight.to(torch.int64) & 0xFFFFFFFF
    shifts = (torch.arange(pf, dtype=torch.int64) * bits).reshape(1, pf, 1)
    q = ((w.unsqueeze(1) >> shifts) & ((1 << bits) - 1)).reshape(size_k, size_n)
    if perm is not None and perm.numel() > 0:
        q = q.index_select(0, perm.to(torch.long))
    return marlin_pack(q, bits)


def awq_marlin_repack(b_q_weight: torch.Tensor, size_k: int, size_n: int, bits: int) -> torch.Tensor:
    """Oracle of the AWQ repack op (csrc/quantization/marlin/awq_marlin_repack.cu:319-381)."""
    pf = 32 // bits
    w = b_q_weight.to(torch.int64) & 0xFFFFFFFF
    shifts = (torch.arange(pf, dtype=torch.int64) * bits)
    vals = (w.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)      # position-major [K, N/pf, pf]
    inv = torch.empty(pf, dtype=torch.long)
    inv[torch.tensor(_ORDER[bits])] = torch.arange(pf)
    q = vals[..., inv].reshape(size_k, size_n)
    return marlin_pack(q, bits)


def permute_bias(bias: torch.Tensor) -> torch.Tensor:
    """Bias as it crosses the op boundary: permuted per 32 by ``scale_perm_single``
    (tests/helpers.py:85-110)."""
    perm = []
    for i in range(4):
        perm.extend([2 * i + j for j in (0, 1, 8, 9, 16, 17, 24, 25)])
    shape = bias.shape
    return bias.reshape(-1, 32)[:, perm].reshape(shape).contiguous()


def unpermute_bias(bias: torch.Tensor) -> torch.Tensor:
    perm = []
    for i in range(4):
        perm.extend([2 * i + j for j in (0, 1, 8, 9, 16, 17, 24, 25)])
    inv = torch.empty(32, dtype=torch.long)
    inv[torch.tensor(perm)] = torch.arange(32)
    shape = bias.shape
    return bias.reshape(-1, 32)[:, inv].reshape(shape).contiguous()


# ---------------------------------------------------------------------------
# quantisers: fp weight [K, N] -> the tensors that cross the op boundary
# ---------------------------------------------------------------------------


def _groups(size_k: int, group_size: int) -> int:
    gs = size_k if group_size == -1 else group_size
    if size_k % gs:
        raise ValueError(f"group_size={gs} must divide size_k={size_k}")
    return gs


def quantize_sym(weight: torch.Tensor, bits: int, group_size: int):
    """u4b8 / u8b128: scale = max|w| / (bias - 1); q = clamp(round(w / s), -bias, bias - 1) + bias
    (tests/helpers.py:641-658).  Returns (q [K,N] int32, scales [G,N] in weight dtype)."""
    bias = 1 << (bits - 1)
    k, n = weight.shape
    gs = _groups(k, group_size)
    r = weight.reshape(k // gs, gs, n)
    max_abs = r.abs().amax(dim=1).clamp_min(1e-6)
    scales = (max_abs / float(bias - 1)).to(weight.dtype)
    q = torch.round(r / scales.unsqueeze(1)).clamp(-bias, bias - 1).to(torch.int32) + bias
    return q.reshape(k, n), scales


def quantize_asym(weight: torch.Tensor, bits: int, group_size: int):
    """u4 / u8 with zero-points: s = (max - min) / qmax, zp = round(-min / s)
    (tests/helpers.py:661-698).  Returns (q, scales, zero_points int32 [G,N], zp_float [G,N]) where
    zp_float = (zp * s) rounded to the weight dtype - the form the GEMM consumes."""
    qmax = (1 << bits) - 1
    k, n = weight.shape
    gs = _groups(k, group_size)
    r = weight.to(torch.float32).reshape(k // gs, gs, n)
    mins, maxs = r.amin(dim=1), r.amax(dim=1)
    scales = ((maxs - mins) / float(qmax)).clamp_min(1e-6)
    zp = torch.round(-mins / scales).clamp(0, qmax).to(torch.int32)
    q = torch.round(r / scales.unsqueeze(1) + zp.unsqueeze(1)).clamp(0, qmax).to(torch.int32)
    s = scales.to(weight.dtype)
    zpf = (zp.to(torch.float32) * s.to(torch.float32)).to(weight.dtype)
    return q.reshape(k, n), s, zp.contiguous(), zpf


def fp8_scale_exponent_bias(dtype: torch.dtype) -> int:
    """Power of two folded into fp8 scales at the boundary: 8 for fp16, 120 for bf16
    (vllm/model_executor/layers/quantization/utils/marlin_utils_fp8.py:28-39)."""
    return 8 if dtype == torch.float16 else 120


def fp8_fuse_exponent_bias(scales: torch.Tensor) -> torch.Tensor:
    """Boundary form of fp8 scales: scale * 2^bias in the scales' own dtype
    (vllm/model_executor/layers/quantization/utils/marlin_utils_fp8.py:28-39)."""
    return scales * (torch.ones_like(scales) * 2) ** fp8_scale_exponent_bias(scales.dtype)


def quantize_fp8(weight: torch.Tensor, group_size: int):
    """fp8-e4m3: s = amax / 448 (tests/helpers.py:890-911).  Returns (raw bytes [K,N] int32,
    boundary scales [G,N] = s * 2^bias in weight dtype, plain scales fp32)."""
    if group_size not in (-1, 128):
        raise ValueError("fp8 supports only group_size -1 or 128")
    k, n = weight.shape
    gs = _groups(k, group_size)
    r = weight.to(torch.float32).reshape(k // gs, gs, n)
    scales = (r.abs().amax(dim=1) / 448.0).clamp_min(1e-6)
    w8 = (r / scales.unsqueeze(1)).to(torch.float8_e4m3fn).reshape(k, n)
    raw = w8.contiguous().view(torch.uint8).to(torch.int32)
    s = scales.to(weight.dtype)
    boundary = (s * float(2.0 ** fp8_scale_exponent_bias(weight.dtype))).to(weight.dtype)
    return raw, boundary, scales


def quantize_e2m1(values: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 code, first table entry on ties (tests/helpers.py:742-770)."""
    table = torch.tensor(E2M1_VALUES, dtype=torch.float32)
    out = torch.empty(values.shape, dtype=torch.int32)
    flat = values.to(torch.float32).reshape(-1)
    res = out.reshape(-1)
    step = 1 << 20
    for i in range(0, flat.numel(), step):
        d = (flat[i:i + step].unsqueeze(-1) - table).abs()
        res[i:i + step] = d.argmin(dim=-1).to(torch.int32)
    return out


def nvfp4_exponent_bias(dtype: torch.dtype) -> int:
    """14 for fp16, 126 for bf16 (marlin_utils_fp4.py:132-144)."""
    return 14 if dtype == torch.float16 else 126


def nvfp4_scale_factor(scales_half: torch.Tensor, a_dtype: torch.dtype) -> float:
    """Power-of-two rescale so that scale * 2^7 >= 2 for non-fp16 activations
    (marlin_utils_fp4.py:30-50)."""
    if a_dtype == torch.float16:
        return 1.0
    ws = scales_half.float() * 128.0
    nz = ws > 0
    if nz.any():
        mn = ws[nz].min()
        if mn < 2:
            return float((2 / mn).log2().ceil().exp2().item())
    return 1.0


def nvfp4_encode_scales(fp8_scales: torch.Tensor, a_dtype: torch.dtype, scale_factor: float | None = None):
    """e4m3 scales [G,N] -> boundary bytes: [0,2,1,3] interleave per 4 along N, times scale_factor,
    times 2^7, fp16 bits << 1, high byte (marlin_utils_fp4.py:53-112)."""
    s = fp8_scales.to(torch.float16)
    s = s.reshape(-1, 4)[:, [0, 2, 1, 3]].reshape(s.shape)
    if scale_factor is None:
        scale_factor = nvfp4_scale_factor(s, a_dtype)
    if scale_factor > 1.0:
        s = (s.float() * scale_factor).to(torch.float16)
    bits = ((s * 128.0).view(torch.int16) << 1).view(torch.float8_e4m3fn)
    return bits[:, 1::2].contiguous(), scale_factor


def nvfp4_process_global_scale(global_scale: torch.Tensor, a_dtype: torch.dtype) -> torch.Tensor:
    """Boundary form of the nvfp4 global scale: g * 2^(bias - 7) (marlin_utils_fp4.py:132-144)."""
    return global_scale * (2.0 ** (nvfp4_exponent_bias(a_dtype) - 7))


def mxfp4_encode_scales(scales: torch.Tensor) -> torch.Tensor:
    """The reference's Marlin-side form of mxfp4 scales for 16-bit activations: [0,2,1,3] interleave per 4
    along N, stored as e8m0 (marlin_utils_fp4.py:115-129)."""
    s = scales.reshape(-1, 4)[:, [0, 2, 1, 3]].reshape(scales.shape)
    return s.to(torch.float8_e8m0fnu)


def nvfp4_decode_scales(scale_bytes: torch.Tensor) -> torch.Tensor:
    """Boundary bytes -> fp32 value (byte << 7 read as fp16) in logical N order
    (tests/helpers.py:825-828)."""
    b = scale_bytes.view(torch.uint8).to(torch.int16) << 7
    v = b.contiguous().view(torch.float16).to(torch.float32)
    return v.reshape(-1, 4)[:, [0, 2, 1, 3]].reshape(scale_bytes.shape)


def quantize_nvfp4(weight: torch.Tensor):
    """nvfp4: e4m3 scale per 16 along K relative to one fp32 global scale
    (tests/helpers.py:831-854,1006-1065).  Returns (q codes [K,N], boundary scale bytes [K/16,N]
    float8_e4m3fn, boundary global scale fp32[1])."""
    k, n = weight.shape
    r = weight.to(torch.float32).reshape(k // 16, 16, n)
    scales = (r.abs().amax(dim=1) / 6.0).clamp_min(1e-6)
    global_scale = (scales.max() / 448.0).to(torch.float32).reshape(1)
    fp8_scales = (scales / global_scale).to(torch.float8_e4m3fn)
    eff = fp8_scales.to(torch.float32) * global_scale
    q = quantize_e2m1(r / eff.unsqueeze(1).clamp_min(1e-12)).reshape(k, n)
    sbytes, sf = nvfp4_encode_scales(fp8_scales, weight.dtype)
    g = global_scale * (2.0 ** (nvfp4_exponent_bias(weight.dtype) - 7))
    g = (g.to(torch.float32) / sf).contiguous()
    return q, sbytes, g


def quantize_mxfp4(weight: torch.Tensor):
    """mxfp4: e8m0 scale = 2^ceil(log2(amax / 6)) per 32 along K (tests/helpers.py:857-887).
    Returns (q codes [K,N], scales [K/32,N] float8_e8m0fnu in natural N order)."""
    k, n = weight.shape
    r = weight.to(torch.float32).reshape(k // 32, 32, n)
    max_abs = r.abs().amax(dim=1)
    inp = torch.where(max_abs > 0, (max_abs / 6.0).clamp_min(2.0 ** -127), torch.ones_like(max_abs))
    e = torch.ceil(torch.log2(inp)).clamp(-127, 127)
    p2 = torch.pow(torch.full_like(e, 2.0), e)
    s8 = p2.to(torch.float8_e8m0fnu)
    eff = s8.to(torch.float32)
    q = quantize_e2m1(r / eff.unsqueeze(1).clamp_min(1e-12)).reshape(k, n)
    return q, s8


# ---------------------------------------------------------------------------
# dequantisers: boundary tensors -> weight [K, N] rounded to out_dtype
# ---------------------------------------------------------------------------


def _expand(t: torch.Tensor, size_k: int) -> torch.Tensor:
    g = t.shape[0]
    return t.to(torch.float32).repeat_interleave(size_k // g, dim=0)


def dequantize(packed: torch.Tensor, scales: torch.Tensor, size_k: int, size_n: int, type_id: int,
               zeros: torch.Tensor | None = None, global_scale: torch.Tensor | None = None,
               out_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Dequantise what the GEMM op receives.  Follows tests/helpers.py:1094-1184,1576-1641:
    u4b8/u8b128 (q - bias) * s;  u4/u8 q * s - zpf;  fp8 e4m3(q) * s / 2^bias;
    nvfp4 e2m1(q) / 2^bias * decode(s) * global;  mxfp4 e2m1(q) * e8m0(s)."""
    scales = scales.reshape(-1, size_n)
    if type_id in (TYPE_U4B8, TYPE_U8B128):
        bits = 4 if type_id == TYPE_U4B8 else 8
        q = marlin_unpack(packed, size_k, size_n, bits).to(torch.float32)
        w = (q - float(1 << (bits - 1))) * _expand(scales, size_k)
    elif type_id in (TYPE_U4, TYPE_U8):
        bits = 4 if type_id == TYPE_U4 else 8
        q = marlin_unpack(packed, size_k, size_n, bits).to(torch.float32)
        w = q * _expand(scales, size_k) - _expand(zeros.reshape(-1, size_n), size_k)
    elif type_id == TYPE_FE4M3:
        q = marlin_unpack(packed, size_k, size_n, 8).to(torch.uint8).contiguous().view(torch.float8_e4m3fn)
        div = float(2.0 ** fp8_scale_exponent_bias(scales.dtype))
        w = q.to(torch.float32) * (_expand(scales, size_k) / div)
    elif type_id == TYPE_FE2M1:
        q = marlin_unpack(packed, size_k, size_n, 4).to(torch.long)
        table = torch.tensor(E2M1_VALUES, dtype=torch.float32)
        if scales.dtype == torch.float8_e4m3fn:
            div = float(2.0 ** nvfp4_exponent_bias(out_dtype))
            dec = nvfp4_decode_scales(scales)
            w = ((table[q].double() / div) * _expand(dec, size_k).double()
                 * global_scale.reshape(-1)[0].double()).to(torch.float32)
        else:
            w = table[q] * _expand(scales, size_k)
    else:
        raise ValueError(f"unsupported type id {type_id}")
    return w.to(out_dtype)


def dense_reference(a: torch.Tensor, w_deq: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 matmul of the activations with the dequantised weight (tests/helpers.py:1749-1760);
    ``bias`` is in logical order."""
    out = torch.matmul(a.to(torch.float32), w_deq.to(torch.float32))
    if bias is not None:
        out = out + bias.to(torch.float32)
    return out


# ---------------------------------------------------------------------------
# MoE routing / align / reference
# ---------------------------------------------------------------------------


def topk_softmax_reference(gating: torch.Tensor, topk: int, renormalize: bool = False,
                           bias: torch.Tensor | None = None):
    """tests/test_marlin_moe.py:111-133 with the kernel's tie rule (lower index wins,
    csrc/moe/topk_softmax_kernels.cu:486-513) made explicit through a stable sort."""
    probs = torch.softmax(gating.to(torch.float32), dim=-1)
    sel = probs if bias is None else probs + bias.to(torch.float32)
    ids = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :topk]
    w = torch.gather(probs, 1, ids)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True).clamp_min(1e-20)
    t = gating.shape[0]
    tei = (torch.arange(t, dtype=torch.int32).unsqueeze(1)
           + torch.arange(topk, dtype=torch.int32).unsqueeze(0) * t)
    return w, ids.to(torch.int32), tei


def moe_align_block_size_reference(topk_ids: torch.Tensor, block_size: int, num_experts: int,
                                   expert_map: torch.Tensor | None = None):
    """Stable per-expert order, padding value = numel (tests/test_marlin_moe.py:194-213).
    Returns full-length buffers shaped like the op's outputs: sorted_ids
    [numel + E*(block-1)] (tail = numel), expert_ids [ceil(len/block)] (tail = -1), total [1].
    With ``expert_map`` (global -> local id, -1 = dropped) ids are remapped first
    (csrc/moe/moe_align_sum_kernels.cu:129-133)."""
    flat = topk_ids.reshape(-1).to(torch.int64)
    numel = flat.numel()
    if expert_map is not None:
        valid = (flat >= 0) & (flat < expert_map.numel())
        mapped = torch.full_like(flat, -1)
        mapped[valid] = expert_map.to(torch.int64)[flat[valid]]
        flat = mapped
    keep = (flat >= 0) & (flat < num_experts)
    idx = torch.nonzero(keep).reshape(-1)
    order = torch.sort(flat[idx], stable=True).indices
    idx_sorted = idx[order]
    counts = torch.bincount(flat[idx], minlength=num_experts)
    padded = (counts + block_size - 1) // block_size * block_size
    starts = torch.cumsum(padded, 0) - padded
    cstarts = torch.cumsum(counts, 0) - counts
    cap = numel + num_experts * (block_size - 1)
    sorted_ids = torch.full((cap,), numel, dtype=torch.int32)
    e_sorted = flat[idx_sorted]
    pos = starts[e_sorted] + (torch.arange(idx_sorted.numel()) - cstarts[e_sorted])
    sorted_ids[pos] = idx_sorted.to(torch.int32)
    nblocks = (cap + block_size - 1) // block_size
    expert_ids = torch.full((nblocks,), -1, dtype=torch.int32)
    blocks = padded // block_size
    expert_ids[: int(blocks.sum())] = torch.repeat_interleave(
        torch.arange(num_experts, dtype=torch.int32), blocks)
    total = torch.tensor([int(padded.sum())], dtype=torch.int32)
    return sorted_ids, expert_ids, total


def moe_gemm_reference(a: torch.Tensor, w_deq: torch.Tensor, topk_ids: torch.Tensor, top_k: int,
                       topk_weights: torch.Tensor | None = None,
                       bias: torch.Tensor | None = None) -> torch.Tensor:
    """One grouped GEMM stage: row sid = t*top_k + j of the output is a[sid // top_k] @ w_deq[e]
    (+ bias[e]) (* topk_weights[sid]) - the scatter/gather rule of
    csrc/moe/marlin_moe_wna16/sm70_marlin_gemm.cuh:3472-3509.  ``w_deq`` [E, K, N]."""
    flat = topk_ids.reshape(-1).to(torch.long)
    rows = flat.numel()
    n = w_deq.shape[2]
    out = torch.zeros((rows, n), dtype=torch.float32)
    af = a.to(torch.float32)
    for e in torch.unique(flat).tolist():
        sel = torch.nonzero(flat == e).reshape(-1)
        r = af[sel // top_k] @ w_deq[e].to(torch.float32)
        if bias is not None:
            r = r + bias[e].to(torch.float32)
        out[sel] = r
    if topk_weights is not None:
        out = out * topk_weights.reshape(-1, 1).to(torch.float32)
    return out


def moe_reference(hidden: torch.Tensor, w1_deq: torch.Tensor, w2_deq: torch.Tensor,
                  topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                  round_dtype: torch.dtype | None = None) -> torch.Tensor:
    """Whole layer: sum_j w_j * (silu(gate) * up) @ w2[e_j] (tests/helpers.py:2039-2060), looped
    per expert instead of per token.  ``round_dtype`` optionally rounds the two intermediate
    tensors the way the two-GEMM driver stores them."""
    t, h = hidden.shape
    k = topk_ids.shape[1]
    flat = topk_ids.reshape(-1).to(torch.long)
    out = torch.zeros((t, h), dtype=torch.float32)
    hf = hidden.to(torch.float32)
    wts = topk_weights.reshape(-1).to(torch.float32)
    for e in torch.unique(flat).tolist():
        sel = torch.nonzero(flat == e).reshape(-1)
        tok = sel // k
        gu = hf[tok] @ w1_deq[e].to(torch.float32)
        if round_dtype is not None:
            gu = gu.to(round_dtype).to(torch.float32)
        gate, up = gu.chunk(2, dim=-1)
        act = torch.nn.functional.silu(gate) * up
        if round_dtype is not None:
            act = act.to(round_dtype).to(torch.float32)
        r = (act @ w2_deq[e].to(torch.float32)) * wts[sel].unsqueeze(1)
        out.index_add_(0, tok, r)
    return out


# ---------------------------------------------------------------------------
# error metrics (acceptance thresholds)
# ---------------------------------------------------------------------------


def mean_rel_err(y: torch.Tensor, ref: torch.Tensor) -> float:
    """mean|y - ref| / mean|ref| (the measure the upstream Marlin tests use)."""
    y, ref = y.to(torch.float32), ref.to(torch.float32)
    return float((y - ref).abs().mean() / ref.abs().mean().clamp_min(1e-30))


def max_abs_err_frac(y: torch.Tensor, ref: torch.Tensor) -> float:
    """max|y - ref| / max|ref|."""
    y, ref = y.to(torch.float32), ref.to(torch.float32)
    return float((y - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def mean_elem_rel_err(y: torch.Tensor, ref: torch.Tensor, eps: float | None = None) -> float:
    """mean(|y - ref| / max(|ref|, eps)): the per-element form.  eps defaults to mean|ref|, so an element
    smaller than the typical output is measured against the typical output, not against itself."""
    y, ref = y.to(torch.float32), ref.to(torch.float32)
    if eps is None:
        eps = float(ref.abs().mean().clamp_min(1e-30))
    return float(((y - ref).abs() / ref.abs().clamp_min(eps)).mean())


def within_tolerance(y: torch.Tensor, ref: torch.Tensor, mean_tol: float = 1e-2,
                     max_tol: float = 5e-2) -> bool:
    return (math.isfinite(mean_rel_err(y, ref)) and mean_rel_err(y, ref) <= mean_tol
            and max_abs_err_frac(y, ref) <= max_tol)
