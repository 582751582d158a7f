"""Seeded problem builders shared by the tests, the smoke check and the benchmark's CPU legs.
Everything is generated on the CPU (so the oracle and the GPU see identical bits) and moved to the
device by the caller."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from oracle import marlin_oracle as mo

FORMATS = ("u4b8", "u4", "u8b128", "u8", "fp8", "nvfp4", "mxfp4")
TYPE_IDS = {"u4b8": mo.TYPE_U4B8, "u4": mo.TYPE_U4, "u8b128": mo.TYPE_U8B128, "u8": mo.TYPE_U8,
            "fp8": mo.TYPE_FE4M3, "nvfp4": mo.TYPE_FE2M1, "mxfp4": mo.TYPE_FE2M1}


def default_group(fmt: str, group_size: int | None) -> int:
    if fmt == "nvfp4":
        return 16
    if fmt == "mxfp4":
        return 32
    return 128 if group_size is None else group_size


@dataclass
class QuantWeight:
    fmt: str
    size_k: int
    size_n: int
    group_size: int
    type_id: int
    packed: torch.Tensor            # int32 [K/16, N*16/pf]
    scales: torch.Tensor            # boundary scales [G, N]
    zeros: torch.Tensor | None = None
    global_scale: torch.Tensor | None = None
    deq: torch.Tensor | None = None  # oracle-dequantised weight [K, N] in the activation dtype
    extra: dict = field(default_factory=dict)


def quantize(weight: torch.Tensor, fmt: str, group_size: int | None = None, want_deq: bool = True,
             pack: bool = True) -> QuantWeight:
    """Quantise ``weight`` [K, N] (fp16/bf16, CPU) to the tensors the GEMM op receives.  With ``pack=False``
    the codes stay in ``extra["q"]`` and ``packed`` is None (the caller repacks them on the GPU)."""
    k, n = weight.shape
    gs = default_group(fmt, group_size)
    zeros = gscale = None
    if fmt in ("u4b8", "u8b128"):
        bits = 4 if fmt == "u4b8" else 8
        q, scales = mo.quantize_sym(weight, bits, gs)
    elif fmt in ("u4", "u8"):
        bits = 4 if fmt == "u4" else 8
        q, scales, _zp, zeros = mo.quantize_asym(weight, bits, gs)
    elif fmt == "fp8":
        bits = 8
        q, scales, _ = mo.quantize_fp8(weight, gs)
    elif fmt == "nvfp4":
        bits = 4
        q, scales, gscale = mo.quantize_nvfp4(weight)
    elif fmt == "mxfp4":
        bits = 4
        q, scales = mo.quantize_mxfp4(weight)
    else:
        raise ValueError(fmt)
    packed = mo.marlin_pack(q, bits) if pack else None
    qw = QuantWeight(fmt, k, n, gs, TYPE_IDS[fmt], packed, scales.contiguous(), zeros, gscale)
    qw.extra["q"] = q
    qw.extra["bits"] = bits
    if want_deq and pack:
        qw.deq = mo.dequantize(packed, scales, k, n, qw.type_id, zeros=zeros, global_scale=gscale,
                               out_dtype=weight.dtype)
    return qw


def make_dense(m: int, k: int, n: int, fmt: str, dtype: torch.dtype, group_size: int | None = None,
               seed: int = 0, want_deq: bool = True):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).to(dtype)
    w = (torch.randn(k, n, generator=g) * 0.02).to(dtype)
    return a, quantize(w, fmt, group_size, want_deq)


def stack_experts(qws: list[QuantWeight]) -> QuantWeight:
    f = qws[0]
    return QuantWeight(
        f.fmt, f.size_k, f.size_n, f.group_size, f.type_id,
        torch.stack([q.packed for q in qws]).contiguous(),
        torch.stack([q.scales for q in qws]).contiguous(),
        None if f.zeros is None else torch.stack([q.zeros for q in qws]).contiguous(),
        None if f.global_scale is None else torch.cat([q.global_scale for q in qws]).contiguous(),
        None if f.deq is None else torch.stack([q.deq for q in qws]).contiguous())


def make_experts(e: int, k: int, n: int, fmt: str, dtype: torch.dtype, group_size: int | None = None,
                 seed: int = 0, want_deq: bool = True, scale: float = 0.02) -> QuantWeight:
    g = torch.Generator().manual_seed(seed)
    qws = []
    for _ in range(e):
        w = (torch.randn(k, n, generator=g) * scale).to(dtype)
        qws.append(quantize(w, fmt, group_size, want_deq))
    return stack_experts(qws)


def to_dev(qw: QuantWeight, device="cuda") -> QuantWeight:
    mv = lambda t: None if t is None else t.to(device)
    return QuantWeight(qw.fmt, qw.size_k, qw.size_n, qw.group_size, qw.type_id, mv(qw.packed), mv(qw.scales),
                       mv(qw.zeros), mv(qw.global_scale), qw.deq, qw.extra)
