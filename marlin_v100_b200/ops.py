"""Host-side mirror of the reference's operator wrappers for the Marlin path.

Same names, argument order and meaning as ``vllm/_custom_ops.py:1163-1321,2133-2169,2286-2301,
2355-2425`` of the reference; failed argument checks raise ``RuntimeError`` with the reference's
message fragments (``csrc/quantization/marlin/marlin.cu:83-506``,
``csrc/moe/marlin_moe_wna16/ops.cu:102-529``).  Tensor-level checks (device, dtype, contiguity,
shapes) live here; everything that only needs pointers and sizes is checked again inside the C ABI.
Every launch goes to the current CUDA stream of the tensor's device; nothing synchronises."""
from __future__ import annotations

import weakref

import torch

from . import _lib
from .scalar_type import ScalarType, scalar_types

_F16, _BF16 = 0, 1
_SCALE_ACT, _SCALE_E4M3, _SCALE_E8M0 = 0, 1, 2


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _act_code(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return _F16
    if dtype == torch.bfloat16:
        return _BF16
    raise RuntimeError("unsupported `a` scalar_type: float16 or bfloat16 activations expected")


def _type_id(b_q_type) -> int:
    return int(b_q_type.id) if hasattr(b_q_type, "id") else int(b_q_type)


def _resolve_format(b_type_id: int, b_scales: torch.Tensor, act_dtype: torch.dtype) -> int:
    lib = _lib.load()
    if b_type_id == scalar_types.float4_e2m1f.id:
        if b_scales.dtype == torch.float8_e4m3fn:
            kind = _SCALE_E4M3
        elif b_scales.dtype == torch.float8_e8m0fnu:
            kind = _SCALE_E8M0
        else:
            raise RuntimeError("When b_type = float4_e2m1f, b_scales must be float8_e4m3fn for NVFP4 "
                               "or float8_e8m0fnu for MXFP4 scales.")
    else:
        kind = _SCALE_ACT
        _check(b_scales.dtype == act_dtype,
               "Marlin expects scales of the activation dtype, except FP4 uses float8_e4m3fn scales "
               "for NVFP4 or float8_e8m0fnu scales for MXFP4.")
    fmt = lib.marlin_b200_format_from_type_id(b_type_id, kind)
    _check(fmt >= 0, "Marlin currently implements only uint4, uint4b8, uint8, uint8b128, fp8_e4m3fn, "
                     "nvfp4, and mxfp4 dense weights.")
    return fmt


# --------------------------------------------------------------------------------------------
# repack
# --------------------------------------------------------------------------------------------

def gptq_marlin_repack(b_q_weight: torch.Tensor, perm: torch.Tensor, size_k: int, size_n: int,
                       num_bits: int, is_a_8bit: bool = False) -> torch.Tensor:
    lib = _lib.load()
    _check(not is_a_8bit, "is_a_8bit=True (8-bit activation layout) is not supported")
    _check(num_bits in (4, 8), f"num_bits must be 4 or 8. Got = {num_bits}")
    pf = 32 // num_bits
    _check(b_q_weight.is_cuda, "b_q_weight is not on GPU")
    _check(b_q_weight.is_contiguous(), "b_q_weight is not contiguous")
    _check(b_q_weight.dtype == torch.int32, "b_q_weight type is not kInt")
    _check(size_k % 16 == 0, f"size_k = {size_k} is not divisible by tile_k_size = 16")
    _check(size_n % 64 == 0, f"size_n = {size_n} is not divisible by tile_n_size = 64")
    _check(b_q_weight.dim() == 2 and b_q_weight.size(0) == size_k // pf and b_q_weight.size(1) == size_n,
           f"Shape mismatch: b_q_weight = {tuple(b_q_weight.shape)}, size_k = {size_k}, "
           f"size_n = {size_n}, pack_factor = {pf}")
    has_perm = perm is not None and perm.numel() > 0
    if has_perm:
        _check(perm.is_cuda, "perm is not on GPU")
        _check(perm.is_contiguous(), "perm is not contiguous")
        _check(perm.dtype == torch.int32, "perm type is not at::kInt")
        _check(perm.numel() == size_k, f"perm.numel() = {perm.numel()} is not size_k = {size_k}")
    with torch.cuda.device(b_q_weight.device):
        out = torch.empty((size_k // 16, size_n * 16 // pf), dtype=torch.int32, device=b_q_weight.device)
        _lib.check(lib.marlin_b200_gptq_repack(_ptr(b_q_weight), _ptr(perm) if has_perm else None,
                                               _ptr(out), size_k, size_n, num_bits,
                                               _stream(b_q_weight.device)))
    return out


def awq_marlin_repack(b_q_weight: torch.Tensor, size_k: int, size_n: int, num_bits: int,
                      is_a_8bit: bool = False) -> torch.Tensor:
    lib = _lib.load()
    _check(not is_a_8bit, "is_a_8bit=True (8-bit activation layout) is not supported")
    _check(num_bits in (4, 8), f"num_bits must be 4 or 8. Got = {num_bits}")
    pf = 32 // num_bits
    _check(b_q_weight.is_cuda, "b_q_weight is not on GPU")
    _check(b_q_weight.is_contiguous(), "b_q_weight is not contiguous")
    _check(b_q_weight.dtype == torch.int32, "b_q_weight type is not kInt")
    _check(size_k % 16 == 0, f"size_k = {size_k} is not divisible by tile_k_size = 16")
    _check(size_n % 64 == 0, f"size_n = {size_n} is not divisible by tile_n_size = 64")
    _check(b_q_weight.dim() == 2 and b_q_weight.size(0) == size_k and b_q_weight.size(1) == size_n // pf,
           f"Shape mismatch: b_q_weight = {tuple(b_q_weight.shape)}, size_k = {size_k}, "
           f"size_n = {size_n}, pack_factor = {pf}")
    with torch.cuda.device(b_q_weight.device):
        out = torch.empty((size_k // 16, size_n * 16 // pf), dtype=torch.int32, device=b_q_weight.device)
        _lib.check(lib.marlin_b200_awq_repack(_ptr(b_q_weight), _ptr(out), size_k, size_n, num_bits,
                                              _stream(b_q_weight.device)))
    return out


def _moe_repack_checks(b_q_weight: torch.Tensor, size_k: int, size_n: int, num_bits: int, is_a_8bit: bool) -> int:
    _check(not is_a_8bit, "is_a_8bit=True (8-bit activation layout) is not supported")
    _check(num_bits in (4, 8), f"num_bits must be 4 or 8. Got = {num_bits}")
    _check(b_q_weight.is_cuda and b_q_weight.is_contiguous() and b_q_weight.dtype == torch.int32,
           "b_q_weight must be a contiguous int32 GPU tensor")
    _check(b_q_weight.dim() == 3, "b_q_weight must be [num_experts, ...]")
    _check(size_k % 16 == 0, f"size_k = {size_k} is not divisible by tile_k_size = 16")
    _check(size_n % 64 == 0, f"size_n = {size_n} is not divisible by tile_n_size = 64")
    return b_q_weight.shape[0]


def gptq_marlin_moe_repack(b_q_weight: torch.Tensor, perm: torch.Tensor | None, size_k: int, size_n: int,
                           num_bits: int, is_a_8bit: bool = False) -> torch.Tensor:
    """All experts of a layer in one launch (the reference loops over the experts in Python:
    vllm/_custom_ops.py:1228-1247).  b_q_weight [E, K / pack_factor, N], perm [E, K] (or empty)."""
    lib = _lib.load()
    e = _moe_repack_checks(b_q_weight, size_k, size_n, num_bits, is_a_8bit)
    pf = 32 // num_bits
    _check(tuple(b_q_weight.shape[1:]) == (size_k // pf, size_n),
           f"Shape mismatch: b_q_weight = {tuple(b_q_weight.shape)}, size_k = {size_k}, size_n = {size_n}, "
           f"pack_factor = {pf}")
    has_perm = perm is not None and perm.numel() > 0
    if has_perm:
        _check(perm.is_cuda and perm.is_contiguous() and perm.dtype == torch.int32,
               "perm must be a contiguous int32 GPU tensor")
        _check(perm.numel() == e * size_k, f"perm.numel() = {perm.numel()} is not num_experts * size_k")
    with torch.cuda.device(b_q_weight.device):
        out = torch.empty((e, size_k // 16, size_n * 16 // pf), dtype=torch.int32, device=b_q_weight.device)
        _lib.check(lib.marlin_b200_gptq_moe_repack(_ptr(b_q_weight), _ptr(perm) if has_perm else None, _ptr(out),
                                                   e, size_k, size_n, num_bits, _stream(b_q_weight.device)))
    return out


def awq_marlin_moe_repack(b_q_weight: torch.Tensor, perm: torch.Tensor | None, size_k: int, size_n: int,
                          num_bits: int, is_a_8bit: bool = False) -> torch.Tensor:
    """All experts of a layer in one launch (vllm/_custom_ops.py:1250-1269; `perm` is unused there too).
    b_q_weight [E, K, N / pack_factor]."""
    lib = _lib.load()
    e = _moe_repack_checks(b_q_weight, size_k, size_n, num_bits, is_a_8bit)
    pf = 32 // num_bits
    _check(tuple(b_q_weight.shape[1:]) == (size_k, size_n // pf),
           f"Shape mismatch: b_q_weight = {tuple(b_q_weight.shape)}, size_k = {size_k}, size_n = {size_n}, "
           f"pack_factor = {pf}")
    with torch.cuda.device(b_q_weight.device):
        out = torch.empty((e, size_k // 16, size_n * 16 // pf), dtype=torch.int32, device=b_q_weight.device)
        _lib.check(lib.marlin_b200_awq_moe_repack(_ptr(b_q_weight), _ptr(out), e, size_k, size_n, num_bits,
                                                  _stream(b_q_weight.device)))
    return out


# --------------------------------------------------------------------------------------------
# scale re-encoders of fp4 / fp8 checkpoints (eager PyTorch in the reference's loaders)
# --------------------------------------------------------------------------------------------

def nvfp4_marlin_process_scales(marlin_scales: torch.Tensor, scale_factor: float | None = None,
                                a_dtype: torch.dtype | None = None) -> tuple[torch.Tensor, float]:
    """nvfp4 block scales [G, N] -> (the S0E5M3 bytes `marlin_gemm` reads, as float8_e4m3fn; scale_factor).
    Mirrors nvfp4_marlin_process_scales (marlin_utils_fp4.py:53-112): [0,2,1,3] interleave per four columns,
    optional power-of-two rescale so that every non-zero scale * 2^7 >= 2 (computed here when `scale_factor`
    is None and the activations are not fp16; the caller divides the global scale by it)."""
    import math
    lib = _lib.load()
    _check(marlin_scales.is_cuda and marlin_scales.dim() == 2, "marlin_scales must be a 2-D GPU tensor")
    _check(marlin_scales.size(1) % 4 == 0, "scale columns must be a multiple of 4")
    half = marlin_scales.to(torch.float16).contiguous()
    dev = half.device
    with torch.cuda.device(dev):
        if scale_factor is None:
            scale_factor = 1.0
            if not (a_dtype is not None and a_dtype == torch.float16):
                mn = torch.empty(1, dtype=torch.float32, device=dev)
                _lib.check(lib.marlin_b200_nvfp4_scale_min(_ptr(half), half.numel(), _ptr(mn), _stream(dev)))
                mn = float(mn.item())
                if math.isfinite(mn) and mn < 2:
                    scale_factor = float(2.0 ** math.ceil(math.log2(2.0 / mn)))
        out = torch.empty(half.shape, dtype=torch.uint8, device=dev)
        _lib.check(lib.marlin_b200_nvfp4_process_scales(_ptr(half), _ptr(out), half.size(0), half.size(1),
                                                        float(scale_factor), _stream(dev)))
    return out.view(torch.float8_e4m3fn), float(scale_factor)


def nvfp4_marlin_process_global_scale(global_scale: torch.Tensor, a_dtype: torch.dtype | None = None) -> torch.Tensor:
    """global_scale * 2^(bias - 7), bias = 14 (fp16) / 126 (bf16) (marlin_utils_fp4.py:132-144); a scalar."""
    a_dtype = global_scale.dtype if a_dtype is None else a_dtype
    _check(a_dtype in (torch.float16, torch.bfloat16), "activations must be fp16 or bf16")
    return global_scale * (2.0 ** ((14 if a_dtype == torch.float16 else 126) - 7))


def mxfp4_marlin_process_scales(marlin_scales: torch.Tensor, input_dtype: torch.dtype | None = None) -> torch.Tensor:
    """The reference's Marlin-side form of mxfp4 scales for 16-bit activations: [0,2,1,3] interleave per four
    columns, as float8_e8m0fnu (marlin_utils_fp4.py:115-129).  `marlin_gemm` of this library takes mxfp4
    scales in natural column order; this is for callers that hold or exchange the reference's form."""
    lib = _lib.load()
    _check(input_dtype is None or input_dtype.itemsize == 2, "only 16-bit activations are supported")
    _check(marlin_scales.is_cuda and marlin_scales.dim() == 2 and marlin_scales.size(1) % 4 == 0,
           "marlin_scales must be a 2-D GPU tensor with a multiple of 4 columns")
    e8 = marlin_scales if marlin_scales.dtype == torch.float8_e8m0fnu else marlin_scales.to(torch.float8_e8m0fnu)
    e8 = e8.contiguous().view(torch.uint8)
    out = torch.empty_like(e8)
    with torch.cuda.device(e8.device):
        _lib.check(lib.marlin_b200_interleave_scale_bytes(_ptr(e8), _ptr(out), e8.size(0), e8.size(1),
                                                          _stream(e8.device)))
    return out.view(torch.float8_e8m0fnu)


def fp8_fused_exponent_bias_into_scales(scales: torch.Tensor) -> torch.Tensor:
    """scales * 2^8 (fp16) / 2^120 (bf16) in the scales' own dtype (marlin_utils_fp8.py:28-39)."""
    lib = _lib.load()
    _check(scales.is_cuda and scales.dtype in (torch.float16, torch.bfloat16), "scales must be fp16 / bf16 on the GPU")
    src = scales.contiguous()
    out = torch.empty_like(src)
    with torch.cuda.device(src.device):
        _lib.check(lib.marlin_b200_fp8_fuse_exponent_bias(_ptr(src), _ptr(out), src.numel(), _act_code(src.dtype),
                                                          _stream(src.device)))
    return out


def gptq_marlin_moe_repack(b_q_weight: torch.Tensor, perm: torch.Tensor, size_k: int, size_n: int,
                           num_bits: int, is_a_8bit: bool = False) -> torch.Tensor:
    """Per-expert repack of ``[E, K/pf, N]`` (reference: vllm/_custom_ops.py:1228-1249)."""
    e = b_q_weight.shape[0]
    out = torch.empty((e, size_k // 16, size_n * (num_bits // 2)), dtype=b_q_weight.dtype,
                      device=b_q_weight.device)
    for i in range(e):
        out[i] = gptq_marlin_repack(b_q_weight[i], perm[i] if perm is not None and perm.numel() else perm,
                                    size_k, size_n, num_bits, is_a_8bit)
    return out


def awq_marlin_moe_repack(b_q_weight: torch.Tensor, perm: torch.Tensor | None, size_k: int, size_n: int,
                          num_bits: int, is_a_8bit: bool = False) -> torch.Tensor:
    """Per-expert repack of ``[E, K, N/pf]`` (reference: vllm/_custom_ops.py:1252-1269)."""
    e = b_q_weight.shape[0]
    out = torch.empty((e, size_k // 16, size_n * (num_bits // 2)), dtype=b_q_weight.dtype,
                      device=b_q_weight.device)
    for i in range(e):
        out[i] = awq_marlin_repack(b_q_weight[i], size_k, size_n, num_bits, is_a_8bit)
    return out


# --------------------------------------------------------------------------------------------
# streaming layout (opt-in; no counterpart in the reference)
# --------------------------------------------------------------------------------------------

# data_ptr -> (size_k, size_n, num_bits) of every live tensor made by `prepare_weights`; an entry is
# dropped when its tensor is freed, so a later allocation at the same address is not mistaken for one.
_PREPARED: dict[int, tuple[int, int, int]] = {}


def _convert_layout(fn_name: str, w: torch.Tensor, size_k: int, size_n: int, num_bits: int) -> torch.Tensor:
    lib = _lib.load()
    _check(w.is_cuda and w.is_contiguous() and w.dtype == torch.int32,
           "packed weights must be a contiguous int32 CUDA tensor")
    _check(w.dim() in (2, 3), "packed weights must be [K/16, N*16/pf] or [E, K/16, N*16/pf]")
    pf = 32 // num_bits
    _check(w.size(-2) == size_k // 16 and w.size(-1) == size_n * 16 // pf,
           f"Shape mismatch: b_q_weight = {tuple(w.shape)}, size_k = {size_k}, size_n = {size_n}")
    experts = w.size(0) if w.dim() == 3 else 1
    with torch.cuda.device(w.device):
        out = torch.empty_like(w)
        _lib.check(getattr(lib, fn_name)(_ptr(w), _ptr(out), size_k, size_n, num_bits, experts, _stream(w.device)))
    return out


def prepare_weights(b_q_weight: torch.Tensor, size_k: int, size_n: int, num_bits: int) -> torch.Tensor:
    """Returns the same codes in the library's streaming layout (every 256-column x 64-k block contiguous,
    codes where the GEMM threads consume them).  Call once after `gptq_marlin_repack` / `awq_marlin_repack`
    and pass the result to `marlin_gemm` in place of the repacked tensor: it is recognised by its address.
    Needs size_k % 128 == 0 and size_n % 256 == 0."""
    out = _convert_layout("marlin_b200_prepare_weights", b_q_weight, size_k, size_n, num_bits)
    ptr = out.data_ptr()
    _PREPARED[ptr] = (size_k, size_n, num_bits)
    weakref.finalize(out, _PREPARED.pop, ptr, None)
    return out


def restore_weights(prepared: torch.Tensor, size_k: int, size_n: int, num_bits: int) -> torch.Tensor:
    """Inverse of `prepare_weights`: the reference layout again, bit for bit."""
    return _convert_layout("marlin_b200_restore_weights", prepared, size_k, size_n, num_bits)


def is_prepared(b_q_weight: torch.Tensor, size_k: int, size_n: int) -> bool:
    entry = _PREPARED.get(b_q_weight.data_ptr())
    return entry is not None and entry[0] == size_k and entry[1] == size_n


# --------------------------------------------------------------------------------------------
# dense GEMM
# --------------------------------------------------------------------------------------------

def _check_act_order_absent(g_idx, perm) -> None:
    if g_idx is not None:
        _check(g_idx.numel() == 0, "Marlin does not support act_order g_idx.")
    if perm is not None:
        _check(perm.numel() == 0, "Marlin does not support act_order perm.")


def _scratch(nbytes: int, device: torch.device) -> torch.Tensor | None:
    if nbytes <= 0:
        return None
    return torch.empty((nbytes,), dtype=torch.uint8, device=device)


def marlin_gemm(a: torch.Tensor, c: torch.Tensor | None, b_q_weight: torch.Tensor,
                b_bias: torch.Tensor | None, b_scales: torch.Tensor, a_scales: torch.Tensor | None,
                global_scale: torch.Tensor | None, b_zeros: torch.Tensor | None,
                g_idx: torch.Tensor | None, perm: torch.Tensor | None, workspace: torch.Tensor,
                b_q_type: ScalarType | int, size_m: int, size_n: int, size_k: int,
                is_k_full: bool = True, use_atomic_add: bool = False, use_fp32_reduce: bool = False,
                is_zp_float: bool = False) -> torch.Tensor:
    """C[size_m, size_n] = a @ dequant(b_q_weight).  ``workspace``, ``is_k_full``, ``use_atomic_add``
    and ``use_fp32_reduce`` are accepted and ignored, as in the reference (marlin.cu:103-106); the
    split-K scratch is allocated here from torch's caching allocator and the caller's workspace is
    never touched."""
    c, call = _gemm_prepare(a, c, b_q_weight, b_bias, b_scales, a_scales, global_scale, b_zeros, g_idx, perm,
                            b_q_type, size_m, size_n, size_k, is_zp_float)
    if call is not None:
        with torch.cuda.device(a.device):
            call(None)
    return c


class PreparedGemm:
    """`marlin_gemm` with its arguments checked and converted once.  Calling the object only enqueues
    the kernels on the current stream of the tensors' device (which must be the current device), for
    loops that run the same layer on the same buffers every step: there the argument checks of
    `marlin_gemm` cost more host time than a decode-sized GEMM takes on the GPU.  The output tensor is
    `.c`; the buffers passed in (and the scratch taken here) must stay alive and in place."""

    def __init__(self, a, c, b_q_weight, b_bias, b_scales, global_scale, b_zeros, b_q_type, size_m, size_n,
                 size_k, is_zp_float=False):
        self.c, self._call = _gemm_prepare(a, c, b_q_weight, b_bias, b_scales, None, global_scale, b_zeros, None,
                                           None, b_q_type, size_m, size_n, size_k, is_zp_float)
        self._keep = (a, b_q_weight, b_bias, b_scales, global_scale, b_zeros)

    def __call__(self, stream: int | None = None) -> torch.Tensor:
        """Enqueues the GEMM on the current stream, or on `stream` (a raw cudaStream_t handle)."""
        if self._call is not None:
            self._call(stream)
        return self.c


class HostPipelinedGemm:
    """Dense GEMM for callers whose activations and results live in pinned host memory (a serving loop
    that receives rows from the host and returns rows to it).  `submit` enqueues copy-in, GEMM and
    copy-out of one call on three streams over `depth` staging slots, so the copies of one call overlap
    the GEMM of its neighbours; nothing synchronises with the host until `synchronize()`.

    `layers` is a list of weight sets, each a dict with `packed`, `scales` and optionally `zeros`,
    `global_scale`, `bias`; `submit(..., layer=i)` picks one.

    `post(c_slot, out_slot)` with `post_shape`: a step that runs behind every GEMM on the compute stream and whose
    output (a per-slot tensor of `post_shape`) is what gets copied to the host instead of the GEMM's own output,
    e.g. the all-gather of a column-parallel layer."""

    def __init__(self, layers, b_q_type, size_m: int, size_n: int, size_k: int, dtype: torch.dtype,
                 device: torch.device, depth: int = 3, post=None, post_shape=None):
        self.depth, self._count = depth, 0
        self.device = device
        self._post = post
        with torch.cuda.device(device):
            self._in, self._run, self._out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
            self._a = [torch.empty((size_m, size_k), dtype=dtype, device=device) for _ in range(depth)]
            self._c = [torch.empty((size_m, size_n), dtype=dtype, device=device) for _ in range(depth)]
            self._g = ([torch.empty(tuple(post_shape), dtype=dtype, device=device) for _ in range(depth)]
                       if post is not None else self._c)
            self._plans = [[PreparedGemm(self._a[s], self._c[s], w["packed"], w.get("bias"), w["scales"],
                                         w.get("global_scale"), w.get("zeros"), b_q_type, size_m, size_n, size_k,
                                         w.get("zeros") is not None) for w in layers] for s in range(depth)]
            self._in_done = [torch.cuda.Event() for _ in range(depth)]
            self._run_done = [torch.cuda.Event() for _ in range(depth)]
            self._out_done = [torch.cuda.Event() for _ in range(depth)]
            start = torch.cuda.Event()
            start.record()           # the staging buffers were created on the current stream
            for st in (self._in, self._run, self._out):
                st.wait_event(start)

    def submit(self, a_host: torch.Tensor, c_host: torch.Tensor, layer: int = 0) -> None:
        """a_host [size_m, size_k] and c_host [size_m, size_n] in pinned host memory; c_host is valid
        after `synchronize()` (or once the event returned by `last_event()` has completed)."""
        s = self._count % self.depth
        reused = self._count >= self.depth
        self._count += 1
        if reused:
            self._in.wait_event(self._run_done[s])   # the GEMM that read this slot's activations is done
        with torch.cuda.stream(self._in):
            self._a[s].copy_(a_host, non_blocking=True)
        self._in_done[s].record(self._in)
        self._run.wait_event(self._in_done[s])
        if reused:
            self._run.wait_event(self._out_done[s])  # this slot's previous result has left the device
        self._plans[s][layer](self._run.cuda_stream)
        if self._post is not None:
            with torch.cuda.stream(self._run):
                self._post(self._c[s], self._g[s])
        self._run_done[s].record(self._run)
        self._out.wait_event(self._run_done[s])
        with torch.cuda.stream(self._out):
            c_host.copy_(self._g[s], non_blocking=True)
        self._out_done[s].record(self._out)

    def capture(self, a_host: torch.Tensor, c_host: torch.Tensor, layers: list[int]) -> torch.cuda.CUDAGraph:
        """A CUDA graph of `len(layers)` pipelined calls on fixed pinned buffers: every call still copies its
        activations in and its result out, but a replay costs the host one launch instead of some fifteen stream
        operations per call (which is what bounds `submit` from Python at decode sizes).  Replay with
        `graph.replay()`; nothing submitted earlier may still be in flight."""
        torch.cuda.synchronize(self.device)
        self._count = 0
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.device(self.device):
            cap = torch.cuda.Stream()
            with torch.cuda.graph(graph, stream=cap):
                for st in (self._in, self._run, self._out):
                    st.wait_stream(cap)
                for layer in layers:
                    self.submit(a_host, c_host, layer)
                for st in (self._in, self._run, self._out):
                    cap.wait_stream(st)
        self._count = 0
        return graph

    def join(self) -> None:
        """Makes the current stream wait for everything submitted so far (no host synchronisation)."""
        cur = torch.cuda.current_stream(self.device)
        for s in range(min(self._count, self.depth)):
            cur.wait_event(self._out_done[s])

    def synchronize(self) -> None:
        self._out.synchronize()


def _gemm_prepare(a, c, b_q_weight, b_bias, b_scales, a_scales, global_scale, b_zeros, g_idx, perm, b_q_type,
                  size_m, size_n, size_k, is_zp_float):
    """Validation, output / scratch allocation and argument conversion of the dense GEMM.  Returns the
    output tensor and a closure that enqueues the work (None when size_m == 0)."""
    lib = _lib.load()
    _check_act_order_absent(g_idx, perm)
    _check(a_scales is None, "a_scales can only be used for 8bit activation.")
    act = _act_code(a.dtype)
    b_type_id = _type_id(b_q_type)
    fmt = _resolve_format(b_type_id, b_scales, a.dtype)
    pf = 8 if fmt in (0, 1, 5, 6) else 4

    _check(a.dim() == 2, "a must be 2-D")
    _check(a.size(0) == size_m, f"Shape mismatch: a.size(0) = {a.size(0)}, size_m = {size_m}")
    _check(a.size(1) == size_k, f"Shape mismatch: a.size(1) = {a.size(1)}, size_k = {size_k}")
    _check(size_k % 16 == 0, f"size_k = {size_k} is not divisible by tile_size = 16")
    _check(b_q_weight.dim() == 2 and size_k // 16 == b_q_weight.size(0),
           f"Shape mismatch: b_q_weight.size(0) = {b_q_weight.size(0)}, size_k = {size_k}, tile_size = 16")
    _check(b_q_weight.size(1) % 16 == 0,
           f"b_q_weight.size(1) = {b_q_weight.size(1)} is not divisible by tile_size = 16")
    actual_n = (b_q_weight.size(1) // 16) * pf
    _check(size_n == actual_n, f"size_n = {size_n}, actual_size_n = {actual_n}")
    _check(a.is_cuda, "A is not on GPU")
    _check(a.stride(1) == 1, "A.stride(1) is not 1")
    _check(a.stride(0) % 8 == 0, "A.stride(0) must divisible by 8")
    _check(a.data_ptr() % 16 == 0, "A must aligned to 16 bytes")
    _check(b_q_weight.is_cuda, "b_q_weight is not on GPU")
    _check(b_q_weight.is_contiguous(), "b_q_weight is not contiguous")
    _check(b_q_weight.dtype == torch.int32, "Marlin expects int32 packed weights.")
    _check(b_scales.is_cuda, "b_scales is not on GPU")
    _check(b_scales.is_contiguous(), "b_scales is not contiguous")

    with torch.cuda.device(a.device):
        if c is not None:
            _check(c.is_cuda, "c is not on GPU")
            _check(c.is_contiguous(), "c is not contiguous")
            _check(c.dtype == a.dtype, "scalar type of a must be the same with c for 16 bit activation")
            _check(c.size(0) == size_m, f"Shape mismatch: c.size(0) = {c.size(0)}, size_m = {size_m}")
            _check(c.size(1) == size_n, f"Shape mismatch: c.size(1) = {c.size(1)}, size_n = {size_n}")
        else:
            c = torch.empty((size_m, size_n), dtype=a.dtype, device=a.device)
        if size_m == 0:
            return c, None

        _check(b_scales.dim() == 2, f"b_scales rank = {b_scales.dim()} is not 2")
        _check(b_scales.size(1) == size_n, f"b_scales dim 1 = {b_scales.size(1)} is not size_n = {size_n}")
        num_groups = b_scales.size(0)
        if num_groups > 1:
            _check(size_k % num_groups == 0,
                   f"size_k = {size_k}, is not divisible by b_scales.size(0) = {num_groups}")

        if global_scale is not None:
            _check(fmt == 5, "Marlin supports global_scale only for nvfp4 format.")
            _check(global_scale.is_cuda, "global_scale is not on GPU")
            _check(global_scale.is_contiguous(), "global_scale is not contiguous")
            _check(global_scale.dtype == torch.float32, "Marlin nvfp4 expects fp32 global_scale.")
            _check(global_scale.numel() == 1, "Marlin nvfp4 expects a single global_scale value.")
        else:
            _check(fmt != 5, "the global_scale parameter must be passed for nvfp4 format.")

        if b_bias is not None:
            _check(b_bias.is_cuda, "b_bias is not on GPU")
            _check(b_bias.is_contiguous(), "b_bias is not contiguous")
            _check(b_bias.dtype == a.dtype, "Marlin bias must have the activation dtype.")
            _check(b_bias.size(0) == size_n, "b_bias.size(0) != size_n")

        has_zp = b_zeros is not None and b_zeros.size(-1) > 0
        _check(not has_zp or fmt in (1, 3),
               "Marlin does not support zero-point metadata for this quant type.")
        if has_zp:
            _check(b_zeros.is_cuda, "b_zeros is not on GPU")
            _check(b_zeros.is_contiguous(), "b_zeros is not contiguous")
            _check(is_zp_float, "Marlin received b_zeros but is_zp_float is false. Packed integer "
                                "zero-points are not supported on the dense uint4/uint8 path.")
            _check(b_zeros.dim() == 2, f"b_zeros rank = {b_zeros.dim()} is not 2")
            _check(b_zeros.dtype == a.dtype, "Marlin uint4/uint8 dense path expects zero points of the "
                                             "activation dtype.")
            _check(b_zeros.size(1) == size_n, f"b_zeros dim 1 = {b_zeros.size(1)} is not size_n = {size_n}")
            _check(b_zeros.size(0) == num_groups,
                   f"b_zeros dim 0 = {b_zeros.size(0)} is not num_groups = {num_groups}")
        else:
            _check(not is_zp_float, "is_zp_float is true but b_zeros was not provided.")
            _check(fmt not in (1, 3), "Marlin uint4/uint8 dense path requires float zero points.")

        fmt_arg = fmt | (_lib.FMT_PREPARED if is_prepared(b_q_weight, size_k, size_n) else 0)
        nbytes = lib.marlin_b200_gemm_scratch_bytes(size_m, size_n, size_k, fmt_arg)
        scratch = _scratch(nbytes, a.device)
        args = (_ptr(a), _ptr(c), _ptr(b_q_weight), _ptr(b_scales), _ptr(b_zeros) if has_zp else None,
                _ptr(b_bias), _ptr(global_scale), act, fmt_arg, size_m, size_n, size_k, a.stride(0), num_groups,
                _ptr(scratch), nbytes)
        device, fn = a.device, lib.marlin_b200_gemm

        def call(stream=None, _scratch_ref=scratch):
            _lib.check(fn(*args, _stream(device) if stream is None else stream))

    return c, call


# --------------------------------------------------------------------------------------------
# MoE
# --------------------------------------------------------------------------------------------

def moe_wna16_marlin_gemm(input: torch.Tensor, output: torch.Tensor | None, b_qweight: torch.Tensor,
                          b_bias: torch.Tensor | None, b_scales: torch.Tensor,
                          a_scales: torch.Tensor | None, global_scale: torch.Tensor | None,
                          b_qzeros: torch.Tensor | None, g_idx: torch.Tensor | None,
                          perm: torch.Tensor | None, workspace: torch.Tensor,
                          sorted_token_ids: torch.Tensor, expert_ids: torch.Tensor,
                          num_tokens_past_padded: torch.Tensor, topk_weights: torch.Tensor,
                          moe_block_size: int, top_k: int, mul_topk_weights: bool,
                          b_q_type: ScalarType | int, size_m: int, size_n: int, size_k: int,
                          is_k_full: bool = True, use_atomic_add: bool = False,
                          use_fp32_reduce: bool = False, is_zp_float: bool = False, thread_k: int = -1,
                          thread_n: int = -1, blocks_per_sm: int = -1, silu_input: bool = False) -> torch.Tensor:
    """Grouped expert GEMM; rows follow ``sorted_token_ids`` (flat route ids ``t * top_k + j``).
    Ignored arguments as in the reference (ops.cu:126-132).  `silu_input` (no counterpart there; expert weights in
    the streaming layout only): `input` is the [size_m, 2 * size_k] gate | up output of the layer's first GEMM and
    silu(gate) * up is what gets multiplied, without a separate SiLU-and-mul pass."""
    lib = _lib.load()
    _check_act_order_absent(g_idx, perm)
    _check(a_scales is None, "a_scales can only be used for 8bit activation.")
    a = input
    act = _act_code(a.dtype)
    b_type_id = _type_id(b_q_type)
    fmt = _resolve_format(b_type_id, b_scales, a.dtype)
    pf = 8 if fmt in (0, 1, 5, 6) else 4
    if moe_block_size != 8:
        _check(moe_block_size % 16 == 0 and 16 <= moe_block_size <= 64,
               f"unsupported moe_block_size={moe_block_size}")
    _check(a.size(0) == size_m, f"Shape mismatch: a.size(0) = {a.size(0)}, size_m = {size_m}")
    _check(a.size(1) == (2 * size_k if silu_input else size_k),
           f"Shape mismatch: a.size(1) = {a.size(1)}, size_k = {size_k}")
    _check(size_k % 16 == 0, f"size_k = {size_k} is not divisible by tile_size = 16")
    _check(b_qweight.dim() == 3, "b_q_weight must be [experts, size_k / 16, size_n * 16 / pack_factor]")
    num_experts = b_qweight.size(0)
    _check(size_k // 16 == b_qweight.size(1),
           f"Shape mismatch: b_q_weight.size(1) = {b_qweight.size(1)}, size_k = {size_k}, tile_size = 16")
    _check(b_qweight.size(2) % 16 == 0,
           f"b_q_weight.size(2) = {b_qweight.size(2)} is not divisible by tile_size = 16")
    actual_n = (b_qweight.size(2) // 16) * pf
    _check(size_n == actual_n, f"size_n = {size_n}, actual_size_n = {actual_n}")
    _check(a.is_cuda, "A is not on GPU")
    _check(a.is_contiguous(), "A is not contiguous")
    _check(b_qweight.is_cuda, "b_q_weight is not on GPU")
    _check(b_qweight.is_contiguous(), "b_q_weight is not contiguous")
    _check(b_qweight.dtype == torch.int32, "Marlin expects int32 packed weights.")
    _check(b_scales.is_cuda, "b_scales is not on GPU")
    _check(b_scales.is_contiguous(), "b_scales is not contiguous")

    with torch.cuda.device(a.device):
        if output is not None:
            c = output
            _check(c.is_cuda, "c is not on GPU")
            _check(c.is_contiguous(), "c is not contiguous")
            _check(c.dtype == a.dtype, "scalar type of a must be the same with c for 16 bit activation")
            _check(c.size(0) == size_m * top_k,
                   f"Shape mismatch: c.size(0) = {c.size(0)}, size_m * topk = {size_m * top_k}")
            _check(c.size(1) == size_n, f"Shape mismatch: c.size(1) = {c.size(1)}, size_n = {size_n}")
        else:
            c = torch.empty((size_m * top_k, size_n), dtype=a.dtype, device=a.device)

        _check(b_scales.dim() == 3, f"b_scales rank = {b_scales.dim()} is not 3")
        _check(b_scales.size(0) == num_experts, "b_scales dim 0 is not the number of experts")
        _check(b_scales.size(2) == size_n, f"b_scales dim 2 = {b_scales.size(2)} is not size_n = {size_n}")
        num_groups = b_scales.size(1)
        if num_groups > 1:
            _check(size_k % num_groups == 0,
                   f"size_k = {size_k}, is not divisible by b_scales.size(1) = {num_groups}")

        if global_scale is not None:
            _check(fmt == 5, "Marlin MoE supports global_scale only for nvfp4 format.")
            _check(global_scale.is_cuda and global_scale.is_contiguous(), "global_scale is not on GPU")
            _check(global_scale.dtype == torch.float32, "Marlin MoE nvfp4 expects fp32 global_scale.")
            _check(global_scale.numel() == num_experts,
                   "Marlin MoE nvfp4 expects global_scale numel = num_experts. Got global_scale.numel() = "
                   f"{global_scale.numel()}, num_experts = {num_experts}")
        else:
            _check(fmt != 5, "the global_scale parameter must be passed for nvfp4 format.")

        if b_bias is not None:
            _check(b_bias.is_cuda and b_bias.is_contiguous(), "b_bias is not on GPU")
            _check(b_bias.dtype == a.dtype, "Marlin bias must have the activation dtype.")
            _check(b_bias.dim() == 2 and b_bias.size(0) == num_experts and b_bias.size(1) == size_n,
                   "b_bias must be [experts, size_n]")

        has_zp = b_qzeros is not None and b_qzeros.size(-1) > 0
        _check(not has_zp or fmt in (1, 3),
               "Marlin does not support zero-point metadata for this quant type.")
        if has_zp:
            _check(b_qzeros.is_cuda and b_qzeros.is_contiguous(), "b_zeros is not on GPU")
            _check(is_zp_float, "Marlin MoE received b_zeros but is_zp_float is false. Packed integer "
                                "zero-points are not supported.")
            _check(b_qzeros.dtype == a.dtype, "Marlin MoE expects zero points of the activation dtype.")
            _check(tuple(b_qzeros.shape) == (num_experts, num_groups, size_n),
                   "b_zeros must be [experts, num_groups, size_n]")
        else:
            _check(not is_zp_float, "is_zp_float is true but b_zeros was not provided.")
            _check(fmt not in (1, 3), "Marlin uint4/uint8 MoE path requires float zero points.")

        for t, name in ((sorted_token_ids, "sorted_token_ids"), (expert_ids, "expert_ids"),
                        (num_tokens_past_padded, "num_tokens_past_padded")):
            _check(t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous GPU tensor")
            _check(t.dtype == torch.int32, f"{name} must be int32")
        _check(topk_weights.is_cuda and topk_weights.is_contiguous() and topk_weights.dtype == torch.float32,
               "topk_weights must be a contiguous fp32 GPU tensor")
        _check(topk_weights.numel() >= size_m * top_k, "topk_weights has fewer than size_m * top_k entries")
        num_sorted = sorted_token_ids.numel()

        if is_prepared(b_qweight, size_k, size_n):
            fmt |= _lib.FMT_PREPARED     # expert weights converted by prepare_weights (decode-sized blocks only)
        _check(not silu_input or (fmt & _lib.FMT_PREPARED),
               "silu_input needs expert weights in the streaming layout")
        if silu_input:
            fmt |= _lib.FMT_SILU_INPUT
        nbytes = lib.marlin_b200_moe_gemm_scratch_bytes(num_sorted, size_n, size_k, fmt)
        scratch = _scratch(nbytes, a.device)
        _lib.check(lib.marlin_b200_moe_gemm(
            _ptr(a), _ptr(c), _ptr(b_qweight), _ptr(b_scales), _ptr(b_qzeros) if has_zp else None,
            _ptr(b_bias), _ptr(global_scale), _ptr(sorted_token_ids), _ptr(expert_ids),
            _ptr(num_tokens_past_padded), _ptr(topk_weights), num_sorted, num_experts,
            moe_block_size, top_k, int(bool(mul_topk_weights)), act, fmt, size_m, size_n, size_k,
            num_groups, _ptr(scratch), nbytes, _stream(a.device)))
    return c


def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_size: int,
                         sorted_token_ids: torch.Tensor, experts_ids: torch.Tensor,
                         num_tokens_post_pad: torch.Tensor,
                         expert_map: torch.Tensor | None = None) -> None:
    """Fills the three caller-allocated outputs (reference: moe_align_sum_kernels.cu:477-569)."""
    lib = _lib.load()
    _check(topk_ids.is_cuda and topk_ids.is_contiguous(), "topk_ids must be a contiguous GPU tensor")
    _check(topk_ids.dtype == torch.int32, "topk_ids must be int32")
    for t in (sorted_token_ids, experts_ids, num_tokens_post_pad):
        _check(t.is_cuda and t.is_contiguous() and t.dtype == torch.int32,
               "align outputs must be contiguous int32 GPU tensors")
    num_global = 0
    if expert_map is not None:
        _check(expert_map.is_cuda and expert_map.is_contiguous() and expert_map.dtype == torch.int32,
               "expert_map must be a contiguous int32 GPU tensor")
        num_global = expert_map.numel()
    numel = topk_ids.numel()
    with torch.cuda.device(topk_ids.device):
        nbytes = lib.marlin_b200_moe_align_scratch_bytes(numel, num_experts)
        scratch = _scratch(nbytes, topk_ids.device)
        _lib.check(lib.marlin_b200_moe_align_block_size(
            _ptr(topk_ids), numel, num_experts, num_global, block_size, _ptr(expert_map),
            _ptr(sorted_token_ids), sorted_token_ids.numel(), _ptr(experts_ids), experts_ids.numel(),
            _ptr(num_tokens_post_pad), _ptr(scratch), nbytes, _stream(topk_ids.device)))


def topk_softmax(topk_weights: torch.Tensor, topk_ids: torch.Tensor, token_expert_indices: torch.Tensor,
                 gating_output: torch.Tensor, renormalize: bool = False,
                 e_score_correction_bias: torch.Tensor | None = None) -> None:
    """Fused softmax + top-k (reference: topk_softmax_kernels.cu:773-809)."""
    lib = _lib.load()
    _check(gating_output.is_cuda and gating_output.is_contiguous(), "gating_output must be contiguous on GPU")
    code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}.get(gating_output.dtype)
    _check(code is not None, "Invalid gating_output type")
    _check(topk_weights.dtype == torch.float32 and topk_weights.is_contiguous(), "topk_weights must be fp32")
    _check(topk_ids.dtype == torch.int32 and topk_ids.is_contiguous(), "topk_indices must be int32")
    _check(token_expert_indices.dtype == torch.int32 and token_expert_indices.is_contiguous(),
           "token_expert_indices must be int32")
    num_experts = gating_output.size(-1)
    num_tokens = gating_output.numel() // max(num_experts, 1)
    topk = topk_weights.size(-1)
    bias = e_score_correction_bias
    if bias is not None:
        _check(bias.is_cuda and bias.is_contiguous() and bias.dtype == torch.float32 and
               bias.numel() == num_experts, "bias must be a contiguous fp32 [num_experts] GPU tensor")
    with torch.cuda.device(gating_output.device):
        _lib.check(lib.marlin_b200_topk_softmax(
            _ptr(gating_output), code, _ptr(bias), _ptr(topk_weights), _ptr(topk_ids),
            _ptr(token_expert_indices), num_tokens, num_experts, topk, int(bool(renormalize)),
            _stream(gating_output.device)))


def silu_and_mul(out: torch.Tensor, x: torch.Tensor) -> None:
    """out = silu(x[..., :d]) * x[..., d:] (reference: fused_moe/activation.py:45-67, eager there)."""
    lib = _lib.load()
    _check(x.is_cuda and x.is_contiguous() and out.is_contiguous(), "silu_and_mul needs contiguous GPU tensors")
    inter = x.size(-1) // 2
    rows = x.numel() // max(x.size(-1), 1)
    with torch.cuda.device(x.device):
        _lib.check(lib.marlin_b200_silu_and_mul(_ptr(x), _ptr(out), rows, inter, _act_code(x.dtype),
                                                _stream(x.device)))


def moe_sum(input: torch.Tensor, output: torch.Tensor) -> None:
    """output[t] = sum_j input[t, j] for input [tokens, top_k, hidden]
    (reference: fused_marlin_moe.py:379-382, torch.sum there)."""
    lib = _lib.load()
    _check(input.is_cuda and input.is_contiguous() and output.is_contiguous(), "moe_sum needs contiguous GPU tensors")
    tokens, top_k, hidden = input.shape
    with torch.cuda.device(input.device):
        _lib.check(lib.marlin_b200_moe_sum(_ptr(input), _ptr(output), tokens, top_k, hidden,
                                           _act_code(input.dtype), _stream(input.device)))


def moe_sum_rows(input: torch.Tensor, rows: torch.Tensor, output: torch.Tensor) -> None:
    """output[t] = sum_j input[rows[t, j]] for input [R, hidden], rows int32 [tokens, top_k]: the top-k
    sum over contributions that sit in another order (the expert-parallel combine)."""
    lib = _lib.load()
    _check(input.is_cuda and input.is_contiguous() and output.is_contiguous() and rows.is_contiguous(),
           "moe_sum_rows needs contiguous GPU tensors")
    _check(rows.dtype == torch.int32, "rows must be int32")
    tokens, top_k = rows.shape
    hidden = input.shape[1]
    with torch.cuda.device(input.device):
        _lib.check(lib.marlin_b200_moe_sum_rows(_ptr(input), _ptr(rows), _ptr(output), tokens, top_k, hidden,
                                                _act_code(input.dtype), _stream(input.device)))


def kernel_status(reset: bool = False) -> int:
    """0 when no pipelined kernel on the current device gave up on one of its bounded waits since the
    last reset (see marlin_b200_kernel_status); synchronises with the device."""
    import ctypes
    lib = _lib.load()
    value = ctypes.c_int(0)
    _lib.check(lib.marlin_b200_kernel_status(ctypes.byref(value), int(reset)))
    return int(value.value)
