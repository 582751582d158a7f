"""ctypes binding of the C ABI in ``include/marlin_b200.h``.

There is no CPU or PyTorch fallback: if the shared library is missing the import of the operators
fails with an error that says how to build it."""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libmarlin_b200.so")

_c = ctypes
_vp, _i64, _int = _c.c_void_p, _c.c_int64, _c.c_int

# name -> (restype, argtypes); mirrors include/marlin_b200.h one to one
SIGNATURES = {
    "marlin_b200_last_error": (_c.c_char_p, []),
    "marlin_b200_version": (_c.c_char_p, []),
    "marlin_b200_launch_count": (_i64, []),
    "marlin_b200_kernel_status": (_int, [_vp, _int]),
    "marlin_b200_format_from_type_id": (_int, [_i64, _int]),
    "marlin_b200_gptq_repack": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "marlin_b200_awq_repack": (_int, [_vp, _vp, _i64, _i64, _int, _vp]),
    "marlin_b200_prepare_weights": (_int, [_vp, _vp, _i64, _i64, _int, _i64, _vp]),
    "marlin_b200_restore_weights": (_int, [_vp, _vp, _i64, _i64, _int, _i64, _vp]),
    "marlin_b200_gemm_scratch_bytes": (_i64, [_i64, _i64, _i64, _int]),
    "marlin_b200_gemm": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _i64, _i64, _i64, _i64,
                                _i64, _vp, _i64, _vp]),
    "marlin_b200_gemm_static_scratch": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _i64, _i64, _i64,
                                               _i64, _i64, _vp]),
    "marlin_b200_moe_gemm_scratch_bytes": (_i64, [_i64, _i64, _i64, _int]),
    "marlin_b200_moe_gemm": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                    _int, _int, _int, _int, _int, _i64, _i64, _i64, _i64, _vp, _i64,
                                    _vp]),
    "marlin_b200_moe_align_scratch_bytes": (_i64, [_i64, _i64]),
    "marlin_b200_moe_align_block_size": (_int, [_vp, _i64, _i64, _i64, _int, _vp, _vp, _i64, _vp, _i64,
                                                _vp, _vp, _i64, _vp]),
    "marlin_b200_topk_softmax": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _vp]),
    "marlin_b200_topk_sigmoid": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _vp]),
    "marlin_b200_batched_moe_align_block_size": (_int, [_i64, _int, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp]),
    "marlin_b200_int4_fp8_preprocess": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "marlin_b200_silu_and_mul": (_int, [_vp, _vp, _i64, _i64, _int, _vp]),
    "marlin_b200_moe_sum": (_int, [_vp, _vp, _i64, _int, _i64, _int, _vp]),
    "marlin_b200_moe_sum_rows": (_int, [_vp, _vp, _vp, _i64, _int, _i64, _int, _vp]),
    "marlin_b200_gptq_moe_repack": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "marlin_b200_awq_moe_repack": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "marlin_b200_nvfp4_scale_min": (_int, [_vp, _i64, _vp, _vp]),
    "marlin_b200_nvfp4_process_scales": (_int, [_vp, _vp, _i64, _i64, _c.c_float, _vp]),
    "marlin_b200_interleave_scale_bytes": (_int, [_vp, _vp, _i64, _i64, _vp]),
    "marlin_b200_fp8_fuse_exponent_bias": (_int, [_vp, _vp, _i64, _int, _vp]),
    "marlin_b200_peer_header_bytes": (_int, []),
    "marlin_b200_peer_alloc": (_int, [_i64, _vp]),
    "marlin_b200_peer_free": (_int, [_vp]),
    "marlin_b200_peer_export": (_int, [_vp, _vp]),
    "marlin_b200_peer_open": (_int, [_vp, _vp]),
    "marlin_b200_peer_close": (_int, [_vp]),
    "marlin_b200_peer_status": (_int, [_vp, _vp, _vp]),
    "marlin_b200_peer_host_word_alloc": (_int, [_vp, _vp]),
    "marlin_b200_peer_host_word_free": (_int, [_vp]),
    "marlin_b200_peer_allgather": (_int, [_vp, _int, _int, _vp, _i64, _i64, _vp, _i64, _vp]),
    "marlin_b200_ep_plan": (_int, [_vp, _int, _int, _vp, _i64, _int, _vp]),
    "marlin_b200_ep_dispatch": (_int, [_vp, _int, _int, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _vp, _vp]),
    "marlin_b200_ep_poll_rows": (_int, [_vp, _int, _int, _vp, _vp, _vp]),
    "marlin_b200_ep_wait": (_int, [_vp, _int, _int, _int, _vp]),
    "marlin_b200_ep_signal": (_int, [_vp, _int, _int, _int, _vp]),
    "marlin_b200_ep_combine": (_int, [_vp, _int, _int, _vp, _vp, _int, _i64, _vp, _int, _int, _vp]),
}

FMT_PREPARED = 0x100  # MARLIN_B200_FMT_PREPARED
FMT_SILU_INPUT = 0x200  # MARLIN_B200_FMT_SILU_INPUT

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m marlin_v100_b200.build` "
                "(needs nvcc with sm_100a support); this package has no fallback path")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int) -> None:
    """Turn a negative status into the RuntimeError the reference raises through TORCH_CHECK."""
    if rc != 0:
        msg = load().marlin_b200_last_error().decode("utf-8", "replace")
        raise RuntimeError(msg or f"marlin_b200 call failed with status {rc}")
