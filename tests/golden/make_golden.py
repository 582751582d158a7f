"""Generate the golden fixtures in this folder from the reference project's own Python helpers.

Run once, in a container that has the reference checked out:

    REFERENCE_ROOT=/path/to/reference python tests/golden/make_golden.py

It imports ``tests.helpers`` / ``tests.quant_utils`` of the reference (pure CPU code), runs them on
small seeded inputs and stores inputs and outputs as ``.npz`` files.  The oracle in ``oracle/`` is
then pinned against these files by ``tests/test_oracle_golden.py``; nothing at test time needs the
reference itself.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu):
        return t.contiguous().view(torch.uint8).numpy()
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy()
    return t.contiguous().numpy()


def main() -> None:
    ref_root = os.environ.get("REFERENCE_ROOT")
    if not ref_root or not os.path.isdir(ref_root):
        raise SystemExit("set REFERENCE_ROOT to a checkout of the reference project (its tests/ helpers are imported)")
    sys.path.insert(0, ref_root)
    from tests import helpers, quant_utils  # noqa: E402  (reference modules)

    st = helpers.scalar_types
    out: dict[str, np.ndarray] = {}

    # --- packed layout, every macro-N class, both bit widths ------------------------------
    for bits in (4, 8):
        for (k, n) in ((32, 64), (48, 128), (32, 192), (64, 256), (32, 320), (32, 512), (16, 768)):
            g = torch.Generator().manual_seed(1000 * bits + k + n)
            q = torch.randint(0, 1 << bits, (k, n), generator=g, dtype=torch.int32)
            perm = quant_utils.get_weight_perm(bits, is_a_8bit=False)
            packed = quant_utils.marlin_weights(q, k, n, bits, perm, is_a_8bit=False)
            tag = f"layout_b{bits}_k{k}_n{n}"
            out[tag + "_q"] = _np(q)
            out[tag + "_packed"] = _np(packed)
            out[tag + "_gptq"] = _np(helpers.gptq_pack(q, bits, k, n))
            out[tag + "_awq"] = _np(helpers.awq_pack(q, bits, k, n))
            qt = st.uint4 if bits == 4 else st.uint8
            out[tag + "_unpacked"] = _np(helpers._marlin_unpack_impl(packed, k, n, qt))

    # --- the reference's deterministic repack input (arange % 2^bits at 128x128) -----------
    for qt, name in ((st.uint4b8, "u4b8"), (st.uint8b128, "u8b128")):
        for act_order in (False, True):
            q, sq, sort_idx = helpers._deterministic_repack_input(
                qt, act_order=act_order, size_k=128, size_n=128, group_size=64, device="cpu")
            perm = quant_utils.get_weight_perm(qt.size_bits, is_a_8bit=False)
            exp = quant_utils.marlin_weights(sq, 128, 128, qt.size_bits, perm, is_a_8bit=False)
            tag = f"repack_{name}_act{int(act_order)}"
            out[tag + "_gptq_in"] = _np(helpers.gptq_pack(q, qt.size_bits, 128, 128))
            out[tag + "_perm"] = _np(sort_idx)
            out[tag + "_expected"] = _np(exp)

    # --- quantise + dequantise per format ---------------------------------------------------
    torch.manual_seed(0)
    k, n = 128, 192
    w16 = (torch.randn(k, n) * 0.02).to(torch.float16)
    out["w16"] = _np(w16)
    a16 = torch.randn(8, k).to(torch.float16)
    out["a16"] = _np(a16)

    for qt, name, gs in ((st.uint4b8, "u4b8", 32), (st.uint4b8, "u4b8", -1),
                         (st.uint8b128, "u8b128", 64), (st.uint8b128, "u8b128", -1)):
        _, qw, sc, *_ = helpers.marlin_quantize(w16, qt, gs, False)
        deq = helpers.marlin_dequantize(qw, sc, k, n, gs, qt)
        tag = f"{name}_g{gs}"
        out[tag + "_qw"], out[tag + "_s"], out[tag + "_deq"] = _np(qw), _np(sc), _np(deq)
        out[tag + "_ref"] = _np(helpers.marlin_dense_reference(a16, qw, sc, k, n, gs, qt))

    for fn, name in ((helpers.marlin_quantize_uint4_zp, "u4"), (helpers.marlin_quantize_uint8_zp, "u8")):
        for gs in (32, -1):
            _, qw, sc, zp, deq = fn(w16, gs)
            tag = f"{name}_g{gs}"
            out[tag + "_qw"], out[tag + "_s"], out[tag + "_zp"], out[tag + "_deq"] = (
                _np(qw), _np(sc), _np(zp), _np(deq))

    for gs in (-1, 128):
        _, qw, sc, *_ = helpers.marlin_quantize_fp8(w16, gs)
        deq = helpers.marlin_dequantize(qw, sc, k, n, gs, st.float8_e4m3fn)
        out[f"fp8_g{gs}_qw"], out[f"fp8_g{gs}_s"], out[f"fp8_g{gs}_deq"] = _np(qw), _np(sc), _np(deq)

    deq, qw, sc, gsc, *_ = helpers.marlin_quantize_nvfp4(w16, 16)
    out["nvfp4_qw"], out["nvfp4_s"], out["nvfp4_g"], out["nvfp4_deq"] = _np(qw), _np(sc), _np(gsc), _np(deq)

    deq_q, qw, sc, *_ = helpers.marlin_quantize_mxfp4(w16, 32)
    deq = helpers.marlin_dequantize_mxfp4(qw, sc, k, n, 32)
    out["mxfp4_qw"], out["mxfp4_s"], out["mxfp4_deq"] = _np(qw), _np(sc), _np(deq)

    # --- bias permutation --------------------------------------------------------------------
    b = torch.arange(192, dtype=torch.float16)
    out["bias_in"], out["bias_perm"] = _np(b), _np(helpers.marlin_permute_bias(b))

    # --- MoE reference on a tiny layer ---------------------------------------------------------
    torch.manual_seed(1)
    hid = torch.randn(5, 64).to(torch.float16)
    w1 = (torch.randn(4, 64, 2 * 32) * 0.1).to(torch.float16)
    w2 = (torch.randn(4, 32, 64) * 0.1).to(torch.float16)
    tw, ti = helpers.make_moe_routing_tensors(tokens=5, experts=4, topk=2, device="cpu",
                                              routing_profile="zipfian")
    out["moe_hidden"], out["moe_w1"], out["moe_w2"] = _np(hid), _np(w1), _np(w2)
    out["moe_topk_w"], out["moe_topk_ids"] = _np(tw), _np(ti)
    out["moe_ref"] = _np(helpers.marlin_moe_reference(hid, w1, w2, tw, ti))

    # --- scalar type ids -------------------------------------------------------------------------
    out["type_ids"] = np.array([st.uint4.id, st.uint4b8.id, st.uint8.id, st.uint8b128.id,
                                st.float4_e2m1f.id, st.float8_e4m3fn.id], dtype=np.int64)

    np.savez_compressed(os.path.join(HERE, "reference_helpers.npz"), **out)
    print(f"wrote {len(out)} arrays")


if __name__ == "__main__":
    main()
