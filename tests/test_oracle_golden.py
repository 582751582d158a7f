"""Pins the CPU oracle against outputs of the reference's own Python helpers (stored fixtures) and
against the literal known-answer inputs of the reference's tests."""
import os

import numpy as np
import pytest
import torch

from oracle import marlin_oracle as mo

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_helpers.npz"))


def T(name, dtype=None):
    t = torch.from_numpy(G[name].copy())
    if dtype is not None:
        t = t.view(dtype)
    return t


LAYOUT = [(b, k, n) for b in (4, 8)
          for (k, n) in ((32, 64), (48, 128), (32, 192), (64, 256), (32, 320), (32, 512), (16, 768))]


@pytest.mark.parametrize("bits,k,n", LAYOUT)
def test_layout_matches_reference(bits, k, n):
    tag = f"layout_b{bits}_k{k}_n{n}"
    q = T(tag + "_q")
    assert torch.equal(mo.marlin_pack(q, bits), T(tag + "_packed"))
    assert torch.equal(mo.marlin_unpack(T(tag + "_packed"), k, n, bits), T(tag + "_unpacked"))
    assert torch.equal(T(tag + "_unpacked"), q)
    assert torch.equal(mo.gptq_pack(q, bits), T(tag + "_gptq"))
    assert torch.equal(mo.awq_pack(q, bits), T(tag + "_awq"))
    assert torch.equal(mo.gptq_marlin_repack(T(tag + "_gptq"), None, k, n, bits), T(tag + "_packed"))
    assert torch.equal(mo.awq_marlin_repack(T(tag + "_awq"), k, n, bits), T(tag + "_packed"))


@pytest.mark.parametrize("name,bits", [("u4b8", 4), ("u8b128", 8)])
@pytest.mark.parametrize("act", [0, 1])
def test_deterministic_repack_known_answer(name, bits, act):
    tag = f"repack_{name}_act{act}"
    perm = T(tag + "_perm") if act else None
    got = mo.gptq_marlin_repack(T(tag + "_gptq_in"), perm, 128, 128, bits)
    assert torch.equal(got, T(tag + "_expected"))


@pytest.mark.parametrize("name,bits,gs", [("u4b8", 4, 32), ("u4b8", 4, -1), ("u8b128", 8, 64), ("u8b128", 8, -1)])
def test_symmetric_quantise_dequantise(name, bits, gs):
    w = T("w16")
    k, n = w.shape
    q, s = mo.quantize_sym(w, bits, gs)
    tag = f"{name}_g{gs}"
    assert torch.equal(mo.marlin_pack(q, bits), T(tag + "_qw"))
    assert torch.equal(s, T(tag + "_s"))
    tid = mo.TYPE_U4B8 if bits == 4 else mo.TYPE_U8B128
    deq = mo.dequantize(T(tag + "_qw"), s, k, n, tid)
    assert torch.equal(deq, T(tag + "_deq"))
    ref = mo.dense_reference(T("a16"), deq)
    torch.testing.assert_close(ref, T(tag + "_ref"), rtol=0, atol=0)


@pytest.mark.parametrize("name,bits", [("u4", 4), ("u8", 8)])
@pytest.mark.parametrize("gs", [32, -1])
def test_zero_point_quantise_dequantise(name, bits, gs):
    w = T("w16")
    k, n = w.shape
    q, s, zp, zpf = mo.quantize_asym(w, bits, gs)
    tag = f"{name}_g{gs}"
    assert torch.equal(mo.marlin_pack(q, bits), T(tag + "_qw"))
    assert torch.equal(s, T(tag + "_s"))
    assert torch.equal(zpf, T(tag + "_zp"))
    tid = mo.TYPE_U4 if bits == 4 else mo.TYPE_U8
    assert torch.equal(mo.dequantize(T(tag + "_qw"), s, k, n, tid, zeros=zpf), T(tag + "_deq"))


@pytest.mark.parametrize("gs", [-1, 128])
def test_fp8(gs):
    w = T("w16")
    k, n = w.shape
    raw, boundary, _ = mo.quantize_fp8(w, gs)
    assert torch.equal(mo.marlin_pack(raw, 8), T(f"fp8_g{gs}_qw"))
    assert torch.equal(boundary, T(f"fp8_g{gs}_s"))
    deq = mo.dequantize(T(f"fp8_g{gs}_qw"), boundary, k, n, mo.TYPE_FE4M3)
    assert torch.equal(deq, T(f"fp8_g{gs}_deq"))


def test_nvfp4():
    w = T("w16")
    k, n = w.shape
    q, sbytes, g = mo.quantize_nvfp4(w)
    assert torch.equal(mo.marlin_pack(q, 4), T("nvfp4_qw"))
    assert torch.equal(sbytes.view(torch.uint8), T("nvfp4_s"))
    assert torch.equal(g, T("nvfp4_g"))
    deq = mo.dequantize(T("nvfp4_qw"), sbytes, k, n, mo.TYPE_FE2M1, global_scale=g)
    assert torch.equal(deq, T("nvfp4_deq"))


def test_mxfp4():
    w = T("w16")
    k, n = w.shape
    q, s8 = mo.quantize_mxfp4(w)
    assert torch.equal(mo.marlin_pack(q, 4), T("mxfp4_qw"))
    assert torch.equal(s8.view(torch.uint8), T("mxfp4_s"))
    deq = mo.dequantize(T("mxfp4_qw"), s8, k, n, mo.TYPE_FE2M1)
    assert torch.equal(deq, T("mxfp4_deq"))


def test_bias_permutation():
    assert torch.equal(mo.permute_bias(T("bias_in")), T("bias_perm"))
    assert torch.equal(mo.unpermute_bias(T("bias_perm")), T("bias_in"))


def test_scalar_type_ids():
    ids = [mo.TYPE_U4, mo.TYPE_U4B8, mo.TYPE_U8, mo.TYPE_U8B128, mo.TYPE_FE2M1, mo.TYPE_FE4M3]
    assert ids == G["type_ids"].tolist()


def test_moe_reference():
    out = mo.moe_reference(T("moe_hidden"), T("moe_w1"), T("moe_w2"), T("moe_topk_w"), T("moe_topk_ids"))
    torch.testing.assert_close(out, T("moe_ref"), rtol=1e-5, atol=1e-6)


def test_topk_known_answer():
    # literal of the reference's test (tests/test_marlin_moe.py:248-271)
    gating = torch.tensor([[0.10, 0.80, -0.20, 0.30], [1.20, -0.40, 0.50, 0.10],
                           [-0.70, 0.60, 0.20, 1.10]], dtype=torch.float16)
    bias = torch.tensor([0.05, -0.10, 0.20, 0.15], dtype=torch.float32)
    w, ids, tei = mo.topk_softmax_reference(gating, 2, True, bias)
    probs = torch.softmax(gating.float(), -1)
    exp_ids = torch.topk(probs + bias, 2, dim=-1).indices
    assert torch.equal(ids, exp_ids.to(torch.int32))
    ew = torch.gather(probs, 1, exp_ids)
    torch.testing.assert_close(w, ew / ew.sum(-1, keepdim=True), rtol=1e-6, atol=1e-7)
    assert tei.tolist() == [[0, 3], [1, 4], [2, 5]]


def test_align_known_answer():
    # literal of the reference's test (tests/test_marlin_moe.py:274-291)
    ids = torch.tensor([[0, 3], [1, 3], [0, 2], [1, 0]], dtype=torch.int32)
    s, e, t = mo.moe_align_block_size_reference(ids, 4, 4)
    assert int(t) == 16
    assert s[:16].tolist() == [0, 4, 7, 8, 2, 6, 8, 8, 5, 8, 8, 8, 1, 3, 8, 8]
    assert e[:4].tolist() == [0, 1, 2, 3]
    assert torch.all(s[16:] == 8) and torch.all(e[4:] == -1)


def test_align_expert_map_and_empty_experts():
    ids = torch.tensor([[5, 1], [7, 5], [2, 2]], dtype=torch.int32)
    emap = torch.tensor([-1, 0, 1, -1, -1, 2, -1, -1], dtype=torch.int32)
    s, e, t = mo.moe_align_block_size_reference(ids, 2, 3, emap)
    # local 0 <- global 1: idx 1; local 1 <- global 2: idx 4,5; local 2 <- global 5: idx 0,3
    assert int(t) == 6
    assert s[:6].tolist() == [1, 6, 4, 5, 0, 3]
    assert e[:3].tolist() == [0, 1, 2]


# --- scale encoders of the fp4 / fp8 paths, fp16 and bf16, against the reference's own functions --------
S = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_scale_encoders.npz"))


def TS(name, dtype=None):
    t = torch.from_numpy(S[name].copy())
    return t if dtype is None else t.view(dtype)


@pytest.mark.parametrize("tag", ["wide", "narrow"])
@pytest.mark.parametrize("dn,dt", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_nvfp4_scale_encoder_matches_reference(tag, dn, dt):
    s = TS(f"nvfp4_{tag}_in", torch.float8_e4m3fn)
    enc, sf = mo.nvfp4_encode_scales(s.to(dt), dt)
    assert sf == float(S[f"nvfp4_{tag}_{dn}_sf"][0])
    assert torch.equal(enc.view(torch.uint8), TS(f"nvfp4_{tag}_{dn}_enc"))
    if tag == "wide":
        assert (sf > 1.0) == (dt == torch.bfloat16)   # only the bf16 path rescales small scales


@pytest.mark.parametrize("dn,dt", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_global_scale_and_fp8_bias_match_reference(dn, dt):
    assert torch.equal(mo.nvfp4_process_global_scale(TS("nvfp4_global_in"), dt), TS(f"nvfp4_global_{dn}"))
    sc = TS(f"fp8_scale_{dn}_in", dt if dt == torch.float16 else None)
    exp = TS(f"fp8_scale_{dn}_out", dt if dt == torch.float16 else None)
    if dt == torch.bfloat16:
        sc, exp = sc.view(torch.bfloat16), exp.view(torch.bfloat16)
    assert torch.equal(mo.fp8_fuse_exponent_bias(sc), exp)


def test_mxfp4_scale_encoder_matches_reference():
    enc = mo.mxfp4_encode_scales(TS("mxfp4_in").to(torch.bfloat16))
    assert torch.equal(enc.view(torch.uint8), TS("mxfp4_enc"))
