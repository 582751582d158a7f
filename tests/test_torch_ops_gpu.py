"""The torch extension modules `_C` / `_moe_C`: the reference's operator schemas, registered by this build and
implemented by libmarlin_b200.so.  The modules are loaded the way the reference loads them (`import vllm._C`,
tests/ops.py:25-37 there) from a scratch package directory holding links to the built files; every hot-path
operator is then called through `torch.ops` and compared with the oracle."""
import importlib
import os
import sys

import pytest
import torch

from oracle import marlin_oracle as mo
from tests import util

pytestmark = pytest.mark.gpu

# Schema strings of the reference (csrc/torch_bindings_marlin.cpp:6-34, csrc/moe/torch_bindings_marlin.cpp:5-54),
# as torch prints them back.
DENSE_SCHEMAS = {
    "marlin_gemm": "_C::marlin_gemm(Tensor a, Tensor? c_or_none, Tensor b_q_weight, Tensor? b_bias_or_none, "
                   "Tensor b_scales, Tensor? a_scales, Tensor? global_scale, Tensor? b_zeros_or_none, "
                   "Tensor? g_idx_or_none, Tensor? perm_or_none, Tensor workspace, int b_type_id, SymInt size_m, "
                   "SymInt size_n, SymInt size_k, bool is_k_full, bool use_atomic_add, bool use_fp32_reduce, "
                   "bool is_zp_float) -> Tensor",
    "gptq_marlin_repack": "_C::gptq_marlin_repack(Tensor b_q_weight, Tensor perm, SymInt size_k, SymInt size_n, "
                          "int num_bits, bool is_a_8bit) -> Tensor",
    "awq_marlin_repack": "_C::awq_marlin_repack(Tensor b_q_weight, SymInt size_k, SymInt size_n, int num_bits, "
                         "bool is_a_8bit) -> Tensor",
    "marlin_int4_fp8_preprocess": "_C::marlin_int4_fp8_preprocess(Tensor qweight, Tensor? qzeros_or_none, "
                                  "bool inplace) -> Tensor",
}
MOE_OPS = ("topk_softmax", "topk_sigmoid", "moe_align_block_size", "batched_moe_align_block_size",
           "moe_wna16_marlin_gemm", "grouped_topk")


@pytest.fixture(scope="module")
def torch_ops(tmp_path_factory):
    from marlin_v100_b200 import build
    paths = build.build_torch_ops()
    pkg = tmp_path_factory.mktemp("site") / "vllm"
    pkg.mkdir()
    (pkg / "__init__.py").write_text("")
    # the three files travel together: the modules find the library next to themselves
    for path in [*paths, build.LIB_PATH]:
        os.symlink(path, pkg / os.path.basename(path))
    sys.path.insert(0, str(pkg.parent))
    try:
        importlib.import_module("vllm._C")       # the reference's load path
        importlib.import_module("vllm._moe_C")
    finally:
        sys.path.remove(str(pkg.parent))
    return torch.ops


def test_schemas_are_the_references(torch_ops):
    for name, schema in DENSE_SCHEMAS.items():
        assert str(getattr(torch_ops._C, name).default._schema) == schema
    for name in ("sm70_cutlass_matmul_probe", "sm70_cutlass_matmul_explicit_warp_probe"):
        assert hasattr(torch_ops._C, name)
    for name in MOE_OPS:
        assert hasattr(torch_ops._moe_C, name)
    s = str(torch_ops._moe_C.moe_wna16_marlin_gemm.default._schema)
    assert "int moe_block_size, int top_k, bool mul_topk_weights, int b_type_id" in s and s.endswith("-> Tensor")


@pytest.mark.parametrize("fmt,dtype,m", [("u4b8", torch.float16, 16), ("u4", torch.bfloat16, 40), ("fp8", torch.bfloat16, 3),
                                         ("nvfp4", torch.float16, 7)])
def test_repack_and_gemm_through_torch_ops(torch_ops, fmt, dtype, m):
    k, n = 512, 768
    a, qw = util.make_dense(m, k, n, fmt, dtype, seed=31)
    bits = qw.extra["bits"]
    q = qw.extra["q"]
    perm = torch.empty(0, dtype=torch.int32, device="cuda")
    packed = torch_ops._C.gptq_marlin_repack(mo.gptq_pack(q, bits).cuda(), perm, k, n, bits, False)
    assert torch.equal(packed.cpu(), qw.packed)
    packed_awq = torch_ops._C.awq_marlin_repack(mo.awq_pack(q, bits).cuda(), k, n, bits, False)
    assert torch.equal(packed_awq.cpu(), qw.packed)
    d = util.to_dev(qw)
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    c = torch.empty(m, n, dtype=dtype, device="cuda")
    out = torch_ops._C.marlin_gemm(a.cuda(), c, packed, None, d.scales, None, d.global_scale, d.zeros, None, None, ws,
                                   qw.type_id, m, n, k, True, False, True, qw.zeros is not None)
    assert out.data_ptr() == c.data_ptr() and ws.numel() == 0      # c_or_none written in place, workspace untouched
    ref = mo.dense_reference(a, qw.deq)
    assert mo.within_tolerance(out.cpu(), ref)
    # the streaming layout through the operator boundary: converted once, recognised by its address
    if fmt in ("u4b8", "u4"):
        prepared = torch_ops._C.marlin_b200_prepare_weights(packed, k, n, bits)
        out2 = torch_ops._C.marlin_gemm(a.cuda(), None, prepared, None, d.scales, None, d.global_scale, d.zeros, None,
                                        None, ws, qw.type_id, m, n, k, True, False, True, qw.zeros is not None)
        assert mo.within_tolerance(out2.cpu(), ref)
        assert torch.equal(torch_ops._C.marlin_b200_restore_weights(prepared, k, n, bits), packed)


def test_error_messages_are_the_references(torch_ops):
    a = torch.zeros(4, 64, dtype=torch.float16, device="cuda")
    w = torch.zeros(4, 100 * 2, dtype=torch.int32, device="cuda")
    s = torch.zeros(1, 100, dtype=torch.float16, device="cuda")
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="b_q_weight.size\\(1\\) = 200 is not divisible by tile_size = 16"):
        torch_ops._C.marlin_gemm(a, None, w, None, s, None, None, None, None, None, ws, mo.TYPE_U4B8, 4, 100, 64, True,
                                 False, True, False)
    g_idx = torch.zeros(64, dtype=torch.int32, device="cuda")
    w = torch.zeros(4, 128 * 2, dtype=torch.int32, device="cuda")
    s = torch.zeros(1, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="does not support act_order g_idx"):
        torch_ops._C.marlin_gemm(a, None, w, None, s, None, None, None, g_idx, None, ws, mo.TYPE_U4B8, 4, 128, 64, True,
                                 False, True, False)


def test_int4_fp8_preprocess_closed_form(torch_ops):
    g = torch.Generator().manual_seed(1)
    q = torch.randint(0, 16, (256, 512), generator=g, dtype=torch.int32)
    packed = (q[:, ::2] * 16 + q[:, 1::2]).to(torch.int8).view(torch.int32).cuda()
    res = torch_ops._C.marlin_int4_fp8_preprocess(packed, None, False)
    want = torch.where(q >= 8, q - 8, 15 - q)
    want = (want[:, ::2] * 16 + want[:, 1::2]).to(torch.int8).view(torch.int32)
    assert torch.equal(res.cpu(), want)
    # AWQ form: zero-points per group of 32 rows, same packing along the columns
    z = torch.randint(0, 16, (8, 512), generator=g, dtype=torch.int32)
    zp = (z[:, ::2] * 16 + z[:, 1::2]).to(torch.int8).view(torch.int32).cuda()
    res = torch_ops._C.marlin_int4_fp8_preprocess(packed, zp, False)
    zfull = z.repeat_interleave(32, dim=0)
    want = torch.where(q >= zfull, q - zfull, 15 - q)
    want = (want[:, ::2] * 16 + want[:, 1::2]).to(torch.int8).view(torch.int32)
    assert torch.equal(res.cpu(), want)


@pytest.mark.parametrize("sigmoid", [False, True])
def test_topk_through_torch_ops(torch_ops, sigmoid):
    t, e, k = 33, 128, 8
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(t, e, generator=g)
    w = torch.empty(t, k, dtype=torch.float32, device="cuda")
    ids = torch.empty(t, k, dtype=torch.int32, device="cuda")
    tei = torch.empty(t, k, dtype=torch.int32, device="cuda")
    op = torch_ops._moe_C.topk_sigmoid if sigmoid else torch_ops._moe_C.topk_softmax
    op(w, ids, tei, logits.cuda(), True, None)
    scores = torch.sigmoid(logits) if sigmoid else torch.softmax(logits, dim=-1)
    rw, rids = torch.topk(scores, k, dim=-1)
    rw = rw / rw.sum(dim=-1, keepdim=True)
    assert torch.equal(ids.cpu().long(), rids)
    assert torch.allclose(w.cpu(), rw, atol=1e-5, rtol=1e-5)
    assert torch.equal(tei.cpu(), (torch.arange(k).view(1, k) * t + torch.arange(t).view(t, 1)).int())


def test_align_and_grouped_gemm_through_torch_ops(torch_ops):
    t, e, k, hidden, n, block = 48, 8, 2, 256, 256, 16
    g = torch.Generator().manual_seed(5)
    ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).int()
    sorted_ids = torch.empty(t * k + e * (block - 1), dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(sorted_ids.numel() // block + 1, dtype=torch.int32, device="cuda")
    num_post = torch.empty(1, dtype=torch.int32, device="cuda")
    torch_ops._moe_C.moe_align_block_size(ids.cuda(), e, block, sorted_ids, expert_ids, num_post, None)
    rs, re_, rn = mo.moe_align_block_size_reference(ids, block, e)
    npp = int(rn)
    assert int(num_post.item()) == npp
    assert torch.equal(sorted_ids.cpu()[:npp], rs[:npp]) and torch.equal(expert_ids.cpu()[:npp // block], re_[:npp // block])
    x = torch.randn(t, hidden, generator=g).to(torch.float16)
    w = util.make_experts(e, hidden, n, "u4b8", torch.float16, seed=6, scale=0.05)
    d = util.to_dev(w)
    tw = torch.rand(t * k, generator=g).float()
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    out = torch_ops._moe_C.moe_wna16_marlin_gemm(x.cuda(), None, d.packed, None, d.scales, None, None, None, None, None,
                                                 ws, sorted_ids, expert_ids, num_post, tw.cuda(), block, k, True,
                                                 w.type_id, t, n, hidden, True, False, True, False, -1, -1, -1)
    ref = mo.moe_gemm_reference(x, w.deq, ids, k, tw)
    assert mo.within_tolerance(out.cpu(), ref)


def test_batched_align_matches_its_definition(torch_ops):
    max_tokens, block = 40, 16
    counts = torch.tensor([0, 5, 40, 16, 17, 0, 1], dtype=torch.int32)
    b = counts.numel()
    per = -(-max_tokens // block)
    sorted_ids = torch.empty(b * per * block, dtype=torch.int32, device="cuda")
    block_ids = torch.empty(b * per, dtype=torch.int32, device="cuda")
    num_post = torch.empty(1, dtype=torch.int32, device="cuda")
    torch_ops._moe_C.batched_moe_align_block_size(max_tokens, block, counts.cuda(), sorted_ids, block_ids, num_post)
    want_ids = torch.full((b * per * block,), b * max_tokens, dtype=torch.int32)
    want_blocks = torch.full((b * per,), -1, dtype=torch.int32)
    off = 0
    for e in range(b):
        c = int(counts[e])
        want_ids[off:off + c] = torch.arange(c, dtype=torch.int32) + e * max_tokens
        nb = -(-c // block)
        want_blocks[off // block:off // block + nb] = e
        off += nb * block
    assert int(num_post.item()) == off
    assert torch.equal(sorted_ids.cpu(), want_ids) and torch.equal(block_ids.cpu(), want_blocks)


def test_grouped_topk_picks_inside_the_best_groups(torch_ops):
    t, e, n_group, topk_group, topk = 16, 64, 8, 3, 6
    g = torch.Generator().manual_seed(9)
    scores = torch.rand(t, e, generator=g)
    bias = torch.zeros(e)
    w, ids = torch_ops._moe_C.grouped_topk(scores.cuda(), n_group, topk_group, topk, True, 2.5, bias.cuda(), 0)
    ids, w = ids.cpu().long(), w.cpu()
    group_scores = scores.view(t, n_group, -1).topk(2, dim=-1)[0].sum(-1)
    best = group_scores.topk(topk_group, dim=-1)[1]
    for row in range(t):
        assert set((ids[row] // (e // n_group)).tolist()) <= set(best[row].tolist())
        picked = scores[row, ids[row]]
        assert torch.allclose(w[row], picked / picked.sum() * 2.5, atol=1e-6)
