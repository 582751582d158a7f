"""Grouped (expert) GEMM on expert weights in the streaming layout: the decode-sized integer-MMA kernel
(blocks of 8, 16 or 32 sorted routes), through the C ABI, against the oracle and against the kernel on the
reference layout.  Tolerance: mean|d| / mean|ref| <= 1e-2 and max|d| <= 5e-2 max|ref|."""
import pytest
import torch

from oracle import marlin_oracle as mo
from tests import util
from tests.test_moe_gpu import _route, check

pytestmark = pytest.mark.gpu


def _ops():
    from marlin_v100_b200 import ops
    return ops


def _fm():
    from marlin_v100_b200 import fused_moe
    return fused_moe


def _moe_gemm_streaming(a, qw, tw, ids, block, top_k, mul, bias=None, emap=None, e_bins=None):
    ops, fm = _ops(), _fm()
    d = util.to_dev(qw)
    e = qw.packed.shape[0]
    bits = 4
    prepared = ops.prepare_weights(d.packed, qw.size_k, qw.size_n, bits)
    assert torch.equal(ops.restore_weights(prepared, qw.size_k, qw.size_n, bits), d.packed)
    s, x, npp = fm.moe_align_block_size(ids.cuda(), block, e_bins or e, None if emap is None else emap.cuda())
    m = a.shape[0]
    c = torch.zeros((m * top_k, qw.size_n), dtype=a.dtype, device="cuda")
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    return ops.moe_wna16_marlin_gemm(a.cuda(), c, prepared, None if bias is None else bias.cuda(), d.scales,
                                     None, d.global_scale, d.zeros, None, None, ws, s, x, npp,
                                     tw.reshape(-1).cuda(), block, top_k, mul, qw.type_id, m, qw.size_n,
                                     qw.size_k, True, False, True, qw.zeros is not None)


@pytest.mark.parametrize("fmt", ["u4b8", "u4"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("block", [8, 16])
def test_grouped_streaming_formats(fmt, dtype, block):
    t, e, k, K, N = 40, 8, 2, 512, 512
    tw, ids = _route(t, e, k, 1)
    a = torch.randn(t, K, generator=torch.Generator().manual_seed(2)).to(dtype)
    qw = util.make_experts(e, K, N, fmt, dtype, seed=3)
    out = _moe_gemm_streaming(a, qw, tw, ids, block, k, True)
    check(out, mo.moe_gemm_reference(a, qw.deq, ids, k, tw))


@pytest.mark.parametrize("t,e,k", [(1, 16, 4), (3, 16, 4), (64, 128, 8), (17, 8, 2)])
@pytest.mark.parametrize("block", [8, 16, 32])
def test_grouped_streaming_tokens_and_experts(t, e, k, block):
    """Few routes per expert, many experts, empty experts; more units than SMs and fewer."""
    K, N = 1024, 768
    tw, ids = _route(t, e, k, 4, zipf=True)
    a = torch.randn(t, K, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    qw = util.make_experts(e, K, N, "u4b8", torch.bfloat16, seed=6)
    out = _moe_gemm_streaming(a, qw, tw, ids, block, k, False)
    check(out, mo.moe_gemm_reference(a, qw.deq, ids, k, None))
    again = _moe_gemm_streaming(a, qw, tw, ids, block, k, False)
    assert torch.equal(out, again)          # the cross-CTA sums keep a fixed order


def test_grouped_streaming_per_channel_bias_and_second_stage():
    t, e, K, N = 50, 4, 256, 256
    g = torch.Generator().manual_seed(8)
    ids = torch.randint(0, e, (t, 1), generator=g, dtype=torch.int32)
    tw = torch.rand(t, 1, generator=g)
    a = torch.randn(t, K, generator=g).to(torch.float16)
    qw = util.make_experts(e, K, N, "u4", torch.float16, group_size=-1, seed=9)
    bias = (torch.randn(e, N, generator=g) * 0.3).to(torch.float16)
    pbias = torch.stack([mo.permute_bias(b) for b in bias])
    out = _moe_gemm_streaming(a, qw, tw, ids, 16, 1, True, bias=pbias)
    check(out, mo.moe_gemm_reference(a, qw.deq, ids, 1, tw, bias))


def test_grouped_streaming_expert_map():
    t, e_global, e_local, k, K, N = 32, 8, 4, 2, 256, 256
    tw, ids = _route(t, e_global, k, 10)
    emap = torch.full((e_global,), -1, dtype=torch.int32)
    emap[4:8] = torch.arange(4, dtype=torch.int32)
    a = torch.randn(t, K, generator=torch.Generator().manual_seed(11)).to(torch.float16)
    qw = util.make_experts(e_local, K, N, "u4b8", torch.float16, seed=12)
    out = _moe_gemm_streaming(a, qw, tw, ids, 16, k, True, emap=emap, e_bins=e_global)
    local = emap[ids.long()]
    ref = torch.zeros(t * k, N)
    keep = (local >= 0).reshape(-1)
    full = mo.moe_gemm_reference(a, qw.deq, local.clamp_min(0), k, tw)
    ref[keep] = full[keep]
    check(out, ref)
    assert torch.all(out.cpu()[~keep] == 0)


def test_grouped_streaming_refuses_what_it_does_not_serve():
    t, e, k, K, N = 300, 4, 2, 256, 256
    tw, ids = _route(t, e, k, 13)
    a = torch.randn(t, K, generator=torch.Generator().manual_seed(14)).to(torch.float16)
    qw = util.make_experts(e, K, N, "u4b8", torch.float16, seed=15)
    with pytest.raises(RuntimeError, match="streaming layout"):
        _moe_gemm_streaming(a, qw, tw, ids, 64, k, True)


@pytest.mark.parametrize("t", [1, 16, 48])
def test_fused_layer_on_streaming_weights(t):
    ops = _ops()
    e, k, H, I = 32, 4, 512, 256
    tw, ids = _route(t, e, k, 20, zipf=True)
    g = torch.Generator().manual_seed(21)
    hidden = torch.randn(t, H, generator=g).to(torch.bfloat16)
    w13 = util.make_experts(e, H, 2 * I, "u4b8", torch.bfloat16, seed=22, scale=0.05)
    w2 = util.make_experts(e, I, H, "u4b8", torch.bfloat16, seed=23, scale=0.05)
    d13, d2 = util.to_dev(w13), util.to_dev(w2)
    s13 = ops.prepare_weights(d13.packed, H, 2 * I, 4)
    s2 = ops.prepare_weights(d2.packed, I, H, 4)
    out = _fm().fused_marlin_moe(hidden.cuda(), d13.packed, d2.packed, None, None, d13.scales, d2.scales,
                                 tw.cuda(), ids.cuda(), w13.type_id, w1_streaming=s13, w2_streaming=s2)
    check(out, mo.moe_reference(hidden, w13.deq, w2.deq, tw, ids, round_dtype=torch.bfloat16))
    assert ops.kernel_status() == 0


def test_silu_on_load_equals_the_separate_pass():
    """The second GEMM with SiLU-and-mul applied where it reads its rows returns the bits of the separate
    SiLU-and-mul pass followed by the same GEMM."""
    ops, fm = _ops(), _fm()
    t, e, inter, H = 24, 8, 256, 512
    g = torch.Generator().manual_seed(40)
    ids = torch.randint(0, e, (t, 1), generator=g, dtype=torch.int32)
    tw = torch.rand(t, 1, generator=g)
    c1 = torch.randn(t, 2 * inter, generator=g).to(torch.bfloat16).cuda()
    qw = util.make_experts(e, inter, H, "u4b8", torch.bfloat16, seed=41)
    d = util.to_dev(qw)
    prepared = ops.prepare_weights(d.packed, inter, H, 4)
    s, x, npp = fm.moe_align_block_size(ids.cuda(), 16, e, None)
    ws = torch.empty(0, dtype=torch.int32, device="cuda")

    def gemm(a, silu):
        c = torch.zeros((t, H), dtype=torch.bfloat16, device="cuda")
        return ops.moe_wna16_marlin_gemm(a, c, prepared, None, d.scales, None, None, None, None, None, ws, s, x, npp,
                                         tw.reshape(-1).cuda(), 16, 1, True, qw.type_id, t, H, inter, True, False,
                                         True, False, silu_input=silu)

    act = torch.empty((t, inter), dtype=torch.bfloat16, device="cuda")
    ops.silu_and_mul(act, c1)
    assert torch.equal(gemm(c1, True), gemm(act, False))
    with pytest.raises(RuntimeError, match="streaming layout"):
        ops.moe_wna16_marlin_gemm(c1, None, d.packed, None, d.scales, None, None, None, None, None, ws, s, x, npp,
                                  tw.reshape(-1).cuda(), 16, 1, True, qw.type_id, t, H, inter, True, False, True,
                                  False, silu_input=True)
