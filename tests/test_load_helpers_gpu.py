"""Load-time helpers against the oracle (which is pinned to the reference's own functions by the golden
fixtures): the batched expert repack and the fp4 / fp8 scale re-encoders.  Everything here is bit-exact."""
import pytest
import torch

from oracle import marlin_oracle as mo

pytestmark = pytest.mark.gpu


def _ops():
    from marlin_v100_b200 import ops
    return ops


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("k,n,e", [(64, 128, 3), (256, 768, 5), (128, 64, 1)])
def test_batched_expert_repack(bits, k, n, e):
    ops = _ops()
    g = torch.Generator().manual_seed(bits * 100 + k + n + e)
    q = torch.randint(0, 1 << bits, (e, k, n), generator=g, dtype=torch.int32)
    want = torch.stack([mo.marlin_pack(q[i], bits) for i in range(e)])
    gptq = torch.stack([mo.gptq_pack(q[i], bits) for i in range(e)]).cuda()
    awq = torch.stack([mo.awq_pack(q[i], bits) for i in range(e)]).cuda()
    assert torch.equal(ops.gptq_marlin_moe_repack(gptq, None, k, n, bits).cpu(), want)
    assert torch.equal(ops.awq_marlin_moe_repack(awq, None, k, n, bits).cpu(), want)
    # the same as the per-expert operator, expert by expert
    empty = torch.empty(0, dtype=torch.int32, device="cuda")
    for i in range(e):
        assert torch.equal(ops.gptq_marlin_repack(gptq[i].contiguous(), empty, k, n, bits).cpu(), want[i])
    # act-order: a different row permutation per expert
    perm = torch.stack([torch.randperm(k, generator=g) for _ in range(e)]).to(torch.int32)
    want_perm = torch.stack([mo.gptq_marlin_repack(gptq[i].cpu(), perm[i], k, n, bits) for i in range(e)])
    assert torch.equal(ops.gptq_marlin_moe_repack(gptq, perm.cuda(), k, n, bits).cpu(), want_perm)


def test_batched_repack_rejects_bad_shapes():
    ops = _ops()
    w = torch.zeros((2, 8, 64), dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="Shape mismatch"):
        ops.gptq_marlin_moe_repack(w, None, 128, 64, 4)
    with pytest.raises(RuntimeError, match="tile_n_size"):
        ops.awq_marlin_moe_repack(w, None, 64, 96, 4)
    assert ops.gptq_marlin_moe_repack(w[:0].contiguous(), None, 64, 64, 4).shape == (0, 4, 128)


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("small", [False, True])
def test_nvfp4_scale_encoder(dt, small):
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    s = torch.rand(40, 256, generator=g) * (0.5 if small else 200.0) + (2.0 ** -8 if small else 4.0)
    s = s.to(torch.float8_e4m3fn)
    s[3, 7] = 0
    want, want_sf = mo.nvfp4_encode_scales(s.to(dt), dt)
    got, sf = ops.nvfp4_marlin_process_scales(s.to(dt).cuda(), None, dt)
    assert sf == want_sf and (sf > 1.0) == (small and dt == torch.bfloat16)
    assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8))
    # a caller-given factor (experts of one layer share it)
    want4, _ = mo.nvfp4_encode_scales(s.to(dt), dt, 4.0)
    got4, sf4 = ops.nvfp4_marlin_process_scales(s.to(dt).cuda(), 4.0, dt)
    assert sf4 == 4.0 and torch.equal(got4.cpu().view(torch.uint8), want4.view(torch.uint8))
    gs = torch.tensor([0.0123, 1.0], dtype=torch.float32)
    assert torch.equal(ops.nvfp4_marlin_process_global_scale(gs.cuda(), dt).cpu(), mo.nvfp4_process_global_scale(gs, dt))


def test_mxfp4_and_fp8_scale_encoders():
    ops = _ops()
    g = torch.Generator().manual_seed(6)
    e8 = torch.pow(2.0, torch.randint(-20, 6, (24, 128), generator=g).float()).to(torch.bfloat16)
    assert torch.equal(ops.mxfp4_marlin_process_scales(e8.cuda(), torch.bfloat16).cpu().view(torch.uint8),
                       mo.mxfp4_encode_scales(e8).view(torch.uint8))
    for dt in (torch.float16, torch.bfloat16):
        sc = (torch.rand(7, 96, generator=g) * 1e-3 + 1e-5).to(dt)
        assert torch.equal(ops.fp8_fused_exponent_bias_into_scales(sc.cuda()).cpu(), mo.fp8_fuse_exponent_bias(sc))


def test_encoded_scales_feed_the_gemm():
    """nvfp4 weights quantised on the CPU, scales encoded on the GPU, GEMM against the oracle."""
    from tests import util
    ops = _ops()
    dt = torch.bfloat16
    a, qw = util.make_dense(8, 512, 512, "nvfp4", dt, seed=12)
    # undo the oracle's encoding to get the checkpoint's e4m3 block scales back, then encode on the GPU
    dec = mo.nvfp4_decode_scales(qw.scales)            # value * 2^7 * scale_factor, logical order
    want_bytes = qw.scales.view(torch.uint8)
    got, _ = ops.nvfp4_marlin_process_scales((dec / 128.0).to(dt).cuda(), 1.0, dt)
    assert torch.equal(got.cpu().view(torch.uint8), want_bytes)
    d = util.to_dev(qw)
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    out = ops.marlin_gemm(a.cuda(), None, d.packed, None, got, None, d.global_scale, None, None, None, ws, qw.type_id,
                          8, 512, 512, True, False, True, False)
    assert mo.within_tolerance(out.cpu(), mo.dense_reference(a, qw.deq))
