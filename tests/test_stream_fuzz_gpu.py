"""Seeded random shapes through the integer-MMA streaming kernel, dense and grouped, against the oracle:
K in multiples of 128 up to 2304, N in multiples of 256 up to 1792, M 1..32, group sizes 128 / 256 / 384 / per
channel where they divide K, both 4-bit integer formats, both activation types, bias on and off.  The split of
the (column group, chunk) units over the SMs changes with every shape (fewer units than SMs, groups owned by one,
two or many CTAs), which is what this is after.  Tolerance as everywhere: mean|d| / mean|ref| <= 1e-2 and
max|d| <= 5e-2 max|ref|."""
import random

import pytest
import torch

from oracle import marlin_oracle as mo
from tests import util

pytestmark = pytest.mark.gpu


def _cases(seed: int, count: int):
    rnd = random.Random(seed)
    out = []
    for i in range(count):
        k = 128 * rnd.randint(1, 18)
        n = 256 * rnd.randint(1, 7)
        groups = [g for g in (128, 256, 384, -1) if g == -1 or k % g == 0]
        out.append((i, rnd.randint(1, 32), k, n, rnd.choice(groups), rnd.choice(["u4b8", "u4"]),
                    rnd.choice([torch.float16, torch.bfloat16]), rnd.random() < 0.4))
    return out


@pytest.mark.parametrize("i,m,k,n,gs,fmt,dtype,with_bias", _cases(2024, 36))
def test_dense_random_shapes(i, m, k, n, gs, fmt, dtype, with_bias):
    from marlin_v100_b200 import ops
    a, qw = util.make_dense(m, k, n, fmt, dtype, group_size=gs, seed=100 + i)
    d = util.to_dev(qw)
    prepared = ops.prepare_weights(d.packed, k, n, 4)
    bias = None
    if with_bias:
        bias = (torch.randn(n, generator=torch.Generator().manual_seed(i)) * 0.3).to(dtype)
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    out = ops.marlin_gemm(a.cuda(), None, prepared, None if bias is None else mo.permute_bias(bias).cuda(), d.scales,
                          None, None, d.zeros, None, None, ws, qw.type_id, m, n, k, True, False, True,
                          qw.zeros is not None)
    ref = mo.dense_reference(a, qw.deq, bias)
    assert mo.within_tolerance(out.cpu(), ref), (mo.mean_rel_err(out.cpu(), ref), mo.max_abs_err_frac(out.cpu(), ref))


@pytest.mark.parametrize("i,m,k,n,gs,fmt,dtype,with_bias", _cases(77, 18))
def test_grouped_random_shapes(i, m, k, n, gs, fmt, dtype, with_bias):
    from marlin_v100_b200 import fused_moe, ops
    rnd = random.Random(1000 + i)
    e, top_k = rnd.choice([2, 4, 8, 16]), rnd.choice([1, 2, 4])
    top_k = min(top_k, e)
    t = m * 3                                    # up to 96 tokens
    block = rnd.choice([8, 16, 32])
    g = torch.Generator().manual_seed(500 + i)
    tw, ids, _ = mo.topk_softmax_reference(torch.randn(t, e, generator=g), top_k, True)
    a = torch.randn(t, k, generator=g).to(dtype)
    qw = util.make_experts(e, k, n, fmt, dtype, group_size=gs, seed=600 + i)
    d = util.to_dev(qw)
    prepared = ops.prepare_weights(d.packed, k, n, 4)
    bias = pbias = None
    if with_bias:
        bias = (torch.randn(e, n, generator=g) * 0.3).to(dtype)
        pbias = torch.stack([mo.permute_bias(b) for b in bias]).cuda()
    s, x, npp = fused_moe.moe_align_block_size(ids.cuda(), block, e, None)
    c = torch.zeros((t * top_k, n), dtype=dtype, device="cuda")
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    out = ops.moe_wna16_marlin_gemm(a.cuda(), c, prepared, pbias, d.scales, None, None, d.zeros, None, None, ws, s, x,
                                    npp, tw.reshape(-1).contiguous().cuda(), block, top_k, True, qw.type_id, t, n, k,
                                    True, False, True, qw.zeros is not None)
    ref = mo.moe_gemm_reference(a, qw.deq, ids, top_k, tw, bias)
    assert mo.within_tolerance(out.cpu(), ref), (mo.mean_rel_err(out.cpu(), ref), mo.max_abs_err_frac(out.cpu(), ref))
    assert ops.kernel_status() == 0
