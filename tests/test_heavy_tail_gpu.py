"""Activations with a heavy tail through the M <= 16 kernels that split activations into integer digits
(`decode_tc_kernel` on the reference layout at K*N >= 2^27, `stream_i8_kernel` on the streaming layout).

Every ordinary row holds one element 2^12 times the size of the rest (512 against 0.125), so the small
elements keep only the low digits of the row's fixed-point form; one row is made of fp16 subnormals only
(its scale is far below every other row's); one row is zero.  The oracle is dequantise + fp32 matmul.

Tolerance: per row mean|d| / mean|ref| <= 1e-2; for the subnormal row, whose outputs are themselves fp16
subnormals, |d| <= one subnormal step (2^-24) + 1e-2 |ref|."""
import pytest
import torch

from oracle import marlin_oracle as mo
from tests import util

pytestmark = pytest.mark.gpu

K, N = 8192, 16384   # K*N = 2^27


@pytest.fixture(scope="module")
def weights():
    out = {}
    for dtype in (torch.float16, torch.bfloat16):
        w = (torch.randn(K, N, generator=torch.Generator().manual_seed(5)) * 0.02).to(dtype)
        out[dtype] = util.quantize(w, "u4b8", 128)
    return out


def activations(m: int, dtype) -> torch.Tensor:
    g = torch.Generator().manual_seed(9)
    a = (torch.rand(m, K, generator=g) - 0.5) * 0.25              # |x| <= 0.125
    spike = torch.randint(0, K, (m,), generator=g)
    a[torch.arange(m), spike] = 512.0 * torch.where(torch.rand(m, generator=g) < 0.5, -1.0, 1.0)
    a = a.to(dtype)
    if m >= 3:
        if dtype == torch.float16:
            a[1] = (torch.randint(-1023, 1024, (K,), generator=g).float() * 2.0 ** -24).to(dtype)   # subnormals
        else:
            a[1] = (torch.randn(K, generator=g) * 1e-30).to(dtype)
        a[2] = 0
    return a


@pytest.mark.parametrize("layout", ["packed", "streaming"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 12, 16, 29])
def test_heavy_tail_rows(weights, dtype, m, layout):
    from marlin_v100_b200 import ops
    qw = weights[dtype]
    d = util.to_dev(qw)
    b = d.packed if layout == "packed" else ops.prepare_weights(d.packed, K, N, 4)
    a = activations(m, dtype)
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    out = ops.marlin_gemm(a.cuda(), None, b, None, d.scales, None, None, None, None, None, ws, qw.type_id,
                          m, N, K, True, False, True, False).cpu().float()
    ref = mo.dense_reference(a, qw.deq)
    assert torch.isfinite(out).all()
    for r in range(m):
        if m >= 3 and r == 2:
            assert torch.count_nonzero(out[r]) == 0
        elif m >= 3 and r == 1 and dtype == torch.float16:
            assert bool(((out[r] - ref[r]).abs() <= 2.0 ** -24 + 1e-2 * ref[r].abs()).all())
        else:
            mre = mo.mean_rel_err(out[r], ref[r])
            assert mre <= 1e-2, f"row {r}: mean_rel={mre:.3e}"
