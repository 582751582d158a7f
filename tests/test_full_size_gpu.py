"""Full-size parity of the dense GEMM: a weight tensor of the benchmark's shapes goes the way a model
loader takes it - quantise on the CPU, pack in the checkpoint format (AWQ for uint4 with zero-points, GPTQ for
the rest), repack on the GPU with `awq_marlin_repack` / `gptq_marlin_repack`, GEMM - and the result is
compared with the CPU oracle (dequantise the GPU-repacked tensor, fp32 matmul).

Shapes: K=8192, N=28672 (uint4 + zero-points group 128; uint8b128 per channel) at M in {1,16,128,1024,4096}
and K=5120, N=25600 (fp8 per channel, mxfp4, nvfp4) at M in {1,32,512}, bf16 activations.  M <= 128: all
columns; larger M: 16 column groups of 256 spread over N (first, last and every seventh or so between).
Both weight layouts are run where the library takes both.

Tolerance (both forms must hold): mean|d| / mean|ref| <= 1e-2 and mean(|d| / max(|ref|, eps)) <= 1e-2 with
eps = mean|ref|; and max|d| <= 5e-2 * max|ref|."""
import functools

import pytest
import torch

from oracle import marlin_oracle as mo
from tests import util

pytestmark = pytest.mark.gpu

CASES = [("u4", 8192, 28672, 128, (1, 16, 128, 1024, 4096)),
         ("u8b128", 8192, 28672, -1, (1, 16, 128, 1024, 4096)),
         ("fp8", 5120, 25600, -1, (1, 32, 512)),
         ("mxfp4", 5120, 25600, 32, (1, 32, 512)),
         ("nvfp4", 5120, 25600, 16, (1, 32, 512))]
PARAMS = [pytest.param(fmt, k, n, gs, m, id=f"{fmt}-k{k}-n{n}-m{m}") for fmt, k, n, gs, ms in CASES for m in ms]


@functools.lru_cache(maxsize=1)
def loaded_weight(fmt: str, k: int, n: int, gs: int):
    """One resident problem at a time: quantised on the CPU, repacked on the GPU, dequantised by the oracle."""
    from marlin_v100_b200 import ops
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(31)
    w = (torch.randn(k, n, generator=g) * 0.02).to(dtype)
    qw = util.quantize(w, fmt, gs, want_deq=False, pack=False)
    del w
    q, bits = qw.extra["q"], qw.extra["bits"]
    if fmt == "u4":   # AWQ checkpoints carry the zero-points
        packed = ops.awq_marlin_repack(mo.awq_pack(q, bits).cuda(), k, n, bits)
    else:
        perm = torch.empty(0, dtype=torch.int32, device="cuda")
        packed = ops.gptq_marlin_repack(mo.gptq_pack(q, bits).cuda(), perm, k, n, bits)
    # the repack kernel against the oracle's packer on the whole tensor
    assert torch.equal(packed.cpu(), mo.marlin_pack(q, bits))
    qw.extra.clear()
    del q
    deq = mo.dequantize(packed.cpu(), qw.scales, k, n, qw.type_id, zeros=qw.zeros, global_scale=qw.global_scale,
                        out_dtype=dtype)
    streaming = ops.prepare_weights(packed, k, n, bits)
    dev = dict(packed=packed, streaming=streaming, scales=qw.scales.cuda(),
               zeros=None if qw.zeros is None else qw.zeros.cuda(),
               gscale=None if qw.global_scale is None else qw.global_scale.cuda())
    return qw, dev, deq


def check(out: torch.Tensor, ref: torch.Tensor, what: str):
    assert torch.isfinite(out).all(), what
    mre, ere, mxe = mo.mean_rel_err(out, ref), mo.mean_elem_rel_err(out, ref), mo.max_abs_err_frac(out, ref)
    assert mre <= 1e-2 and ere <= 1e-2 and mxe <= 5e-2, f"{what}: mean_rel={mre:.3e} elem_rel={ere:.3e} max_frac={mxe:.3e}"


@pytest.mark.parametrize("fmt,k,n,gs,m", PARAMS)
def test_full_size_dense(fmt, k, n, gs, m):
    from marlin_v100_b200 import ops
    qw, dev, deq = loaded_weight(fmt, k, n, gs)
    a = torch.randn(m, k, generator=torch.Generator().manual_seed(100 + m)).to(torch.bfloat16)
    if m <= 128:
        cols = torch.arange(n)
    else:
        groups = sorted(set([0, n // 256 - 1] + list(range(3, n // 256, 7))))[:16]
        cols = torch.cat([torch.arange(g * 256, (g + 1) * 256) for g in groups])
    ref = mo.dense_reference(a, deq[:, cols])
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    for layout in ("packed", "streaming"):
        out = ops.marlin_gemm(a.cuda(), None, dev[layout], None, dev["scales"], None, dev["gscale"], dev["zeros"],
                              None, None, ws, qw.type_id, m, n, k, True, False, True, dev["zeros"] is not None)
        assert tuple(out.shape) == (m, n) and out.dtype == torch.bfloat16
        check(out.cpu()[:, cols].float(), ref, f"{layout} layout")
