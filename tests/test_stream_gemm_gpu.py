"""The streaming weight layout and the weight-streaming GEMM that reads it, through the C ABI.

Layout: `prepare_weights` must hold exactly the codes of the reference layout (unpack(streaming) ==
unpack(reference) == q, checked against the oracle's statement of the layout) and `restore_weights` must be
its exact inverse.  GEMM: same tolerance as the reference-layout path, mean|y - ref| / mean|ref| <= 1e-2 and
max|y - ref| <= 5e-2 * max|ref| against dequantise -> fp32 matmul."""
import pytest
import torch

from oracle import marlin_oracle as mo
from tests import util

pytestmark = pytest.mark.gpu

MEAN_TOL, MAX_TOL = 1e-2, 5e-2


def _ops():
    from marlin_v100_b200 import ops
    return ops


def run_prepared(a, qw, bias=None, c=None):
    ops = _ops()
    d = util.to_dev(qw)
    bits = qw.extra["bits"]
    prepared = ops.prepare_weights(d.packed, qw.size_k, qw.size_n, bits)
    assert ops.is_prepared(prepared, qw.size_k, qw.size_n) and not ops.is_prepared(d.packed, qw.size_k, qw.size_n)
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    out = ops.marlin_gemm(a.cuda(), c, prepared, None if bias is None else mo.permute_bias(bias).cuda(),
                          d.scales, None, d.global_scale, d.zeros, None, None, ws, qw.type_id,
                          a.shape[0], qw.size_n, qw.size_k, True, False, True, qw.zeros is not None)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    return out


def check(out, ref):
    assert torch.isfinite(out.float()).all()
    mre, mxe = mo.mean_rel_err(out.cpu(), ref), mo.max_abs_err_frac(out.cpu(), ref)
    assert mre <= MEAN_TOL and mxe <= MAX_TOL, f"mean_rel={mre:.3e} max_frac={mxe:.3e}"


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("k,n,experts", [(128, 256, 1), (512, 768, 1), (4096, 4096, 1), (256, 512, 3)])
def test_layout_is_a_bijection_on_the_codes(bits, k, n, experts):
    ops = _ops()
    g = torch.Generator().manual_seed(k + n + bits)
    q = torch.randint(0, 1 << bits, (experts, k, n), generator=g, dtype=torch.int32)
    ref_layout = torch.stack([mo.marlin_pack(q[e], bits) for e in range(experts)])
    want = torch.stack([mo.stream_layout_pack(q[e], bits) for e in range(experts)])
    if experts == 1:
        ref_layout, want = ref_layout[0], want[0]
    prepared = ops.prepare_weights(ref_layout.cuda(), k, n, bits)
    assert torch.equal(prepared.cpu(), want)                       # unpack(streaming) == q, by the oracle's statement
    back = ops.restore_weights(prepared, k, n, bits)
    assert torch.equal(back.cpu(), ref_layout)                     # exact inverse
    one = want if experts == 1 else want[0]
    assert torch.equal(mo.stream_layout_unpack(one, k, n, bits), q[0])


def test_layout_refuses_other_shapes():
    ops = _ops()
    w = torch.zeros(64 // 16, 320 * 2, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="size_k % 128 == 0 and size_n % 256 == 0"):
        ops.prepare_weights(w, 64, 320, 4)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fmt", util.FORMATS)
@pytest.mark.parametrize("m", [1, 16, 40, 128])
def test_formats(fmt, dtype, m):
    a, qw = util.make_dense(m, 512, 512, fmt, dtype, seed=1)
    out = run_prepared(a, qw)
    assert out.dtype == dtype and tuple(out.shape) == (m, 512)
    check(out, mo.dense_reference(a, qw.deq))


@pytest.mark.parametrize("fmt,gs", [("u4b8", -1), ("u4b8", 16), ("u4b8", 32), ("u4b8", 64), ("u4b8", 256), ("u4", -1),
                                    ("u4", 64), ("u8b128", -1), ("u8b128", 128), ("u8", 32), ("u8", 128),
                                    ("fp8", -1), ("fp8", 128)])
def test_group_sizes(fmt, gs):
    a, qw = util.make_dense(8, 512, 256, fmt, torch.float16, group_size=gs, seed=2)
    check(run_prepared(a, qw), mo.dense_reference(a, qw.deq))


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 15, 16, 17, 24, 33, 48, 64, 65, 100, 128, 129, 257])
def test_odd_m(m):
    a, qw = util.make_dense(m, 512, 768, "u4b8", torch.float16, seed=3)
    check(run_prepared(a, qw), mo.dense_reference(a, qw.deq))


@pytest.mark.parametrize("fmt", ["u4b8", "u4", "nvfp4", "u8b128"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bias(fmt, dtype):
    a, qw = util.make_dense(6, 256, 512, fmt, dtype, seed=6)
    bias = (torch.randn(512, generator=torch.Generator().manual_seed(7)) * 0.5).to(dtype)
    check(run_prepared(a, qw, bias=bias), mo.dense_reference(a, qw.deq, bias))


@pytest.mark.parametrize("m,k,n", [(16, 4096, 4096), (64, 4096, 4096), (16, 2048, 2560), (100, 1024, 9216)])
def test_column_groups_shared_between_ctas(m, k, n):
    """Shapes whose (column group, chunk) units do not divide by the SM count: partial sums go through the
    scratch and the last CTA of a column group adds them.  Two runs must agree bit for bit."""
    a, qw = util.make_dense(m, k, n, "u4", torch.bfloat16, seed=5)
    out1 = run_prepared(a, qw)
    out2 = run_prepared(a, qw)
    assert torch.equal(out1, out2)
    check(out1, mo.dense_reference(a, qw.deq))


def test_without_scratch_every_cta_takes_whole_column_groups():
    from marlin_v100_b200 import _lib
    ops = _ops()
    lib = _lib.load()
    m, k, n = 16, 1024, 2048
    a, qw = util.make_dense(m, k, n, "u4b8", torch.float16, seed=9)
    d = util.to_dev(qw)
    prepared = ops.prepare_weights(d.packed, k, n, 4)
    out = torch.empty(m, n, dtype=torch.float16, device="cuda")
    a_dev = a.cuda()
    _lib.check(lib.marlin_b200_gemm(a_dev.data_ptr(), out.data_ptr(), prepared.data_ptr(), d.scales.data_ptr(), None,
                                    None, None, 0, 0 | _lib.FMT_PREPARED, m, n, k, k, k // 128, None, 0,
                                    torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    check(out, mo.dense_reference(a, qw.deq))


def test_strided_a_and_preallocated_c():
    a, qw = util.make_dense(4, 256, 256, "u4b8", torch.float16, seed=8)
    ops = _ops()
    d = util.to_dev(qw)
    prepared = ops.prepare_weights(d.packed, 256, 256, 4)
    big = torch.zeros(4, 512, dtype=torch.float16, device="cuda")
    big[:, :256] = a.cuda()
    c = torch.full((4, 256), 7.0, dtype=torch.float16, device="cuda")
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    out = ops.marlin_gemm(big[:, :256], c, prepared, None, d.scales, None, None, None, None, None, ws, qw.type_id,
                          4, 256, 256)
    assert out.data_ptr() == c.data_ptr()
    check(out, mo.dense_reference(a, qw.deq))


def test_grouped_gemm_takes_the_flag_only_for_decode_blocks():
    """Expert weights in the streaming layout are served for blocks of 8 / 16 / 32 routes (tests/test_moe_stream_gpu.py);
    any other block size is refused with a message that names the reference layout."""
    from marlin_v100_b200 import _lib
    lib = _lib.load()
    dev = torch.zeros(4096, dtype=torch.int32, device="cuda")
    ptr = dev.data_ptr()
    rc = lib.marlin_b200_moe_gemm(ptr, ptr, ptr, ptr, None, None, None, ptr, ptr, ptr, ptr, 64, 1, 64, 1, 0, 0,
                                  0 | _lib.FMT_PREPARED, 1, 256, 128, 1, None, 0, None)
    assert rc == -1 and b"reference layout" in lib.marlin_b200_last_error()
