"""Dense marlin_gemm parity against dequantise -> fp32 matmul (the oracle), through the C ABI.

Tolerance (stated by the task): mean|y - ref| / mean|ref| <= 1e-2 and max|y - ref| <= 5e-2 * max|ref|."""
import pytest
import torch

from oracle import marlin_oracle as mo
from tests import util

pytestmark = pytest.mark.gpu

MEAN_TOL, MAX_TOL = 1e-2, 5e-2


def _ops():
    from marlin_v100_b200 import ops
    return ops


def run_gemm(a, qw, bias=None, c=None):
    ops = _ops()
    d = util.to_dev(qw)
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    out = ops.marlin_gemm(a.cuda(), c, d.packed, None if bias is None else mo.permute_bias(bias).cuda(),
                          d.scales, None, d.global_scale, d.zeros, None, None, ws, qw.type_id,
                          a.shape[0], qw.size_n, qw.size_k, True, False, True, qw.zeros is not None)
    assert ws.numel() == 0
    return out


def check(out, ref):
    assert torch.isfinite(out.float()).all()
    mre, mxe = mo.mean_rel_err(out.cpu(), ref), mo.max_abs_err_frac(out.cpu(), ref)
    assert mre <= MEAN_TOL and mxe <= MAX_TOL, f"mean_rel={mre:.3e} max_frac={mxe:.3e}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fmt", util.FORMATS)
@pytest.mark.parametrize("m", [1, 16])
def test_formats_small(fmt, dtype, m):
    a, qw = util.make_dense(m, 512, 512, fmt, dtype, seed=1)
    out = run_gemm(a, qw)
    assert out.dtype == dtype and tuple(out.shape) == (m, 512)
    check(out, mo.dense_reference(a, qw.deq))


@pytest.mark.parametrize("fmt,gs", [("u4b8", -1), ("u4b8", 32), ("u4b8", 64), ("u4", -1), ("u4", 64),
                                    ("u8b128", -1), ("u8b128", 128), ("u8", 32), ("fp8", -1), ("fp8", 128)])
def test_group_sizes(fmt, gs):
    a, qw = util.make_dense(8, 256, 256, fmt, torch.float16, group_size=gs, seed=2)
    check(run_gemm(a, qw), mo.dense_reference(a, qw.deq))


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 15, 16, 17, 24, 33, 48, 64, 100, 128, 257])
def test_odd_m(m):
    a, qw = util.make_dense(m, 512, 768, "u4b8", torch.float16, seed=3)
    check(run_gemm(a, qw), mo.dense_reference(a, qw.deq))


@pytest.mark.parametrize("n", [64, 128, 192, 256, 320, 384, 640, 832, 1152])
@pytest.mark.parametrize("fmt", ["u4b8", "u8b128", "mxfp4"])
def test_alignment_n(n, fmt):
    a, qw = util.make_dense(5, 256, n, fmt, torch.float16, seed=4)
    check(run_gemm(a, qw), mo.dense_reference(a, qw.deq))


@pytest.mark.parametrize("k", [32, 64, 96, 160, 2048 + 32])
def test_short_and_ragged_k(k):
    a, qw = util.make_dense(4, k, 256, "u4b8", torch.float16, group_size=32, seed=5)
    check(run_gemm(a, qw), mo.dense_reference(a, qw.deq))


@pytest.mark.parametrize("fmt", ["u4b8", "u4", "nvfp4"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bias(fmt, dtype):
    a, qw = util.make_dense(6, 256, 512, fmt, dtype, seed=6)
    bias = (torch.randn(512, generator=torch.Generator().manual_seed(7)) * 0.5).to(dtype)
    check(run_gemm(a, qw, bias=bias), mo.dense_reference(a, qw.deq, bias))


def test_config1_shape_fp16_u4b8():
    # first configuration of the headline benchmark: M=16, K=N=4096, group 128, seed 0
    a, qw = util.make_dense(16, 4096, 4096, "u4b8", torch.float16, seed=0)
    check(run_gemm(a, qw), mo.dense_reference(a, qw.deq))


def test_strided_a_and_preallocated_c():
    a, qw = util.make_dense(4, 256, 256, "u4b8", torch.float16, seed=8)
    big = torch.zeros(4, 512, dtype=torch.float16, device="cuda")
    big[:, :256] = a.cuda()
    av = big[:, :256]
    ops = _ops()
    d = util.to_dev(qw)
    c = torch.full((4, 256), 7.0, dtype=torch.float16, device="cuda")
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    out = ops.marlin_gemm(av, c, d.packed, None, d.scales, None, None, None, None, None, ws, qw.type_id,
                          4, 256, 256)
    assert out.data_ptr() == c.data_ptr()
    check(out, mo.dense_reference(a, qw.deq))


def test_m_zero_returns_empty():
    a, qw = util.make_dense(1, 64, 64, "u4b8", torch.float16, group_size=32, seed=9)
    d = util.to_dev(qw)
    ops = _ops()
    out = ops.marlin_gemm(a.cuda()[:0], None, d.packed, None, d.scales, None, None, None, None, None,
                          torch.empty(0, dtype=torch.int32, device="cuda"), qw.type_id, 0, 64, 64)
    assert tuple(out.shape) == (0, 64)


def test_linearity_full_size():
    """Size-independent property at a full benchmark shape: the op is linear in A."""
    k, n = 8192, 28672
    g = torch.Generator().manual_seed(11)
    q = torch.randint(0, 16, (k, n), generator=g, dtype=torch.int32)
    packed = mo.marlin_pack(q, 4).cuda()
    scales = (torch.rand(k // 128, n, generator=g) * 0.01 + 0.001).to(torch.bfloat16).cuda()
    zeros = (torch.rand(k // 128, n, generator=g) * 0.1).to(torch.bfloat16).cuda()
    a1 = torch.randn(16, k, generator=g).to(torch.bfloat16)
    a2 = torch.randn(16, k, generator=g).to(torch.bfloat16)
    ops = _ops()
    ws = torch.empty(0, dtype=torch.int32, device="cuda")

    def f(a):
        return ops.marlin_gemm(a.cuda(), None, packed, None, scales, None, None, zeros, None, None, ws,
                               mo.TYPE_U4, 16, n, k, True, False, True, True).float()

    y1, y2, y12 = f(a1), f(a2), f((a1.float() + a2.float()).to(torch.bfloat16))
    ref = y1 + y2
    # a1 + a2 is rounded to bf16 before the call: allow that rounding on top of the output rounding
    assert mo.mean_rel_err(y12.cpu(), ref.cpu()) < 2e-2
    # run-to-run determinism (the split-K reduction is ordered)
    assert torch.equal(f(a1), y1)


@pytest.mark.parametrize("m", [9, 16])
@pytest.mark.parametrize("fmt,dtype,group", [("u4b8", torch.float16, 128), ("u4", torch.bfloat16, 128),
                                             ("u4b8", torch.bfloat16, -1), ("u4", torch.float16, 1024)])
def test_large_matrix_9_to_16_rows(fmt, dtype, m, group):
    """K * N = 2^27 with 9-16 rows is served by the integer-MMA kernel (codes as bytes in tensor memory,
    activations as 7-bit digit planes): parity against (q - zero) * scale in fp32, all columns."""
    k, n = 8192, 16384
    g = torch.Generator().manual_seed(5)
    q = torch.randint(0, 16, (k, n), generator=g, dtype=torch.int32)
    packed = mo.marlin_pack(q, 4).cuda()
    ng = 1 if group == -1 else k // group
    scales = (torch.rand(ng, n, generator=g) * 0.01 + 0.001).to(dtype)
    a = torch.randn(m, k, generator=g).to(dtype)
    # a few large activations: the digit planes are relative to the row maximum
    a[:, 7] *= 40.0
    zeros = None
    if fmt == "u4":
        zeros = (torch.randint(0, 16, (ng, n), generator=g).float() * scales.float()).to(dtype)
    ops = _ops()
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    out = ops.marlin_gemm(a.cuda(), None, packed, None, scales.cuda(), None, None,
                          None if zeros is None else zeros.cuda(), None, None, ws,
                          mo.TYPE_U4 if fmt == "u4" else mo.TYPE_U4B8, m, n, k, True, False, True, zeros is not None)
    rep = k // ng
    sc = scales.cuda().float().repeat_interleave(rep, dim=0)
    w = q.cuda().float()
    if fmt == "u4":
        w = w * sc - zeros.cuda().float().repeat_interleave(rep, dim=0)
    else:
        w = (w - 8.0) * sc
    ref = a.cuda().float() @ w
    check(out, ref.cpu())


@pytest.mark.parametrize("m", [17, 64, 200, 300])
@pytest.mark.parametrize("fmt,dtype", [("u4b8", torch.float16), ("u4", torch.bfloat16), ("u8b128", torch.float16),
                                       ("fp8", torch.bfloat16), ("nvfp4", torch.float16), ("mxfp4", torch.bfloat16)])
def test_k_slices_few_column_tiles(fmt, dtype, m):
    """More than 16 rows on a matrix of four 256-column tiles: the tensor-memory kernel cuts K into slices
    (fp32 partials, summed in slice order, bias and the nvfp4 global scale applied after the sum)."""
    k, n = 4096, 1024
    a, qw = util.make_dense(m, k, n, fmt, dtype, seed=21)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(22)).to(dtype)
    out = run_gemm(a, qw, bias=bias)
    check(out, mo.dense_reference(a, qw.deq, bias=bias))
    again = run_gemm(a, qw, bias=bias)
    assert torch.equal(out, again), "the slice sum must be bit-identical from run to run"


@pytest.mark.parametrize("m,dtype", [(32, torch.float16), (130, torch.bfloat16)])
def test_stream_k_many_column_tiles(m, dtype):
    """86 column tiles on a 148-SM GPU: the (tile, chunk) units are cut into one equal range per SM, tiles
    shared by two CTAs are summed from fp32 partial tiles in CTA order (128-row tiles at 32 rows, 256-row
    tiles at 130).  Parity against (q - 8) * scale in fp32 with bias, all columns, and bit-equality of two runs."""
    k, n, group = 4096, 22016, 128
    g = torch.Generator().manual_seed(31)
    q = torch.randint(0, 16, (k, n), generator=g, dtype=torch.int32)
    packed = mo.marlin_pack(q, 4).cuda()
    scales = (torch.rand(k // group, n, generator=g) * 0.01 + 0.001).to(dtype)
    a = torch.randn(m, k, generator=g).to(dtype)
    bias = torch.randn(n, generator=g).to(dtype)
    ops = _ops()
    ws = torch.empty(0, dtype=torch.int32, device="cuda")

    def run():
        return ops.marlin_gemm(a.cuda(), None, packed, mo.permute_bias(bias).cuda(), scales.cuda(), None, None, None,
                               None, None, ws, mo.TYPE_U4B8, m, n, k)

    out = run()
    w = (q.cuda().float() - 8.0) * scales.cuda().float().repeat_interleave(group, dim=0)
    ref = a.cuda().float() @ w + bias.cuda().float()
    check(out, ref.cpu())
    assert torch.equal(out, run())


def test_k_slices_need_scratch_room():
    """The C ABI takes fewer k slices when the scratch buffer is small, down to none: all three give the
    oracle's result."""
    from marlin_v100_b200 import _lib
    lib = _lib.load()
    m, k, n = 64, 4096, 1024
    a, qw = util.make_dense(m, k, n, "u4b8", torch.float16, seed=23)
    ref = mo.dense_reference(a, qw.deq)
    d = util.to_dev(qw)
    a_d = a.cuda()
    full = lib.marlin_b200_gemm_scratch_bytes(m, n, k, 0)  # format 0 = u4b8, activation type 0 = fp16
    assert full >= 2 * m * n * 4
    stream = torch.cuda.current_stream().cuda_stream
    for nbytes in (full, 2 * m * n * 4 + 64, 1024):
        scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        c = torch.empty(m, n, dtype=torch.float16, device="cuda")
        rc = lib.marlin_b200_gemm(a_d.data_ptr(), c.data_ptr(), d.packed.data_ptr(), d.scales.data_ptr(), None, None,
                                  None, 0, 0, m, n, k, k, d.scales.shape[0], scratch.data_ptr(), nbytes, stream)
        assert rc == 0, lib.marlin_b200_last_error()
        torch.cuda.synchronize()
        check(c, ref)


@pytest.mark.parametrize("kw,match", [
    (dict(g_idx=True), "does not support act_order g_idx"),
    (dict(perm=True), "does not support act_order perm"),
    (dict(size_n=100), "size_n = 100, actual_size_n"),
    (dict(size_m=3), "Shape mismatch: a.size"),
    (dict(zp_on_b8=True), "does not support zero-point"),
])
def test_argument_errors(kw, match):
    a, qw = util.make_dense(2, 64, 64, "u4b8", torch.float16, group_size=32, seed=10)
    d = util.to_dev(qw)
    ops = _ops()
    one = torch.ones(4, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match=match):
        ops.marlin_gemm(a.cuda(), None, d.packed, None, d.scales, None, None,
                        d.scales if kw.get("zp_on_b8") else None,
                        one if kw.get("g_idx") else None, one if kw.get("perm") else None,
                        torch.empty(0, dtype=torch.int32, device="cuda"), qw.type_id,
                        kw.get("size_m", 2), kw.get("size_n", 64), 64, True, False, True,
                        bool(kw.get("zp_on_b8")))


@pytest.mark.parametrize("fmt,dtype,m,k,n,gs", [
    ("fp8", torch.bfloat16, 1, 5120, 3200, -1),      # a column shard of 25600 / 8
    ("fp8", torch.bfloat16, 32, 5120, 3200, -1),
    ("mxfp4", torch.bfloat16, 16, 1024, 3200, None),
    ("nvfp4", torch.float16, 16, 512, 320, None),
    ("u4", torch.bfloat16, 64, 1024, 832, 128),
    ("u4b8", torch.float16, 300, 512, 1152, 128),
    ("u8b128", torch.float16, 128, 512, 192, -1),
])
def test_n_not_a_multiple_of_256_takes_the_padded_path(fmt, dtype, m, k, n, gs):
    """size_n % 256 != 0 with a scratch buffer of the advertised size: the operands are copied into the
    256-column form of a matrix padded to the next multiple of 256 columns and the regular kernels run on it
    (more than the one launch of the shape-agnostic kernel), with a bias crossing the boundary as well."""
    from marlin_v100_b200 import _lib
    lib = _lib.load()
    a, qw = util.make_dense(m, k, n, fmt, dtype, group_size=gs, seed=21)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(22)) * 0.5).to(dtype)
    run_gemm(a, qw, bias=bias)   # warm-up: tensor maps, function attributes
    before = lib.marlin_b200_launch_count()
    out = run_gemm(a, qw, bias=bias)
    launches = lib.marlin_b200_launch_count() - before
    assert tuple(out.shape) == (m, n)
    check(out, mo.dense_reference(a, qw.deq, bias))
    assert launches >= 4, f"{launches} launches: the padded path did not run"
