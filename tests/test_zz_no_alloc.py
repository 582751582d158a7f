"""The allocation-free dense GEMM entry point (scratch inside the library image).

Some callers of this library cannot allocate device memory at the point where they run a GEMM: a
serving runtime with a memory plan fixed at start-up, a plugin that receives tensors but no
allocator, host code that runs while somebody else captures the stream.  For them
`marlin_b200_gemm_static_scratch` keeps the split-K partial sums in a fixed array of the loaded
library.  The test calls it twice in a row through the C ABI and compares with the regular entry
point (caller-provided scratch) on the same inputs: both run the same kernels in the same order, so
the outputs must be bit-identical; the oracle tolerance is checked as well.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test."""
import pytest
import torch

from oracle import marlin_oracle as mo
from tests import util

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt,dtype,m", [("u4b8", torch.float16, 16), ("u4", torch.bfloat16, 5)])
def test_static_scratch_matches_regular_entry_point(fmt, dtype, m):
    from marlin_v100_b200 import _lib
    lib = _lib.load()
    # 2048 x 2560: ten column groups of 256 over 32 chunks = 320 units on 148 SMs, so the column
    # groups are split across CTAs and the partial sums really go through the scratch
    k, n = 2048, 2560
    a, qw = util.make_dense(m, k, n, fmt, dtype, seed=21)
    d = util.to_dev(qw)
    a_dev = a.cuda()
    act = 0 if dtype == torch.float16 else 1
    fmt_code = lib.marlin_b200_format_from_type_id(qw.type_id, 0)
    stream = torch.cuda.current_stream().cuda_stream
    groups = d.scales.shape[0]
    zeros = None if d.zeros is None else d.zeros.data_ptr()

    nbytes = lib.marlin_b200_gemm_scratch_bytes(m, n, k, fmt_code)
    assert nbytes > 0
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    ref_out = torch.empty(m, n, dtype=dtype, device="cuda")
    _lib.check(lib.marlin_b200_gemm(a_dev.data_ptr(), ref_out.data_ptr(), d.packed.data_ptr(), d.scales.data_ptr(),
                                    zeros, None, None, act, fmt_code, m, n, k, a_dev.stride(0), groups,
                                    scratch.data_ptr(), nbytes, stream))
    outs = []
    for _ in range(2):  # two calls in a row share the built-in array
        out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        before = torch.cuda.memory_allocated()
        _lib.check(lib.marlin_b200_gemm_static_scratch(a_dev.data_ptr(), out.data_ptr(), d.packed.data_ptr(),
                                                       d.scales.data_ptr(), zeros, None, None, act, fmt_code, m, n,
                                                       k, a_dev.stride(0), groups, stream))
        assert torch.cuda.memory_allocated() == before
        outs.append(out)
    torch.cuda.synchronize()
    for out in outs:
        assert torch.equal(out, ref_out)
        assert mo.within_tolerance(out.cpu(), mo.dense_reference(a, qw.deq))


def _random_problem(m, k, n, dtype, seed):
    """Random codes and scales made on the device: the comparison below is between two entry points
    of the library, so no oracle (and no CPU quantiser) is needed."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(m, k, generator=g, device="cuda").to(dtype)
    packed = torch.randint(-2**31, 2**31 - 1, (k // 16, n * 2), generator=g, device="cuda", dtype=torch.int32)
    scales = (torch.rand(k // 128, n, generator=g, device="cuda") * 0.01 + 0.002).to(dtype)
    return a, packed, scales


# (m, k, n): the M > 16 kernel cutting K into slices that fit the built-in 6 MiB; a shape where no cut
# fits (whole tiles); 12 rows on a matrix of 2^27 weights (the integer-MMA kernel: its digit planes sit
# behind the partial sums in the scratch)
@pytest.mark.parametrize("m,k,n", [(64, 4096, 4096), (64, 4096, 22016), (12, 8192, 16384)])
def test_static_scratch_larger_shapes(m, k, n):
    from marlin_v100_b200 import _lib
    lib = _lib.load()
    dtype = torch.float16
    a, packed, scales = _random_problem(m, k, n, dtype, seed=m + n)
    stream = torch.cuda.current_stream().cuda_stream
    six_mib = 6 << 20
    scratch = torch.empty(six_mib, dtype=torch.uint8, device="cuda")
    ref_out = torch.empty(m, n, dtype=dtype, device="cuda")
    _lib.check(lib.marlin_b200_gemm(a.data_ptr(), ref_out.data_ptr(), packed.data_ptr(), scales.data_ptr(), None,
                                    None, None, 0, 0, m, n, k, k, k // 128, scratch.data_ptr(), six_mib, stream))
    for _ in range(2):
        out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        before = torch.cuda.memory_allocated()
        _lib.check(lib.marlin_b200_gemm_static_scratch(a.data_ptr(), out.data_ptr(), packed.data_ptr(),
                                                       scales.data_ptr(), None, None, None, 0, 0, m, n, k, k,
                                                       k // 128, stream))
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert torch.equal(out, ref_out)
    assert not torch.isnan(ref_out.float()).any()


def test_static_scratch_refuses_what_does_not_fit():
    """K so large that the M <= 16 kernels' fixed need (SMs * 32 KiB + 48 * K + 256) passes 6 MiB."""
    from marlin_v100_b200 import _lib
    lib = _lib.load()
    m, k, n = 4, 65536, 256
    a, packed, scales = _random_problem(m, k, n, torch.float16, seed=5)
    out = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    rc = lib.marlin_b200_gemm_static_scratch(a.data_ptr(), out.data_ptr(), packed.data_ptr(), scales.data_ptr(),
                                             None, None, None, 0, 0, m, n, k, k, k // 128,
                                             torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    msg = lib.marlin_b200_last_error()
    assert b"built-in scratch holds 6291456 bytes" in msg and b"marlin_b200_gemm" in msg


def test_static_scratch_argument_error_is_reported():
    from marlin_v100_b200 import _lib
    lib = _lib.load()
    rc = lib.marlin_b200_gemm_static_scratch(None, None, None, None, None, None, None, 0, 0, 1, 100, 64, 64, 1, None)
    assert rc == -1 and b"size_n % 64 == 0" in lib.marlin_b200_last_error()
