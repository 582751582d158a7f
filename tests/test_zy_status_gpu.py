"""After the other GPU tests of the session no pipelined kernel may have given up on a wait."""
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu


def test_no_kernel_gave_up_on_a_wait():
    from marlin_v100_b200 import ops
    # one call through each pipelined kernel family, then the status word
    for m in (4, 16, 200):
        a, qw = util.make_dense(m, 512, 512, "u4b8", torch.float16, 128)
        d = util.to_dev(qw)
        ws = torch.empty(0, dtype=torch.int32, device="cuda")
        ops.marlin_gemm(a.cuda(), None, d.packed, None, d.scales, None, None, None, None, None, ws, qw.type_id,
                        m, 512, 512)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
