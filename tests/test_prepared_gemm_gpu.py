"""The prepared-call form of the dense GEMM gives the same bits as the operator call."""
import pytest
import torch

from oracle import marlin_oracle as mo
from tests import util

pytestmark = pytest.mark.gpu


def test_prepared_gemm_matches_operator_call():
    from marlin_v100_b200 import ops
    a, qw = util.make_dense(16, 512, 512, "u4", torch.bfloat16, 128)
    d = util.to_dev(qw)
    a = a.cuda()
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    ref = ops.marlin_gemm(a, None, d.packed, None, d.scales, None, None, d.zeros, None, None, ws, qw.type_id,
                          16, 512, 512, True, False, True, True)
    plan = ops.PreparedGemm(a, None, d.packed, None, d.scales, None, d.zeros, qw.type_id, 16, 512, 512, True)
    out1 = plan().clone()
    a.mul_(2.0)          # same buffers, new contents: the plan reads them at call time
    out2 = plan().clone()
    torch.cuda.synchronize()
    assert torch.equal(out1, ref)
    assert mo.mean_rel_err(out2.float().cpu(), 2.0 * ref.float().cpu()) < 1e-2
    with pytest.raises(RuntimeError):
        ops.PreparedGemm(a, None, d.packed, None, d.scales, None, d.zeros, qw.type_id, 16, 500, 512, True)


def test_host_pipelined_gemm_matches_operator_call():
    from marlin_v100_b200 import ops
    a, qw = util.make_dense(16, 512, 512, "u4b8", torch.float16, 128)
    d = util.to_dev(qw)
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    pipe = ops.HostPipelinedGemm([dict(packed=d.packed, scales=d.scales)], qw.type_id, 16, 512, 512, torch.float16,
                                 torch.device("cuda", torch.cuda.current_device()), depth=2)
    g = torch.Generator().manual_seed(9)
    ins = [torch.randn(16, 512, generator=g).to(torch.float16).pin_memory() for _ in range(5)]
    outs = [torch.empty(16, 512, dtype=torch.float16).pin_memory() for _ in range(5)]
    for x, y in zip(ins, outs):            # more calls than slots: the slots are reused
        pipe.submit(x, y)
    pipe.synchronize()
    for x, y in zip(ins, outs):
        ref = ops.marlin_gemm(x.cuda(), None, d.packed, None, d.scales, None, None, None, None, None, ws,
                              qw.type_id, 16, 512, 512)
        assert torch.equal(y, ref.cpu())


def test_host_pipeline_captured_in_a_graph():
    """The same pipelined calls captured once and replayed: every replay copies the activations in and the
    results out again, so a changed host buffer shows in the next replay."""
    from marlin_v100_b200 import ops
    a, qw = util.make_dense(16, 512, 512, "u4b8", torch.float16, 128)
    d = util.to_dev(qw)
    prepared = ops.prepare_weights(d.packed, 512, 512, 4)
    ws = torch.empty(0, dtype=torch.int32, device="cuda")
    layers = [dict(packed=d.packed, scales=d.scales), dict(packed=prepared, scales=d.scales)]
    pipe = ops.HostPipelinedGemm(layers, qw.type_id, 16, 512, 512, torch.float16,
                                 torch.device("cuda", torch.cuda.current_device()), depth=3)
    x = torch.randn(16, 512, generator=torch.Generator().manual_seed(3)).to(torch.float16).pin_memory()
    y = torch.empty(16, 512, dtype=torch.float16).pin_memory()
    graph = pipe.capture(x, y, [0, 1, 0, 1, 0])          # five calls, the last one on layer 0
    for scale in (1.0, 0.5):
        x.mul_(scale)
        graph.replay()
        torch.cuda.synchronize()
        ref = ops.marlin_gemm(x.cuda(), None, d.packed, None, d.scales, None, None, None, None, None, ws,
                              qw.type_id, 16, 512, 512)
        assert torch.equal(y, ref.cpu())
    # the eager form still works afterwards
    pipe.submit(x, y, layer=1)
    pipe.synchronize()
    ref = ops.marlin_gemm(x.cuda(), None, prepared, None, d.scales, None, None, None, None, None, ws, qw.type_id,
                          16, 512, 512)
    assert torch.equal(y, ref.cpu())
