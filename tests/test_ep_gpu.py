"""Expert-parallel layer on GPUs: world size 1 must equal the plain fused layer; with two or more
GPUs a torchrun job checks the NCCL dispatch / combine against the CPU oracle."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from oracle import marlin_oracle as mo
from tests import util

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_world1_equals_fused_layer():
    from marlin_v100_b200 import fused_moe, parallel
    e, k, hdim, inter, t = 8, 2, 256, 128, 40
    g = torch.Generator().manual_seed(2)
    hidden = torch.randn(t, hdim, generator=g).to(torch.float16)
    logits = torch.randn(t, e, generator=g)
    w13 = util.make_experts(e, hdim, 2 * inter, "u4b8", torch.float16, seed=3, scale=0.05)
    w2 = util.make_experts(e, inter, hdim, "u4b8", torch.float16, seed=4, scale=0.05)
    d13, d2 = util.to_dev(w13), util.to_dev(w2)
    tw, ids, _ = fused_moe.fused_topk(logits.cuda(), k, True)
    layer = parallel.ExpertParallelMoE.from_marlin_weights(d13.packed, d2.packed, d13.scales, d2.scales,
                                                           w13.type_id, e)
    out = layer.forward(hidden.cuda(), tw, ids)
    rtw, rids, _ = mo.topk_softmax_reference(logits, k, True)
    ref = mo.moe_reference(hidden, w13.deq, w2.deq, rtw, rids, round_dtype=torch.float16)
    assert mo.within_tolerance(out.cpu(), ref)


def test_peer_arena_single_rank():
    """World size 1: the peer-memory kernels run against this rank's own arena (every flag is its own)."""
    from marlin_v100_b200 import fused_moe, parallel
    e, k, hdim, inter, t = 8, 2, 256, 128, 24
    g = torch.Generator().manual_seed(2)
    hidden = torch.randn(t, hdim, generator=g).to(torch.float16)
    logits = torch.randn(t, e, generator=g)
    w13 = util.make_experts(e, hdim, 2 * inter, "u4b8", torch.float16, seed=3, scale=0.05)
    w2 = util.make_experts(e, inter, hdim, "u4b8", torch.float16, seed=4, scale=0.05)
    d13, d2 = util.to_dev(w13), util.to_dev(w2)
    tw, ids, _ = fused_moe.fused_topk(logits.cuda(), k, True)
    layer = parallel.ExpertParallelMoE.from_marlin_weights(d13.packed, d2.packed, d13.scales, d2.scales,
                                                           w13.type_id, e)
    want = layer.forward(hidden.cuda(), tw, ids)
    layer.enable_peer_memory(t * k, hdim, torch.float16)
    for _ in range(3):
        got = layer.forward(hidden.cuda(), tw, ids)
        assert torch.equal(got, want)
    assert layer.arena.status() == (0, 3)
    bad = ids.clone()
    bad[1, 1] = e + 3
    with pytest.raises(RuntimeError, match="outside"):
        layer.forward(hidden.cuda(), tw, bad)
    assert torch.equal(layer.forward(hidden.cuda(), tw, ids), want)
    # a buffer too small for the step is reported, not overrun
    small = parallel.ExpertParallelMoE.from_marlin_weights(d13.packed, d2.packed, d13.scales, d2.scales,
                                                           w13.type_id, e)
    small.enable_peer_memory(t * k - 8, hdim, torch.float16)
    with pytest.raises(RuntimeError, match="status 16"):
        small.forward(hidden.cuda(), tw, ids)
    small.close()
    layer.close()


def _run_worker(script: str, n: int):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                           "--master-addr", "127.0.0.1", "--master-port", str(port),
                           os.path.join(ROOT, "tests", script)], capture_output=True, text=True, env=env, timeout=600)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_multi_gpu_column_parallel_peer_gather():
    r = _run_worker("tp_worker.py", min(torch.cuda.device_count(), 4))
    assert r.returncode == 0 and "TP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_multi_gpu_dispatch_combine():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", str(port),
                        os.path.join(ROOT, "tests", "ep_worker.py")], capture_output=True, text=True, env=env,
                       timeout=600)
    assert r.returncode == 0 and "EP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
