"""Repack parity: bit-exact against the oracle / the stored reference outputs, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from oracle import marlin_oracle as mo

pytestmark = pytest.mark.gpu

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_helpers.npz"))


def _ops():
    from marlin_v100_b200 import ops
    return ops


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("k,n", [(32, 64), (48, 128), (32, 192), (64, 256), (32, 320), (32, 512), (16, 768)])
def test_repack_matches_reference_fixture(bits, k, n):
    ops = _ops()
    tag = f"layout_b{bits}_k{k}_n{n}"
    exp = torch.from_numpy(G[tag + "_packed"].copy())
    got = ops.gptq_marlin_repack(torch.from_numpy(G[tag + "_gptq"].copy()).cuda(),
                                 torch.empty(0, dtype=torch.int32, device="cuda"), k, n, bits)
    assert torch.equal(got.cpu(), exp)
    got = ops.awq_marlin_repack(torch.from_numpy(G[tag + "_awq"].copy()).cuda(), k, n, bits)
    assert torch.equal(got.cpu(), exp)


@pytest.mark.parametrize("name,bits", [("u4b8", 4), ("u8b128", 8)])
@pytest.mark.parametrize("act", [0, 1])
def test_deterministic_known_answer(name, bits, act):
    ops = _ops()
    tag = f"repack_{name}_act{act}"
    perm = torch.from_numpy(G[tag + "_perm"].copy()).cuda() if act else torch.empty(0, dtype=torch.int32, device="cuda")
    got = ops.gptq_marlin_repack(torch.from_numpy(G[tag + "_gptq_in"].copy()).cuda(), perm, 128, 128, bits)
    assert torch.equal(got.cpu(), torch.from_numpy(G[tag + "_expected"].copy()))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("k,n", [(4096, 4096), (1024, 3200), (512, 28672)])
def test_repack_large_random(bits, k, n):
    ops = _ops()
    g = torch.Generator().manual_seed(k + n + bits)
    q = torch.randint(0, 1 << bits, (k, n), generator=g, dtype=torch.int32)
    exp = mo.marlin_pack(q, bits)
    got = ops.gptq_marlin_repack(mo.gptq_pack(q, bits).cuda(), torch.empty(0, dtype=torch.int32, device="cuda"), k, n, bits)
    assert torch.equal(got.cpu(), exp)
    got = ops.awq_marlin_repack(mo.awq_pack(q, bits).cuda(), k, n, bits)
    assert torch.equal(got.cpu(), exp)
    # unpack(packed) == q : the layout round trip, independent of the packer
    assert torch.equal(mo.marlin_unpack(got.cpu(), k, n, bits), q)


def test_repack_act_order_random():
    ops = _ops()
    k, n, bits = 256, 512, 4
    g = torch.Generator().manual_seed(5)
    q = torch.randint(0, 16, (k, n), generator=g, dtype=torch.int32)
    perm = torch.randperm(k, generator=g).to(torch.int32)
    exp = mo.gptq_marlin_repack(mo.gptq_pack(q, bits), perm, k, n, bits)
    got = ops.gptq_marlin_repack(mo.gptq_pack(q, bits).cuda(), perm.cuda(), k, n, bits)
    assert torch.equal(got.cpu(), exp)


def test_repack_errors():
    ops = _ops()
    w = torch.zeros((16, 64), dtype=torch.int32, device="cuda")
    e = torch.empty(0, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="not divisible by tile_k_size"):
        ops.gptq_marlin_repack(w, e, 120, 64, 4)
    with pytest.raises(RuntimeError, match="not divisible by tile_n_size"):
        ops.gptq_marlin_repack(w, e, 128, 96, 4)
    with pytest.raises(RuntimeError, match="num_bits must be 4 or 8"):
        ops.gptq_marlin_repack(w, e, 128, 64, 3)
    with pytest.raises(RuntimeError, match="Shape mismatch"):
        ops.awq_marlin_repack(w, 128, 64, 4)
