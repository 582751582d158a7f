"""World-size-2 checks of the multi-GPU plumbing on CPU ranks (gloo): the dispatch / combine index
math of the expert-parallel layer and the column split of the dense layer, each against a
single-process computation of the same seeded problem."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from marlin_v100_b200 import parallel


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    g = torch.Generator().manual_seed(7)
    t, h, e, k = 24, 16, 8, 3
    hidden = torch.randn(t, h, generator=g)
    experts = torch.randn(e, h, h, generator=g) * 0.3
    logits = torch.randn(t, e, generator=g)
    w, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    return hidden, experts, w, ids.to(torch.int32)


def _reference(hidden, experts, w, ids):
    out = torch.zeros_like(hidden)
    for t in range(hidden.shape[0]):
        for j in range(ids.shape[1]):
            out[t] += w[t, j] * torch.tanh(hidden[t] @ experts[ids[t, j]])
    return out


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hidden, experts, w, ids = _problem()
        per_rank = experts.shape[0] // world
        # experts placed by a load table; this rank stacks the experts of its slots in slot order
        slot = parallel.balanced_expert_placement(torch.tensor([9.0, 8, 1, 1, 1, 1, 1, 1]), world)
        expert_of_slot = torch.argsort(slot)
        mine = experts[expert_of_slot[rank * per_rank:(rank + 1) * per_rank]]

        def compute(rows, local_expert, weights):
            out = torch.empty_like(rows)
            for i in range(rows.shape[0]):
                out[i] = weights[i] * torch.tanh(rows[i] @ mine[int(local_expert[i])])
            return out

        layer = parallel.ExpertParallelMoE(compute, experts.shape[0], expert_slot=slot)
        tok = hidden.shape[0] // world
        sl = slice(rank * tok, (rank + 1) * tok)
        out = layer.forward(hidden[sl], w[sl], ids[sl])
        ref = _reference(hidden, experts, w, ids)[sl]
        ok_moe = torch.allclose(out, ref, atol=1e-5)
        # an expert id outside the table on ONE rank: both ranks raise before the row exchange
        bad = ids[sl].clone()
        if rank == 1:
            bad[0, 0] = experts.shape[0]
        try:
            layer.forward(hidden[sl], w[sl], bad)
            ok_moe = False
        except RuntimeError as err:
            ok_moe = ok_moe and "outside" in str(err)

        # dense column split
        g = torch.Generator().manual_seed(3)
        x = torch.randn(5, 32, generator=g)
        wt = torch.randn(32, 256, generator=g)
        lo, hi = parallel.column_slice(256, rank, world)
        dense = parallel.ColumnParallelMarlinLinear(lambda a, o: o.copy_(a @ wt[:, lo:hi]), 256)
        ok_dense = torch.allclose(dense.forward(x), x @ wt, atol=1e-5)
        results[rank] = (ok_moe, ok_dense)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_expert_parallel_and_column_parallel_world2():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: (True, True), 1: (True, True)}


def test_single_process_paths():
    hidden, experts, w, ids = _problem()

    def compute(rows, local_expert, weights):
        return torch.stack([weights[i] * torch.tanh(rows[i] @ experts[int(local_expert[i])])
                            for i in range(rows.shape[0])])

    layer = parallel.ExpertParallelMoE(compute, experts.shape[0])
    assert torch.allclose(layer.forward(hidden, w, ids), _reference(hidden, experts, w, ids), atol=1e-5)
    with pytest.raises(ValueError):
        parallel.column_slice(192, 0, 4)
    assert parallel.column_slice(512, 1, 4) == (128, 256)


def test_dispatch_plan_orders_routes_by_slot():
    ids = torch.tensor([[5, 0], [2, 7], [1, 6]], dtype=torch.int32)
    w = torch.arange(6, dtype=torch.float32).reshape(3, 2)
    plan = parallel.make_dispatch_plan(ids, w, experts_per_rank=8, world=1)
    assert plan.order.tolist() == [1, 4, 2, 0, 5, 3]
    assert plan.local_expert.tolist() == [0, 1, 2, 5, 6, 7]
    assert plan.weights.tolist() == [1.0, 4.0, 2.0, 0.0, 5.0, 3.0]
    assert plan.send_counts == [6] and plan.recv_counts == [6]
    # a placement table: expert e lives in slot 7 - e
    slot = torch.arange(7, -1, -1, dtype=torch.int32)
    plan = parallel.make_dispatch_plan(ids, w, experts_per_rank=8, world=1, expert_slot=slot)
    assert plan.order.tolist() == [3, 5, 0, 2, 4, 1]
    assert plan.local_expert.tolist() == [0, 1, 2, 5, 6, 7]


def test_dispatch_plan_rejects_ids_outside_the_table():
    w = torch.ones(2, 2)
    for bad in (8, -1):
        plan = parallel.make_dispatch_plan(torch.tensor([[0, bad], [1, 2]], dtype=torch.int32), w, 8, 1)
        with pytest.raises(RuntimeError, match="outside"):
            plan.send_counts


def test_balanced_expert_placement():
    load = torch.tensor([10.0, 9.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0])
    slot = parallel.balanced_expert_placement(load, 2)
    assert sorted(slot.tolist()) == list(range(8))
    per_rank = [sum(float(load[e]) for e in range(8) if int(slot[e]) // 4 == r) for r in range(2)]
    assert max(per_rank) <= 13.0          # contiguous shards would put 21 of 25 on rank 0
    assert int(slot[0]) // 4 != int(slot[1]) // 4
    with pytest.raises(ValueError):
        parallel.balanced_expert_placement(load, 3)
    with pytest.raises(ValueError):
        parallel.ExpertParallelMoE(lambda *a: None, 8, expert_slot=torch.zeros(8, dtype=torch.int32))
