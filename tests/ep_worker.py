"""Worker of the multi-GPU expert-parallel check: launched with torchrun, one rank per GPU.
Every rank builds the same seeded layer on the CPU, keeps its expert shard and its token shard,
runs the expert-parallel layer (NCCL all-to-all dispatch / combine around the local fused expert
layer) and compares its tokens with the CPU oracle of the whole layer."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import marlin_oracle as mo  # noqa: E402
from tests import util  # noqa: E402
from marlin_v100_b200 import fused_moe, parallel  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    fmt, dtype = "mxfp4", torch.bfloat16
    e, k, hdim, inter, tokens = 8 * world, 4, 256, 128, 32 * world
    g = torch.Generator().manual_seed(5)
    hidden = torch.randn(tokens, hdim, generator=g).to(dtype)
    # a skewed router: the first experts draw most routes, so contiguous shards would load rank 0 most
    logits = torch.randn(tokens, e, generator=g) + torch.linspace(2.0, -2.0, e)
    w13 = util.make_experts(e, hdim, 2 * inter, fmt, dtype, seed=6, scale=0.05)
    w2 = util.make_experts(e, inter, hdim, fmt, dtype, seed=7, scale=0.05)
    per = e // world
    # experts placed by expected load; this rank stacks the experts of its slots in slot order
    slot = parallel.balanced_expert_placement(torch.softmax(logits, -1).sum(0), world)
    sl_e = torch.argsort(slot)[rank * per:(rank + 1) * per]
    tok = tokens // world
    sl_t = slice(rank * tok, (rank + 1) * tok)
    dev = "cuda"
    layer = parallel.ExpertParallelMoE.from_marlin_weights(
        w13.packed[sl_e].to(dev), w2.packed[sl_e].to(dev), w13.scales[sl_e].to(dev), w2.scales[sl_e].to(dev),
        w13.type_id, e, expert_slot=slot)
    tw, ids, _ = fused_moe.fused_topk(logits[sl_t].to(dev), k, True)
    out = layer.forward(hidden[sl_t].to(dev), tw, ids)
    torch.cuda.synchronize()
    rtw, rids, _ = mo.topk_softmax_reference(logits, k, True)
    ref = mo.moe_reference(hidden, w13.deq, w2.deq, rtw, rids, round_dtype=dtype)[sl_t]
    ok = torch.equal(ids.cpu(), rids[sl_t]) and mo.within_tolerance(out.cpu(), ref)
    # the placement must spread the routes: no rank receives more than 1.5x its even share
    ok = ok and layer.last_recv_rows <= 1.5 * tokens * k / world
    why = "" if ok else "collective transport; "

    # the same layer over peer-mapped memory: same bits, step after step
    layer.enable_peer_memory(tokens * k, hdim, dtype)
    for step in range(3):
        out_peer = layer.forward(hidden[sl_t].to(dev), tw, ids)
        torch.cuda.synchronize()
        if not torch.equal(out_peer, out):
            ok, why = False, why + f"peer transport differs at step {step}; "
    # an expert id outside the table on ONE rank: every rank raises, and the next step still works
    bad = ids.clone()
    if rank == world - 1:
        bad[0, 0] = e
    try:
        layer.forward(hidden[sl_t].to(dev), tw, bad)
        ok, why = False, why + "invalid id not reported; "
    except RuntimeError as err:
        if "outside" not in str(err):
            ok, why = False, why + f"unexpected error {err}; "
    out_peer = layer.forward(hidden[sl_t].to(dev), tw, ids)
    torch.cuda.synchronize()
    if not torch.equal(out_peer, out) or layer.arena.status()[0] != 0:
        ok, why = False, why + "step after the refused one differs; "
    layer.close()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EP_OK" if int(flag) == 1 else f"EP_FAIL mean_rel={mo.mean_rel_err(out.cpu(), ref):.3e}", flush=True)
    if why:
        print(f"rank {rank}: {why}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
