"""Worker of the multi-GPU column-parallel check: launched with torchrun, one rank per GPU.  Every rank
quantises its own column slice of the same seeded weight, runs the dense layer with the peer-memory
all-gather (eagerly and as a captured graph that is replayed) and compares all columns with the CPU oracle
and with the NCCL form of the same layer."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import marlin_oracle as mo  # noqa: E402
from tests import util  # noqa: E402
from marlin_v100_b200 import ops, parallel  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dtype, m, k, n = torch.bfloat16, 12, 1024, 512 * world
    g = torch.Generator().manual_seed(21)
    w = (torch.randn(k, n, generator=g) * 0.02).to(dtype)
    xs = [torch.randn(m, k, generator=g).to(dtype) for _ in range(4)]
    lo, hi = parallel.column_slice(n, rank, world)
    qw = util.quantize(w[:, lo:hi].contiguous(), "u4b8", 128)
    d = util.to_dev(qw)
    ws = torch.empty(0, dtype=torch.int32, device="cuda")

    def gemm(x, out):
        ops.marlin_gemm(x, out, d.packed, None, d.scales, None, None, None, None, None, ws, qw.type_id,
                        x.shape[0], hi - lo, k, True, False, True, False)

    # reference: every rank's slice dequantised by the oracle
    deq = [None] * world
    dist.all_gather_object(deq, qw.deq)
    w_deq = torch.cat(deq, dim=1)
    ok, why = True, ""
    nccl = parallel.ColumnParallelMarlinLinear(gemm, n)
    peer = parallel.ColumnParallelMarlinLinear(gemm, n, use_peer_memory=True, max_m=16, dtype=dtype)
    for i, x in enumerate(xs):
        got = peer.forward(x.cuda()).clone()
        want = nccl.forward(x.cuda())
        torch.cuda.synchronize()
        if not torch.equal(got, want):
            ok, why = False, why + f"eager step {i} differs from the collective form; "
        if not mo.within_tolerance(got.cpu(), mo.dense_reference(x, w_deq)):
            ok, why = False, why + f"eager step {i} outside tolerance; "
    # captured: three steps per graph, replayed twice (the step counter lives on the device)
    x_dev = xs[0].cuda()
    keep = torch.empty((3, m, n), dtype=dtype, device="cuda")
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for j in range(3):
                keep[j].copy_(peer.forward(x_dev))
    for _ in range(2):
        dist.barrier()
        graph.replay()
        torch.cuda.synchronize()
        want = nccl.forward(x_dev)
        for j in range(3):
            if not torch.equal(keep[j], want):
                ok, why = False, why + f"replayed step {j} differs; "
    if peer.arena.status()[0] != 0:
        ok, why = False, why + f"arena status {peer.arena.status()}; "
    peer.arena.close()
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if why:
        print(f"rank {rank}: {why}", flush=True)
    if rank == 0:
        print("TP_OK" if int(flag) == 1 else "TP_FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
