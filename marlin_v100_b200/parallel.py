"""Multi-GPU layouts of the Marlin path: one process per GPU, `torch.distributed` for the plumbing.

The reference has no distributed code (`vllm/distributed/__init__.py:4-25` is a world-size-1 stub);
what it offers are the hooks this module builds on: `expert_map` / zero-filled rows in the fused
expert layer (`fused_marlin_moe.py:170-171`, `csrc/moe/moe_align_sum_kernels.cu:129-133`) and an op
whose output columns are independent (`csrc/quantization/marlin/marlin.cu:356-359`: any column count
that is a multiple of 64 is legal).

* `ColumnParallelMarlinLinear`: N is cut into `world` contiguous slices; every rank quantises /
  repacks its own slice (the packed layout depends on `size_n`), runs the local GEMM into its part of
  a `[world, M, N/world]` buffer and the ranks all-gather in place.
* `ExpertParallelMoE`: tokens are data-parallel, experts are sharded contiguously.  Routing is local;
  one all-to-all of row counts, one of rows (+ local expert id and router weight per row) to the ranks
  that own the experts, the local fused expert layer with top_k = 1, one all-to-all back, and the
  top-k contributions of every token are summed where the token lives.

Both classes take a `compute` callable so the index plumbing can be exercised on CPU ranks (gloo)
with a plain PyTorch stand-in; on GPUs the default is the CUDA library.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


# --------------------------------------------------------------------------------------------------
# dense: column split + all-gather
# --------------------------------------------------------------------------------------------------

def column_slice(n: int, rank: int, world: int) -> tuple[int, int]:
    """Columns [lo, hi) owned by `rank`; every slice must keep the op's N % 64 == 0 contract."""
    if n % world or (n // world) % 64:
        raise ValueError(f"N = {n} cannot be split over {world} ranks in multiples of 64 columns")
    per = n // world
    return rank * per, (rank + 1) * per


class ColumnParallelMarlinLinear:
    """y[M, N] = x[M, K] @ W[K, N] with W's columns sharded over the ranks of `group`."""

    def __init__(self, gemm: Callable[[torch.Tensor, torch.Tensor], None], n_total: int, group=None):
        """`gemm(x, out_slice)` runs this rank's local GEMM into `out_slice` [M, N/world]."""
        self.gemm, self.n_total, self.group = gemm, n_total, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.lo, self.hi = column_slice(n_total, self.rank, self.world)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        m = x.shape[0]
        per = self.hi - self.lo
        gathered = torch.empty((self.world, m, per), dtype=x.dtype, device=x.device)
        self.gemm(x, gathered[self.rank])
        if self.world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), gathered[self.rank].reshape(-1), group=self.group)
        # [world, M, per] -> [M, world * per]
        return gathered.permute(1, 0, 2).reshape(m, self.n_total)


# --------------------------------------------------------------------------------------------------
# MoE: expert parallel dispatch / combine
# --------------------------------------------------------------------------------------------------

class DispatchPlan:
    """Routes of this rank sorted by the rank that owns their expert.  The row counts per destination are
    exchanged with an asynchronous all-to-all that is started first; `send_counts` / `recv_counts` (the
    one host synchronisation of the layer) are only resolved when they are first read, so the caller can
    put more device work (the row gather) in front of that synchronisation."""

    def __init__(self, order, local_expert, weights, send, recv, work):
        self.order = order                # [T*k] route indices sorted by destination rank (stable)
        self.local_expert = local_expert  # [T*k] expert id inside the destination rank, in `order` order
        self.weights = weights            # [T*k] router weight, in `order` order
        self._send, self._recv, self._work, self._counts = send, recv, work, None

    def _resolve(self):
        if self._counts is None:
            if self._work is not None:
                self._work.wait()
            self._counts = torch.stack((self._send, self._recv)).tolist()
        return self._counts

    @property
    def send_counts(self) -> list[int]:   # rows sent to each rank
        return self._resolve()[0]

    @property
    def recv_counts(self) -> list[int]:   # rows received from each rank
        return self._resolve()[1]


def make_dispatch_plan(topk_ids: torch.Tensor, topk_weights: torch.Tensor, experts_per_rank: int, world: int,
                       group=None) -> DispatchPlan:
    """Sorts the (token, route) pairs by the rank that owns their expert and exchanges the counts."""
    flat = topk_ids.reshape(-1).to(torch.int64)
    dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
    send = torch.bincount(dest, minlength=world)[:world]
    recv = torch.empty_like(send)
    work = None
    if world > 1:
        work = dist.all_to_all_single(recv, send, group=group, async_op=True)
    else:
        recv.copy_(send)
    order = torch.sort(dest, stable=True).indices
    local_expert = (flat - dest * experts_per_rank)[order].to(torch.int32)
    return DispatchPlan(order, local_expert, topk_weights.reshape(-1)[order].to(torch.float32), send, recv, work)


def _all_to_all_rows(rows: torch.Tensor, send_counts: list[int], recv_counts: list[int], group) -> torch.Tensor:
    out = torch.empty((sum(recv_counts),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=group)
    else:
        out.copy_(rows)
    return out


class ExpertParallelMoE:
    """Fused expert layer with the experts sharded over the ranks of `group`.

    compute(rows [R, H], local_expert int32 [R], weights fp32 [R]) -> [R, H] must return, for every
    received row, weight * expert(local_expert)(row).  The default built by `from_marlin_weights`
    runs moe_align_block_size + the two grouped GEMMs + SiLU-and-mul of the CUDA library with
    top_k = 1."""

    def __init__(self, compute: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
                 num_experts: int, group=None):
        self.compute, self.num_experts, self.group = compute, num_experts, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts cannot be sharded evenly over {self.world} ranks")
        self.experts_per_rank = num_experts // self.world

    @classmethod
    def from_marlin_weights(cls, w13, w2, w13_scale, w2_scale, quant_type_id: int, num_experts: int, group=None,
                            w13_zeros=None, w2_zeros=None, global_scale1=None, global_scale2=None):
        """w13 / w2: this rank's experts ([E/world, ...]) in the packed layout of the grouped GEMM."""
        from . import fused_moe

        def compute(rows, local_expert, weights):
            if rows.shape[0] == 0:
                return rows.new_empty(rows.shape)
            return fused_moe.fused_marlin_moe(rows, w13, w2, None, None, w13_scale, w2_scale,
                                              weights.reshape(-1, 1).contiguous(), local_expert.reshape(-1, 1).contiguous(),
                                              quant_type_id, global_scale1=global_scale1, global_scale2=global_scale2,
                                              w1_zeros=w13_zeros, w2_zeros=w2_zeros)

        return cls(compute, num_experts, group)

    def forward(self, hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        """hidden [T, H] (this rank's tokens), topk_* [T, k] with GLOBAL expert ids -> [T, H]."""
        t, h = hidden.shape
        k = topk_ids.shape[1]
        plan = make_dispatch_plan(topk_ids, topk_weights, self.experts_per_rank, self.world, self.group)
        # everything that does not need the split sizes goes in front of the plan's host synchronisation
        token_of = torch.div(plan.order, k, rounding_mode="floor")
        send_rows = hidden.index_select(0, token_of)
        # local expert id and router weight of every row travel together (two fp32 per row; ids are small
        # integers, exact in fp32)
        meta = torch.stack((plan.local_expert.to(torch.float32), plan.weights), dim=1)
        # the contributions come back in `order` order: row inv[t * k + j] is route j of token t
        inv = torch.empty_like(plan.order)
        inv[plan.order] = torch.arange(t * k, device=plan.order.device, dtype=plan.order.dtype)
        recv_rows = _all_to_all_rows(send_rows, plan.send_counts, plan.recv_counts, self.group)
        recv_meta = _all_to_all_rows(meta, plan.send_counts, plan.recv_counts, self.group)
        recv_expert = recv_meta[:, 0].to(torch.int32)
        recv_weight = recv_meta[:, 1].contiguous()
        out_rows = self.compute(recv_rows, recv_expert, recv_weight)
        back = _all_to_all_rows(out_rows, plan.recv_counts, plan.send_counts, self.group)
        return self._sum_routes(back, inv.view(t, k), hidden)

    @staticmethod
    def _sum_routes(back: torch.Tensor, inv: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
        if back.is_cuda:
            from . import ops
            out = torch.empty_like(like)
            ops.moe_sum_rows(back.contiguous(), inv.to(torch.int32).contiguous(), out)
            return out
        return back.float()[inv.reshape(-1)].view(inv.shape[0], inv.shape[1], -1).sum(dim=1).to(like.dtype)
