"""Multi-GPU layouts of the Marlin path: one process per GPU, `torch.distributed` for the plumbing.

The reference has no distributed code (`vllm/distributed/__init__.py:4-25` is a world-size-1 stub);
what it offers are the hooks this module builds on: `expert_map` / zero-filled rows in the fused
expert layer (`fused_marlin_moe.py:170-171`, `csrc/moe/moe_align_sum_kernels.cu:129-133`) and an op
whose output columns are independent (`csrc/quantization/marlin/marlin.cu:356-359`: any column count
that is a multiple of 64 is legal).

* `ColumnParallelMarlinLinear`: N is cut into `world` contiguous slices; every rank quantises /
  repacks its own slice (the packed layout depends on `size_n`), runs the local GEMM into its part of
  a `[world, M, N/world]` buffer and the ranks all-gather in place.
* `ExpertParallelMoE`: tokens are data-parallel, experts are sharded (contiguously, or by a placement
  table that evens out the routes per rank: `balanced_expert_placement`).  Routing is local; one
  all-to-all of row counts, one of rows (+ local expert id and router weight per row) to the ranks that
  own the experts, the local fused expert layer with top_k = 1, one all-to-all back, and the top-k
  contributions of every token are summed where the token lives.

Both classes take a `compute` callable so the index plumbing can be exercised on CPU ranks (gloo)
with a plain PyTorch stand-in; on GPUs the default is the CUDA library.

Transport.  The portable form of both layers moves data with `torch.distributed` collectives (NCCL on
GPUs, gloo on CPU ranks).  On the GPUs of one node both layers can instead use the library's own kernels
over peer-mapped memory (`PeerArena`, `use_peer_memory=True`): the all-gather of the dense layer is one
kernel that stores this rank's slice into every rank's buffer, and the expert-parallel layer stores every
route's row straight into the owning rank's receive buffer and reads the contributions back with peer
loads, with no collective library call and no stream synchronisation in the step.
"""
from __future__ import annotations

import ctypes
from typing import Callable

import torch
import torch.distributed as dist


# --------------------------------------------------------------------------------------------------
# peer-mapped memory of the ranks of one node
# --------------------------------------------------------------------------------------------------

class _DeviceBytes:
    """Lets torch wrap a raw device allocation (no copy) through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._owner = owner


class PeerArena:
    """One device allocation per rank that every rank of `group` (all on one node) maps into its own address
    space (CUDA IPC).  The first `header_bytes` belong to the library's kernels; the rest is laid out by the
    layer that owns the arena, identically on every rank.  Collective: every rank must construct it."""

    def __init__(self, nbytes: int, group=None, device: torch.device | None = None):
        from . import _lib
        self._lib = lib = _lib.load()
        self._check = _lib.check
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.header_bytes = lib.marlin_b200_peer_header_bytes()
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self._opened: list[int] = []
        with torch.cuda.device(self.device):
            base = ctypes.c_void_p()
            self._check(lib.marlin_b200_peer_alloc(self.nbytes, ctypes.byref(base)))
            self.base = base.value
            handle = ctypes.create_string_buffer(64)
            self._check(lib.marlin_b200_peer_export(self.base, handle))
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
            ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    ptrs.append(self.base)
                    continue
                peer = ctypes.c_void_p()
                self._check(lib.marlin_b200_peer_open(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(peer)))
                self._opened.append(peer.value)
                ptrs.append(peer.value)
        self.table = (ctypes.c_void_p * self.world)(*ptrs)
        self._bytes = torch.as_tensor(_DeviceBytes(self.base, self.nbytes, self), device=self.device)
        if self.world > 1:
            dist.barrier(group=group)

    def tensor(self, offset: int, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """A tensor over the local arena at `offset` (a multiple of 256 behind the header)."""
        if offset < self.header_bytes or offset % 256:
            raise ValueError("arena offsets are multiples of 256 bytes behind the library's header")
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if offset + nbytes > self.nbytes:
            raise ValueError("tensor does not fit the arena")
        return self._bytes[offset:offset + nbytes].view(dtype).view(shape)

    def status(self) -> tuple[int, int]:
        """(status, steps completed); 0 = no wait of this arena's kernels has given up.  Synchronous."""
        st, ep = ctypes.c_int(0), ctypes.c_int(0)
        with torch.cuda.device(self.device):
            self._check(self._lib.marlin_b200_peer_status(self.base, ctypes.byref(st), ctypes.byref(ep)))
        return int(st.value), int(ep.value)

    def close(self):
        """Collective: unmaps the peers' arenas and frees this rank's once every rank has stopped using them."""
        if self.base is None:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.group)
            for ptr in self._opened:
                self._lib.marlin_b200_peer_close(ptr)
            self._opened = []
            if self.world > 1:
                dist.barrier(group=self.group)
            self._bytes = None
            self._lib.marlin_b200_peer_free(self.base)
            self.base = None


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

    def __init__(self, gemm: Callable[[torch.Tensor, torch.Tensor], None], n_total: int, group=None,
                 use_peer_memory: bool = False, max_m: int = 16, dtype: torch.dtype = torch.bfloat16):
        """`gemm(x, out_slice)` runs this rank's local GEMM into `out_slice` [M, N/world].
        `use_peer_memory`: gather with the library's peer-store kernel (GPUs of one node, M <= max_m); the
        buffers are allocated once, here, and the step has no host synchronisation (it can be captured)."""
        self.gemm, self.n_total, self.group = gemm, n_total, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.lo, self.hi = column_slice(n_total, self.rank, self.world)
        self.arena = None
        if use_peer_memory and self.world > 1:
            per = self.hi - self.lo
            self._slice_bytes = max_m * per * torch.empty((), dtype=dtype).element_size()
            self.max_m, self.dtype = max_m, dtype
            self.arena = PeerArena(4096 + 4 * self.world * self._slice_bytes, group)
            self._local = torch.empty((max_m, per), dtype=dtype, device=self.arena.device)
            self._out = torch.empty((max_m, n_total), dtype=dtype, device=self.arena.device)

    def gather(self, local: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Peer-memory all-gather of this rank's [M, N/world] block (contiguous, M <= max_m) into `out` [M, N]
        (default: the layer's own output buffer): one kernel, no host synchronisation."""
        from . import _lib
        m, per = local.shape
        a = self.arena
        out = self._out[:m] if out is None else out
        _lib.check(a._lib.marlin_b200_peer_allgather(a.table, self.rank, self.world, local.data_ptr(),
                                                     m * per * local.element_size(), 4096, out.data_ptr(), m,
                                                     torch.cuda.current_stream(a.device).cuda_stream))
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        m = x.shape[0]
        per = self.hi - self.lo
        if self.arena is not None and m <= self.max_m and x.dtype == self.dtype:
            local = self._local[:m]
            self.gemm(x, local)
            return self.gather(local)
        gathered = torch.empty((self.world, m, per), dtype=x.dtype, device=x.device)
        self.gemm(x, gathered[self.rank])
        if self.world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), gathered[self.rank].reshape(-1), group=self.group)
        # [world, M, per] -> [M, world * per]
        return gathered.permute(1, 0, 2).reshape(m, self.n_total)


# --------------------------------------------------------------------------------------------------
# MoE: expert parallel dispatch / combine
# --------------------------------------------------------------------------------------------------

def balanced_expert_placement(expected_load: torch.Tensor, world: int) -> torch.Tensor:
    """Expert -> slot table (slot = rank * experts_per_rank + index on that rank) that evens out the routes per
    rank: experts are taken in order of decreasing expected load (router statistics; any non-negative
    weights) and each goes to the rank with the smallest load so far that still has a free slot (longest
    processing time first).  Deterministic; returns int32 [E].  With contiguous shards a skewed router sends
    most routes to a few ranks and the busiest rank bounds the layer."""
    load = expected_load.detach().to(torch.float64).cpu()
    e = load.numel()
    if e % world:
        raise ValueError(f"{e} experts cannot be sharded evenly over {world} ranks")
    per = e // world
    order = sorted(range(e), key=lambda i: (-float(load[i]), i))
    rank_load, rank_fill = [0.0] * world, [0] * world
    slot = torch.empty(e, dtype=torch.int32)
    for ex in order:
        r = min((r for r in range(world) if rank_fill[r] < per), key=lambda r: (rank_load[r], r))
        slot[ex] = r * per + rank_fill[r]
        rank_fill[r] += 1
        rank_load[r] += float(load[ex])
    return slot


class DispatchPlan:
    """Routes of this rank sorted by the slot (owning rank, then expert on that rank) of their expert.  The row
    counts per destination are exchanged with an asynchronous all-to-all that is started first;
    `send_counts` / `recv_counts` (the one host synchronisation of the layer) are only resolved when they are
    first read, so the caller can put more device work (the row gather) in front of that synchronisation."""

    def __init__(self, order, local_expert, weights, send, recv, work):
        self.order = order                # [T*k] route indices sorted by destination slot (stable)
        self.local_expert = local_expert  # [T*k] expert id inside the destination rank, in `order` order
        self.weights = weights            # [T*k] router weight, in `order` order
        self._send, self._recv, self._work, self._counts = send, recv, work, None

    def _resolve(self):
        if self._counts is None:
            if self._work is not None:
                self._work.wait()
            both = torch.stack((self._send, self._recv)).tolist()     # [2][world][2]: (rows, invalid routes)
            if any(c[1] for c in both[0]) or any(c[1] for c in both[1]):
                # every rank sees the same flags (they travelled with the counts), so every rank raises here,
                # before the row exchange: none is left waiting inside a collective
                raise RuntimeError("expert-parallel dispatch: topk_ids holds expert ids outside [0, num_experts)")
            self._counts = [[c[0] for c in both[0]], [c[0] for c in both[1]]]
        return self._counts

    @property
    def send_counts(self) -> list[int]:   # rows sent to each rank
        return self._resolve()[0]

    @property
    def recv_counts(self) -> list[int]:   # rows received from each rank
        return self._resolve()[1]


def make_dispatch_plan(topk_ids: torch.Tensor, topk_weights: torch.Tensor, experts_per_rank: int, world: int,
                       group=None, expert_slot: torch.Tensor | None = None) -> DispatchPlan:
    """Sorts the (token, route) pairs by the slot of their expert and exchanges the counts.  `expert_slot`
    (int32 [E], expert -> rank * experts_per_rank + index on the rank) defaults to contiguous shards.  On CUDA
    the sort is the library's stable counting sort (`moe_align_block_size` with blocks of one route and the
    slot table as its expert map): one kernel instead of a general sort."""
    num_experts = experts_per_rank * world
    flat = topk_ids.reshape(-1)
    numel = flat.numel()
    dev = flat.device
    if flat.is_cuda:
        from . import ops
        if expert_slot is None:
            expert_slot = torch.arange(num_experts, dtype=torch.int32, device=dev)
        order32 = torch.empty(numel, dtype=torch.int32, device=dev)
        slot_sorted = torch.empty(numel + 1, dtype=torch.int32, device=dev)
        num_valid = torch.empty(1, dtype=torch.int32, device=dev)
        ops.moe_align_block_size(flat.to(torch.int32).contiguous(), num_experts, 1, order32, slot_sorted, num_valid,
                                 expert_slot)
        slot_sorted = slot_sorted[:numel]
        valid = slot_sorted >= 0            # routes with an id outside the table are dropped by the sort
        order = order32.clamp_max(max(numel - 1, 0)).to(torch.int64)
    else:
        ids = flat.to(torch.int64)
        ok = (ids >= 0) & (ids < num_experts)
        slot_all = ids.clamp(0, num_experts - 1)
        if expert_slot is not None:
            slot_all = expert_slot.to(torch.int64)[slot_all]
        slot_all = torch.where(ok, slot_all, torch.full_like(slot_all, num_experts))   # invalid ones sort last
        srt = torch.sort(slot_all, stable=True)
        order, slot_sorted = srt.indices, srt.values.to(torch.int32)
        valid = srt.values < num_experts
        slot_sorted = torch.where(valid, slot_sorted, torch.full_like(slot_sorted, -1))
    dest = torch.where(valid, torch.div(slot_sorted, experts_per_rank, rounding_mode="floor"),
                       torch.full_like(slot_sorted, world)).to(torch.int64)
    counts = torch.bincount(dest, minlength=world + 1)
    send = torch.stack((counts[:world], counts[world:world + 1].expand(world)), dim=1).contiguous()   # [world, 2]
    recv = torch.empty_like(send)
    work = None
    if world > 1:
        work = dist.all_to_all_single(recv, send, group=group, async_op=True)
    else:
        recv.copy_(send)
    local_expert = torch.remainder(slot_sorted.clamp_min(0), experts_per_rank).to(torch.int32)
    return DispatchPlan(order, local_expert, topk_weights.reshape(-1)[order].to(torch.float32), send, recv, work)


def _all_to_all_rows(rows: torch.Tensor, send_counts: list[int], recv_counts: list[int], group, async_op=False):
    out = torch.empty((sum(recv_counts),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    work = None
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        work = dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts,
                                      input_split_sizes=send_counts, group=group, async_op=async_op)
    else:
        out.copy_(rows[:sum(send_counts)])
    return (out, work) if async_op else out


class ExpertParallelMoE:
    """Fused expert layer with the experts sharded over the ranks of `group`.

    compute(rows [R, H], local_expert int32 [R], weights fp32 [R]) -> [R, H] must return, for every
    received row, weight * expert(local_expert)(row).  The default built by `from_marlin_weights`
    runs moe_align_block_size + the two grouped GEMMs + SiLU-and-mul of the CUDA library with
    top_k = 1.

    `expert_slot` (int32 [E]) places expert e at index `expert_slot[e] % experts_per_rank` of rank
    `expert_slot[e] // experts_per_rank`; this rank's weight tensors must be stacked in that order.  Default:
    contiguous shards.  `balanced_expert_placement` builds a table from router statistics."""

    def __init__(self, compute: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
                 num_experts: int, group=None, expert_slot: torch.Tensor | None = None):
        self.compute, self.num_experts, self.group = compute, num_experts, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts cannot be sharded evenly over {self.world} ranks")
        self.experts_per_rank = num_experts // self.world
        if expert_slot is not None:
            if sorted(expert_slot.tolist()) != list(range(num_experts)):
                raise ValueError("expert_slot must be a permutation of range(num_experts)")
            expert_slot = expert_slot.to(torch.int32).contiguous()
        self.expert_slot = expert_slot
        self.last_recv_rows = 0   # rows this rank's experts received in the last forward (load report)
        self.record_phases = False   # CUDA events between the phases of every forward, read by phase_ms()
        self._marks = []
        self.arena = None

    def enable_peer_memory(self, capacity_rows: int, hidden: int, dtype: torch.dtype, device=None):
        """Collective.  Switches the layer to the library's peer-memory kernels (GPUs of one node): receive and
        output buffers of `capacity_rows` rows are allocated once on every rank and mapped by all ranks.
        `capacity_rows` bounds the routes one rank can receive in a step (tokens of all ranks * top_k is always
        enough); a step that exceeds it raises."""
        row_bytes = hidden * torch.empty((), dtype=dtype).element_size()
        if row_bytes % 16:
            raise ValueError("hidden size must give rows of a multiple of 16 bytes")
        up = lambda v: (v + 255) // 256 * 256
        off_rows = 4096
        off_expert = up(off_rows + capacity_rows * row_bytes)
        off_weight = up(off_expert + capacity_rows * 4)
        off_out = up(off_weight + capacity_rows * 4)
        self.arena = PeerArena(off_out + capacity_rows * row_bytes, self.group, device)
        a = self.arena
        self._layout = (ctypes.c_int64 * 6)(off_rows, off_expert, off_weight, off_out, capacity_rows, row_bytes)
        self._recv_rows = a.tensor(off_rows, (capacity_rows, hidden), dtype)
        self._recv_expert = a.tensor(off_expert, (capacity_rows,), torch.int32)
        self._recv_weight = a.tensor(off_weight, (capacity_rows,), torch.float32)
        self._out_rows = a.tensor(off_out, (capacity_rows, hidden), dtype)
        host, dev = ctypes.c_void_p(), ctypes.c_void_p()
        with torch.cuda.device(a.device):
            a._check(a._lib.marlin_b200_peer_host_word_alloc(ctypes.byref(host), ctypes.byref(dev)))
        self._host_word, self._host_word_dev = host.value, dev.value
        self._step = 0
        if self.expert_slot is None:
            self.expert_slot = torch.arange(self.num_experts, dtype=torch.int32, device=a.device)
        else:
            self.expert_slot = self.expert_slot.to(a.device)

    def close(self):
        """Collective: releases the peer-memory buffers."""
        if self.arena is not None:
            self.arena.close()
            self.arena._lib.marlin_b200_peer_host_word_free(self._host_word)
            self.arena = None

    def _forward_peer(self, hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        from . import ops
        a, lib = self.arena, self.arena._lib
        t, h = hidden.shape
        k = topk_ids.shape[1]
        numel = t * k
        dev = hidden.device
        if not (hidden.is_contiguous() and topk_ids.is_contiguous() and topk_weights.is_contiguous()):
            raise RuntimeError("the expert-parallel layer takes contiguous tensors")
        if hidden.dtype != self._recv_rows.dtype or h != self._recv_rows.shape[1]:
            raise RuntimeError("hidden does not match the shape / dtype the peer buffers were made for")
        ids32 = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
        w32 = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.to(torch.float32)
        order = torch.empty(numel, dtype=torch.int32, device=dev)
        slot_sorted = torch.empty(numel + 1, dtype=torch.int32, device=dev)
        num_valid = torch.empty(1, dtype=torch.int32, device=dev)
        position = torch.empty(numel, dtype=torch.int32, device=dev)
        out = torch.empty_like(hidden)
        ops.moe_align_block_size(ids32, self.num_experts, 1, order, slot_sorted, num_valid, self.expert_slot)
        stream = torch.cuda.current_stream(dev).cuda_stream
        rank, world, per = self.rank, self.world, self.experts_per_rank
        a._check(lib.marlin_b200_ep_plan(a.table, rank, world, slot_sorted.data_ptr(), numel, per, stream))
        a._check(lib.marlin_b200_ep_dispatch(a.table, rank, world, self._layout, hidden.data_ptr(), order.data_ptr(),
                                             slot_sorted.data_ptr(), w32.data_ptr(), position.data_ptr(), k, per,
                                             self._host_word_dev, stream))
        self._step += 1
        rows, invalid, status = ctypes.c_int64(0), ctypes.c_int(0), ctypes.c_int(0)
        # the row total arrives through mapped host memory while the dispatch kernel is still copying rows
        a._check(lib.marlin_b200_ep_poll_rows(self._host_word, self._step, 10000, ctypes.byref(rows),
                                              ctypes.byref(invalid), ctypes.byref(status)))
        self._mark("plan")
        if status.value:
            raise RuntimeError(f"expert-parallel step {self._step}: peer-memory status {status.value} "
                               "(1 + phase of a wait that gave up after two seconds, or 16 = receive capacity)")
        if invalid.value:
            # every rank sees the same count: all close the step and raise
            a._check(lib.marlin_b200_ep_signal(a.table, rank, world, 3, stream))
            a._check(lib.marlin_b200_ep_combine(a.table, rank, world, self._layout, position.data_ptr(), k, t,
                                                out.data_ptr(), ops._act_code(hidden.dtype), 1, stream))
            raise RuntimeError("expert-parallel dispatch: topk_ids holds expert ids outside [0, num_experts)")
        r = int(rows.value)
        self.last_recv_rows = r
        a._check(lib.marlin_b200_ep_wait(a.table, rank, world, 2, stream))
        self._mark("dispatch")
        if r > 0:
            out_rows = self._out_rows[:r]
            if getattr(self.compute, "takes_out", False):
                self.compute(self._recv_rows[:r], self._recv_expert[:r], self._recv_weight[:r], out=out_rows)
            else:
                out_rows.copy_(self.compute(self._recv_rows[:r], self._recv_expert[:r], self._recv_weight[:r]))
        self._mark("experts")
        a._check(lib.marlin_b200_ep_signal(a.table, rank, world, 3, stream))
        a._check(lib.marlin_b200_ep_combine(a.table, rank, world, self._layout, position.data_ptr(), k, t,
                                            out.data_ptr(), ops._act_code(hidden.dtype), 0, stream))
        self._mark("combine")
        return out

    @classmethod
    def from_marlin_weights(cls, w13, w2, w13_scale, w2_scale, quant_type_id: int, num_experts: int, group=None,
                            w13_zeros=None, w2_zeros=None, global_scale1=None, global_scale2=None,
                            expert_slot: torch.Tensor | None = None):
        """w13 / w2: this rank's experts ([E/world, ...], in slot order) in the packed layout of the grouped GEMM."""
        from . import fused_moe

        def compute(rows, local_expert, weights, out=None):
            if rows.shape[0] == 0:
                return rows.new_empty(rows.shape)
            return fused_moe.fused_marlin_moe(rows, w13, w2, None, None, w13_scale, w2_scale,
                                              weights.reshape(-1, 1).contiguous(), local_expert.reshape(-1, 1).contiguous(),
                                              quant_type_id, global_scale1=global_scale1, global_scale2=global_scale2,
                                              w1_zeros=w13_zeros, w2_zeros=w2_zeros, output=out)

        compute.takes_out = True

        if expert_slot is not None:
            expert_slot = expert_slot.to(w13.device)
        return cls(compute, num_experts, group, expert_slot)

    def _mark(self, name: str):
        if self.record_phases and torch.cuda.is_available():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((name, ev))

    def phase_ms(self) -> dict:
        """Device time of the phases of the last forward run with `record_phases` set (after a synchronise):
        plan (sort, counts and their exchange, row gather), dispatch (all-to-all of rows and metadata),
        experts (the local fused layer), combine (all-to-all back and the per-token sum)."""
        out = {}
        for (_, e0), (name, e1) in zip(self._marks[:-1], self._marks[1:]):
            out[name] = e0.elapsed_time(e1)
        return out

    def forward(self, hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        """hidden [T, H] (this rank's tokens), topk_* [T, k] with GLOBAL expert ids -> [T, H]."""
        self._marks = []
        self._mark("start")
        if self.arena is not None:
            return self._forward_peer(hidden, topk_weights, topk_ids)
        t, h = hidden.shape
        k = topk_ids.shape[1]
        slot = self.expert_slot
        if slot is not None and slot.device != topk_ids.device:
            slot = self.expert_slot = slot.to(topk_ids.device)
        plan = make_dispatch_plan(topk_ids, topk_weights, self.experts_per_rank, self.world, self.group, slot)
        # everything that does not need the split sizes goes in front of the plan's host synchronisation
        token_of = torch.div(plan.order, k, rounding_mode="floor")
        send_rows = hidden.index_select(0, token_of)
        # local expert id and router weight of every row travel together (two fp32 per row; ids are small
        # integers, exact in fp32)
        meta = torch.stack((plan.local_expert.to(torch.float32), plan.weights), dim=1)
        # the contributions come back in `order` order: row inv[t * k + j] is route j of token t
        inv = torch.empty_like(plan.order)
        inv[plan.order] = torch.arange(t * k, device=plan.order.device, dtype=plan.order.dtype)
        send_counts, recv_counts = plan.send_counts, plan.recv_counts
        self._mark("plan")
        # the small exchange is queued first and not waited for until the rows are in flight too
        recv_meta, meta_work = _all_to_all_rows(meta, send_counts, recv_counts, self.group, async_op=True)
        recv_rows = _all_to_all_rows(send_rows, send_counts, recv_counts, self.group)
        if meta_work is not None:
            meta_work.wait()
        self.last_recv_rows = int(sum(recv_counts))
        recv_expert = recv_meta[:, 0].to(torch.int32)
        recv_weight = recv_meta[:, 1].contiguous()
        self._mark("dispatch")
        out_rows = self.compute(recv_rows, recv_expert, recv_weight)
        self._mark("experts")
        back = _all_to_all_rows(out_rows, recv_counts, send_counts, self.group)
        out = self._sum_routes(back, inv.view(t, k), hidden)
        self._mark("combine")
        return out

    @staticmethod
    def _sum_routes(back: torch.Tensor, inv: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
        if back.is_cuda:
            from . import ops
            out = torch.empty_like(like)
            ops.moe_sum_rows(back.contiguous(), inv.to(torch.int32).contiguous(), out)
            return out
        return back.float()[inv.reshape(-1)].view(inv.shape[0], inv.shape[1], -1).sum(dim=1).to(like.dtype)
