"""Two-GEMM fused expert layer on top of the operator mirror.

Mirrors ``fused_marlin_moe`` / ``moe_align_block_size`` of the reference
(vllm/model_executor/layers/fused_moe/fused_marlin_moe.py:217-382,
vllm/model_executor/layers/fused_moe/moe_align_block_size.py:8-34): align -> GEMM-1 (gate|up) ->
SiLU-and-mul -> GEMM-2 with the router weight -> sum over the top-k routes.  The activation and the
sum, eager PyTorch in the reference, are CUDA kernels of this library."""
from __future__ import annotations

import torch

from . import ops
from .scalar_type import scalar_types

_BIT4 = (scalar_types.uint4.id, scalar_types.uint4b8.id, scalar_types.float4_e2m1f.id)


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int,
                         expert_map: torch.Tensor | None = None,
                         ignore_invalid_experts: bool = False):
    """Allocates and fills (sorted_ids, expert_ids, num_tokens_post_pad)."""
    max_padded = topk_ids.numel() + num_experts * (block_size - 1)
    dev = topk_ids.device
    sorted_ids = torch.empty((max_padded,), dtype=torch.int32, device=dev)
    expert_ids = torch.empty((max_padded // block_size + 1,), dtype=torch.int32, device=dev)
    num_post = torch.empty((1,), dtype=torch.int32, device=dev)
    ops.moe_align_block_size(topk_ids, num_experts, block_size, sorted_ids, expert_ids, num_post, expert_map)
    return sorted_ids, expert_ids, num_post


def fused_topk(gating_output: torch.Tensor, topk: int, renormalize: bool,
               bias: torch.Tensor | None = None):
    """softmax + top-k (reference wrapper: tests/helpers.py:314-332)."""
    t = gating_output.shape[0]
    dev = gating_output.device
    w = torch.empty((t, topk), dtype=torch.float32, device=dev)
    ids = torch.empty((t, topk), dtype=torch.int32, device=dev)
    tei = torch.empty((t, topk), dtype=torch.int32, device=dev)
    ops.topk_softmax(w, ids, tei, gating_output, renormalize, bias)
    return w, ids, tei


def select_block_size_m(m: int, topk: int, num_experts: int) -> int:
    """First of 8,16,32,48,64 with m*topk/E/block < 0.9 (fused_marlin_moe.py:319-321)."""
    block = 64
    for block in (8, 16, 32, 48, 64):
        if m * topk / num_experts / block < 0.9:
            break
    return block


def fused_marlin_moe(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                     bias1: torch.Tensor | None, bias2: torch.Tensor | None, w1_scale: torch.Tensor,
                     w2_scale: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                     quant_type_id: int, apply_router_weight_on_input: bool = False,
                     global_num_experts: int = -1, expert_map: torch.Tensor | None = None,
                     global_scale1: torch.Tensor | None = None, global_scale2: torch.Tensor | None = None,
                     w1_zeros: torch.Tensor | None = None, w2_zeros: torch.Tensor | None = None,
                     is_w1_zp_float: bool | None = None, is_w2_zp_float: bool | None = None,
                     workspace: torch.Tensor | None = None, output: torch.Tensor | None = None,
                     inplace: bool = False, block_size_m: int | None = None,
                     w1_streaming: torch.Tensor | None = None,
                     w2_streaming: torch.Tensor | None = None) -> torch.Tensor:
    """hidden [M, K] -> [M, K].  w1 [E, K/16, 2N*16/pf] (gate|up), w2 [E, N/16, K*16/pf].

    `w1_streaming` / `w2_streaming` (no counterpart in the reference): the same expert weights converted once by
    `ops.prepare_weights`.  When both are given and the routing leaves at most 32 routes per block (the decode
    regime, where the layer is bound by streaming the weights of the experts that are hit), the two GEMMs run
    on them with the integer-MMA streaming kernel; larger batches use `w1` / `w2` as before."""
    num_bits = 4 if quant_type_id in _BIT4 else 8
    m, k = hidden_states.shape
    e = w1.size(0)
    topk = topk_ids.size(1)
    n = w2.size(1) * 16
    assert w1.size(1) * 16 == k, "Hidden size mismatch w1"
    assert w2.size(2) // (num_bits // 2) == k, "Hidden size mismatch w2"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert hidden_states.dtype in (torch.float16, torch.bfloat16)
    assert topk_weights.dtype == torch.float32
    if block_size_m is None:
        block_size_m = select_block_size_m(m, topk, e)
    if global_num_experts == -1:
        global_num_experts = e
    if is_w1_zp_float is None:
        is_w1_zp_float = w1_zeros is not None
    if is_w2_zp_float is None:
        is_w2_zp_float = w2_zeros is not None
    dev = hidden_states.device
    if workspace is None:
        workspace = torch.empty(0, dtype=torch.int32, device=dev)

    streaming = w1_streaming is not None and w2_streaming is not None and block_size_m <= 32
    if streaming:
        w1, w2 = w1_streaming, w2_streaming
    sorted_ids, expert_ids, num_post = moe_align_block_size(topk_ids, block_size_m, global_num_experts,
                                                            expert_map)
    flat_w = topk_weights.reshape(-1).contiguous()
    # routes of experts that are not on this rank are skipped by both GEMMs: their rows must read as 0
    zero_fill = expert_map is not None
    alloc = torch.zeros if zero_fill else torch.empty
    c1 = alloc((m * topk, 2 * n), dtype=hidden_states.dtype, device=dev)
    ops.moe_wna16_marlin_gemm(hidden_states, c1, w1, bias1, w1_scale, None, global_scale1, w1_zeros, None,
                              None, workspace, sorted_ids, expert_ids, num_post, flat_w, block_size_m,
                              topk, apply_router_weight_on_input, quant_type_id, m, 2 * n, k, True, False,
                              True, is_w1_zp_float)
    if streaming:
        act = c1     # SiLU-and-mul is applied where the second GEMM reads its rows
    else:
        act = torch.empty((m * topk, n), dtype=hidden_states.dtype, device=dev)
        ops.silu_and_mul(act, c1)
    if topk == 1:
        # one route per row: the second GEMM writes the result itself, there is nothing to sum
        if output is None:
            output = hidden_states if inplace else torch.empty_like(hidden_states)
        if zero_fill:
            output.zero_()
        c3 = output
    else:
        c3 = alloc((m * topk, k), dtype=hidden_states.dtype, device=dev)
    ops.moe_wna16_marlin_gemm(act, c3, w2, bias2, w2_scale, None, global_scale2, w2_zeros, None, None,
                              workspace, sorted_ids, expert_ids, num_post, flat_w, block_size_m, 1,
                              not apply_router_weight_on_input, quant_type_id, m * topk, k, n, True, False,
                              True, is_w2_zp_float, silu_input=streaming)
    if topk == 1:
        return output
    if output is None:
        output = hidden_states if inplace else torch.empty_like(hidden_states)
    ops.moe_sum(c3.view(m, topk, k), output)
    return output
