// torch extension module `_moe_C`: the fused-MoE operators under the reference's schemas
// (csrc/moe/torch_bindings_marlin.cpp:4-57 of the reference), implemented by libmarlin_b200.so.
// Built as `_moe_C.abi3.so`; dropped into the reference's package it is what `import vllm._moe_C` loads.
#include <limits>
#include <tuple>

#include "binding_common.h"

namespace {
using namespace mb200_torch;

int gating_code(const at::Tensor& g) {
  switch (g.scalar_type()) {
    case at::kHalf: return 0;
    case at::kBFloat16: return 1;
    case at::kFloat: return 2;
    default: TORCH_CHECK(false, "Invalid gating_output type");
  }
}

template <bool SIGMOID>
void topk_scores(at::Tensor& topk_weights, at::Tensor& topk_indices, at::Tensor& token_expert_indices,
                 at::Tensor& gating_output, bool renormalize, OptTensor bias) {
  TORCH_CHECK(gating_output.is_cuda() && gating_output.is_contiguous(), "gating_output must be contiguous on GPU");
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat && topk_weights.is_contiguous(), "topk_weights must be fp32");
  TORCH_CHECK(topk_indices.scalar_type() == at::kInt && topk_indices.is_contiguous(), "topk_indices must be int32");
  TORCH_CHECK(token_expert_indices.scalar_type() == at::kInt && token_expert_indices.is_contiguous(),
              "token_expert_indices must be int32");
  const int64_t num_experts = gating_output.size(-1);
  const int64_t num_tokens = num_experts > 0 ? gating_output.numel() / num_experts : 0;
  const int64_t topk = topk_weights.size(-1);
  const float* bias_ptr = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->scalar_type() == at::kFloat &&
                    bias->numel() == num_experts, "bias must be a contiguous fp32 [num_experts] GPU tensor");
    bias_ptr = bias->data_ptr<float>();
  }
  const c10::cuda::OptionalCUDAGuard guard(device_of(gating_output));
  auto fn = SIGMOID ? marlin_b200_topk_sigmoid : marlin_b200_topk_softmax;
  check_rc(fn(gating_output.data_ptr(), gating_code(gating_output), bias_ptr, topk_weights.data_ptr<float>(),
              topk_indices.data_ptr<int32_t>(), token_expert_indices.data_ptr<int32_t>(), num_tokens, num_experts,
              (int)topk, renormalize ? 1 : 0, stream_of(gating_output)));
}

void topk_softmax(at::Tensor& topk_weights, at::Tensor& topk_indices, at::Tensor& token_expert_indices,
                  at::Tensor& gating_output, bool renormalize, OptTensor bias) {
  topk_scores<false>(topk_weights, topk_indices, token_expert_indices, gating_output, renormalize, bias);
}
void topk_sigmoid(at::Tensor& topk_weights, at::Tensor& topk_indices, at::Tensor& token_expert_indices,
                  at::Tensor& gating_output, bool renormalize, OptTensor bias) {
  topk_scores<true>(topk_weights, topk_indices, token_expert_indices, gating_output, renormalize, bias);
}

void moe_align_block_size(at::Tensor topk_ids, int64_t num_experts, int64_t block_size, at::Tensor sorted_token_ids,
                          at::Tensor experts_ids, at::Tensor num_tokens_post_pad, OptTensor maybe_expert_map) {
  TORCH_CHECK(topk_ids.is_cuda() && topk_ids.is_contiguous(), "topk_ids must be a contiguous GPU tensor");
  TORCH_CHECK(topk_ids.scalar_type() == at::kInt, "topk_ids must be int32");
  for (const at::Tensor* t : {&sorted_token_ids, &experts_ids, &num_tokens_post_pad})
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kInt,
                "align outputs must be contiguous int32 GPU tensors");
  int64_t num_global = 0;
  const int32_t* map = nullptr;
  if (maybe_expert_map.has_value()) {
    const at::Tensor& m = maybe_expert_map.value();
    TORCH_CHECK(m.is_cuda() && m.is_contiguous() && m.scalar_type() == at::kInt,
                "expert_map must be a contiguous int32 GPU tensor");
    num_global = m.numel();
    map = m.data_ptr<int32_t>();
  }
  const int64_t numel = topk_ids.numel();
  const c10::cuda::OptionalCUDAGuard guard(device_of(topk_ids));
  const int64_t nbytes = marlin_b200_moe_align_scratch_bytes(numel, num_experts);
  at::Tensor scratch = scratch_like(topk_ids, nbytes);
  check_rc(marlin_b200_moe_align_block_size(topk_ids.data_ptr<int32_t>(), numel, num_experts, num_global,
                                            (int)block_size, map, sorted_token_ids.data_ptr<int32_t>(),
                                            sorted_token_ids.numel(), experts_ids.data_ptr<int32_t>(),
                                            experts_ids.numel(), num_tokens_post_pad.data_ptr<int32_t>(),
                                            nbytes > 0 ? scratch.data_ptr() : nullptr, nbytes, stream_of(topk_ids)));
}

void batched_moe_align_block_size(int64_t max_tokens_per_batch, int64_t block_size, at::Tensor const& expert_num_tokens,
                                  at::Tensor sorted_token_ids, at::Tensor experts_ids, at::Tensor num_tokens_post_pad) {
  const at::Tensor* all[4] = {&expert_num_tokens, &sorted_token_ids, &experts_ids, &num_tokens_post_pad};
  for (const at::Tensor* t : all)
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kInt,
                "batched align tensors must be contiguous int32 GPU tensors");
  TORCH_CHECK(num_tokens_post_pad.numel() == 1, "num_tokens_post_pad must have one element");
  const c10::cuda::OptionalCUDAGuard guard(device_of(expert_num_tokens));
  check_rc(marlin_b200_batched_moe_align_block_size(
      max_tokens_per_batch, (int)block_size, expert_num_tokens.data_ptr<int32_t>(), expert_num_tokens.numel(),
      sorted_token_ids.data_ptr<int32_t>(), sorted_token_ids.numel(), experts_ids.data_ptr<int32_t>(),
      experts_ids.numel(), num_tokens_post_pad.data_ptr<int32_t>(), stream_of(expert_num_tokens)));
}

at::Tensor moe_wna16_marlin_gemm(at::Tensor& a, OptTensor c_or_none, at::Tensor& b_q_weight,
                                 OptTensor const& b_bias_or_none, at::Tensor& b_scales, OptTensor const& a_scales_or_none,
                                 OptTensor const& global_scale_or_none, OptTensor const& b_zeros_or_none,
                                 OptTensor const& g_idx_or_none, OptTensor const& perm_or_none, at::Tensor& workspace,
                                 at::Tensor& sorted_token_ids, at::Tensor& expert_ids,
                                 at::Tensor& num_tokens_past_padded, at::Tensor& topk_weights, int64_t moe_block_size,
                                 int64_t top_k, bool mul_topk_weights, int64_t b_type_id, int64_t size_m, int64_t size_n,
                                 int64_t size_k, bool is_k_full, bool use_atomic_add, bool use_fp32_reduce,
                                 bool is_zp_float, int64_t thread_k, int64_t thread_n, int64_t blocks_per_sm) {
  (void)workspace; (void)is_k_full; (void)use_atomic_add; (void)use_fp32_reduce;
  (void)thread_k; (void)thread_n; (void)blocks_per_sm;                         // accepted and ignored
  check_no_act_order(g_idx_or_none, perm_or_none);
  TORCH_CHECK(!a_scales_or_none.has_value(), "a_scales can only be used for 8bit activation.");
  const int act = act_code(a);
  const int fmt = resolve_format(b_type_id, b_scales, a);
  const int pf = (fmt == MARLIN_B200_FMT_U8B128 || fmt == MARLIN_B200_FMT_U8 || fmt == MARLIN_B200_FMT_FP8) ? 4 : 8;
  if (moe_block_size != 8)
    TORCH_CHECK(moe_block_size % 16 == 0 && moe_block_size >= 16 && moe_block_size <= 64,
                "unsupported moe_block_size=", moe_block_size);
  TORCH_CHECK(a.size(0) == size_m, "Shape mismatch: a.size(0) = ", a.size(0), ", size_m = ", size_m);
  TORCH_CHECK(a.size(1) == size_k, "Shape mismatch: a.size(1) = ", a.size(1), ", size_k = ", size_k);
  TORCH_CHECK(size_k % 16 == 0, "size_k = ", size_k, " is not divisible by tile_size = 16");
  TORCH_CHECK(b_q_weight.dim() == 3, "b_q_weight must be [experts, size_k / 16, size_n * 16 / pack_factor]");
  const int64_t num_experts = b_q_weight.size(0);
  TORCH_CHECK(size_k / 16 == b_q_weight.size(1), "Shape mismatch: b_q_weight.size(1) = ", b_q_weight.size(1),
              ", size_k = ", size_k, ", tile_size = 16");
  TORCH_CHECK(b_q_weight.size(2) % 16 == 0, "b_q_weight.size(2) = ", b_q_weight.size(2),
              " is not divisible by tile_size = 16");
  const int64_t actual_n = (b_q_weight.size(2) / 16) * pf;
  TORCH_CHECK(size_n == actual_n, "size_n = ", size_n, ", actual_size_n = ", actual_n);
  TORCH_CHECK(a.is_cuda(), "A is not on GPU");
  TORCH_CHECK(a.is_contiguous(), "A is not contiguous");
  TORCH_CHECK(b_q_weight.is_cuda(), "b_q_weight is not on GPU");
  TORCH_CHECK(b_q_weight.is_contiguous(), "b_q_weight is not contiguous");
  TORCH_CHECK(b_q_weight.scalar_type() == at::kInt, "Marlin expects int32 packed weights.");
  TORCH_CHECK(b_scales.is_cuda(), "b_scales is not on GPU");
  TORCH_CHECK(b_scales.is_contiguous(), "b_scales is not contiguous");

  const c10::cuda::OptionalCUDAGuard guard(device_of(a));
  at::Tensor c;
  if (c_or_none.has_value()) {
    c = c_or_none.value();
    TORCH_CHECK(c.is_cuda(), "c is not on GPU");
    TORCH_CHECK(c.is_contiguous(), "c is not contiguous");
    TORCH_CHECK(c.scalar_type() == a.scalar_type(), "scalar type of a must be the same with c for 16 bit activation");
    TORCH_CHECK(c.size(0) == size_m * top_k, "Shape mismatch: c.size(0) = ", c.size(0), ", size_m * topk = ",
                size_m * top_k);
    TORCH_CHECK(c.size(1) == size_n, "Shape mismatch: c.size(1) = ", c.size(1), ", size_n = ", size_n);
  } else {
    c = at::empty({size_m * top_k, size_n}, a.options());
  }
  TORCH_CHECK(b_scales.dim() == 3, "b_scales rank = ", b_scales.dim(), " is not 3");
  TORCH_CHECK(b_scales.size(0) == num_experts, "b_scales dim 0 is not the number of experts");
  TORCH_CHECK(b_scales.size(2) == size_n, "b_scales dim 2 = ", b_scales.size(2), " is not size_n = ", size_n);
  const int64_t num_groups = b_scales.size(1);
  if (num_groups > 1)
    TORCH_CHECK(size_k % num_groups == 0, "size_k = ", size_k, ", is not divisible by b_scales.size(1) = ", num_groups);

  const float* global_scale = nullptr;
  if (global_scale_or_none.has_value()) {
    const at::Tensor& gs = global_scale_or_none.value();
    TORCH_CHECK(fmt == MARLIN_B200_FMT_NVFP4, "Marlin MoE supports global_scale only for nvfp4 format.");
    TORCH_CHECK(gs.is_cuda() && gs.is_contiguous(), "global_scale is not on GPU");
    TORCH_CHECK(gs.scalar_type() == at::kFloat, "Marlin MoE nvfp4 expects fp32 global_scale.");
    TORCH_CHECK(gs.numel() == num_experts, "Marlin MoE nvfp4 expects global_scale numel = num_experts. Got "
                "global_scale.numel() = ", gs.numel(), ", num_experts = ", num_experts);
    global_scale = gs.data_ptr<float>();
  } else {
    TORCH_CHECK(fmt != MARLIN_B200_FMT_NVFP4, "the global_scale parameter must be passed for nvfp4 format.");
  }
  const void* bias = nullptr;
  if (b_bias_or_none.has_value()) {
    const at::Tensor& b = b_bias_or_none.value();
    TORCH_CHECK(b.is_cuda() && b.is_contiguous(), "b_bias is not on GPU");
    TORCH_CHECK(b.scalar_type() == a.scalar_type(), "Marlin bias must have the activation dtype.");
    TORCH_CHECK(b.dim() == 2 && b.size(0) == num_experts && b.size(1) == size_n, "b_bias must be [experts, size_n]");
    bias = b.data_ptr();
  }
  const bool zp_format = fmt == MARLIN_B200_FMT_U4 || fmt == MARLIN_B200_FMT_U8;
  const bool has_zp = b_zeros_or_none.has_value() && b_zeros_or_none->size(-1) > 0;
  TORCH_CHECK(!has_zp || zp_format, "Marlin does not support zero-point metadata for this quant type.");
  const void* zeros = nullptr;
  if (has_zp) {
    const at::Tensor& z = b_zeros_or_none.value();
    TORCH_CHECK(z.is_cuda() && z.is_contiguous(), "b_zeros is not on GPU");
    TORCH_CHECK(is_zp_float, "Marlin MoE received b_zeros but is_zp_float is false. Packed integer zero-points are "
                             "not supported.");
    TORCH_CHECK(z.scalar_type() == a.scalar_type(), "Marlin MoE expects zero points of the activation dtype.");
    TORCH_CHECK(z.dim() == 3 && z.size(0) == num_experts && z.size(1) == num_groups && z.size(2) == size_n,
                "b_zeros must be [experts, num_groups, size_n]");
    zeros = z.data_ptr();
  } else {
    TORCH_CHECK(!is_zp_float, "is_zp_float is true but b_zeros was not provided.");
    TORCH_CHECK(!zp_format, "Marlin uint4/uint8 MoE path requires float zero points.");
  }
  for (const at::Tensor* t : {&sorted_token_ids, &expert_ids, &num_tokens_past_padded}) {
    TORCH_CHECK(t->is_cuda() && t->is_contiguous(), "routing tensors must be contiguous GPU tensors");
    TORCH_CHECK(t->scalar_type() == at::kInt, "routing tensors must be int32");
  }
  TORCH_CHECK(topk_weights.is_cuda() && topk_weights.is_contiguous() && topk_weights.scalar_type() == at::kFloat,
              "topk_weights must be a contiguous fp32 GPU tensor");
  TORCH_CHECK(topk_weights.numel() >= size_m * top_k, "topk_weights has fewer than size_m * top_k entries");
  const int64_t num_sorted = sorted_token_ids.numel();
  const int64_t nbytes = marlin_b200_moe_gemm_scratch_bytes(num_sorted, size_n, size_k, fmt);
  at::Tensor scratch = scratch_like(a, nbytes);
  check_rc(marlin_b200_moe_gemm(a.data_ptr(), c.data_ptr(), b_q_weight.data_ptr<int32_t>(), b_scales.data_ptr(), zeros,
                                bias, global_scale, sorted_token_ids.data_ptr<int32_t>(), expert_ids.data_ptr<int32_t>(),
                                num_tokens_past_padded.data_ptr<int32_t>(), topk_weights.data_ptr<float>(), num_sorted,
                                num_experts, (int)moe_block_size, (int)top_k, mul_topk_weights ? 1 : 0, act, fmt, size_m,
                                size_n, size_k, num_groups, nbytes > 0 ? scratch.data_ptr() : nullptr, nbytes,
                                stream_of(a)));
  return c;
}

// Group-limited routing (csrc/moe/grouped_topk_kernels.cu:987-1090 of the reference).  Outside the Marlin hot
// path; kept available as a composition of library operators: scores (optionally through a sigmoid) plus bias
// pick the groups by the sum of their two best experts, then the experts inside the chosen groups; the weights
// are the unbiased scores, optionally renormalised, times the scaling factor.
std::tuple<at::Tensor, at::Tensor> grouped_topk(at::Tensor const& scores, int64_t n_group, int64_t topk_group,
                                                int64_t topk, bool renormalize, double routed_scaling_factor,
                                                at::Tensor const& bias, int64_t scoring_func) {
  TORCH_CHECK(scores.dim() == 2, "scores must be a 2D Tensor");
  const int64_t num_tokens = scores.size(0), num_experts = scores.size(1);
  TORCH_CHECK(n_group > 0, "n_group must be positive");
  TORCH_CHECK(topk > 0, "topk must be positive");
  TORCH_CHECK(topk_group > 0, "topk_group must be positive");
  TORCH_CHECK(topk_group <= n_group, "topk_group must be <= n_group");
  TORCH_CHECK(num_experts % n_group == 0, "num_experts should be divisible by n_group");
  TORCH_CHECK(n_group <= 32, "n_group should be smaller than or equal to 32 for now");
  TORCH_CHECK(topk <= 32, "topk should be smaller than or equal to 32 for now");
  TORCH_CHECK(topk <= topk_group * (num_experts / n_group), "topk must be <= topk_group * (num_experts / n_group)");
  TORCH_CHECK(scoring_func == 0 || scoring_func == 1, "scoring_func must be SCORING_NONE (0) or SCORING_SIGMOID (1)");
  const c10::cuda::OptionalCUDAGuard guard(device_of(scores));
  at::Tensor s = scores.to(at::kFloat);
  if (scoring_func == 1) s = at::sigmoid(s);
  at::Tensor choice = s + bias.to(at::kFloat).unsqueeze(0);
  const int64_t per_group = num_experts / n_group;
  at::Tensor group_scores =
      std::get<0>(at::topk(choice.view({num_tokens, n_group, per_group}), per_group < 2 ? per_group : 2, -1)).sum(-1);
  at::Tensor group_idx = std::get<1>(at::topk(group_scores, topk_group, -1, true, false));
  at::Tensor group_mask = at::zeros_like(group_scores).scatter_(1, group_idx, 1.0);
  at::Tensor mask = group_mask.unsqueeze(-1).expand({num_tokens, n_group, per_group}).reshape({num_tokens, num_experts});
  at::Tensor masked = choice.masked_fill(mask == 0, -std::numeric_limits<float>::infinity());
  at::Tensor ids = std::get<1>(at::topk(masked, topk, -1, true, true));
  at::Tensor weights = at::gather(s, 1, ids);
  if (renormalize) weights = weights / (weights.sum(-1, true) + 1e-20);
  weights = weights * routed_scaling_factor;
  return {weights.contiguous(), ids.to(at::kInt).contiguous()};
}

}  // namespace

TORCH_LIBRARY(_moe_C, m) {
  m.def(
      "topk_softmax(Tensor! topk_weights, Tensor! topk_indices, Tensor! "
      "token_expert_indices, Tensor gating_output, bool renormalize, Tensor? "
      "bias) -> ()");
  m.def(
      "topk_sigmoid(Tensor! topk_weights, Tensor! topk_indices, Tensor! "
      "token_expert_indices, Tensor gating_output, bool renormalize, Tensor? "
      "bias) -> ()");
  m.def(
      "moe_align_block_size(Tensor topk_ids, int num_experts,"
      "                     int block_size, Tensor! sorted_token_ids,"
      "                     Tensor! experts_ids,"
      "                     Tensor! num_tokens_post_pad,"
      "                     Tensor? maybe_expert_map) -> ()");
  m.def(
      "batched_moe_align_block_size(int max_tokens_per_batch,"
      "                     int block_size, Tensor expert_num_tokens,"
      "                     Tensor! sorted_token_ids,"
      "                     Tensor! experts_ids,"
      "                     Tensor! num_tokens_post_pad) -> ()");
  m.def(
      "moe_wna16_marlin_gemm(Tensor! a, Tensor? c_or_none,"
      "Tensor! b_q_weight, Tensor? b_bias_or_none,"
      "Tensor! b_scales, Tensor? a_scales, Tensor? global_scale, Tensor? "
      "b_zeros_or_none,"
      "Tensor? g_idx_or_none, Tensor? perm_or_none, Tensor! workspace,"
      "Tensor sorted_token_ids,"
      "Tensor! expert_ids, Tensor! num_tokens_past_padded,"
      "Tensor! topk_weights, int moe_block_size, int top_k, "
      "bool mul_topk_weights, int b_type_id,"
      "int size_m, int size_n, int size_k,"
      "bool is_k_full, bool use_atomic_add,"
      "bool use_fp32_reduce, bool is_zp_float,"
      "int thread_k, int thread_n, int blocks_per_sm) -> Tensor");
  m.def(
      "grouped_topk(Tensor scores, int n_group, int "
      "topk_group, int topk, bool renormalize, float "
      "routed_scaling_factor, Tensor bias, int scoring_func) -> (Tensor, "
      "Tensor)");
}

TORCH_LIBRARY_IMPL(_moe_C, CUDA, m) {
  m.impl("topk_softmax", &topk_softmax);
  m.impl("topk_sigmoid", &topk_sigmoid);
  m.impl("moe_align_block_size", &moe_align_block_size);
  m.impl("batched_moe_align_block_size", &batched_moe_align_block_size);
  m.impl("moe_wna16_marlin_gemm", &moe_wna16_marlin_gemm);
  m.impl("grouped_topk", &grouped_topk);
}

MB200_REGISTER_EXTENSION(_moe_C)
