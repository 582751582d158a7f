// torch extension module `_C`: the dense Marlin operators under the reference's schemas
// (csrc/torch_bindings_marlin.cpp:5-37 of the reference), implemented by libmarlin_b200.so.
// Built as `_C.abi3.so`; dropped into the reference's package it is what `import vllm._C` loads.
#include <mutex>
#include <unordered_map>

#include "binding_common.h"

namespace {
using namespace mb200_torch;

// Weight tensors that marlin_b200_prepare_weights returned, by address.  An entry lives as long as its tensor's
// storage: the storage's deleter removes it, so a later allocation at the same address is not mistaken for one.
struct Prepared { int64_t size_k, size_n; int num_bits; };
std::mutex g_mutex;
std::unordered_map<const void*, Prepared> g_prepared;

bool is_prepared(const at::Tensor& w, int64_t size_k, int64_t size_n) {
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_prepared.find(w.data_ptr());
  return it != g_prepared.end() && it->second.size_k == size_k && it->second.size_n == size_n;
}

at::Tensor marlin_gemm(at::Tensor& a, OptTensor c_or_none, at::Tensor& b_q_weight, OptTensor const& b_bias_or_none,
                       at::Tensor& b_scales, OptTensor const& a_scales_or_none, OptTensor const& global_scale_or_none,
                       OptTensor const& b_zeros_or_none, OptTensor const& g_idx_or_none, OptTensor const& perm_or_none,
                       at::Tensor& workspace, int64_t b_type_id, int64_t size_m, int64_t size_n, int64_t size_k,
                       bool is_k_full, bool use_atomic_add, bool use_fp32_reduce, bool is_zp_float) {
  (void)workspace; (void)is_k_full; (void)use_atomic_add; (void)use_fp32_reduce;   // accepted and ignored
  check_no_act_order(g_idx_or_none, perm_or_none);
  TORCH_CHECK(!a_scales_or_none.has_value(), "a_scales can only be used for 8bit activation.");
  const int act = act_code(a);
  const int fmt = resolve_format(b_type_id, b_scales, a);
  const int pf = (fmt == MARLIN_B200_FMT_U8B128 || fmt == MARLIN_B200_FMT_U8 || fmt == MARLIN_B200_FMT_FP8) ? 4 : 8;

  TORCH_CHECK(a.dim() == 2, "a must be 2-D");
  TORCH_CHECK(a.size(0) == size_m, "Shape mismatch: a.size(0) = ", a.size(0), ", size_m = ", size_m);
  TORCH_CHECK(a.size(1) == size_k, "Shape mismatch: a.size(1) = ", a.size(1), ", size_k = ", size_k);
  TORCH_CHECK(size_k % 16 == 0, "size_k = ", size_k, " is not divisible by tile_size = 16");
  TORCH_CHECK(b_q_weight.dim() == 2 && size_k / 16 == b_q_weight.size(0), "Shape mismatch: b_q_weight.size(0) = ",
              b_q_weight.size(0), ", size_k = ", size_k, ", tile_size = 16");
  TORCH_CHECK(b_q_weight.size(1) % 16 == 0, "b_q_weight.size(1) = ", b_q_weight.size(1),
              " is not divisible by tile_size = 16");
  const int64_t actual_n = (b_q_weight.size(1) / 16) * pf;
  TORCH_CHECK(size_n == actual_n, "size_n = ", size_n, ", actual_size_n = ", actual_n);
  TORCH_CHECK(a.is_cuda(), "A is not on GPU");
  TORCH_CHECK(a.stride(1) == 1, "A.stride(1) is not 1");
  TORCH_CHECK(a.stride(0) % 8 == 0, "A.stride(0) must divisible by 8");
  TORCH_CHECK(((uintptr_t)a.data_ptr()) % 16 == 0, "A must aligned to 16 bytes");
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
    TORCH_CHECK(c.size(0) == size_m, "Shape mismatch: c.size(0) = ", c.size(0), ", size_m = ", size_m);
    TORCH_CHECK(c.size(1) == size_n, "Shape mismatch: c.size(1) = ", c.size(1), ", size_n = ", size_n);
  } else {
    c = at::empty({size_m, size_n}, a.options());
  }
  if (size_m == 0) return c;

  TORCH_CHECK(b_scales.dim() == 2, "b_scales rank = ", b_scales.dim(), " is not 2");
  TORCH_CHECK(b_scales.size(1) == size_n, "b_scales dim 1 = ", b_scales.size(1), " is not size_n = ", size_n);
  const int64_t num_groups = b_scales.size(0);
  if (num_groups > 1)
    TORCH_CHECK(size_k % num_groups == 0, "size_k = ", size_k, ", is not divisible by b_scales.size(0) = ", num_groups);

  const float* global_scale = nullptr;
  if (global_scale_or_none.has_value()) {
    const at::Tensor& gs = global_scale_or_none.value();
    TORCH_CHECK(fmt == MARLIN_B200_FMT_NVFP4, "Marlin supports global_scale only for nvfp4 format.");
    TORCH_CHECK(gs.is_cuda() && gs.is_contiguous(), "global_scale is not on GPU");
    TORCH_CHECK(gs.scalar_type() == at::kFloat, "Marlin nvfp4 expects fp32 global_scale.");
    TORCH_CHECK(gs.numel() == 1, "Marlin nvfp4 expects a single global_scale value.");
    global_scale = gs.data_ptr<float>();
  } else {
    TORCH_CHECK(fmt != MARLIN_B200_FMT_NVFP4, "the global_scale parameter must be passed for nvfp4 format.");
  }
  const void* bias = nullptr;
  if (b_bias_or_none.has_value()) {
    const at::Tensor& b = b_bias_or_none.value();
    TORCH_CHECK(b.is_cuda(), "b_bias is not on GPU");
    TORCH_CHECK(b.is_contiguous(), "b_bias is not contiguous");
    TORCH_CHECK(b.scalar_type() == a.scalar_type(), "Marlin bias must have the activation dtype.");
    TORCH_CHECK(b.size(0) == size_n, "b_bias.size(0) != size_n");
    bias = b.data_ptr();
  }
  const bool zp_format = fmt == MARLIN_B200_FMT_U4 || fmt == MARLIN_B200_FMT_U8;
  const bool has_zp = b_zeros_or_none.has_value() && b_zeros_or_none->size(-1) > 0;
  TORCH_CHECK(!has_zp || zp_format, "Marlin does not support zero-point metadata for this quant type.");
  const void* zeros = nullptr;
  if (has_zp) {
    const at::Tensor& z = b_zeros_or_none.value();
    TORCH_CHECK(z.is_cuda(), "b_zeros is not on GPU");
    TORCH_CHECK(z.is_contiguous(), "b_zeros is not contiguous");
    TORCH_CHECK(is_zp_float, "Marlin received b_zeros but is_zp_float is false. Packed integer zero-points are not "
                             "supported on the dense uint4/uint8 path.");
    TORCH_CHECK(z.dim() == 2, "b_zeros rank = ", z.dim(), " is not 2");
    TORCH_CHECK(z.scalar_type() == a.scalar_type(), "Marlin uint4/uint8 dense path expects zero points of the "
                                                    "activation dtype.");
    TORCH_CHECK(z.size(1) == size_n, "b_zeros dim 1 = ", z.size(1), " is not size_n = ", size_n);
    TORCH_CHECK(z.size(0) == num_groups, "b_zeros dim 0 = ", z.size(0), " is not num_groups = ", num_groups);
    zeros = z.data_ptr();
  } else {
    TORCH_CHECK(!is_zp_float, "is_zp_float is true but b_zeros was not provided.");
    TORCH_CHECK(!zp_format, "Marlin uint4/uint8 dense path requires float zero points.");
  }

  const int fmt_arg = fmt | (is_prepared(b_q_weight, size_k, size_n) ? MARLIN_B200_FMT_PREPARED : 0);
  const int64_t nbytes = marlin_b200_gemm_scratch_bytes(size_m, size_n, size_k, fmt_arg);
  at::Tensor scratch = scratch_like(a, nbytes);
  check_rc(marlin_b200_gemm(a.data_ptr(), c.data_ptr(), b_q_weight.data_ptr<int32_t>(), b_scales.data_ptr(), zeros,
                            bias, global_scale, act, fmt_arg, size_m, size_n, size_k, a.stride(0), num_groups,
                            nbytes > 0 ? scratch.data_ptr() : nullptr, nbytes, stream_of(a)));
  return c;
}

void check_repack_input(const at::Tensor& w, int64_t size_k, int64_t size_n, int64_t num_bits, bool is_a_8bit) {
  TORCH_CHECK(!is_a_8bit, "is_a_8bit=True (8-bit activation layout) is not supported");
  TORCH_CHECK(num_bits == 4 || num_bits == 8, "num_bits must be 4 or 8. Got = ", num_bits);
  TORCH_CHECK(w.is_cuda(), "b_q_weight is not on GPU");
  TORCH_CHECK(w.is_contiguous(), "b_q_weight is not contiguous");
  TORCH_CHECK(w.scalar_type() == at::kInt, "b_q_weight type is not kInt");
  TORCH_CHECK(size_k % 16 == 0, "size_k = ", size_k, " is not divisible by tile_k_size = 16");
  TORCH_CHECK(size_n % 64 == 0, "size_n = ", size_n, " is not divisible by tile_n_size = 64");
}

at::Tensor gptq_marlin_repack(at::Tensor& b_q_weight, at::Tensor& perm, int64_t size_k, int64_t size_n,
                              int64_t num_bits, bool is_a_8bit) {
  check_repack_input(b_q_weight, size_k, size_n, num_bits, is_a_8bit);
  const int64_t pf = 32 / num_bits;
  TORCH_CHECK(b_q_weight.dim() == 2 && b_q_weight.size(0) == size_k / pf && b_q_weight.size(1) == size_n,
              "Shape mismatch: b_q_weight = ", b_q_weight.sizes(), ", size_k = ", size_k, ", size_n = ", size_n,
              ", pack_factor = ", pf);
  const bool has_perm = perm.numel() > 0;
  if (has_perm) {
    TORCH_CHECK(perm.is_cuda(), "perm is not on GPU");
    TORCH_CHECK(perm.is_contiguous(), "perm is not contiguous");
    TORCH_CHECK(perm.scalar_type() == at::kInt, "perm type is not at::kInt");
    TORCH_CHECK(perm.numel() == size_k, "perm.numel() = ", perm.numel(), " is not size_k = ", size_k);
  }
  const c10::cuda::OptionalCUDAGuard guard(device_of(b_q_weight));
  at::Tensor out = at::empty({size_k / 16, size_n * 16 / pf}, b_q_weight.options());
  check_rc(marlin_b200_gptq_repack(b_q_weight.data_ptr<int32_t>(), has_perm ? perm.data_ptr<int32_t>() : nullptr,
                                   out.data_ptr<int32_t>(), size_k, size_n, (int)num_bits, stream_of(b_q_weight)));
  return out;
}

at::Tensor awq_marlin_repack(at::Tensor& b_q_weight, int64_t size_k, int64_t size_n, int64_t num_bits,
                             bool is_a_8bit) {
  check_repack_input(b_q_weight, size_k, size_n, num_bits, is_a_8bit);
  const int64_t pf = 32 / num_bits;
  TORCH_CHECK(b_q_weight.dim() == 2 && b_q_weight.size(0) == size_k && b_q_weight.size(1) == size_n / pf,
              "Shape mismatch: b_q_weight = ", b_q_weight.sizes(), ", size_k = ", size_k, ", size_n = ", size_n,
              ", pack_factor = ", pf);
  const c10::cuda::OptionalCUDAGuard guard(device_of(b_q_weight));
  at::Tensor out = at::empty({size_k / 16, size_n * 16 / pf}, b_q_weight.options());
  check_rc(marlin_b200_awq_repack(b_q_weight.data_ptr<int32_t>(), out.data_ptr<int32_t>(), size_k, size_n,
                                  (int)num_bits, stream_of(b_q_weight)));
  return out;
}

at::Tensor marlin_int4_fp8_preprocess(at::Tensor& qweight, OptTensor qzeros_or_none, bool inplace) {
  TORCH_CHECK(qweight.is_cuda(), "qweight is not on GPU");
  TORCH_CHECK(qweight.scalar_type() == at::kInt, "qweight.dtype != torch.int32");
  TORCH_CHECK(qweight.is_contiguous(), "qweight is not contiguous");
  const c10::cuda::OptionalCUDAGuard guard(device_of(qweight));
  at::Tensor out = inplace ? qweight : at::empty_like(qweight);
  if (!qzeros_or_none.has_value()) {
    TORCH_CHECK(qweight.numel() * 8 % 256 == 0, "qweight.numel() * 8 % 256 != 0");
    check_rc(marlin_b200_int4_fp8_preprocess(qweight.data_ptr<int32_t>(), nullptr, out.data_ptr<int32_t>(), 1,
                                             qweight.numel(), 1, stream_of(qweight)));
  } else {
    const at::Tensor& qzeros = qzeros_or_none.value();
    TORCH_CHECK(qweight.dim() == 2 && qzeros.dim() == 2, "qweight and qzeros must be 2-D");
    TORCH_CHECK(qweight.size(0) % 32 == 0, "size_k % 32 != 0");
    TORCH_CHECK(qzeros.is_cuda(), "qzeros is not on GPU");
    TORCH_CHECK(qzeros.scalar_type() == at::kInt, "qweight.dtype != torch.int32");
    TORCH_CHECK(qzeros.is_contiguous(), "qzeros is not contiguous");
    TORCH_CHECK(qzeros.device() == qweight.device(), "qzeros is not on the same device with qweight");
    TORCH_CHECK(qweight.size(1) == qzeros.size(1), "qweight.size(1) != qzeros.size(1)");
    TORCH_CHECK(qweight.size(0) % qzeros.size(0) == 0, "qweight.size(0) % qzeros.size(0) != 0");
    check_rc(marlin_b200_int4_fp8_preprocess(qweight.data_ptr<int32_t>(), qzeros.data_ptr<int32_t>(),
                                             out.data_ptr<int32_t>(), qweight.size(0), qweight.size(1), qzeros.size(0),
                                             stream_of(qweight)));
  }
  return out;
}

// The two probe operators exercise the reference's SM70 CUTLASS mainloop; there is nothing for them to probe here.
at::Tensor sm70_cutlass_matmul_probe(at::Tensor&, at::Tensor&, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                                     int64_t) {
  TORCH_CHECK(false, "sm70_cutlass_matmul_probe is a diagnostic of the SM70 build and is not available in the B200 build");
}
at::Tensor sm70_cutlass_matmul_explicit_warp_probe(at::Tensor&, at::Tensor&, int64_t, int64_t, int64_t, int64_t, int64_t,
                                                   int64_t, int64_t) {
  TORCH_CHECK(false, "sm70_cutlass_matmul_explicit_warp_probe is a diagnostic of the SM70 build and is not available "
                     "in the B200 build");
}

// ---- additions without a counterpart in the reference: the streaming weight layout ----
at::Tensor convert_layout(at::Tensor& w, int64_t size_k, int64_t size_n, int64_t num_bits, bool to_stream) {
  TORCH_CHECK(w.is_cuda() && w.is_contiguous() && w.scalar_type() == at::kInt,
              "packed weights must be a contiguous int32 CUDA tensor");
  TORCH_CHECK(w.dim() == 2 || w.dim() == 3, "packed weights must be [K/16, N*16/pf] or [E, K/16, N*16/pf]");
  TORCH_CHECK(num_bits == 4 || num_bits == 8, "num_bits must be 4 or 8. Got = ", num_bits);
  const int64_t pf = 32 / num_bits;
  TORCH_CHECK(w.size(-2) == size_k / 16 && w.size(-1) == size_n * 16 / pf, "Shape mismatch: b_q_weight = ", w.sizes(),
              ", size_k = ", size_k, ", size_n = ", size_n);
  const int64_t experts = w.dim() == 3 ? w.size(0) : 1;
  const c10::cuda::OptionalCUDAGuard guard(device_of(w));
  at::Tensor out = at::empty_like(w);
  if (to_stream)
    check_rc(marlin_b200_prepare_weights(w.data_ptr<int32_t>(), out.data_ptr<int32_t>(), size_k, size_n, (int)num_bits,
                                         experts, stream_of(w)));
  else
    check_rc(marlin_b200_restore_weights(w.data_ptr<int32_t>(), out.data_ptr<int32_t>(), size_k, size_n, (int)num_bits,
                                         experts, stream_of(w)));
  return out;
}

at::Tensor marlin_b200_prepare_weights_op(at::Tensor& b_q_weight, int64_t size_k, int64_t size_n, int64_t num_bits) {
  at::Tensor inner = convert_layout(b_q_weight, size_k, size_n, num_bits, true);
  void* ptr = inner.data_ptr();
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_prepared[ptr] = Prepared{size_k, size_n, (int)num_bits};
  }
  // a view of the same memory whose deleter forgets the entry and then lets go of the allocation
  return at::from_blob(ptr, inner.sizes(), inner.strides(),
                       [inner](void* p) mutable {
                         std::lock_guard<std::mutex> lock(g_mutex);
                         g_prepared.erase(p);
                       },
                       inner.options());
}

at::Tensor marlin_b200_restore_weights_op(at::Tensor& prepared, int64_t size_k, int64_t size_n, int64_t num_bits) {
  return convert_layout(prepared, size_k, size_n, num_bits, false);
}

}  // namespace

TORCH_LIBRARY(_C, ops) {
  ops.def(
      "marlin_gemm(Tensor a, Tensor? c_or_none, Tensor b_q_weight, "
      "Tensor? b_bias_or_none,Tensor b_scales, "
      "Tensor? a_scales, Tensor? global_scale, Tensor? b_zeros_or_none, "
      "Tensor? g_idx_or_none, Tensor? perm_or_none, Tensor workspace, "
      "int b_type_id, SymInt size_m, SymInt size_n, SymInt size_k, "
      "bool is_k_full, bool use_atomic_add, bool use_fp32_reduce, "
      "bool is_zp_float) -> Tensor");
  ops.def(
      "gptq_marlin_repack(Tensor b_q_weight, Tensor perm, "
      "SymInt size_k, SymInt size_n, int num_bits, bool is_a_8bit) -> Tensor");
  ops.def(
      "awq_marlin_repack(Tensor b_q_weight, SymInt size_k, "
      "SymInt size_n, int num_bits, bool is_a_8bit) -> Tensor");
  ops.def(
      "marlin_int4_fp8_preprocess(Tensor qweight, "
      "Tensor? qzeros_or_none, bool inplace) -> Tensor");
  ops.def(
      "sm70_cutlass_matmul_probe(Tensor a, Tensor b, int cta_m, int cta_n, "
      "int cta_k, int warps, int stages, int a_path, int b_path) -> Tensor");
  ops.def(
      "sm70_cutlass_matmul_explicit_warp_probe(Tensor a, Tensor b, "
      "int cta_m, int cta_n, int cta_k, int warps, "
      "int warp_m, int warp_n, int warp_k) -> Tensor");
  // no counterpart in the reference: one-time conversion to / from the streaming weight layout
  ops.def("marlin_b200_prepare_weights(Tensor b_q_weight, SymInt size_k, SymInt size_n, int num_bits) -> Tensor");
  ops.def("marlin_b200_restore_weights(Tensor prepared, SymInt size_k, SymInt size_n, int num_bits) -> Tensor");
}

TORCH_LIBRARY_IMPL(_C, CUDA, m) {
  m.impl("marlin_gemm", &marlin_gemm);
  m.impl("gptq_marlin_repack", &gptq_marlin_repack);
  m.impl("awq_marlin_repack", &awq_marlin_repack);
  m.impl("marlin_int4_fp8_preprocess", &marlin_int4_fp8_preprocess);
  m.impl("sm70_cutlass_matmul_probe", &sm70_cutlass_matmul_probe);
  m.impl("sm70_cutlass_matmul_explicit_warp_probe", &sm70_cutlass_matmul_explicit_warp_probe);
  m.impl("marlin_b200_prepare_weights", &marlin_b200_prepare_weights_op);
  m.impl("marlin_b200_restore_weights", &marlin_b200_restore_weights_op);
}

MB200_REGISTER_EXTENSION(_C)
