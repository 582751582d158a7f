// Shared helpers of the two torch extension modules (_C, _moe_C): they register the reference project's
// operator schemas (csrc/torch_bindings_marlin.cpp, csrc/moe/torch_bindings_marlin.cpp there) and forward every
// call to the C ABI of libmarlin_b200.so on the current CUDA stream of the tensors' device.
#pragma once

#include <Python.h>

#include <ATen/ATen.h>
#include <ATen/DeviceGuard.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <optional>

#include "marlin_b200.h"

namespace mb200_torch {

using OptTensor = std::optional<at::Tensor>;

inline void check_rc(int rc) { TORCH_CHECK(rc == 0, marlin_b200_last_error()); }

inline void* stream_of(const at::Tensor& t) {
  return (void*)at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}

inline int act_code(const at::Tensor& a) {
  if (a.scalar_type() == at::kHalf) return MARLIN_B200_F16;
  if (a.scalar_type() == at::kBFloat16) return MARLIN_B200_BF16;
  TORCH_CHECK(false, "unsupported `a` scalar_type: float16 or bfloat16 activations expected");
}

// weight format from the reference's ScalarType id and the scale tensor's element type
inline int resolve_format(int64_t b_type_id, const at::Tensor& b_scales, const at::Tensor& a) {
  int kind = MARLIN_B200_SCALE_ACT;
  if (b_scales.scalar_type() == at::kFloat8_e4m3fn) kind = MARLIN_B200_SCALE_E4M3;
  else if (b_scales.scalar_type() == at::kFloat8_e8m0fnu) kind = MARLIN_B200_SCALE_E8M0;
  else
    TORCH_CHECK(b_scales.scalar_type() == a.scalar_type(),
                "Marlin expects scales of the activation dtype, except FP4 uses float8_e4m3fn scales for NVFP4 or "
                "float8_e8m0fnu scales for MXFP4.");
  const int fmt = marlin_b200_format_from_type_id(b_type_id, kind);
  TORCH_CHECK(fmt >= 0, "Marlin currently implements only uint4, uint4b8, uint8, uint8b128, fp8_e4m3fn, nvfp4, "
                        "and mxfp4 weights.");
  return fmt;
}

inline void check_no_act_order(const OptTensor& g_idx, const OptTensor& perm) {
  if (g_idx.has_value()) TORCH_CHECK(g_idx->numel() == 0, "Marlin does not support act_order g_idx.");
  if (perm.has_value()) TORCH_CHECK(perm->numel() == 0, "Marlin does not support act_order perm.");
}

inline at::Tensor scratch_like(const at::Tensor& a, int64_t nbytes) {
  return at::empty({nbytes > 0 ? nbytes : 0}, a.options().dtype(at::kByte));   // caching allocator: capture-safe
}

}  // namespace mb200_torch

// The module object itself is empty: importing the file runs the static TORCH_LIBRARY initialisers, which is
// all the reference's loaders (`import vllm._C`, tests/ops.py:25-37 there) rely on.
#define MB200_REGISTER_EXTENSION(NAME)                                                            \
  PyMODINIT_FUNC PyInit_##NAME() {                                                                 \
    static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, #NAME, nullptr, 0, nullptr};        \
    return PyModule_Create(&module);                                                               \
  }
