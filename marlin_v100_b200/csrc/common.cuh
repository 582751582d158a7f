// Shared definitions of the B200 Marlin library: formats, the packed-weight index math and the
// per-element decoders every kernel agrees on.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/marlin_b200.h"

namespace mb200 {

enum Format : int {
  kU4B8 = MARLIN_B200_FMT_U4B8,
  kU4 = MARLIN_B200_FMT_U4,
  kU8B128 = MARLIN_B200_FMT_U8B128,
  kU8 = MARLIN_B200_FMT_U8,
  kFP8 = MARLIN_B200_FMT_FP8,
  kNVFP4 = MARLIN_B200_FMT_NVFP4,
  kMXFP4 = MARLIN_B200_FMT_MXFP4,
};

__host__ __device__ constexpr int format_bits(int f) {
  return (f == kU8B128 || f == kU8 || f == kFP8) ? 8 : 4;
}
__host__ __device__ constexpr bool format_has_zp(int f) { return f == kU4 || f == kU8; }
__host__ __device__ constexpr bool format_scale_is_byte(int f) { return f == kNVFP4 || f == kMXFP4; }

// Host-side error plumbing (abi.cu owns the storage).
void set_error(const char* fmt, ...);
int sm_count();  // SMs of the current device, cached
void count_launches(int n);  // bumps the process-wide kernel launch counter

#define MB_CHECK(cond, ...)             \
  do {                                  \
    if (!(cond)) {                      \
      ::mb200::set_error(__VA_ARGS__);  \
      return MARLIN_B200_EINVAL;        \
    }                                   \
  } while (0)

#define MB_CUDA(expr)                                                                  \
  do {                                                                                 \
    cudaError_t e__ = (expr);                                                          \
    if (e__ != cudaSuccess) {                                                          \
      ::mb200::set_error("CUDA error %s at %s:%d", cudaGetErrorString(e__), __FILE__, \
                         __LINE__);                                                    \
      return MARLIN_B200_ECUDA;                                                        \
    }                                                                                  \
  } while (0)

// ---------------------------------------------------------------------------------------------
// Packed layout.  One row of the packed tensor holds 16 consecutive k.  Columns are cut into groups
// of macro_n (256, 128 or 64) columns; with g = macro_n / 64 and pf = 32 / bits values per word the
// word that holds (k, n) is
//   row  k / 16
//   col  (n / macro_n) * g * W + ((k % 16) * (64 / pf) + (n % 64) / pf) * g + (n % macro_n) / 64
// with W = 1024 / pf, and inside the word the value sits at position pos(n % pf):
//   4-bit positions hold n%8 = 0,2,4,6,1,3,5,7;  8-bit positions hold n%4 = 0,2,1,3.
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline int macro_n_of(int64_t size_n) {
  return (size_n % 256 == 0) ? 256 : (size_n % 128 == 0) ? 128 : 64;
}

__host__ __device__ inline int nibble_pos(int j) { return (j & 1) * 4 + (j >> 1); }  // j = n % 8
__host__ __device__ inline int byte_pos(int j) { return (j & 1) * 2 + (j >> 1); }    // j = n % 4

template <int BITS>
__host__ __device__ inline int64_t packed_col(int lk, int n, int g) {
  constexpr int pf = 32 / BITS;
  constexpr int W = 1024 / pf;
  const int macro = g * 64;
  const int grp = n / macro;
  const int sub = (n % macro) / 64;
  const int nv = (n % 64) / pf;
  return (int64_t)grp * g * W + (int64_t)(lk * (64 / pf) + nv) * g + sub;
}

// ---------------------------------------------------------------------------------------------
// Scalar decoders (used by the generic kernel and as the definition the fast kernels follow).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float e2m1_value(int code) {
  // sign(1) exp(2) man(1): 0, .5, 1, 1.5, 2, 3, 4, 6
  const int e = (code >> 1) & 3, m = code & 1;
  float v = (e == 0) ? 0.5f * m : (1.0f + 0.5f * m) * (float)(1 << (e - 1));
  return (code & 8) ? -v : v;
}

__device__ __forceinline__ float e4m3_value(int b) {
  const int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
  float v = (e == 0) ? ldexpf((float)m, -9) : ldexpf(1.0f + m * 0.125f, e - 7);
  return s ? -v : v;
}

// nvfp4 block scale byte: value = fp16 whose bits are (byte << 7).
__device__ __forceinline__ float s0e5m3_value(int b) {
  return __half2float(__ushort_as_half((unsigned short)(b << 7)));
}

__device__ __forceinline__ float e8m0_value(int b) { return ldexpf(1.0f, b - 127); }

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Position of column n inside a row of the nvfp4 scale tensor ([0,2,1,3] interleave per 4).
__host__ __device__ inline int64_t nvfp4_scale_col(int64_t n) {
  const int j = (int)(n & 3);
  return (n & ~(int64_t)3) + ((j == 1) ? 2 : (j == 2) ? 1 : j);
}

// Un-permute the bias index: the bias crosses the boundary permuted per 32 columns.
__host__ __device__ inline int64_t bias_index(int64_t n) {
  // stored[p] = logical[perm[p]] with perm = for i in 0..3: 2i + {0,1,8,9,16,17,24,25}
  const int l = (int)(n & 31);
  const int i = (l & 7) >> 1;
  const int jj = (l >> 3) * 2 + (l & 1);
  return (n & ~(int64_t)31) + i * 8 + jj;
}

struct GemmArgs {
  const void* a;
  void* c;
  const int32_t* bq;
  const void* scales;
  const void* zeros;
  const void* bias;
  const float* global_scale;
  int act_dtype;
  int format;
  int64_t size_m;  // rows of A
  int64_t size_n;
  int64_t size_k;
  int64_t a_stride;
  int64_t num_groups;
  // grouped (MoE) part; sorted_ids == nullptr means dense
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post_pad;
  const float* topk_weights;
  int64_t num_sorted;
  int64_t num_experts;
  int block_size;
  int top_k;
  int mul_topk;
  void* scratch;
  int64_t scratch_bytes;
  cudaStream_t stream;
  bool prepared;  // b_q_weight is in the streaming layout (stream_layout.cuh)
  bool silu_input;  // grouped, streaming layout: `a` is [size_m, 2 * size_k] gate | up, SiLU-and-mul applied on load
};

// kernel launchers (one per translation unit)
int launch_gemm_generic(const GemmArgs& g);
// size_n % 256 != 0: operands copied into the 256-column form of a matrix padded to N' columns (gemm_pad.cu)
bool gemm_pad_applies(const GemmArgs& g);
int64_t gemm_pad_scratch_bytes(int64_t m, int64_t n, int64_t k, int format, int64_t inner);
int gemm_pad_prepare(const GemmArgs& g, GemmArgs* padded);   // 1: the scratch buffer cannot hold it
int gemm_pad_finish(const GemmArgs& g, const GemmArgs& padded);
int launch_gemm_decode(const GemmArgs& g);          // returns 1 if the shape is not handled
int64_t gemm_decode_scratch_bytes(int64_t m, int64_t n, int64_t k, int format);
int launch_gemm_decode_tc(const GemmArgs& g);       // returns 1 if the shape is not handled
int launch_gemm_tc(const GemmArgs& g);              // returns 1 if the shape is not handled
int launch_gemm_stream_f16(const GemmArgs& g);      // weights in the streaming layout
int launch_gemm_stream_bf16(const GemmArgs& g);
int64_t gemm_stream_scratch_bytes(int64_t m, int64_t n, int64_t k);
bool gemm_stream_i8_accepts(const GemmArgs& g);     // integer-MMA kernel for M <= 32, 4-bit integer formats
bool gemm_stream_i8_grouped_accepts(const GemmArgs& g);   // its grouped (expert) form: blocks of 8 / 16 / 32 routes
int launch_gemm_stream_i8_grouped(const GemmArgs& g);
int64_t gemm_stream_i8_grouped_scratch_bytes(int64_t num_sorted, int64_t n, int64_t k);
int launch_gemm_stream_i8(const GemmArgs& g);
int64_t gemm_stream_i8_scratch_bytes(int64_t m, int64_t n, int64_t k);
int64_t gemm_tc_scratch_bytes(int64_t m, int64_t n, int64_t k);
// give-up words of the three pipelined kernel families (0 = every wait completed)
int read_decode_status(int* value, bool reset);
int read_tc_status(int* value, bool reset);
int read_decode_tc_status(int* value, bool reset);
int read_stream_status_f16(int* value, bool reset);
int read_stream_status_bf16(int* value, bool reset);
int read_stream_i8_status(int* value, bool reset);

}  // namespace mb200
