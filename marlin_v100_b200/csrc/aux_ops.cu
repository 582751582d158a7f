// Small integer operators that the reference registers next to the GEMMs.
//
//  * marlin_b200_int4_fp8_preprocess: per 4-bit code, value >= zero ? value - zero : 15 - value, with zero = 8
//    (symmetric checkpoints) or the code's own AWQ zero-point
//    (csrc/quantization/marlin/marlin_int4_fp8_preprocess.cu:8-56 of the reference).  One thread per packed
//    word of eight codes, any tensor shape.
//  * scale re-encoders of the fp4 / fp8 checkpoints, which the reference runs as eager PyTorch at load time
//    (vllm/model_executor/layers/quantization/utils/marlin_utils_fp4.py:30-129, marlin_utils_fp8.py:28-39):
//    nvfp4 block scales -> the S0E5M3 bytes the GEMM reads (with the power-of-two rescale and its minimum
//    search), the [0,2,1,3] byte interleave of mxfp4 scales, fp8 scales times 2^bias.
//  * marlin_b200_batched_moe_align_block_size: block lists for tokens that are already grouped by expert
//    (csrc/moe/moe_align_sum_kernels.cu:22-78,571-596).  Every output position finds its expert by a
//    search in the prefix sums, so the kernel is one pass over the outputs on any number of CTAs.
#include "common.cuh"

namespace mb200 {
namespace {

// per nibble: v >= z ? v - z : 15 - v
__device__ __forceinline__ uint32_t preprocess_word(uint32_t v, uint32_t z) {
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t a = (v >> (4 * i)) & 15u, b = (z >> (4 * i)) & 15u;
    out |= ((a >= b) ? (a - b) : (15u - a)) << (4 * i);
  }
  return out;
}

__global__ void __launch_bounds__(256) int4_fp8_preprocess_kernel(const uint32_t* __restrict__ in,
                                                                  const uint32_t* __restrict__ zeros,
                                                                  uint32_t* __restrict__ out, int64_t total,
                                                                  int64_t words_per_row, int64_t rows_per_zero) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    uint32_t z = 0x88888888u;
    if (zeros != nullptr) {
      const int64_t row = i / words_per_row, col = i % words_per_row;
      z = zeros[(row / rows_per_zero) * words_per_row + col];
    }
    out[i] = preprocess_word(in[i], z);
  }
}

__global__ void __launch_bounds__(256) batched_align_kernel(const int32_t* __restrict__ counts, int num_batches,
                                                            int max_tokens, int block_size,
                                                            int32_t* __restrict__ sorted_ids, int64_t sorted_size,
                                                            int32_t* __restrict__ block_ids, int64_t num_blocks,
                                                            int32_t* __restrict__ num_post_pad) {
  extern __shared__ int s_off[];   // num_batches + 1 padded prefix sums (in tokens)
  __shared__ int s_scan[256];
  const int tid = threadIdx.x;
  // inclusive scan of the padded counts, 256 per round
  int carry = 0;
  for (int b0 = 0; b0 < num_batches; b0 += 256) {
    const int b = b0 + tid;
    int v = 0;
    if (b < num_batches) v = (counts[b] + block_size - 1) / block_size * block_size;
    s_scan[tid] = v;
    __syncthreads();
    for (int o = 1; o < 256; o <<= 1) {
      const int t = (tid >= o) ? s_scan[tid - o] : 0;
      __syncthreads();
      s_scan[tid] += t;
      __syncthreads();
    }
    if (b < num_batches) s_off[b + 1] = carry + s_scan[tid];
    carry += s_scan[255];
    __syncthreads();
  }
  if (tid == 0) {
    s_off[0] = 0;
    if (blockIdx.x == 0) *num_post_pad = carry;
  }
  __syncthreads();
  const int total = carry;
  const int sentinel = num_batches * max_tokens;
  const int64_t gsize = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + tid; i < sorted_size; i += gsize) {
    int value = sentinel;
    if (i < total) {
      int lo = 0, hi = num_batches;   // the batch b with s_off[b] <= i < s_off[b + 1]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= (int)i) lo = mid; else hi = mid;
      }
      const int local = (int)i - s_off[lo];
      if (local < counts[lo]) value = lo * max_tokens + local;
    }
    sorted_ids[i] = value;
  }
  for (int64_t j = (int64_t)blockIdx.x * blockDim.x + tid; j < num_blocks; j += gsize) {
    int value = -1;
    const int64_t pos = j * block_size;
    if (pos < total) {
      int lo = 0, hi = num_batches;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= (int)pos) lo = mid; else hi = mid;
      }
      value = lo;
    }
    block_ids[j] = value;
  }
}

// smallest non-zero value of h * 2^7 over all scales, as float bits (positive floats order like unsigned ints)
__global__ void __launch_bounds__(256) nvfp4_scale_min_kernel(const __half* __restrict__ in, int64_t count,
                                                              unsigned int* __restrict__ min_bits) {
  unsigned int best = 0x7f800000u;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = __half2float(in[i]) * 128.f;
    if (v > 0.f) best = min(best, __float_as_uint(v));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
  if ((threadIdx.x & 31) == 0 && best != 0x7f800000u) atomicMin(min_bits, best);
}

// out[r][4 q + j] = encode(in[r][4 q + {0,2,1,3}[j]]): times scale_factor (rounded to half), times 2^7 in half,
// the half's bits shifted left by one, high byte
__global__ void __launch_bounds__(256) nvfp4_process_scales_kernel(const __half* __restrict__ in,
                                                                   uint8_t* __restrict__ out, int64_t count,
                                                                   float scale_factor) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(i & 3);
    const int64_t src = (i & ~(int64_t)3) + ((j == 1) ? 2 : (j == 2) ? 1 : j);
    __half h = in[src];
    if (scale_factor > 1.f) h = __float2half_rn(__half2float(h) * scale_factor);
    h = __hmul(h, __float2half_rn(128.f));
    const unsigned short bits = (unsigned short)(__half_as_ushort(h) << 1);
    out[i] = (uint8_t)(bits >> 8);
  }
}

__global__ void __launch_bounds__(256) interleave_bytes4_kernel(const uint8_t* __restrict__ in,
                                                                uint8_t* __restrict__ out, int64_t count) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(i & 3);
    out[i] = in[(i & ~(int64_t)3) + ((j == 1) ? 2 : (j == 2) ? 1 : j)];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) fp8_fuse_bias_kernel(const T* __restrict__ in, T* __restrict__ out,
                                                            int64_t count, float factor) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = from_float<T>(to_float<T>(in[i]) * factor);
}

int elementwise_grid(int64_t count) {
  const int64_t want = (count + 255) / 256, cap = (int64_t)sm_count() * 16;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace
}  // namespace mb200

using namespace mb200;

// Smallest non-zero scale times 2^7 of an nvfp4 scale tensor (fp16), written to *min_out as a float (+inf when
// every scale is zero).  The caller derives the rescale: 2^ceil(log2(2 / min)) when min < 2, else 1.
extern "C" int marlin_b200_nvfp4_scale_min(const void* scales_half, int64_t count, float* min_out, void* stream) {
  MB_CHECK(count >= 0 && min_out != nullptr, "bad arguments");
  auto s = (cudaStream_t)stream;
  const unsigned int inf_bits = 0x7f800000u;
  MB_CUDA(cudaMemcpyAsync(min_out, &inf_bits, sizeof(inf_bits), cudaMemcpyHostToDevice, s));
  if (count == 0) return 0;
  MB_CHECK(scales_half != nullptr, "null tensor pointer");
  nvfp4_scale_min_kernel<<<elementwise_grid(count), 256, 0, s>>>((const __half*)scales_half, count,
                                                                 reinterpret_cast<unsigned int*>(min_out));
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

// nvfp4 block scales (fp16 values of the e4m3 scales, [rows][cols], cols % 4 == 0) -> the bytes the GEMM reads.
extern "C" int marlin_b200_nvfp4_process_scales(const void* scales_half, uint8_t* out, int64_t rows, int64_t cols,
                                                float scale_factor, void* stream) {
  MB_CHECK(rows >= 0 && cols >= 0 && cols % 4 == 0, "scale columns must be a multiple of 4");
  MB_CHECK(scale_factor >= 1.f, "scale_factor must be a power of two >= 1");
  const int64_t count = rows * cols;
  if (count == 0) return 0;
  MB_CHECK(scales_half != nullptr && out != nullptr, "null tensor pointer");
  nvfp4_process_scales_kernel<<<elementwise_grid(count), 256, 0, (cudaStream_t)stream>>>(
      (const __half*)scales_half, out, count, scale_factor);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

// The [0,2,1,3] interleave per four columns of one-byte scales (mxfp4's e8m0 bytes in the reference's own form).
extern "C" int marlin_b200_interleave_scale_bytes(const uint8_t* in, uint8_t* out, int64_t rows, int64_t cols,
                                                  void* stream) {
  MB_CHECK(rows >= 0 && cols >= 0 && cols % 4 == 0, "scale columns must be a multiple of 4");
  const int64_t count = rows * cols;
  if (count == 0) return 0;
  MB_CHECK(in != nullptr && out != nullptr && in != out, "null or aliased tensor pointer");
  interleave_bytes4_kernel<<<elementwise_grid(count), 256, 0, (cudaStream_t)stream>>>(in, out, count);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

// fp8 scales times 2^8 (fp16) or 2^120 (bf16), rounded to the scales' own type; out may be in.
extern "C" int marlin_b200_fp8_fuse_exponent_bias(const void* in, void* out, int64_t count, int act_dtype,
                                                  void* stream) {
  MB_CHECK(count >= 0, "negative size");
  MB_CHECK(act_dtype == MARLIN_B200_F16 || act_dtype == MARLIN_B200_BF16, "scales must be fp16 or bf16");
  if (count == 0) return 0;
  MB_CHECK(in != nullptr && out != nullptr, "null tensor pointer");
  auto s = (cudaStream_t)stream;
  if (act_dtype == MARLIN_B200_F16)
    fp8_fuse_bias_kernel<__half><<<elementwise_grid(count), 256, 0, s>>>((const __half*)in, (__half*)out, count, 256.f);
  else
    fp8_fuse_bias_kernel<__nv_bfloat16><<<elementwise_grid(count), 256, 0, s>>>(
        (const __nv_bfloat16*)in, (__nv_bfloat16*)out, count, 1.329227995784916e36f);   // 2^120
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

extern "C" int marlin_b200_int4_fp8_preprocess(const int32_t* qweight, const int32_t* qzeros, int32_t* out,
                                               int64_t rows, int64_t words_per_row, int64_t zero_rows,
                                               void* stream) {
  MB_CHECK(rows >= 0 && words_per_row >= 0, "negative size");
  const int64_t total = rows * words_per_row;
  if (total == 0) return 0;
  MB_CHECK(qweight != nullptr && out != nullptr, "null tensor pointer");
  int64_t rows_per_zero = 1;
  if (qzeros != nullptr) {
    MB_CHECK(zero_rows >= 1 && rows % zero_rows == 0, "qweight.size(0) %% qzeros.size(0) != 0");
    rows_per_zero = rows / zero_rows;
    MB_CHECK(rows_per_zero % 8 == 0, "group_size %% 8 != 0");
  }
  const int64_t want = (total + 255) / 256, cap = (int64_t)sm_count() * 16;
  int4_fp8_preprocess_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint32_t*>(qweight), reinterpret_cast<const uint32_t*>(qzeros),
      reinterpret_cast<uint32_t*>(out), total, words_per_row, rows_per_zero);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

extern "C" int marlin_b200_batched_moe_align_block_size(int64_t max_tokens_per_batch, int block_size,
                                                        const int32_t* expert_num_tokens, int64_t num_batches,
                                                        int32_t* sorted_token_ids, int64_t sorted_size,
                                                        int32_t* block_ids, int64_t num_blocks,
                                                        int32_t* num_tokens_post_pad, void* stream) {
  MB_CHECK(block_size > 0 && max_tokens_per_batch >= 0, "block_size must be positive");
  MB_CHECK(num_batches >= 1 && num_batches <= 8192, "number of experts %lld out of range (1..8192)",
           (long long)num_batches);
  MB_CHECK(num_batches * max_tokens_per_batch < (1ll << 31), "batch sizes do not fit 32-bit ids");
  const int64_t blocks_per_batch = (max_tokens_per_batch + block_size - 1) / block_size;
  MB_CHECK(sorted_size == blocks_per_batch * num_batches * block_size,
           "sorted_token_ids has %lld entries, expected %lld", (long long)sorted_size,
           (long long)(blocks_per_batch * num_batches * block_size));
  MB_CHECK(num_blocks == sorted_size / block_size, "experts_ids has %lld entries, expected %lld",
           (long long)num_blocks, (long long)(sorted_size / block_size));
  MB_CHECK(expert_num_tokens != nullptr && sorted_token_ids != nullptr && block_ids != nullptr &&
               num_tokens_post_pad != nullptr, "null tensor pointer");
  const int64_t want = (sorted_size + 255) / 256 + 1, cap = (int64_t)sm_count() * 4;
  batched_align_kernel<<<(unsigned)(want < cap ? want : cap), 256, (size_t)(num_batches + 1) * 4,
                         (cudaStream_t)stream>>>(expert_num_tokens, (int)num_batches, (int)max_tokens_per_batch,
                                                 block_size, sorted_token_ids, sorted_size, block_ids, num_blocks,
                                                 num_tokens_post_pad);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}
