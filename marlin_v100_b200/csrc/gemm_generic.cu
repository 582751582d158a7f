// Shape-agnostic GEMM kernel (CUDA cores, fp32 accumulate).
//
// Handles every legal shape (size_n % 64 == 0, size_k % 16 == 0, any M, dense or grouped) and is
// the path taken when no specialised kernel accepts the problem.  A CTA owns a 32-row x 64-column
// output tile and walks K in steps of 16: the packed words of the step are decoded once into shared
// memory (rounded to the activation type, exactly as the dequantise-then-matmul definition does),
// the activation rows are gathered beside them, and each thread accumulates a 2 x 4 patch.
#include "common.cuh"

namespace mb200 {
namespace {

constexpr int TM = 32;
constexpr int TN = 64;
constexpr int TK = 16;

template <typename T, int FMT>
__device__ __forceinline__ float decode_weight(uint32_t word, int j, float s, float z) {
  // j = n % pf (logical position in the word)
  if constexpr (FMT == kU4B8) {
    const int q = (word >> (4 * nibble_pos(j))) & 15;
    return to_float<T>(from_float<T>((float)(q - 8) * s));
  } else if constexpr (FMT == kU4) {
    const int q = (word >> (4 * nibble_pos(j))) & 15;
    return to_float<T>(from_float<T>((float)q * s - z));
  } else if constexpr (FMT == kU8B128) {
    const int q = (word >> (8 * byte_pos(j))) & 255;
    return to_float<T>(from_float<T>((float)(q - 128) * s));
  } else if constexpr (FMT == kU8) {
    const int q = (word >> (8 * byte_pos(j))) & 255;
    return to_float<T>(from_float<T>((float)q * s - z));
  } else if constexpr (FMT == kFP8) {
    const int q = (word >> (8 * byte_pos(j))) & 255;
    return to_float<T>(from_float<T>(e4m3_value(q) * s));
  } else {  // nvfp4 (s already holds decode(scale) * global / 2^bias) and mxfp4
    const int q = (word >> (4 * nibble_pos(j))) & 15;
    return to_float<T>(from_float<T>(e2m1_value(q) * s));
  }
}

template <typename T, int FMT>
__global__ void __launch_bounds__(256) gemm_generic_kernel(GemmArgs g) {
  constexpr int BITS = format_bits(FMT);
  constexpr int PF = 32 / BITS;
  __shared__ float sW[TK][TN + 1];
  __shared__ float sA[TM][TK + 1];
  __shared__ int sArow[TM];
  __shared__ int sCrow[TM];

  const int tid = threadIdx.x;
  const bool moe = g.sorted_ids != nullptr;
  const int n0 = blockIdx.y * TN;
  int expert = 0;

  // ---- which rows does this CTA own -----------------------------------------------------
  if (!moe) {
    const int64_t r0 = (int64_t)blockIdx.x * TM;
    if (tid < TM) {
      const int64_t r = r0 + tid;
      sArow[tid] = (r < g.size_m) ? (int)r : -1;
      sCrow[tid] = (r < g.size_m) ? (int)r : -1;
    }
  } else {
    const int sub_per_block = (g.block_size + TM - 1) / TM;
    const int blk = blockIdx.x / sub_per_block;
    const int sub = blockIdx.x % sub_per_block;
    const int64_t first = (int64_t)blk * g.block_size;
    if (first >= g.num_post_pad[0] || first >= g.num_sorted) return;
    expert = g.expert_ids[blk];
    if (expert < 0 || expert >= g.num_experts) return;
    if (tid < TM) {
      const int r = sub * TM + tid;
      int arow = -1, crow = -1;
      if (r < g.block_size && first + r < g.num_sorted) {
        const int sid = g.sorted_ids[first + r];
        if (sid >= 0 && (int64_t)sid < g.size_m * g.top_k) {
          arow = sid / g.top_k;
          crow = sid;
        }
      }
      sArow[tid] = arow;
      sCrow[tid] = crow;
    }
  }
  __syncthreads();

  const int gN = macro_n_of(g.size_n) / 64;
  const int64_t row_words = g.size_n * 16 / PF;
  const int64_t group_size = g.size_k / g.num_groups;
  const int32_t* bq = g.bq + (int64_t)expert * (g.size_k / 16) * row_words;
  const int64_t sbase = (int64_t)expert * g.num_groups * g.size_n;
  const T* scales = reinterpret_cast<const T*>(g.scales);
  const uint8_t* scales8 = reinterpret_cast<const uint8_t*>(g.scales);
  const T* zeros = reinterpret_cast<const T*>(g.zeros);
  const T* A = reinterpret_cast<const T*>(g.a);
  float fmt_mul = 1.0f;
  if constexpr (FMT == kFP8) fmt_mul = (sizeof(T) == 2 && std::is_same<T, __half>::value) ? ldexpf(1.f, -8) : ldexpf(1.f, -120);
  float gscale = 1.0f;
  if constexpr (FMT == kNVFP4) {
    // the e2m1 decoder yields true values; fold the 2^-bias of the boundary contract here
    gscale = g.global_scale[moe ? expert : 0] *
             (std::is_same<T, __half>::value ? ldexpf(1.f, -14) : ldexpf(1.f, -126));
  }

  float acc[2][4] = {};
  const int ty = tid / 16, tx = tid % 16;
  const int wl = tid / 16;        // lk handled when decoding
  const int wn = (tid % 16) * 4;  // first of 4 columns handled when decoding

  for (int64_t k0 = 0; k0 < g.size_k; k0 += TK) {
    // ---- decode 16 x 64 weights ------------------------------------------------------------
    {
      const int n = n0 + wn;
      const int64_t col = packed_col<BITS>(wl, n, gN);
      const uint32_t word = (uint32_t)bq[(k0 / 16) * row_words + col];
      const int64_t grp = (k0 + wl) / group_size;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float s, z = 0.f;
        if constexpr (FMT == kNVFP4) {
          // value = e2m1 / 2^bias * decode(byte) * global: products of powers of two and short
          // mantissas, exact in fp32 up to the final rounding
          s = s0e5m3_value(scales8[sbase + grp * g.size_n + nvfp4_scale_col(n + i)]) * gscale;
        } else if constexpr (FMT == kMXFP4) {
          s = e8m0_value(scales8[sbase + grp * g.size_n + n + i]);
        } else {
          s = to_float<T>(scales[sbase + grp * g.size_n + n + i]) * fmt_mul;
          if constexpr (format_has_zp(FMT)) z = to_float<T>(zeros[sbase + grp * g.size_n + n + i]);
        }
        sW[wl][wn + i] = decode_weight<T, FMT>(word, (n + i) % PF, s, z);
      }
    }
    // ---- gather 32 x 16 activations -----------------------------------------------------------
    for (int i = tid; i < TM * TK; i += 256) {
      const int r = i / TK, kk = i % TK;
      const int arow = sArow[r];
      sA[r][kk] = (arow >= 0) ? to_float<T>(A[(int64_t)arow * g.a_stride + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      const float a0 = sA[ty * 2][kk], a1 = sA[ty * 2 + 1][kk];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float w = sW[kk][tx * 4 + j];
        acc[0][j] = fmaf(a0, w, acc[0][j]);
        acc[1][j] = fmaf(a1, w, acc[1][j]);
      }
    }
    __syncthreads();
  }

  // ---- epilogue ------------------------------------------------------------------------------
  T* C = reinterpret_cast<T*>(g.c);
  const T* bias = reinterpret_cast<const T*>(g.bias);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int crow = sCrow[ty * 2 + i];
    if (crow < 0) continue;
    float tw = 1.f;
    if (moe && g.mul_topk) tw = g.topk_weights[crow];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      float v = acc[i][j];
      if (bias != nullptr) {
        float b = to_float<T>(bias[(int64_t)expert * g.size_n + bias_index(n)]);
        if constexpr (FMT == kNVFP4) {
          // the reference scales the bias by the expert's global scale when it also applies the
          // router weight (sm70_marlin_gemm.cuh:3490-3504); the accumulator already carries it
          if (moe && g.mul_topk) b *= g.global_scale[expert];
        }
        v += b;
      }
      C[(int64_t)crow * g.size_n + n] = from_float<T>(v * tw);
    }
  }
}

template <typename T>
int launch_t(const GemmArgs& g) {
  dim3 grid;
  if (g.sorted_ids == nullptr) {
    grid = dim3((unsigned)((g.size_m + TM - 1) / TM), (unsigned)(g.size_n / TN));
  } else {
    const int64_t blocks = g.num_sorted / g.block_size;
    const int sub = (g.block_size + TM - 1) / TM;
    if (blocks == 0) return 0;
    grid = dim3((unsigned)(blocks * sub), (unsigned)(g.size_n / TN));
  }
  switch (g.format) {
#define CASE(F)                                                          \
  case F:                                                                \
    gemm_generic_kernel<T, F><<<grid, 256, 0, g.stream>>>(g);            \
    break;
    CASE(kU4B8) CASE(kU4) CASE(kU8B128) CASE(kU8) CASE(kFP8) CASE(kNVFP4) CASE(kMXFP4)
#undef CASE
    default:
      set_error("unsupported format %d", g.format);
      return MARLIN_B200_EINVAL;
  }
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

}  // namespace

int launch_gemm_generic(const GemmArgs& g) {
  if (g.act_dtype == MARLIN_B200_F16) return launch_t<__half>(g);
  return launch_t<__nv_bfloat16>(g);
}

}  // namespace mb200
