// Routing helpers of the fused expert layer: softmax top-k gating, stable token sorting into
// expert blocks, and the two elementwise glue steps (SiLU-and-mul, top-k sum).
#include "common.cuh"

namespace mb200 {
namespace {

// ---------------------------------------------------------------------------------------------
// moe_align_block_size
//
// Stable counting sort of the flat route indices by (mapped) expert id, each expert padded to a
// multiple of block_size.  Three steps: (1) every CTA histograms its chunk of CHUNK routes and the
// output buffer is pre-filled with the padding value; (2) one CTA turns the per-chunk histograms
// into per-chunk start offsets, pads, scans the experts and writes expert_ids / the total;
// (3) every CTA re-reads its chunk and places each route at start[chunk][expert] + (number of
// earlier routes of that expert inside the chunk), which keeps ascending order inside an expert.
// Small inputs run all three steps in a single CTA.
// ---------------------------------------------------------------------------------------------
constexpr int CHUNK = 1024;
constexpr int MAX_SMEM_EXPERTS = 2048;

__device__ __forceinline__ int map_expert(const int32_t* ids, int64_t i, const int32_t* emap,
                                          int num_global, int num_experts) {
  int e = ids[i];
  if (emap != nullptr) e = (e >= 0 && e < num_global) ? emap[e] : -1;
  return (e >= 0 && e < num_experts) ? e : -1;
}

// Places the routes of one chunk.  cnt[] holds, per expert, the next free slot.
__device__ void place_chunk(const int32_t* ids, int64_t begin, int64_t end, const int32_t* emap,
                            int num_global, int num_experts, int* cnt, int32_t* sorted) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int64_t base = begin; base < end; base += blockDim.x) {
    const int64_t i = base + threadIdx.x;
    const int e = (i < end) ? map_expert(ids, i, emap, num_global, num_experts) : -1;
    for (int w = 0; w < nwarps; ++w) {
      if (w == warp) {
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        if (e >= 0) {
          const int rank = __popc(peers & ((1u << lane) - 1u));
          const int old = cnt[e];
          __syncwarp(peers);
          if (rank == 0) cnt[e] = old + __popc(peers);
          sorted[old + rank] = (int32_t)i;
        }
      }
      __syncthreads();
    }
  }
}

// Exclusive scan of padded counts + expert_ids + total, by one CTA.  counts[] in shared memory is
// replaced by the start of every expert.
__device__ void scan_and_write_experts(int* counts, int num_experts, int block_size,
                                       int32_t* expert_ids, int64_t expert_ids_capacity,
                                       int32_t* total_out, int* s_total) {
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < num_experts; ++e) {
      const int padded = (counts[e] + block_size - 1) / block_size * block_size;
      counts[e] = run;
      run += padded;
    }
    counts[num_experts] = run;
    *s_total = run;
    *total_out = run;
  }
  __syncthreads();
  const int nblocks = *s_total / block_size;
  for (int64_t b = threadIdx.x; b < expert_ids_capacity; b += blockDim.x) {
    int e = -1;
    if (b < nblocks) {
      const int pos = (int)b * block_size;
      int lo = 0, hi = num_experts;  // last expert with start <= pos and start(e+1) > pos
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (counts[mid] <= pos) lo = mid; else hi = mid;
      }
      // skip experts with zero blocks that share the same start
      while (lo + 1 <= num_experts && counts[lo + 1] <= pos) ++lo;
      e = lo;
    }
    expert_ids[b] = e;
  }
}

__global__ void __launch_bounds__(1024) align_single_cta_kernel(
    const int32_t* ids, int64_t numel, int num_experts, int num_global, int block_size,
    const int32_t* emap, int32_t* sorted, int64_t sorted_capacity, int32_t* expert_ids,
    int64_t expert_ids_capacity, int32_t* total_out) {
  extern __shared__ int smem[];
  int* counts = smem;  // [num_experts + 1]
  __shared__ int s_total;
  for (int e = threadIdx.x; e <= num_experts; e += blockDim.x) counts[e] = 0;
  for (int64_t i = threadIdx.x; i < sorted_capacity; i += blockDim.x) sorted[i] = (int32_t)numel;
  __syncthreads();
  for (int64_t i = threadIdx.x; i < numel; i += blockDim.x) {
    const int e = map_expert(ids, i, emap, num_global, num_experts);
    if (e >= 0) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  scan_and_write_experts(counts, num_experts, block_size, expert_ids, expert_ids_capacity, total_out,
                         &s_total);
  __syncthreads();
  place_chunk(ids, 0, numel, emap, num_global, num_experts, counts, sorted);
}

__global__ void __launch_bounds__(1024) align_hist_kernel(const int32_t* ids, int64_t numel,
                                                          int num_experts, int num_global,
                                                          const int32_t* emap, int* hist,
                                                          int32_t* sorted, int64_t sorted_capacity) {
  extern __shared__ int smem[];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) smem[e] = 0;
  __syncthreads();
  const int64_t begin = (int64_t)blockIdx.x * CHUNK;
  const int64_t end = begin + CHUNK < numel ? begin + CHUNK : numel;
  for (int64_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const int e = map_expert(ids, i, emap, num_global, num_experts);
    if (e >= 0) atomicAdd(&smem[e], 1);
  }
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < sorted_capacity;
       i += (int64_t)gridDim.x * blockDim.x)
    sorted[i] = (int32_t)numel;
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x)
    hist[(int64_t)blockIdx.x * num_experts + e] = smem[e];
}

__global__ void __launch_bounds__(1024) align_scan_kernel(int* hist, int num_chunks, int num_experts,
                                                          int block_size, int32_t* expert_ids,
                                                          int64_t expert_ids_capacity,
                                                          int32_t* total_out) {
  extern __shared__ int smem[];
  int* counts = smem;
  __shared__ int s_total;
  // per expert: turn the chunk histograms into exclusive prefixes (in place), keep the total
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < num_chunks; ++c) {
      const int v = hist[(int64_t)c * num_experts + e];
      hist[(int64_t)c * num_experts + e] = run;
      run += v;
    }
    counts[e] = run;
  }
  __syncthreads();
  scan_and_write_experts(counts, num_experts, block_size, expert_ids, expert_ids_capacity, total_out,
                         &s_total);
  __syncthreads();
  // fold the expert start into every chunk prefix
  for (int64_t i = threadIdx.x; i < (int64_t)num_chunks * num_experts; i += blockDim.x)
    hist[i] += counts[i % num_experts];
}

__global__ void __launch_bounds__(1024) align_place_kernel(const int32_t* ids, int64_t numel,
                                                           int num_experts, int num_global,
                                                           const int32_t* emap, const int* hist,
                                                           int32_t* sorted) {
  extern __shared__ int smem[];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x)
    smem[e] = hist[(int64_t)blockIdx.x * num_experts + e];
  __syncthreads();
  const int64_t begin = (int64_t)blockIdx.x * CHUNK;
  const int64_t end = begin + CHUNK < numel ? begin + CHUNK : numel;
  place_chunk(ids, begin, end, emap, num_global, num_experts, smem, sorted);
}

// ---------------------------------------------------------------------------------------------
// topk_softmax: one warp per row.  Lane l owns columns c*128 + l*4 + i (i < 4), the mapping of the
// reference kernel for fp32 logits (topk_softmax_kernels.cu:567-588), so that partial sums follow
// the same order; max and sum are xor-butterflies; each of the k rounds picks the largest remaining
// probability, the lower index winning ties.
// ---------------------------------------------------------------------------------------------
constexpr int MAX_COLS_PER_LANE = 32;  // up to 1024 experts

template <typename T>
__device__ __forceinline__ float load_logit(const T* p) { return to_float<T>(*p); }
template <>
__device__ __forceinline__ float load_logit<float>(const float* p) { return *p; }

// SIGMOID: the scores are 1 / (1 + exp(-x)) per expert instead of the softmax over the row (topk_sigmoid of the
// reference, csrc/moe/topk_softmax_kernels.cu:436-441); selection, bias and renormalisation are the same.
template <typename T, bool SIGMOID>
__global__ void __launch_bounds__(128) topk_softmax_kernel(const T* __restrict__ gating,
                                                           const float* __restrict__ bias,
                                                           float* __restrict__ weights,
                                                           int32_t* __restrict__ indices,
                                                           int32_t* __restrict__ tei,
                                                           int64_t num_tokens, int num_experts,
                                                           int topk, int renormalize) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= num_tokens) return;
  const int chunks = (num_experts + 127) / 128;
  float p[MAX_COLS_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int c = 0; c < MAX_COLS_PER_LANE / 4; ++c) {
    if (c < chunks) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = c * 128 + lane * 4 + i;
        const float v = (col < num_experts) ? load_logit<T>(gating + row * num_experts + col) : -INFINITY;
        p[c * 4 + i] = v;
        mx = fmaxf(mx, v);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if constexpr (SIGMOID) {
#pragma unroll
    for (int c = 0; c < MAX_COLS_PER_LANE / 4; ++c)
      if (c < chunks) {
#pragma unroll
        for (int i = 0; i < 4; ++i) p[c * 4 + i] = 1.0f / (1.0f + __expf(-p[c * 4 + i]));
      }
  } else {
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < MAX_COLS_PER_LANE / 4; ++c) {
      if (c < chunks) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float e = expf(p[c * 4 + i] - mx);
          p[c * 4 + i] = e;
          sum += e;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
#pragma unroll
    for (int c = 0; c < MAX_COLS_PER_LANE / 4; ++c)
      if (c < chunks) {
#pragma unroll
        for (int i = 0; i < 4; ++i) p[c * 4 + i] *= inv;
      }
  }

  // selection scores (probability + optional bias); taken entries become -inf
  float s[MAX_COLS_PER_LANE];
#pragma unroll
  for (int c = 0; c < MAX_COLS_PER_LANE / 4; ++c)
    if (c < chunks) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = c * 128 + lane * 4 + i;
        s[c * 4 + i] = (col < num_experts) ? (bias ? p[c * 4 + i] + bias[col] : p[c * 4 + i]) : -INFINITY;
      }
    }

  float wsum = 0.f;
  float my_w = 0.f;  // lane j keeps the weight of the j-th pick (topk <= 32)
  for (int j = 0; j < topk; ++j) {
    float best = -INFINITY, bestp = 0.f;
    int besti = 0x7fffffff;
#pragma unroll
    for (int c = 0; c < MAX_COLS_PER_LANE / 4; ++c)
      if (c < chunks) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = c * 128 + lane * 4 + i;
          if (s[c * 4 + i] > best) {  // strict: the first (lowest) column wins inside a lane
            best = s[c * 4 + i];
            besti = col;
            bestp = p[c * 4 + i];
          }
        }
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      const float op = __shfl_xor_sync(0xffffffffu, bestp, o);
      if (ob > best || (ob == best && oi < besti)) {
        best = ob;
        besti = oi;
        bestp = op;
      }
    }
    // remove the winner
#pragma unroll
    for (int c = 0; c < MAX_COLS_PER_LANE / 4; ++c)
      if (c < chunks) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (c * 128 + lane * 4 + i == besti) s[c * 4 + i] = -INFINITY;
      }
    wsum += bestp;
    if (lane == j) my_w = bestp;
    if (lane == 0) {
      indices[row * topk + j] = besti;
      tei[row * topk + j] = (int32_t)(j * num_tokens + row);
    }
  }
  if (lane < topk) {
    if (renormalize) my_w = my_w / fmaxf(wsum, 1e-20f);
    weights[row * topk + lane] = my_w;
  }
}

// ---------------------------------------------------------------------------------------------
// elementwise glue
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) silu_and_mul_kernel(const T* __restrict__ in, T* __restrict__ out,
                                                           int64_t rows, int64_t inter) {
  // 8 elements (16 bytes) per thread step
  const int64_t vec_per_row = inter / 8;
  const int64_t total = rows * vec_per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / vec_per_row, v = idx % vec_per_row;
    const uint4 g4 = *reinterpret_cast<const uint4*>(in + r * 2 * inter + v * 8);
    const uint4 u4 = *reinterpret_cast<const uint4*>(in + r * 2 * inter + inter + v * 8);
    const T* gp = reinterpret_cast<const T*>(&g4);
    const T* up = reinterpret_cast<const T*>(&u4);
    uint4 o4;
    T* op = reinterpret_cast<T*>(&o4);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float x = to_float<T>(gp[i]);
      // round silu(x) to the storage type before the product, as the eager reference does
      const float sl = to_float<T>(from_float<T>(x / (1.f + expf(-x))));
      op[i] = from_float<T>(sl * to_float<T>(up[i]));
    }
    *reinterpret_cast<uint4*>(out + r * inter + v * 8) = o4;
  }
}

// rows == nullptr: in is [tokens, top_k, hidden].  Otherwise rows[t * top_k + j] is the row of `in` that
// holds the contribution of route j of token t (rows of an all-to-all that came back in sender order).
template <typename T>
__global__ void __launch_bounds__(256) moe_sum_kernel(const T* __restrict__ in, T* __restrict__ out,
                                                      const int32_t* __restrict__ rows, int64_t tokens, int top_k,
                                                      int64_t hidden) {
  const int64_t vec_per_row = hidden / 8;
  const int64_t total = tokens * vec_per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / vec_per_row, v = idx % vec_per_row;
    float acc[8] = {};
    for (int j = 0; j < top_k; ++j) {
      const int64_t row = rows != nullptr ? (int64_t)rows[t * top_k + j] : t * top_k + j;
      const uint4 x4 = *reinterpret_cast<const uint4*>(in + row * hidden + v * 8);
      const T* xp = reinterpret_cast<const T*>(&x4);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += to_float<T>(xp[i]);
    }
    uint4 o4;
    T* op = reinterpret_cast<T*>(&o4);
#pragma unroll
    for (int i = 0; i < 8; ++i) op[i] = from_float<T>(acc[i]);
    *reinterpret_cast<uint4*>(out + t * hidden + v * 8) = o4;
  }
}

int grid_for(int64_t total, int threads) {
  const int64_t want = (total + threads - 1) / threads;
  const int64_t cap = (int64_t)sm_count() * 8;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" int64_t marlin_b200_moe_align_scratch_bytes(int64_t numel, int64_t num_experts) {
  const int64_t chunks = (numel + CHUNK - 1) / CHUNK;
  return (chunks * num_experts + 64) * (int64_t)sizeof(int);
}

extern "C" int marlin_b200_moe_align_block_size(
    const int32_t* topk_ids, int64_t numel, int64_t num_experts, int64_t num_global_experts,
    int block_size, const int32_t* expert_map, int32_t* sorted_token_ids, int64_t sorted_capacity,
    int32_t* expert_ids, int64_t expert_ids_capacity, int32_t* num_tokens_post_pad, void* scratch,
    int64_t scratch_bytes, void* stream) {
  MB_CHECK(block_size > 0, "block_size must be positive, got %d", block_size);
  MB_CHECK(num_experts > 0 && num_experts <= MAX_SMEM_EXPERTS, "num_experts = %lld out of range (1..%d)",
           (long long)num_experts, MAX_SMEM_EXPERTS);
  MB_CHECK(numel < (1ll << 31), "numel too large");
  MB_CHECK(scratch == nullptr || ((uintptr_t)scratch & 255) == 0, "scratch must be aligned to 256 bytes");
  const int64_t need = numel + num_experts * (block_size - 1);
  MB_CHECK(sorted_capacity >= (numel == 0 ? 0 : need) || sorted_capacity >= need,
           "sorted_token_ids has %lld entries, needs %lld", (long long)sorted_capacity, (long long)need);
  auto s = (cudaStream_t)stream;
  const size_t smem = (size_t)(num_experts + 1) * sizeof(int);
  if (numel <= 4 * CHUNK) {
    align_single_cta_kernel<<<1, 1024, smem, s>>>(topk_ids, numel, (int)num_experts,
                                                  (int)num_global_experts, block_size, expert_map,
                                                  sorted_token_ids, sorted_capacity, expert_ids,
                                                  expert_ids_capacity, num_tokens_post_pad);
    MB_CUDA(cudaGetLastError());
    count_launches(1);
    return 0;
  }
  if (scratch_bytes < marlin_b200_moe_align_scratch_bytes(numel, num_experts) || scratch == nullptr) {
    set_error("moe_align scratch too small: %lld < %lld", (long long)scratch_bytes,
              (long long)marlin_b200_moe_align_scratch_bytes(numel, num_experts));
    return MARLIN_B200_ESCRATCH;
  }
  const int chunks = (int)((numel + CHUNK - 1) / CHUNK);
  int* hist = reinterpret_cast<int*>(scratch);
  align_hist_kernel<<<chunks, 1024, smem, s>>>(topk_ids, numel, (int)num_experts,
                                               (int)num_global_experts, expert_map, hist,
                                               sorted_token_ids, sorted_capacity);
  align_scan_kernel<<<1, 1024, smem, s>>>(hist, chunks, (int)num_experts, block_size, expert_ids,
                                          expert_ids_capacity, num_tokens_post_pad);
  align_place_kernel<<<chunks, 1024, smem, s>>>(topk_ids, numel, (int)num_experts,
                                                (int)num_global_experts, expert_map, hist,
                                                sorted_token_ids);
  MB_CUDA(cudaGetLastError());
  count_launches(3);
  return 0;
}

namespace {
template <bool SIGMOID>
int launch_topk(const void* gating, int gating_dtype, const float* bias, float* topk_weights, int32_t* topk_indices,
                int32_t* token_expert_indices, int64_t num_tokens, int64_t num_experts, int topk, int renormalize,
                void* stream) {
  MB_CHECK(num_experts >= 1 && num_experts <= 128 * (MAX_COLS_PER_LANE / 4),
           "num_experts = %lld not supported (1..%d)", (long long)num_experts,
           128 * (MAX_COLS_PER_LANE / 4));
  MB_CHECK(topk >= 1 && topk <= 32 && topk <= num_experts, "topk = %d not supported", topk);
  if (num_tokens == 0) return 0;
  auto s = (cudaStream_t)stream;
  const unsigned grid = (unsigned)((num_tokens + 3) / 4);
  switch (gating_dtype) {
    case MARLIN_B200_F16:
      topk_softmax_kernel<__half, SIGMOID><<<grid, 128, 0, s>>>((const __half*)gating, bias, topk_weights,
                                                                topk_indices, token_expert_indices, num_tokens,
                                                                (int)num_experts, topk, renormalize);
      break;
    case MARLIN_B200_BF16:
      topk_softmax_kernel<__nv_bfloat16, SIGMOID><<<grid, 128, 0, s>>>(
          (const __nv_bfloat16*)gating, bias, topk_weights, topk_indices, token_expert_indices,
          num_tokens, (int)num_experts, topk, renormalize);
      break;
    case 2:
      topk_softmax_kernel<float, SIGMOID><<<grid, 128, 0, s>>>((const float*)gating, bias, topk_weights,
                                                               topk_indices, token_expert_indices, num_tokens,
                                                               (int)num_experts, topk, renormalize);
      break;
    default:
      MB_CHECK(false, "unsupported gating dtype %d", gating_dtype);
  }
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}
}  // namespace

extern "C" int marlin_b200_topk_softmax(const void* gating, int gating_dtype, const float* bias,
                                        float* topk_weights, int32_t* topk_indices,
                                        int32_t* token_expert_indices, int64_t num_tokens,
                                        int64_t num_experts, int topk, int renormalize, void* stream) {
  return launch_topk<false>(gating, gating_dtype, bias, topk_weights, topk_indices, token_expert_indices, num_tokens,
                            num_experts, topk, renormalize, stream);
}

extern "C" int marlin_b200_topk_sigmoid(const void* gating, int gating_dtype, const float* bias,
                                        float* topk_weights, int32_t* topk_indices,
                                        int32_t* token_expert_indices, int64_t num_tokens,
                                        int64_t num_experts, int topk, int renormalize, void* stream) {
  return launch_topk<true>(gating, gating_dtype, bias, topk_weights, topk_indices, token_expert_indices, num_tokens,
                           num_experts, topk, renormalize, stream);
}

extern "C" int marlin_b200_silu_and_mul(const void* in, void* out, int64_t rows, int64_t inter,
                                        int act_dtype, void* stream) {
  MB_CHECK(inter % 8 == 0, "silu_and_mul needs the intermediate size to be a multiple of 8, got %lld",
           (long long)inter);
  if (rows == 0 || inter == 0) return 0;
  auto s = (cudaStream_t)stream;
  const int grid = grid_for(rows * inter / 8, 256);
  if (act_dtype == MARLIN_B200_F16)
    silu_and_mul_kernel<__half><<<grid, 256, 0, s>>>((const __half*)in, (__half*)out, rows, inter);
  else
    silu_and_mul_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)in,
                                                            (__nv_bfloat16*)out, rows, inter);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

extern "C" int marlin_b200_moe_sum(const void* in, void* out, int64_t tokens, int top_k, int64_t hidden,
                                   int act_dtype, void* stream) {
  return marlin_b200_moe_sum_rows(in, nullptr, out, tokens, top_k, hidden, act_dtype, stream);
}

extern "C" int marlin_b200_moe_sum_rows(const void* in, const int32_t* rows, void* out, int64_t tokens, int top_k,
                                        int64_t hidden, int act_dtype, void* stream) {
  MB_CHECK(hidden % 8 == 0, "moe_sum needs the hidden size to be a multiple of 8, got %lld",
           (long long)hidden);
  if (tokens == 0 || hidden == 0) return 0;
  auto s = (cudaStream_t)stream;
  const int grid = grid_for(tokens * hidden / 8, 256);
  if (act_dtype == MARLIN_B200_F16)
    moe_sum_kernel<__half><<<grid, 256, 0, s>>>((const __half*)in, (__half*)out, rows, tokens, top_k, hidden);
  else
    moe_sum_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, rows,
                                                       tokens, top_k, hidden);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}
