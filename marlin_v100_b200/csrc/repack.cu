// Weight repack: GPTQ (packed along K) and AWQ (packed along N) checkpoints -> packed layout of the
// GEMM kernels.  Integer work only; output is bit-identical to the reference layout.
//
// One thread produces one output word.  Threads are numbered so that a warp reads consecutive
// input words (the input side is the wide one for GPTQ: pf words per output word).
#include "common.cuh"

namespace mb200 {
namespace {

template <int BITS, bool HAS_PERM>
__global__ void __launch_bounds__(256) gptq_repack_kernel(const uint32_t* __restrict__ in,
                                                          const int32_t* __restrict__ perm,
                                                          uint32_t* __restrict__ out, int64_t size_k,
                                                          int64_t size_n, int g, int64_t num_experts) {
  // experts are stacked: in [E][K / PF][N], perm [E][K], out [E][K / 16][N * 16 / PF]
  constexpr int PF = 32 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  const int64_t words_per_k = size_n / PF;
  const int64_t total = size_k * words_per_k;
  for (int64_t gidx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gidx < total * num_experts;
       gidx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t ex = gidx / total, idx = gidx % total;
    const int64_t k = idx / words_per_k;
    const int64_t nw = idx % words_per_k;
    const int64_t n = nw * PF;
    const int64_t ksrc = HAS_PERM ? (int64_t)perm[ex * size_k + k] : k;
    const uint32_t* src = in + ex * (size_k / PF) * size_n + (ksrc / PF) * size_n + n;
    const int shift = (int)(ksrc % PF) * BITS;
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < PF; ++j) {
      const uint32_t v = (src[j] >> shift) & MASK;
      const int pos = (BITS == 4) ? nibble_pos(j) : byte_pos(j);
      word |= v << (pos * BITS);
    }
    const int64_t row_words = size_n * 16 / PF;
    out[ex * total + (k / 16) * row_words + packed_col<BITS>((int)(k % 16), (int)n, g)] = word;
  }
}

template <int BITS>
__global__ void __launch_bounds__(256) awq_repack_kernel(const uint32_t* __restrict__ in,
                                                         uint32_t* __restrict__ out, int64_t size_k,
                                                         int64_t size_n, int g, int64_t num_experts) {
  // The AWQ word already carries the values in the output order, so this is a word permutation.
  constexpr int PF = 32 / BITS;
  const int64_t words_per_k = size_n / PF;
  const int64_t total = size_k * words_per_k;
  const int64_t row_words = size_n * 16 / PF;
  for (int64_t gidx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gidx < total * num_experts;
       gidx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t ex = gidx / total, idx = gidx % total;
    const int64_t k = idx / words_per_k;
    const int64_t nw = idx % words_per_k;
    out[ex * total + (k / 16) * row_words + packed_col<BITS>((int)(k % 16), (int)(nw * PF), g)] = in[gidx];
  }
}

int check_shape(int64_t size_k, int64_t size_n, int num_bits) {
  MB_CHECK(num_bits == 4 || num_bits == 8, "num_bits must be 4 or 8. Got = %d", num_bits);
  MB_CHECK(size_k % 16 == 0, "size_k = %lld is not divisible by tile_k_size = 16", (long long)size_k);
  MB_CHECK(size_n % 64 == 0, "size_n = %lld is not divisible by tile_n_size = 64", (long long)size_n);
  return 0;
}

}  // namespace
}  // namespace mb200

using namespace mb200;

namespace {
int gptq_repack_any(const int32_t* b_q_weight, const int32_t* perm, int32_t* out, int64_t num_experts, int64_t size_k,
                    int64_t size_n, int num_bits, void* stream) {
  if (int rc = check_shape(size_k, size_n, num_bits)) return rc;
  MB_CHECK(num_experts >= 0, "negative expert count");
  if (size_k == 0 || size_n == 0 || num_experts == 0) return 0;
  MB_CHECK(b_q_weight != nullptr && out != nullptr, "null tensor pointer");
  const int g = macro_n_of(size_n) / 64;
  const int64_t total = num_experts * size_k * size_n * num_bits / 32;
  const int blocks = (int)((total + 255) / 256 < (int64_t)sm_count() * 16 ? (total + 255) / 256
                                                                           : (int64_t)sm_count() * 16);
  auto s = (cudaStream_t)stream;
  auto in = reinterpret_cast<const uint32_t*>(b_q_weight);
  auto o = reinterpret_cast<uint32_t*>(out);
  if (num_bits == 4) {
    if (perm) gptq_repack_kernel<4, true><<<blocks, 256, 0, s>>>(in, perm, o, size_k, size_n, g, num_experts);
    else gptq_repack_kernel<4, false><<<blocks, 256, 0, s>>>(in, perm, o, size_k, size_n, g, num_experts);
  } else {
    if (perm) gptq_repack_kernel<8, true><<<blocks, 256, 0, s>>>(in, perm, o, size_k, size_n, g, num_experts);
    else gptq_repack_kernel<8, false><<<blocks, 256, 0, s>>>(in, perm, o, size_k, size_n, g, num_experts);
  }
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

int awq_repack_any(const int32_t* b_q_weight, int32_t* out, int64_t num_experts, int64_t size_k, int64_t size_n,
                   int num_bits, void* stream) {
  if (int rc = check_shape(size_k, size_n, num_bits)) return rc;
  MB_CHECK(num_experts >= 0, "negative expert count");
  if (size_k == 0 || size_n == 0 || num_experts == 0) return 0;
  MB_CHECK(b_q_weight != nullptr && out != nullptr, "null tensor pointer");
  const int g = macro_n_of(size_n) / 64;
  const int64_t total = num_experts * size_k * size_n * num_bits / 32;
  const int blocks = (int)((total + 255) / 256 < (int64_t)sm_count() * 16 ? (total + 255) / 256
                                                                           : (int64_t)sm_count() * 16);
  auto s = (cudaStream_t)stream;
  auto in = reinterpret_cast<const uint32_t*>(b_q_weight);
  auto o = reinterpret_cast<uint32_t*>(out);
  if (num_bits == 4) awq_repack_kernel<4><<<blocks, 256, 0, s>>>(in, o, size_k, size_n, g, num_experts);
  else awq_repack_kernel<8><<<blocks, 256, 0, s>>>(in, o, size_k, size_n, g, num_experts);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}
}  // namespace

extern "C" int marlin_b200_gptq_repack(const int32_t* b_q_weight, const int32_t* perm, int32_t* out,
                                       int64_t size_k, int64_t size_n, int num_bits, void* stream) {
  return gptq_repack_any(b_q_weight, perm, out, 1, size_k, size_n, num_bits, stream);
}

extern "C" int marlin_b200_awq_repack(const int32_t* b_q_weight, int32_t* out, int64_t size_k,
                                      int64_t size_n, int num_bits, void* stream) {
  return awq_repack_any(b_q_weight, out, 1, size_k, size_n, num_bits, stream);
}

// All experts of a layer in one launch: b_q_weight [E][...], perm [E][size_k] (or NULL), out [E][size_k / 16][...].
extern "C" int marlin_b200_gptq_moe_repack(const int32_t* b_q_weight, const int32_t* perm, int32_t* out,
                                           int64_t num_experts, int64_t size_k, int64_t size_n, int num_bits,
                                           void* stream) {
  return gptq_repack_any(b_q_weight, perm, out, num_experts, size_k, size_n, num_bits, stream);
}

extern "C" int marlin_b200_awq_moe_repack(const int32_t* b_q_weight, int32_t* out, int64_t num_experts,
                                          int64_t size_k, int64_t size_n, int num_bits, void* stream) {
  return awq_repack_any(b_q_weight, out, num_experts, size_k, size_n, num_bits, stream);
}
