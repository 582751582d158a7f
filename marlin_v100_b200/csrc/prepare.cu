// Conversion between the reference packed layout and the streaming layout (stream_layout.cuh), both
// directions.  Integer work only: every code keeps its value, only its place changes, so
// unpack(streaming) == unpack(reference) and restore(prepare(x)) == x bit for bit.
//
// One thread produces one output word by gathering its 8 (4-bit) or 4 (8-bit) codes; the scattered reads
// stay inside one 64-k x 256-column block (8 / 16 KiB), i.e. in cache.  One-time work at weight load.
#include "common.cuh"
#include "stream_layout.cuh"

namespace mb200 {
namespace {

template <int BITS>
__global__ void __launch_bounds__(256) to_stream_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out,
                                                        int64_t size_k, int64_t size_n, int64_t words_per_expert,
                                                        int64_t total_words) {
  constexpr int PF = 32 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  const int64_t kblocks = size_k / stream::kBlockK;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_words;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = idx / words_per_expert, w = idx % words_per_expert;
    const uint32_t* src = in + e * words_per_expert;
    int64_t block, k0, n0;
    int dk[PF], hi[PF];
    if (BITS == 4) {
      block = w / 2048;
      const int r = (int)(w % 2048), slab = r / 128, lane = (r % 128) / 4, j = r % 4;
      k0 = (block % kblocks) * 64 + j * 16 + (lane % 4) * 4;
      n0 = (block / kblocks) * 256 + slab * 16 + lane / 4;
#pragma unroll
      for (int p = 0; p < PF; ++p) { dk[p] = ((p >> 1) & 1) * 2 + (p >> 2); hi[p] = p & 1; }
    } else {
      block = w / 4096;
      const int r = (int)(w % 4096), slab = r / 256, r2 = r % 256, lane = (r2 % 128) / 4, q = r2 % 4;
      const int j = (r2 / 128) * 2 + (q >> 1), y = q & 1;
      k0 = (block % kblocks) * 64 + j * 16 + (lane % 4) * 4 + y * 2;
      n0 = (block / kblocks) * 256 + slab * 16 + lane / 4;
#pragma unroll
      for (int p = 0; p < PF; ++p) { dk[p] = p & 1; hi[p] = p >> 1; }
    }
    uint32_t word = 0;
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      int64_t rw;
      int rs;
      stream::reference_pos<BITS>(k0 + dk[p], n0 + 8 * hi[p], size_n, &rw, &rs);
      word |= ((src[rw] >> rs) & MASK) << (BITS * p);
    }
    out[idx] = word;
  }
}

template <int BITS>
__global__ void __launch_bounds__(256) from_stream_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out,
                                                          int64_t size_k, int64_t size_n, int64_t words_per_expert,
                                                          int64_t total_words) {
  constexpr int PF = 32 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  constexpr int W = 1024 / PF;
  const int macro = macro_n_of(size_n), g = macro / 64;
  const int64_t row_words = size_n * 16 / PF;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_words;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = idx / words_per_expert, w = idx % words_per_expert;
    const uint32_t* src = in + e * words_per_expert;
    const int64_t row = w / row_words, col = w % row_words;
    const int64_t grp = col / (g * W);
    const int r = (int)(col % (g * W)), sub = r % g, r2 = r / g, nv = r2 % (64 / PF), lk = r2 / (64 / PF);
    const int64_t k = row * 16 + lk;
    const int64_t n0 = grp * macro + sub * 64 + nv * PF;
    uint32_t word = 0;
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      const int j = (BITS == 4) ? ((p & 3) * 2 + (p >> 2)) : ((p & 1) * 2 + (p >> 1));
      int64_t sw;
      int ss;
      stream::stream_pos<BITS>(k, n0 + j, size_k, &sw, &ss);
      word |= ((src[sw] >> ss) & MASK) << (BITS * p);
    }
    out[idx] = word;
  }
}

int convert(const int32_t* src, int32_t* dst, int64_t size_k, int64_t size_n, int num_bits, int64_t num_experts,
            bool to_stream, cudaStream_t s) {
  MB_CHECK(num_bits == 4 || num_bits == 8, "num_bits must be 4 or 8. Got = %d", num_bits);
  MB_CHECK(num_experts >= 1, "num_experts must be positive");
  MB_CHECK(stream::layout_accepts(size_k, size_n),
           "the streaming layout needs size_k %% 128 == 0 and size_n %% 256 == 0 (size_k = %lld, size_n = %lld)",
           (long long)size_k, (long long)size_n);
  MB_CHECK(src != nullptr && dst != nullptr && src != dst, "source and destination must be two different buffers");
  MB_CHECK(((uintptr_t)src % 16) == 0 && ((uintptr_t)dst % 16) == 0, "buffers must be aligned to 16 bytes");
  const int64_t wpe = size_k * size_n * num_bits / 32;
  const int64_t total = wpe * num_experts;
  const int64_t want = (total + 255) / 256, cap = (int64_t)sm_count() * 32;
  const int blocks = (int)(want < cap ? want : cap);
  auto in = reinterpret_cast<const uint32_t*>(src);
  auto out = reinterpret_cast<uint32_t*>(dst);
  if (to_stream) {
    if (num_bits == 4) to_stream_kernel<4><<<blocks, 256, 0, s>>>(in, out, size_k, size_n, wpe, total);
    else to_stream_kernel<8><<<blocks, 256, 0, s>>>(in, out, size_k, size_n, wpe, total);
  } else {
    if (num_bits == 4) from_stream_kernel<4><<<blocks, 256, 0, s>>>(in, out, size_k, size_n, wpe, total);
    else from_stream_kernel<8><<<blocks, 256, 0, s>>>(in, out, size_k, size_n, wpe, total);
  }
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

}  // namespace
}  // namespace mb200

extern "C" int marlin_b200_prepare_weights(const int32_t* b_q_weight, int32_t* out, int64_t size_k, int64_t size_n,
                                           int num_bits, int64_t num_experts, void* stream) {
  return mb200::convert(b_q_weight, out, size_k, size_n, num_bits, num_experts, true, (cudaStream_t)stream);
}

extern "C" int marlin_b200_restore_weights(const int32_t* prepared, int32_t* out, int64_t size_k, int64_t size_n,
                                           int num_bits, int64_t num_experts, void* stream) {
  return mb200::convert(prepared, out, size_k, size_n, num_bits, num_experts, false, (cudaStream_t)stream);
}
