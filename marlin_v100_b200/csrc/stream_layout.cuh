// The streaming weight layout: a second, opt-in arrangement of the same packed codes, made once per weight
// tensor by marlin_b200_prepare_weights (inverse: marlin_b200_restore_weights).  It holds exactly the bytes of
// the reference layout (csrc/quantization/marlin/gptq_marlin_repack.cu:399-469 in the reference project), only
// in another order, chosen for the weight-streaming GEMM kernel:
//
//  * Every (256-column group, 64-k) block is one contiguous run of 8 KiB (4-bit) / 16 KiB (8-bit), and the
//    blocks of a column group follow each other along k.  A CTA that streams a range of k of one column group
//    reads one linear byte range; in the reference layout the same data is 2 KiB / 4 KiB runs that lie
//    size_n * 8 bytes apart, which costs a third of the DRAM bandwidth.
//  * Inside a block the codes sit where the kernel's threads need them: a 32-bit word holds, for two weight
//    columns 8 apart, the codes of four consecutive k (4-bit) or of two consecutive k (8-bit) in the order
//    the register-level decoders of codes.cuh expect ("k pair in the two 16-bit halves"), so a decoded
//    register is directly one 32-bit column of the tensor-memory operand and no byte transposes are needed.
//
// Block order: [column group][k / 64].  Inside a block: [tile = column / 128][quadrant = column / 32 % 4]
// [half = column / 16 % 2] then 32 "lanes" of 16 bytes (4-bit) or 2 x 32 lanes of 16 bytes (8-bit); lane =
// (column % 8) * 4 + (k % 16) / 4; the column's bit 3 selects which of the word's two columns it is.
#pragma once

#include "common.cuh"

namespace mb200 {
namespace stream {

constexpr int kGroupN = 256;   // columns per block
constexpr int kBlockK = 64;    // k per block

__host__ __device__ inline bool layout_accepts(int64_t size_k, int64_t size_n) {
  return size_k > 0 && size_n > 0 && size_k % 128 == 0 && size_n % kGroupN == 0;
}

// Position of code (k, n): index of the 32-bit word in the tensor and the bit offset inside the word.
template <int BITS>
__host__ __device__ inline void stream_pos(int64_t k, int64_t n, int64_t size_k, int64_t* word, int* shift) {
  const int64_t block = (n / kGroupN) * (size_k / kBlockK) + k / kBlockK;
  const int nl = (int)(n % kGroupN);
  const int slab = nl >> 4;                 // (tile, quadrant, half)
  const int hi = (nl >> 3) & 1, g8 = nl & 7;
  const int kl = (int)(k % kBlockK);
  const int j = kl >> 4, t = (kl >> 2) & 3, e = kl & 3;
  const int lane = g8 * 4 + t;
  if (BITS == 4) {
    *word = block * 2048 + slab * 128 + lane * 4 + j;
    *shift = 4 * ((e & 1) * 4 + (e >> 1) * 2 + hi);
  } else {
    *word = block * 4096 + slab * 256 + (j >> 1) * 128 + lane * 4 + (j & 1) * 2 + (e >> 1);
    *shift = 8 * (hi * 2 + (e & 1));
  }
}

// Position of code (k, n) in the reference layout.
template <int BITS>
__host__ __device__ inline void reference_pos(int64_t k, int64_t n, int64_t size_n, int64_t* word, int* shift) {
  constexpr int PF = 32 / BITS;
  const int g = macro_n_of(size_n) / 64;
  const int64_t row_words = size_n * 16 / PF;
  *word = (k / 16) * row_words + packed_col<BITS>((int)(k % 16), (int)n, g);
  const int j = (int)(n % PF);
  *shift = BITS * ((BITS == 4) ? nibble_pos(j) : byte_pos(j));
}

}  // namespace stream
}  // namespace mb200
