// Decode-sized GEMM (M <= 32 rows) for 4-bit integer weights in the streaming layout (stream_layout.cuh):
// integer MMAs on 8-bit operands, weights as the tensor-memory operand.
//
//   C[M, N] = A[M, K] * dequant(Wq)[K, N] (+ bias)      (reference operator: csrc/quantization/marlin/marlin.cu:83)
//
// Why integers: a tcgen05.mma whose 128-row operand comes from tensor memory costs about 45 cycles of the SM
// partitions' issue bandwidth whatever its N, so the number of MMAs per weight byte bounds the stream.  With
// 8-bit operands (kind::i8, K = 32) a 16 KiB chunk takes 8 MMAs and two logic instructions per packed word;
// with 16-bit operands it takes 16 MMAs and fifteen instructions per word.
//
// The contraction runs transposed, D[n, m] = sum_k W[k, n] * A[m, k]: the 128 rows of an MMA are 128 weight
// columns, its N = 16 / 32 / 64 are two digit planes of 8 / 16 / 32 token columns, accumulation is exact (s32).
//  * Weights.  A word of the streaming layout holds the codes of two columns (8 apart) at four k, one column
//    in the low nibbles, the other in the high nibbles of its bytes.  `w & 0x0f0f0f0f` is the first column's
//    byte quadruple (byte = q); `(w ^ 0x80808080) & 0xf0f0f0f0` the second one's (byte = 16 (q - 8) as a signed
//    byte).  Byte = alpha (q - beta) with (alpha, beta) = (1, 0) or (16, 8), fixed per tensor-memory lane.
//  * Activations.  act_digits_kernel (in front, chained by programmatic dependent launch) rewrites every row as
//    two signed 8-bit digits, a = 2^(e-7) (d1 + d2 / 2^8), e from the row maximum (|d1| <= 127): 16 bits of
//    fixed point under the row maximum, i.e. exact for every bf16 element within 2^-8 of the row maximum (fp16:
//    2^-5), absolute error <= 2^(e-16) otherwise; the row factor 2^(e-7) is exact.  Digits are stored in the k
//    order in which the weight bytes land in tensor memory (a fixed permutation inside every 128 k).  The kernel
//    also leaves, per row and 128-k chunk, the sum of the row's digits (what the zero-point and offset terms
//    multiply), and it clears the column-group counters of the reduction.
// Scales are applied after the MMA, per 128-k chunk: with V = 256 D1 + D2 (an exact integer) and SA the chunk's
// digit sum, acc += (s / (256 alpha)) V + (s (beta - zero) - zs) SA  (zero = 8 for u4b8; zs = zero-point times
// scale as passed for u4).  The row factor and the bias are applied once per column group.
//
// Work split: persistent CTAs, one per SM, each owning a contiguous range of (256-column group, 128-k chunk)
// units = one linear range of weight bytes.  Column groups shared between CTAs leave fp32 partial sums in
// scratch; the CTA that arrives last at the group's counter adds them in CTA order (no waiting; bit-identical
// from run to run).
//
// Warps (768 threads; 80 registers each, nothing spills): 0-7 epilogue (tile = warp / 4, 32-lane quadrant =
// warp % 4) | 8-15 dequant (quadrant = warp % 4; warps 8-11 take the even chunks of the CTA's sequence, 12-15 the odd
// ones, each warp both tiles and both 16-lane halves: one group's wait for its tensor-memory stores overlaps the
// other group's loads and conversion) | 16 weight producer | 17 and 19 MMA issuers on two different SM partitions
// (issuing is what an MMA of this size costs; up to 16 rows each takes every other chunk with both 128-column tiles,
// at 32 rows each takes one tile of every chunk; 17 owns the tensor memory) | 18 producer of the small per-chunk
// operands (digit tile, digit sums, scale and zero rows) | 20-23 cross-CTA sums of the column groups shared with
// other CTAs (one thread waits for the epilogue's partial sums, the others block in a named barrier).
// Four operand stages and eight (up to 8 rows), four (up to 16) or two (up to 32) accumulator buffers in tensor memory: the
// round trip MMA -> epilogue -> next MMA on the same buffer (about 1500 cycles) bounds the rate at one chunk per
// round trip / buffers.
// A stage's 16 KiB of packed weights are released as soon as the dequant warps have read them and refilled at
// once, so all six stages (96 KiB per SM; eight stages measured 0.6 us slower per GEMM, eleven 1.5 us, bare copies
// lose bandwidth beyond 128 KiB in flight per SM too) cover the DRAM latency; the small operands (7 KiB, served by
// L2) stay until the chunk's MMAs and epilogue are done.
// Every wait is bounded; a wait that gives up raises the CTA's abort flag, the kernel drains, frees its tensor
// memory and reports through g_si8_status.
//
// Grouped (expert) form, GROUPED = true (reference operator: csrc/moe/marlin_moe_wna16/ops.cu:102): the same kernel
// where a "column group" is (block of 8 / 16 / 32 routes of the sorted route list, 256 columns of the block's expert).
// The digit kernel writes the planes in sorted order (row r = activation row sorted_ids[r] / top_k, optionally
// SiLU-and-mul of a [rows, 2 K] gate | up tensor on the way), the weight producer offsets its stream by the
// block's expert, scale rows are the expert's, and the epilogue / reduce warps scatter rows to C[sorted_id] with the
// top-k weight and the expert's bias.  The number of blocks is read from num_tokens_post_pad on the device, after
// the kernels in front have completed; min(units, launched CTAs) CTAs take part.

#include "codes.cuh"
#include "common.cuh"
#include "stream_layout.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace mb200 {
namespace {

using codes::kHalf;
using stream::kGroupN;

constexpr int KCH = 128;
constexpr int NDIG = 2;
constexpr int DQ_WARPS = 8;
constexpr int TSTAGES = 4;
constexpr int RAW_BYTES = KCH * kGroupN / 2;          // 16 KiB
constexpr int A_COLS = 64;                            // per operand stage: 2 tiles x 32 columns (128 k bytes)
constexpr int DCOL = TSTAGES * A_COLS;
constexpr int TMEM_COLS = 512;

// TOKH = 1: up to 8 token rows, TOKH = 2: up to 16, TOKH = 4: up to 32 (one pass over the weights for 17-32 rows:
// the MMAs take 64 token columns, the epilogue works through the rows eight at a time, two accumulator buffers).
// An epilogue thread owns one weight column and all token
// rows (twice the epilogue warps with 8 rows each were measured slower for 16 rows: 51 against 47 us, the
// register budget of 28 warps makes the epilogue spill).
template <int TOKH>
struct Cfg {
  static constexpr int NTOK = 8 * TOKH;
  static constexpr int STAGES = 6;   // 96 KiB of weights in flight per SM: measured ahead of 8 and of 4 stages, and 11 were slower still
  static constexpr int NUM_BARS_FIXED = 5 * STAGES + TSTAGES + 2;
  static constexpr int NCOL = NDIG * NTOK;                 // token columns of an MMA
  static constexpr int EPI_WARPS = 8;
  static constexpr int DQ_WARP0 = EPI_WARPS;
  static constexpr int PROD_WARP = DQ_WARP0 + DQ_WARPS, MMA_WARP = PROD_WARP + 1, META_WARP = PROD_WARP + 2,
                       MMA_WARP2 = PROD_WARP + 3;
  static constexpr int REDUCE_WARP = PROD_WARP + 4;          // four warps
  static constexpr int THREADS = (PROD_WARP + 8) * 32;
  static constexpr int ACT_BYTES = NCOL * KCH;             // digit rows x 128 k
  static constexpr int OFF_ACT = RAW_BYTES;
  static constexpr int OFF_S = OFF_ACT + ACT_BYTES;
  static constexpr int OFF_Z = OFF_S + kGroupN * 2;
  static constexpr int OFF_SA = OFF_Z + kGroupN * 2;       // NTOK floats
  static constexpr int STAGE_BYTES = (OFF_SA + (NTOK * 4 > 64 ? NTOK * 4 : 64) + 1023) / 1024 * 1024;
  static constexpr int DBUF_COLS = 2 * NCOL;               // two tiles
  static constexpr int DBUFS = 256 / DBUF_COLS;            // 8, 4 or 2 accumulator buffers
  static constexpr int NUM_BARS = NUM_BARS_FIXED + DBUFS;
  static constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + NUM_BARS * 8 + 64;
  static_assert(DCOL + DBUFS * DBUF_COLS <= TMEM_COLS, "tensor memory budget");
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
  static_assert(OFF_ACT % 1024 == 0, "the digit tile is a swizzled operand tile");
};

struct I8Params {
  const uint8_t* w;
  void* c;
  const void* bias;
  float* partials;          // [CTA][2][NTOK][256] fp32
  int* counters;            // one per column group, zero on entry
  const float* row_scale;   // [NTOK]
  const float* chunk_sums;  // [K / 128][NTOK]
  int M, N, K;
  int num_groups;
  int cps;                  // chunks per scale row
  int kc, ng;
  int num_ctas;
  uint32_t tx_bytes;        // bytes of the small operands of a chunk
  // grouped (expert) form: a "column group" is (block of NTOK sorted routes, 256 columns of the block's expert)
  const int32_t* sorted_ids;    // [row_capacity] route ids in expert order, >= num_routes for padding
  const int32_t* expert_ids;    // [row_capacity / NTOK] expert of every block (-1: not on this rank)
  const int32_t* num_post_pad;  // [1] sorted rows in use (a multiple of NTOK)
  const float* topk_weights;    // [num_routes] or NULL
  int num_routes;               // size_m * top_k
  int row_capacity;             // rows of the digit planes and the row factors
  int sum_stride;               // row stride of the digit sums (row capacity rounded up to 16)
  int ngc;                      // column groups per expert
  int rows_per_expert;          // scale rows per expert
  int mul_topk;
};

__device__ int g_si8_status = 0;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void reduce_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Wait for a barrier that has usually completed already (the small operands of a chunk, a free accumulator buffer,
// the chunk's MMAs seen from the epilogue): one plain try_wait first, the parking wait only if that fails.  A
// try_wait with a suspend hint costs 150-300 cycles even when the phase is complete; on waits that usually block the
// extra try costs more than it saves (measured per wait: -0.8 us per GEMM at 16 rows, -0.5 us at one row with this
// choice; +0.9 us at one row with the plain try in front of every wait).
__device__ __forceinline__ bool mbar_wait_likely(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t hint_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_park(bar, parity, abort_flag, hint_ns);
}
// Arrival by one lane of a converged warp without a divergent branch around it.
__device__ __forceinline__ void mbar_arrive_if(uint32_t bar, bool pred) {
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 st;\n\tsetp.ne.u32 p, %1, 0;\n\t"
               "@p mbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar), "r"((uint32_t)pred) : "memory");
}
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ int64_t range_start(int64_t p, int64_t U, int64_t P) { return p * U / P; }
__device__ __forceinline__ int64_t unit_owner(int64_t u, int64_t U, int64_t P) { return ((u + 1) * P - 1) / U; }

// kind::i8 instruction descriptor: s32 accumulate, signed 8-bit A and B, both K-major, M = 128, N = NCOL
template <int NCOL>
__device__ __forceinline__ constexpr uint32_t instr_desc_i8() {
  uint32_t d = 0;
  d |= 2u << 4;
  d |= 1u << 7;
  d |= 1u << 10;
  d |= (uint32_t)(NCOL >> 3) << 17;
  d |= (uint32_t)(128 >> 4) << 24;
  return d;
}
__device__ __forceinline__ void mma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t desc_lo, uint32_t desc_hi,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 d;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 d, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], d, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x4(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
template <typename T>
__device__ __forceinline__ T lds_as(uint32_t addr) {
  const unsigned short v = (unsigned short)lds16(addr);
  return *reinterpret_cast<const T*>(&v);
}

// Position, inside its 128-k chunk, of the digit (and weight byte) of k: the dequant thread t = k % 16 / 4 of a
// lane pair holds, for the 16-k run j = k % 64 / 16 of 64-k block h, the word whose bytes are k % 4 = 0, 2, 1, 3;
// that word becomes column 2 t + (j % 2) of the MMA's 32-k block 2 h + j / 2.
__host__ __device__ inline int digit_pos(int k_local) {
  const int h = k_local >> 6, j = (k_local >> 4) & 3, t = (k_local >> 2) & 3, e = k_local & 3;
  const int b = ((e & 1) << 1) | (e >> 1);
  return 32 * (2 * h + (j >> 1)) + 8 * t + 4 * (j & 1) + b;
}

// ---- activations -> digit planes -----------------------------------------------------------------------
// digits: int8 [2 * rows][K], row d * rows + m; rows of absent tokens are zero.
// 128 threads at no more than 32 registers: such a block fits into what a resident CTA of the GEMM kernel leaves
// of an SM's register file (24 warps x 80 registers), so the blocks of the next call can sit beside the running
// GEMM and the GEMM of this call can start beside them.
constexpr int AD_THREADS = 128;

// GROUPED: one block row per sorted route (grid.x = row capacity); row r converts activation row
// sorted_ids[r] / top_k; padding entries and rows beyond *num_post_pad are left alone (their outputs are dropped).
// SILU (grouped form only): the activation rows are the [rows, 2 K] gate | up output of the expert layer's first
// GEMM and the value converted is silu(gate) * up, rounded to T at the two places where the separate
// SiLU-and-mul kernel rounds (silu, then the product).
template <typename T>
__device__ __forceinline__ float silu_mul_rounded(T gate, T up) {
  const float x = to_float<T>(gate);
  const float sl = to_float<T>(from_float<T>(x / (1.f + expf(-x))));
  return to_float<T>(from_float<T>(sl * to_float<T>(up)));
}

template <typename T, bool GROUPED, bool SILU = false>
__global__ void __launch_bounds__(AD_THREADS, GROUPED ? 4 : 16) act_digits_kernel(const T* __restrict__ a, int64_t a_stride, int M, int K,
                                                         int8_t* __restrict__ digits, float* __restrict__ row_scale,
                                                         float* __restrict__ chunk_sums, int* __restrict__ counters,
                                                         int num_counters, const int32_t* __restrict__ sorted_ids,
                                                         const int32_t* __restrict__ num_post_pad, int top_k,
                                                         int num_routes, int sum_stride) {
  // grid (token rows, parts): every block finds the maximum of its whole row (the row is small and cached), then
  // converts its own part of the row, so that the conversion of a row is spread over several SMs
  const int m = blockIdx.x, tid = threadIdx.x, ntok = gridDim.x;
  const int part = blockIdx.y, parts = gridDim.y;
  // Launched with programmatic stream serialisation: the blocks may become resident while the kernel in front
  // (the GEMM of the previous call, or any producer of the activations) still runs, so nothing in global memory
  // is read or written before that kernel has completed; the GEMM behind may be scheduled at once (its weight
  // stream does not depend on this kernel, its digit loads wait for this kernel's completion).
  pdl_release_dependents();
  pdl_wait_prior_grid();
  if (m == 0 && part == 0)
    for (int i = tid; i < num_counters; i += AD_THREADS) counters[i] = 0;
  __shared__ float s_red[AD_THREADS / 32];
  __shared__ float s_max;
  const int vecs = K / 8;
  const int v_begin = part * (vecs / parts), v_end = v_begin + vecs / parts;   // a multiple of 16 vectors (one chunk)
  int src_row = m;
  if constexpr (GROUPED) {
    if (m >= *num_post_pad) return;
    const int sid = sorted_ids[m];
    if (sid >= num_routes) return;
    src_row = sid / top_k;
  }
  if (!GROUPED && m >= M) {
    for (int v = v_begin + tid; v < v_end; v += AD_THREADS)
#pragma unroll
      for (int d = 0; d < NDIG; ++d) *reinterpret_cast<uint2*>(digits + (int64_t)(d * ntok + m) * K + v * 8) = make_uint2(0, 0);
    for (int c = v_begin / 16 + tid; c < v_end / 16; c += AD_THREADS) chunk_sums[c * sum_stride + m] = 0.f;
    if (tid == 0 && part == 0) row_scale[m] = 0.f;
    return;
  }
  const T* row = a + (int64_t)src_row * a_stride;
  float mx = 0.f;
  for (int v = tid; v < vecs; v += AD_THREADS) {
    const uint4 q = *reinterpret_cast<const uint4*>(row + v * 8);
    const T* e = reinterpret_cast<const T*>(&q);
    if constexpr (SILU) {
      const uint4 qu = *reinterpret_cast<const uint4*>(row + K + v * 8);
      const T* eu = reinterpret_cast<const T*>(&qu);
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(silu_mul_rounded<T>(e[i], eu[i])));
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(to_float<T>(e[i])));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) s_red[tid >> 5] = mx;
  __syncthreads();
  if (tid == 0) {
    float t = s_red[0];
    for (int i = 1; i < AD_THREADS / 32; ++i) t = fmaxf(t, s_red[i]);
    s_max = t;
  }
  __syncthreads();
  mx = s_max;
  int e = 0;
  const bool finite = mx > 0.f && mx < 3.0e38f;
  if (finite) {
    (void)frexpf(mx, &e);                                   // mx = f * 2^e, f in [0.5, 1)
    if (ldexpf(mx, 7 - e) >= 127.49f) ++e;                  // keep the first digit inside [-127, 127]
  }
  // x = a * 2^(7 - e), |x| < 127.5; two exact power-of-two multiplies keep the factors in range
  const float f1 = ldexpf(1.f, (7 - e) / 2), f2 = ldexpf(1.f, (7 - e) - (7 - e) / 2);
  if (tid == 0 && part == 0) row_scale[m] = finite ? ldexpf(1.f, e - 7) : 0.f;
  // K / 8 vectors, 16 per chunk; the threads of a pass cover 8 whole chunks
  for (int v0 = v_begin; v0 < v_end; v0 += AD_THREADS) {
    const int v = v0 + tid;
    float sum = 0.f;
    if (v < v_end) {
      const uint4 q = *reinterpret_cast<const uint4*>(row + v * 8);
      const T* el = reinterpret_cast<const T*>(&q);
      uint4 qu = make_uint4(0, 0, 0, 0);
      if constexpr (SILU) qu = *reinterpret_cast<const uint4*>(row + K + v * 8);
      const T* eu = reinterpret_cast<const T*>(&qu);
      uint32_t out[NDIG][2] = {};
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float val = SILU ? silu_mul_rounded<T>(el[i], eu[i]) : to_float<T>(el[i]);
        const float x = finite ? val * f1 * f2 : 0.f;
        const float d1 = rintf(x);
        const float d2 = fminf(fmaxf(rintf((x - d1) * 256.f), -127.f), 127.f);
        s1 += d1; s2 += d2;
        const float dd[2] = {d1, d2};
        const int b = (((i & 3) & 1) << 1) | ((i & 3) >> 1);   // byte of k % 4 inside its word: 0, 2, 1, 3
#pragma unroll
        for (int d = 0; d < NDIG; ++d) out[d][i >> 2] |= ((uint32_t)(int)dd[d] & 0xffu) << (8 * b);
      }
      sum = s1 + s2 * (1.f / 256.f);
      const int chunk = v >> 4, kl = (v & 15) * 8;
      const int p0 = digit_pos(kl), p1 = digit_pos(kl + 4);
#pragma unroll
      for (int d = 0; d < NDIG; ++d) {
        int8_t* dst = digits + (int64_t)(d * ntok + m) * K + chunk * KCH;
        *reinterpret_cast<uint32_t*>(dst + p0) = out[d][0];
        *reinterpret_cast<uint32_t*>(dst + p1) = out[d][1];
      }
    }
    // the 16 vectors of a chunk sit in 16 consecutive lanes
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (v < v_end && (tid & 15) == 0) chunk_sums[(v >> 4) * sum_stride + m] = sum;
  }
}

template <typename T, int FMT, int TOKH, bool GROUPED>
__global__ void __launch_bounds__(Cfg<TOKH>::THREADS, 1)
stream_i8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmS,
                 const __grid_constant__ CUtensorMap tmZ, const I8Params p) {
  using C = Cfg<TOKH>;
  constexpr int NTOK = C::NTOK, NCOL = C::NCOL, EPI_WARPS = C::EPI_WARPS, DQ_WARP0 = C::DQ_WARP0,
                PROD_WARP = C::PROD_WARP, MMA_WARP = C::MMA_WARP, META_WARP = C::META_WARP, MMA_WARP2 = C::MMA_WARP2,
                REDUCE_WARP = C::REDUCE_WARP, STAGES = C::STAGES, NUM_BARS_FIXED = C::NUM_BARS_FIXED,
                STAGE_BYTES = C::STAGE_BYTES, OFF_ACT = C::OFF_ACT, OFF_S = C::OFF_S, OFF_Z = C::OFF_Z,
                OFF_SA = C::OFF_SA, DBUF_COLS = C::DBUF_COLS, DBUFS = C::DBUFS, NUM_BARS = C::NUM_BARS;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = base + STAGES * STAGE_BYTES;
  auto full = [&](int s) { return bar0 + 8u * s; };                       // the stage's packed weights have landed
  auto fullm = [&](int s) { return bar0 + 8u * (4 * STAGES + TSTAGES + s); };  // ... its small operands
  auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };           // the epilogue is done with the stage
  auto mma_done = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };    // the chunk's MMAs have completed
  auto a_ready = [&](int t) { return bar0 + 8u * (3 * STAGES + t); };     // operand stage written
  auto raw_free = [&](int s) { return bar0 + 8u * (3 * STAGES + TSTAGES + s); };  // packed weights read
  auto part_ready = [&](int r) { return bar0 + 8u * (5 * STAGES + TSTAGES + r); };  // a partial sum is in scratch
  auto d_free = [&](int b) { return bar0 + 8u * (NUM_BARS_FIXED + b); };
  const uint32_t tmem_slot = bar0 + 8u * NUM_BARS;
  auto drain_bar = [&](int w) { return bar0 + 8u * NUM_BARS + 16u + 8u * w; };   // give-up path of the MMA issuers

  __shared__ int s_abort;
  __shared__ int s_last;
  // The CTA visits its units in up to three runs: the part of a column group that it enters midway, the part
  // of a group that it starts but does not finish, then its whole groups.  The groups shared with other CTAs
  // come first so that their cross-CTA sums are formed while every CTA still streams.
  __shared__ int s_run_g[3], s_run_c[3], s_run_len[3];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int ng_total = p.ng;
  if constexpr (GROUPED) {
    // the block count comes from the routing kernels in front: nothing is read before they have completed
    pdl_wait_prior_grid();
    ng_total = (*p.num_post_pad / NTOK) * p.ngc;
  }
  const int64_t U = (int64_t)ng_total * p.kc;
  // every CTA that takes part owns at least one unit (the owners of a group are then consecutive CTAs); in the
  // grouped form the unit count is only known here, so the surplus CTAs of the launch stay idle
  const int num_ctas = (int)((U < p.num_ctas) ? (U > 0 ? U : 1) : p.num_ctas);
  int64_t u0 = 0, u1 = 0;
  if ((int)blockIdx.x < num_ctas) {
    u0 = range_start(blockIdx.x, U, num_ctas);
    u1 = range_start(blockIdx.x + 1, U, num_ctas);
  }
  const int total = (int)(u1 - u0);
  if (tid == 0) {
    const int c0 = (int)(u0 % p.kc), e1 = (int)(u1 % p.kc);
    const int n_head = (c0 != 0) ? ((total < p.kc - c0) ? total : p.kc - c0) : 0;
    const int rem = total - n_head;
    const int n_tail = (rem > 0 && e1 != 0) ? ((rem < e1) ? rem : e1) : 0;
    const int64_t ru[3] = {u0, u1 - n_tail, u0 + n_head};
    const int rl[3] = {n_head, n_tail, total - n_head - n_tail};
    for (int r = 0; r < 3; ++r) {
      s_run_g[r] = (int)(ru[r] / p.kc);
      s_run_c[r] = (int)(ru[r] % p.kc);
      s_run_len[r] = rl[r];
    }
    s_abort = 0;
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmS);
    if constexpr (format_has_zp(FMT)) prefetch_tensormap(&tmZ);
  }
  if (warp == 1) {
    // barriers in the order of the accessors above; every lane initialises its share
    for (int i = lane; i < NUM_BARS; i += 32) {
      int count;
      if (i < STAGES) count = 1;                                        // full
      else if (i < 2 * STAGES) count = EPI_WARPS;                       // empty
      else if (i < 3 * STAGES) count = (NTOK == 32) ? 2 : 1;            // mma_done
      else if (i < 3 * STAGES + TSTAGES) count = DQ_WARPS / 2;          // a_ready
      else if (i < 4 * STAGES + TSTAGES) count = DQ_WARPS / 2;          // raw_free
      else if (i < 5 * STAGES + TSTAGES) count = 1;                     // fullm
      else count = EPI_WARPS;                                           // part_ready, d_free
      mbar_init(bar0 + 8u * i, count);
    }
    if (lane < 2) mbar_init(drain_bar(lane), 1);
    fence_barrier_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = lds32(tmem_slot);

  pdl_release_dependents();

  if (warp == PROD_WARP) {
    // ---------------- weight producer: one linear 16 KiB copy per chunk ----------------
    if (lane == 0) {
      int s = 0, i = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int r = 0; r < 3 && ok; ++r) {
        const uint8_t* src = p.w + ((int64_t)s_run_g[r] * p.kc + s_run_c[r]) * RAW_BYTES;   // a run is linear
        const int len = s_run_len[r];
        int g = s_run_g[r], c = s_run_c[r];
        for (int j = 0; j < len; ++j, ++i) {
          // the ring is filled in two steps: two copies at once, the rest when the first has landed, so that no SM's
          // first chunk queues behind other SMs' sixth (-0.3 us at 16 rows)
          if (i == 2 && !mbar_wait_park(full(0), 0, &s_abort, 2000)) { atomicExch(&g_si8_status, 1); ok = false; break; }
          if (i >= STAGES && !mbar_wait_park(raw_free(s), ph ^ 1u, &s_abort, 2000)) { atomicExch(&g_si8_status, 1); ok = false; break; }
          mbar_arrive_expect_tx(full(s), RAW_BYTES);
          if constexpr (GROUPED) {
            // group g = (block, column group of the block's expert): linear inside the group only
            if (j == 0 || c == 0) {
              int e = p.expert_ids[g / p.ngc];
              if (e < 0) e = 0;   // a block of an expert that is not here: any weights do, its rows are dropped
              src = p.w + (((int64_t)e * p.ngc + g % p.ngc) * p.kc) * RAW_BYTES;
            }
            bulk_load(base + s * STAGE_BYTES, src + (int64_t)c * RAW_BYTES, RAW_BYTES, full(s));
            if (++c == p.kc) { c = 0; ++g; }
          } else {
            bulk_load(base + s * STAGE_BYTES, src + (int64_t)j * RAW_BYTES, RAW_BYTES, full(s));
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      // after a give-up nobody waits for the copies this thread issued last, and a CTA must not exit with copies on
      // their way into its shared memory
      if (s_abort != 0) drain_copies(full, STAGES, i);
    }
  } else if (warp == META_WARP) {
    // ---------------- producer of the digit tile, the digit sums and the scale / zero rows ----------------
    if (lane == 0) {
      pdl_wait_prior_grid();   // digits and sums come from the kernel in front
      int s = 0, i = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int r = 0; r < 3 && ok; ++r) {
      int g = s_run_g[r], c = s_run_c[r];
      const int len = s_run_len[r];
      for (int j = 0; j < len; ++j, ++i) {
        if (i >= STAGES && !mbar_wait_park(empty(s), ph ^ 1u, &s_abort, 2000)) { atomicExch(&g_si8_status, 9); ok = false; break; }
        const uint32_t st = base + s * STAGE_BYTES;
        mbar_arrive_expect_tx(fullm(s), p.tx_bytes);
        int srow = (p.num_groups == 1) ? 0 : c / p.cps;
        int col = g * kGroupN;
        if constexpr (GROUPED) {
          const int blk = g / p.ngc;
          int e = p.expert_ids[blk];
          if (e < 0) e = 0;
          tma_load_3d(st + OFF_ACT, &tmA, fullm(s), c * KCH, blk * NTOK, 0);   // both digit planes of the block's rows
          bulk_load(st + OFF_SA, p.chunk_sums + (int64_t)c * p.sum_stride + blk * NTOK, NTOK * 4, fullm(s));
          srow += e * p.rows_per_expert;
          col = (g % p.ngc) * kGroupN;
        } else {
          tma_load_2d(st + OFF_ACT, &tmA, fullm(s), c * KCH, 0);
          bulk_load(st + OFF_SA, p.chunk_sums + (int64_t)c * NTOK, NTOK * 4, fullm(s));
        }
        tma_load_2d(st + OFF_S, &tmS, fullm(s), col, srow);
        if constexpr (format_has_zp(FMT)) tma_load_2d(st + OFF_Z, &tmZ, fullm(s), col, srow);
        if (++c == p.kc) { c = 0; ++g; }
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
      }
      if (s_abort != 0) drain_copies(fullm, STAGES, i);
    }
  } else if (warp == MMA_WARP || warp == MMA_WARP2) {
    // ---------------- MMA issuers: alternate chunks, both 128-column tiles, 4 blocks of 32 k per tile ----------------
    // A cycle-stamped run showed the issuer's loop as the period of the whole pipeline: its three barrier waits cost
    // the lone thread 150-300 cycles each even when they are already satisfied.  Each issuer therefore takes every
    // other chunk with both tiles (three waits per eight MMAs instead of per four); chunks use different operand
    // stages and accumulator buffers, so the two threads need no order between them.
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_i8<NCOL>();
      const int which = (warp == MMA_WARP) ? 0 : 1;
      const uint64_t desc0 = kmajor_sw128_desc(base + OFF_ACT);
      const uint32_t desc_lo = (uint32_t)desc0, desc_hi = (uint32_t)(desc0 >> 32);
      if constexpr (NTOK == 32) {
        // 32 rows (two accumulator buffers): one tile per issuer and every chunk, measured 0.3 us ahead there
        int s = 0, t = 0, b = 0;
        uint32_t ph = 0, tph = 0, bph = 0;
        for (int i = 0; i < total; ++i) {
          if (!mbar_wait_likely(d_free(b), bph ^ 1u, &s_abort, 2000)) { atomicExch(&g_si8_status, 2); break; }
          if (!mbar_wait_likely(fullm(s), ph, &s_abort, 2000)) { atomicExch(&g_si8_status, 3); break; }
          if (!mbar_wait_park(a_ready(t), tph, &s_abort, 2000)) { atomicExch(&g_si8_status, 4); break; }
          tc_fence_after();
          const uint32_t dlo = desc_lo + (uint32_t)((s * STAGE_BYTES) >> 4);
          const uint32_t a_base = tmem + t * A_COLS + which * 32;
          const uint32_t d_addr = tmem + DCOL + b * DBUF_COLS + which * NCOL;
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) mma_i8_ts(d_addr, a_base + kb * 8, dlo + kb * 2, desc_hi, idesc, kb == 0 ? 0u : 1u);
          tc_commit(mma_done(s));
          if (++s == STAGES) { s = 0; ph ^= 1u; }
          if (++t == TSTAGES) { t = 0; tph ^= 1u; }
          if (++b == DBUFS) { b = 0; bph ^= 1u; }
        }
      } else {
      int s = which % STAGES, t = which % TSTAGES, b = which % DBUFS;
      uint32_t ph = 0, tph = 0, bph = 0;
      for (int i = which; i < total; i += 2) {
        if (!mbar_wait_likely(d_free(b), bph ^ 1u, &s_abort, 2000)) { atomicExch(&g_si8_status, 2); break; }
        if (!mbar_wait_likely(fullm(s), ph, &s_abort, 2000)) { atomicExch(&g_si8_status, 3); break; }
        if (!mbar_wait_park(a_ready(t), tph, &s_abort, 2000)) { atomicExch(&g_si8_status, 4); break; }
        tc_fence_after();
        const uint32_t dlo = desc_lo + (uint32_t)((s * STAGE_BYTES) >> 4);
        const uint32_t a_base = tmem + t * A_COLS;
        const uint32_t d_addr = tmem + DCOL + b * DBUF_COLS;
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            mma_i8_ts(d_addr + tile * NCOL, a_base + tile * 32 + kb * 8, dlo + kb * 2, desc_hi, idesc, kb == 0 ? 0u : 1u);
        tc_commit(mma_done(s));
        s += 2;
        if (s >= STAGES) { s -= STAGES; ph ^= 1u; }
        t += 2;
        if (t >= TSTAGES) { t -= TSTAGES; tph ^= 1u; }
        b += 2;
        if (b >= DBUFS) { b -= DBUFS; bph ^= 1u; }
      }
      }
      // after a give-up nobody waits for this thread's MMAs: the tensor memory is freed only once they have completed
      if (s_abort != 0) {
        tc_commit(drain_bar(which));
        drain_barrier(drain_bar(which), 0);
      }
    }
  } else if (warp < EPI_WARPS) {
    // ---------------- epilogue: per chunk, scale the integer sums into fp32 registers ----------------
    // thread = one weight column (tensor-memory lane) x NTOK token rows
    const int tile = (warp >> 2) & 1, quad = warp & 3;
    const int nl = tile * 128 + quad * 32 + lane;          // column inside the group = tensor-memory lane
    const bool hi_lane = (lane & 8) != 0;                   // second column of its packed word: byte = 16 (q - 8)
    const float inv_alpha = hi_lane ? 1.f / 16.f : 1.f;
    const float beta_minus_zero = (hi_lane ? 8.f : 0.f) - (FMT == kU4B8 ? 8.f : 0.f);
    T* Cout = reinterpret_cast<T*>(p.c);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    float acc[NTOK];
    bool ok = true, first_segment = true;
    int s = 0, seg_c0 = 0, db = 0;
    uint32_t ph = 0;
    for (int r = 0; r < 3; ++r) {
    int g = s_run_g[r], c = s_run_c[r];
    const int len = s_run_len[r];
    for (int j = 0; j < len; ++j) {
      const bool seg_start = (j == 0) || (c == 0);
      const bool seg_end = (j == len - 1) || (c == p.kc - 1);
      if (seg_start) {
        seg_c0 = c;
#pragma unroll
        for (int m = 0; m < NTOK; ++m) acc[m] = 0.f;
      }
      if (ok && !mbar_wait_likely(fullm(s), ph, &s_abort, 2000)) { atomicExch(&g_si8_status, 5); ok = false; }
      const uint32_t st = base + s * STAGE_BYTES;
      float sv = 0.f, zv = 0.f;
      if (ok) {
        sv = to_float<T>(lds_as<T>(st + OFF_S + nl * 2));
        if constexpr (format_has_zp(FMT)) zv = to_float<T>(lds_as<T>(st + OFF_Z + nl * 2));
      }
      if (ok && !mbar_wait_likely(mma_done(s), ph, &s_abort, 2000)) { atomicExch(&g_si8_status, 6); ok = false; }
      if constexpr (NTOK == 32) {
        // eight rows at a time: load both digit planes of the eight, fold them into the running sums, next eight
        const float t0 = sv * inv_alpha * (1.f / 256.f);
        const float cfix = sv * beta_minus_zero - zv;
        if (ok) {
          tc_fence_after();
          const uint32_t dbase = tmem + ((uint32_t)(32 * quad) << 16) + DCOL + db * DBUF_COLS + tile * NCOL;
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            uint32_t va[8], vb[8];
            tmem_ld8(dbase + 8 * q8, va);
            tmem_ld8(dbase + NTOK + 8 * q8, vb);
            // the digit-sum term does not need the integer sums: it runs while they are on their way
            const uint4 sa0 = lds128(st + OFF_SA + q8 * 32), sa1 = lds128(st + OFF_SA + q8 * 32 + 16);
            const float sa[8] = {__uint_as_float(sa0.x), __uint_as_float(sa0.y), __uint_as_float(sa0.z),
                                 __uint_as_float(sa0.w), __uint_as_float(sa1.x), __uint_as_float(sa1.y),
                                 __uint_as_float(sa1.z), __uint_as_float(sa1.w)};
#pragma unroll
            for (int m = 0; m < 8; ++m) acc[8 * q8 + m] = fmaf(cfix, sa[m], acc[8 * q8 + m]);
            tmem_ld_wait();
#pragma unroll
            for (int m = 0; m < 8; ++m) {
              const int vv = (int)va[m] * 256 + (int)vb[m];   // exact: |D1| < 2^22
              acc[8 * q8 + m] = fmaf(t0, (float)vv, acc[8 * q8 + m]);
            }
          }
          tc_fence_before();
        }
        __syncwarp();
        mbar_arrive_if(d_free(db), lane == 0);
      } else {
      int v[NTOK];
      if (ok) {
        tc_fence_after();
        const uint32_t dbase = tmem + ((uint32_t)(32 * quad) << 16) + DCOL + db * DBUF_COLS + tile * NCOL;
        uint32_t va[NTOK], vb[NTOK];
        if constexpr (NTOK == 8) {
          tmem_ld8(dbase, va);
          tmem_ld8(dbase + NTOK, vb);
        } else {
          tmem_ld16(dbase, va);
          tmem_ld16(dbase + NTOK, vb);
        }
        // 16 rows: the digit-sum term does not need the integer sums and runs while they are on their way
        // (-0.2 us per GEMM; with 8 rows the same order measured +0.4 us)
        const float cfix = sv * beta_minus_zero - zv;
        if constexpr (NTOK == 16) {
#pragma unroll
        for (int q = 0; q < NTOK / 4; ++q) {   // the chunk's digit sums of the token rows (same for every lane)
          const uint4 sa = lds128(st + OFF_SA + q * 16);
          acc[4 * q + 0] = fmaf(cfix, __uint_as_float(sa.x), acc[4 * q + 0]);
          acc[4 * q + 1] = fmaf(cfix, __uint_as_float(sa.y), acc[4 * q + 1]);
          acc[4 * q + 2] = fmaf(cfix, __uint_as_float(sa.z), acc[4 * q + 2]);
          acc[4 * q + 3] = fmaf(cfix, __uint_as_float(sa.w), acc[4 * q + 3]);
        }
        }
        tmem_ld_wait();
        tc_fence_before();
#pragma unroll
        for (int m = 0; m < NTOK; ++m) v[m] = (int)va[m] * 256 + (int)vb[m];   // exact: |D1| < 2^22
      }
      // the accumulator buffer goes back before the arithmetic: the next MMA on it need not wait for that
      __syncwarp();
      mbar_arrive_if(d_free(db), lane == 0);
      if (ok) {
        const float t0 = sv * inv_alpha * (1.f / 256.f);
        if constexpr (NTOK == 16) {
#pragma unroll
          for (int m = 0; m < NTOK; ++m) acc[m] = fmaf(t0, (float)v[m], acc[m]);
        } else {
          const float cfix = sv * beta_minus_zero - zv;
#pragma unroll
          for (int q = 0; q < NTOK / 4; ++q) {
            const uint4 sa = lds128(st + OFF_SA + q * 16);
            acc[4 * q + 0] = fmaf(t0, (float)v[4 * q + 0], fmaf(cfix, __uint_as_float(sa.x), acc[4 * q + 0]));
            acc[4 * q + 1] = fmaf(t0, (float)v[4 * q + 1], fmaf(cfix, __uint_as_float(sa.y), acc[4 * q + 1]));
            acc[4 * q + 2] = fmaf(t0, (float)v[4 * q + 2], fmaf(cfix, __uint_as_float(sa.z), acc[4 * q + 2]));
            acc[4 * q + 3] = fmaf(t0, (float)v[4 * q + 3], fmaf(cfix, __uint_as_float(sa.w), acc[4 * q + 3]));
          }
        }
      }
      }
      __syncwarp();
      mbar_arrive_if(empty(s), lane == 0);
      if (++db == DBUFS) db = 0;
      if (seg_end) {
        const bool whole = (seg_c0 == 0) && (c == p.kc - 1);
        if (first_segment) pdl_wait_prior_grid();   // the row factors come from the kernel in front
        if constexpr (GROUPED) {
          const int blk = g / p.ngc, e = p.expert_ids[blk];
          const int n = (g % p.ngc) * kGroupN + nl;
          if (ok && s_abort == 0) {
            if (whole) {
              const float bv = (bias != nullptr && e >= 0) ? to_float<T>(bias[(int64_t)e * p.N + bias_index(n)]) : 0.f;
#pragma unroll
              for (int m = 0; m < NTOK; ++m) {
                const int sid = p.sorted_ids[blk * NTOK + m];
                if (sid < p.num_routes && e >= 0) {
                  float v = fmaf(acc[m], p.row_scale[blk * NTOK + m], bv);
                  if (p.mul_topk) v *= p.topk_weights[sid];
                  Cout[(int64_t)sid * p.N + n] = from_float<T>(v);
                }
              }
            } else {
              float* P = p.partials + ((int64_t)blockIdx.x * 2 + (seg_c0 == 0 ? 1 : 0)) * (NTOK * kGroupN);
#pragma unroll
              for (int m = 0; m < NTOK; ++m) P[m * kGroupN + nl] = acc[m] * p.row_scale[blk * NTOK + m];
            }
          }
        } else {
        const int n = g * kGroupN + nl;
        if (ok && s_abort == 0) {
          if (whole) {
            const float bv = (bias != nullptr) ? to_float<T>(bias[bias_index(n)]) : 0.f;
#pragma unroll
            for (int m = 0; m < NTOK; ++m)
              if (m < p.M) Cout[(int64_t)m * p.N + n] = from_float<T>(fmaf(acc[m], p.row_scale[m], bv));
          } else {
            // slot 1: the run that starts the group (c = 0) but ends early; slot 0: a run that enters it midway
            float* P = p.partials + ((int64_t)blockIdx.x * 2 + (seg_c0 == 0 ? 1 : 0)) * (NTOK * kGroupN);
#pragma unroll
            for (int m = 0; m < NTOK; ++m)
              if (m < p.M) P[m * kGroupN + nl] = acc[m] * p.row_scale[m];
          }
        }
        }
        if (!whole) {   // runs 0 and 1: the reduce warp takes it from here
          __syncwarp();
          mbar_arrive_if(part_ready(r), lane == 0);
        }
        first_segment = false;
      }
      if (++c == p.kc) { c = 0; ++g; }
      if (++s == STAGES) { s = 0; ph ^= 1u; }
    }
    }
  } else if (warp >= REDUCE_WARP) {
    // ---------------- cross-CTA sums of the column groups shared with other CTAs (four warps) ----------------
    // Whoever arrives last at a group's counter adds the partial sums, always in CTA order, and writes C.
    // Warps of their own, so that the epilogue warps (and with them the whole chunk pipeline) never wait for
    // the fence, the atomic and the loads.
    T* Cout = reinterpret_cast<T*>(p.c);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const int rt = tid - REDUCE_WARP * 32;
    bool waited = false;
    for (int r = 0; r < 2; ++r) {
      if (s_run_len[r] == 0) continue;
      const int g = s_run_g[r];
      // one thread waits for the epilogue warps (polling with short sleeps: a parked wait wakes up about half a
      // microsecond late, and this wait is on the critical path of the CTA's last run); the other 127 block in the
      // named barrier below, which costs no issue slots
      const int64_t ua = (int64_t)g * p.kc;
      const int64_t pa = unit_owner(ua, U, num_ctas), pb = unit_owner(ua + p.kc - 1, U, num_ctas);
      if (rt == 0) {
        int last = -1;
        if (mbar_wait_sleep(part_ready(r), 0, &s_abort, 100)) last = 0;
        else atomicExch(&g_si8_status, 10);
        if (last == 0) pdl_wait_prior_grid();   // the counters were cleared by the kernel in front
        if (last == 0 && s_abort == 0) {
          // One release-acquire atomic instead of fence, atomic, fence: the release is cumulative over the epilogue
          // warps' stores (ordered before this thread by part_ready), the acquire covers the other owners' stores
          // for every thread behind the barrier below.
          int old;
          asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + g) : "memory");
          last = (old == (int)(pb - pa)) ? 1 : 0;
        }
        s_last = last;
      }
      reduce_barrier();
      const int last = s_last;
      reduce_barrier();
      if (last < 0) break;
      if (!last) continue;
      if (!waited) { pdl_wait_prior_grid(); waited = true; }   // nothing is stored before the kernel in front is done
      constexpr int64_t SLOT = NTOK * kGroupN;
      // the first owner holds the group's first chunks (slot 1), every other one a run from midway (slot 0)
      const float4* first = reinterpret_cast<const float4*>(p.partials + (pa * 2 + 1) * SLOT);
      const int total4 = (GROUPED ? NTOK : p.M) * (kGroupN / 4);
      const int blk = GROUPED ? g / p.ngc : 0;
      const int ex = GROUPED ? p.expert_ids[blk] : 0;
      const int gcol = GROUPED ? g % p.ngc : g;
      for (int e0 = rt; e0 < total4; e0 += 128 * 4) {
        float4 sum[4];
#pragma unroll
        for (int uu = 0; uu < 4; ++uu) {
          const int e = e0 + 128 * uu;
          sum[uu] = (e < total4) ? __ldcg(first + e) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int64_t o = pa + 1; o <= pb; ++o) {
          const float4* src = reinterpret_cast<const float4*>(p.partials + (o * 2) * SLOT);
          float4 v4[4];
#pragma unroll
          for (int uu = 0; uu < 4; ++uu) {
            const int e = e0 + 128 * uu;
            v4[uu] = (e < total4) ? __ldcg(src + e) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int uu = 0; uu < 4; ++uu) {
            sum[uu].x += v4[uu].x; sum[uu].y += v4[uu].y; sum[uu].z += v4[uu].z; sum[uu].w += v4[uu].w;
          }
        }
#pragma unroll
        for (int uu = 0; uu < 4; ++uu) {
          const int e = e0 + 128 * uu;
          if (e < total4) {
            const int m = e / (kGroupN / 4), col = (e % (kGroupN / 4)) * 4;
            const int nn = gcol * kGroupN + col;
            int64_t out_row = m;
            float wgt = 1.f;
            if constexpr (GROUPED) {
              const int sid = p.sorted_ids[blk * NTOK + m];
              if (sid >= p.num_routes || ex < 0) continue;
              out_row = sid;
              if (p.mul_topk) wgt = p.topk_weights[sid];
            }
            float bv[4] = {0.f, 0.f, 0.f, 0.f};
            if (bias != nullptr) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) bv[q4] = to_float<T>(bias[(GROUPED ? (int64_t)ex * p.N : 0) + bias_index(nn + q4)]);
            }
            T o4[4];
            o4[0] = from_float<T>((sum[uu].x + bv[0]) * wgt);
            o4[1] = from_float<T>((sum[uu].y + bv[1]) * wgt);
            o4[2] = from_float<T>((sum[uu].z + bv[2]) * wgt);
            o4[3] = from_float<T>((sum[uu].w + bv[3]) * wgt);
            *reinterpret_cast<uint2*>(Cout + out_row * p.N + nn) = *reinterpret_cast<const uint2*>(o4);
          }
        }
      }
      if (rt == 0) p.counters[g] = 0;
    }
  } else if (warp < DQ_WARP0 + DQ_WARPS) {
    // ---------------- dequant: per 16-lane half, 8 packed words -> 16 byte quadruples -> one store ----------------
    // Two groups of four warps take alternate chunks (a warp converts both 128-column tiles of its lane quarter),
    // so that one group's wait for its tensor-memory stores overlaps the other group's loads and conversion.
    const int quad = warp & 3, grp = (warp - DQ_WARP0) >> 2;
    const uint32_t woff = (uint32_t)(quad * 2 * 512 + lane * 16);   // tile 1 is 4096 bytes, half 1 512 bytes further on
    const uint32_t t_lane = (uint32_t)(32 * quad) << 16;
    bool ok = true;
    int s = grp, t = grp, ms = grp;
    uint32_t ph = 0, mph = 0;
    for (int i = grp; i < total; i += 2) {
      if (ok && !mbar_wait_park(full(s), ph, &s_abort, 2000)) { atomicExch(&g_si8_status, 7); ok = false; }
      const uint32_t st = base + s * STAGE_BYTES;
      uint4 x[2][2][2] = {};
      if (ok) {
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            x[tile][half][0] = lds128(st + woff + tile * 4096 + half * 512);
            x[tile][half][1] = lds128(st + RAW_BYTES / 2 + woff + tile * 4096 + half * 512);
          }
      }
      __syncwarp();
      mbar_arrive_if(raw_free(s), lane == 0);
      // the operand stage is free once the MMAs of the chunk that used it last have completed
      if (i >= TSTAGES) {
        if (ok && !mbar_wait_park(mma_done(ms), mph, &s_abort, 2000)) { atomicExch(&g_si8_status, 8); ok = false; }
        ms += 2;
        if (ms >= STAGES) { ms -= STAGES; mph ^= 1u; }
      }
      if (ok) {
        tc_fence_after();
        // registers 4 b .. 4 b + 3 of a store: (lane g: columns 2t, 2t + 1 of 32-k block b), (lane g + 8: same)
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const uint32_t w[8] = {x[tile][half][0].x, x[tile][half][0].y, x[tile][half][0].z, x[tile][half][0].w,
                                   x[tile][half][1].x, x[tile][half][1].y, x[tile][half][1].z, x[tile][half][1].w};
            uint32_t r[16];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              r[4 * b + 0] = w[2 * b] & 0x0f0f0f0fu;
              r[4 * b + 1] = w[2 * b + 1] & 0x0f0f0f0fu;
              r[4 * b + 2] = (w[2 * b] ^ 0x80808080u) & 0xf0f0f0f0u;
              r[4 * b + 3] = (w[2 * b + 1] ^ 0x80808080u) & 0xf0f0f0f0u;
            }
            tmem_st_16x256b_x4(tmem + t_lane + ((uint32_t)(16 * half) << 16) + t * A_COLS + tile * 32, r);
          }
        tmem_st_wait();
        tc_fence_before();
      }
      __syncwarp();
      mbar_arrive_if(a_ready(t), lane == 0);
      s += 2;
      if (s >= STAGES) { s -= STAGES; ph ^= 1u; }
      t += 2;
      if (t >= TSTAGES) t -= TSTAGES;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------
int64_t counters_bytes(int64_t n) { return ((n / kGroupN) * 4 + 255) & ~(int64_t)255; }
int64_t partial_bytes(int rows = 16) { return (int64_t)sm_count() * 2 * rows * kGroupN * (int64_t)sizeof(float); }

template <typename T, int FMT, int TOKH>
int launch_one(const GemmArgs& g) {
  using C = Cfg<TOKH>;
  constexpr int NCOL = C::NCOL, NTOK = C::NTOK;
  const int64_t K = g.size_k, N = g.size_n;
  const int m = (int)g.size_m;
  I8Params p{};
  p.w = reinterpret_cast<const uint8_t*>(g.bq);
  p.c = g.c; p.bias = g.bias;
  p.M = m; p.N = (int)N; p.K = (int)K;
  p.num_groups = (int)g.num_groups;
  p.kc = (int)(K / KCH);
  p.ng = (int)(N / kGroupN);
  p.cps = (g.num_groups == 1) ? p.kc : (int)((K / g.num_groups) / KCH);
  const int64_t U = (int64_t)p.ng * p.kc;
  // scratch: counters | partial sums | digit planes | row factors | per-chunk digit sums
  uint8_t* sc = reinterpret_cast<uint8_t*>(g.scratch);
  const int64_t cb = counters_bytes(N), pb = partial_bytes(NTOK <= 16 ? 16 : 32);
  p.counters = reinterpret_cast<int*>(sc);
  p.partials = reinterpret_cast<float*>(sc + cb);
  int8_t* digits = reinterpret_cast<int8_t*>(sc + cb + pb);
  float* row_scale = reinterpret_cast<float*>(digits + (int64_t)(NTOK <= 16 ? 32 : 64) * K);   // two planes of 16 / 32 rows
  float* chunk_sums = row_scale + 64;
  p.row_scale = row_scale;
  p.chunk_sums = chunk_sums;
  p.num_ctas = (int)(U < sm_count() ? U : sm_count());
  p.tx_bytes = C::ACT_BYTES + NTOK * 4 + kGroupN * 2 * (format_has_zp(FMT) ? 2 : 1);   // small operands of a chunk

  int parts = 1;   // as many parts per row as leave every part whole chunks and at least one pass of the block
  while (parts < 8 && K % (KCH * parts * 2) == 0 && K / (parts * 2) >= 8 * AD_THREADS) parts *= 2;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(NTOK, parts);
    cfg.blockDim = dim3(AD_THREADS);
    cfg.stream = g.stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MB_CUDA(cudaLaunchKernelEx(&cfg, act_digits_kernel<T, false>, reinterpret_cast<const T*>(g.a), g.a_stride, m, (int)K,
                               digits, row_scale, chunk_sums, p.counters, p.ng, (const int32_t*)nullptr,
                               (const int32_t*)nullptr, 1, 0, NTOK));
    count_launches(1);
  }
  CUtensorMap tmA, tmS, tmZ;
  {
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)g.num_groups};
    const uint64_t strides[1] = {(uint64_t)N * 2};
    const uint32_t box[2] = {kGroupN, 1};
    if (int rc = cached_tensor_map(&tmS, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, g.scales, dims, strides, box,
                                   CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
    tmZ = tmS;
    if (format_has_zp(FMT)) {
      if (int rc = cached_tensor_map(&tmZ, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, g.zeros, dims, strides, box,
                                     CU_TENSOR_MAP_SWIZZLE_NONE))
        return rc;
    }
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)NCOL};
    const uint64_t strides[1] = {(uint64_t)K};
    const uint32_t box[2] = {KCH, NCOL};
    if (int rc = cached_tensor_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, digits, dims, strides, box,
                                   CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  static bool attr_set[64] = {};
  int dev = 0;
  MB_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    MB_CUDA(cudaFuncSetAttribute(stream_i8_kernel<T, FMT, TOKH, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.num_ctas);
  cfg.blockDim = dim3(C::THREADS);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = g.stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MB_CUDA(cudaLaunchKernelEx(&cfg, stream_i8_kernel<T, FMT, TOKH, false>, tmA, tmS, tmZ, p));
  count_launches(1);
  return 0;
}

// ---- grouped (expert) form --------------------------------------------------------------------------------
// scratch: counters | partial sums | digit planes [2][rows][K] | row factors [rows] | digit sums [K / 128][rows]
int64_t grouped_counters_bytes(int64_t rows, int64_t n) { return ((rows / 8) * (n / kGroupN) * 4 + 255) & ~(int64_t)255; }

template <typename T, int FMT, int TOKH>
int launch_grouped(const GemmArgs& g) {
  using C = Cfg<TOKH>;
  constexpr int NTOK = C::NTOK;
  const int64_t K = g.size_k, N = g.size_n, R = g.num_sorted;
  I8Params p{};
  p.w = reinterpret_cast<const uint8_t*>(g.bq);
  p.c = g.c; p.bias = g.bias;
  p.M = (int)g.size_m; p.N = (int)N; p.K = (int)K;
  p.num_groups = (int)g.num_groups;
  p.kc = (int)(K / KCH);
  p.ngc = (int)(N / kGroupN);
  p.ng = 0;
  p.cps = (g.num_groups == 1) ? p.kc : (int)((K / g.num_groups) / KCH);
  p.rows_per_expert = (int)g.num_groups;
  p.sorted_ids = g.sorted_ids; p.expert_ids = g.expert_ids; p.num_post_pad = g.num_post_pad;
  p.topk_weights = g.topk_weights; p.mul_topk = g.mul_topk;
  p.num_routes = (int)(g.size_m * g.top_k);
  p.row_capacity = (int)R;
  p.sum_stride = (int)((R + 15) & ~(int64_t)15);
  uint8_t* sc = reinterpret_cast<uint8_t*>(g.scratch);
  const int64_t cb = grouped_counters_bytes(R, N), pb = partial_bytes(32);
  p.counters = reinterpret_cast<int*>(sc);
  p.partials = reinterpret_cast<float*>(sc + cb);
  int8_t* digits = reinterpret_cast<int8_t*>(sc + cb + pb);
  const int64_t digit_bytes = (2 * R * K + 255) & ~(int64_t)255;
  float* row_scale = reinterpret_cast<float*>(digits + digit_bytes);
  float* chunk_sums = row_scale + ((R + 63) & ~(int64_t)63);
  p.row_scale = row_scale;
  p.chunk_sums = chunk_sums;
  p.num_ctas = sm_count();
  p.tx_bytes = C::ACT_BYTES + NTOK * 4 + kGroupN * 2 * (format_has_zp(FMT) ? 2 : 1);

  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  int parts = 1;
  while (parts < 4 && K % (KCH * parts * 2) == 0 && K / (parts * 2) >= 8 * AD_THREADS) parts *= 2;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)R, parts);
    cfg.blockDim = dim3(AD_THREADS);
    cfg.stream = g.stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int num_counters = (int)((R / NTOK) * p.ngc);
    auto kern = g.silu_input ? act_digits_kernel<T, true, true> : act_digits_kernel<T, true, false>;
    MB_CUDA(cudaLaunchKernelEx(&cfg, kern, reinterpret_cast<const T*>(g.a), g.a_stride, (int)g.size_m,
                               (int)K, digits, row_scale, chunk_sums, p.counters, num_counters, g.sorted_ids,
                               g.num_post_pad, g.top_k, p.num_routes, p.sum_stride));
    count_launches(1);
  }
  CUtensorMap tmA, tmS, tmZ;
  {
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)(g.num_groups * g.num_experts)};
    const uint64_t strides[1] = {(uint64_t)N * 2};
    const uint32_t box[2] = {kGroupN, 1};
    if (int rc = cached_tensor_map(&tmS, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, g.scales, dims, strides, box,
                                   CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
    tmZ = tmS;
    if (format_has_zp(FMT)) {
      if (int rc = cached_tensor_map(&tmZ, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, g.zeros, dims, strides, box,
                                     CU_TENSOR_MAP_SWIZZLE_NONE))
        return rc;
    }
  }
  {
    // digit planes [2][rows][K]: one box = both planes of a block's rows over one 128-k chunk
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)R, 2};
    const uint64_t strides[2] = {(uint64_t)K, (uint64_t)R * K};
    const uint32_t box[3] = {KCH, (uint32_t)NTOK, 2};
    if (int rc = cached_tensor_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, digits, dims, strides, box,
                                   CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  static bool attr_set[64] = {};
  int dev = 0;
  MB_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    MB_CUDA(cudaFuncSetAttribute(stream_i8_kernel<T, FMT, TOKH, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.num_ctas);
  cfg.blockDim = dim3(C::THREADS);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = g.stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MB_CUDA(cudaLaunchKernelEx(&cfg, stream_i8_kernel<T, FMT, TOKH, true>, tmA, tmS, tmZ, p));
  count_launches(1);
  return 0;
}

template <typename T>
int launch_grouped_dtype(const GemmArgs& g) {
  switch (g.format) {
    case kU4B8: return g.block_size == 8 ? launch_grouped<T, kU4B8, 1>(g) : g.block_size == 16 ? launch_grouped<T, kU4B8, 2>(g) : launch_grouped<T, kU4B8, 4>(g);
    case kU4: return g.block_size == 8 ? launch_grouped<T, kU4, 1>(g) : g.block_size == 16 ? launch_grouped<T, kU4, 2>(g) : launch_grouped<T, kU4, 4>(g);
  }
  return 1;
}

template <typename T>
int launch_dtype(const GemmArgs& g) {
  switch (g.format) {
    case kU4B8: return g.size_m <= 8 ? launch_one<T, kU4B8, 1>(g) : g.size_m <= 16 ? launch_one<T, kU4B8, 2>(g) : launch_one<T, kU4B8, 4>(g);
    case kU4: return g.size_m <= 8 ? launch_one<T, kU4, 1>(g) : g.size_m <= 16 ? launch_one<T, kU4, 2>(g) : launch_one<T, kU4, 4>(g);
  }
  return 1;
}

}  // namespace

// counters, partial sums, then the digit planes (32 x K), the 16 row factors and K / 128 x 16 chunk sums
int64_t gemm_stream_i8_scratch_bytes(int64_t m, int64_t n, int64_t k) {
  if (m <= 0 || !stream::layout_accepts(k, n)) return 0;
  const int rows = m <= 16 ? 16 : 32;
  return counters_bytes(n) + partial_bytes(rows) + 2 * rows * k + 256 + (k / KCH) * rows * 4;
}

bool gemm_stream_i8_accepts(const GemmArgs& g) {
  if (g.sorted_ids != nullptr || !g.prepared) return false;
  if (g.format != kU4B8 && g.format != kU4) return false;
  if (g.size_m <= 0 || g.size_m > 32 || !stream::layout_accepts(g.size_k, g.size_n)) return false;
  if (g.num_groups > 1 && (g.size_k / g.num_groups) % KCH != 0) return false;
  if (g.global_scale != nullptr) return false;
  return g.scratch != nullptr && g.scratch_bytes >= gemm_stream_i8_scratch_bytes(g.size_m, g.size_n, g.size_k);
}

// grouped form: expert weights [E][...] in the streaming layout, blocks of 8, 16 or 32 sorted routes
int64_t gemm_stream_i8_grouped_scratch_bytes(int64_t num_sorted, int64_t n, int64_t k) {
  if (num_sorted <= 0 || !stream::layout_accepts(k, n)) return 0;
  return grouped_counters_bytes(num_sorted, n) + partial_bytes(32) + ((2 * num_sorted * k + 255) & ~(int64_t)255) +
         ((num_sorted + 63) & ~(int64_t)63) * 4 + (k / KCH) * ((num_sorted + 15) & ~(int64_t)15) * 4 + 256;
}

bool gemm_stream_i8_grouped_accepts(const GemmArgs& g) {
  if (g.sorted_ids == nullptr || !g.prepared) return false;
  if (g.format != kU4B8 && g.format != kU4) return false;
  if (g.block_size != 8 && g.block_size != 16 && g.block_size != 32) return false;
  if (g.num_sorted < g.block_size || !stream::layout_accepts(g.size_k, g.size_n)) return false;
  if (g.num_groups > 1 && (g.size_k / g.num_groups) % KCH != 0) return false;
  if (g.global_scale != nullptr) return false;
  return g.scratch != nullptr &&
         g.scratch_bytes >= gemm_stream_i8_grouped_scratch_bytes(g.num_sorted, g.size_n, g.size_k);
}

int launch_gemm_stream_i8_grouped(const GemmArgs& g) {
  if (g.act_dtype == MARLIN_B200_F16) return launch_grouped_dtype<__half>(g);
  return launch_grouped_dtype<__nv_bfloat16>(g);
}

int launch_gemm_stream_i8(const GemmArgs& g) {
  if (g.act_dtype == MARLIN_B200_F16) return launch_dtype<__half>(g);
  return launch_dtype<__nv_bfloat16>(g);
}

int read_stream_i8_status(int* value, bool reset) {
  MB_CUDA(cudaMemcpyFromSymbol(value, g_si8_status, sizeof(int)));
  if (reset && *value != 0) {
    const int zero = 0;
    MB_CUDA(cudaMemcpyToSymbol(g_si8_status, &zero, sizeof(int)));
  }
  return 0;
}

}  // namespace mb200
