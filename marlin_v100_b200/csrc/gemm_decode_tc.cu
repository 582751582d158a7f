// Decode-sized GEMM (M <= 16 rows) on the tcgen05 tensor cores: integer MMAs on 8-bit operands, weights
// as the tensor-memory operand.
//
//   C[M, N] = A[M, K] * dequant(Wq)[K, N]          (reference operator: csrc/quantization/marlin/marlin.cu:83)
//
// The contraction runs transposed, D[n, m] = sum_k W[k, n] * A[m, k]: the 128 rows of an MMA are 128
// weight columns, the MMA's N are token columns.  Both operands are 8-bit integers (kind::i8, exact
// 32-bit accumulation):
//
//  * Weights.  A 4-bit code becomes a byte with one logic instruction per four codes: the low nibbles
//    of a word are kept as they are (byte = q), the high nibbles are kept in place with their top bit
//    flipped (byte = 16 (q - 8) as a signed byte).  Bytes are written to tensor memory with
//    tcgen05.st; the M-side operand of tcgen05.mma may live there, so unpacked weights never touch
//    shared memory.  Byte = alpha (q - beta) with (alpha, beta) = (1, 0) or (16, 8), fixed per lane.
//  * Activations.  A small kernel in front rewrites every row as three signed 7-bit digits,
//    a = 2^(e-6) (d1 + d2 / 2^7 + d3 / 2^14), e from the row maximum: exact for every element within
//    2^-10 of the row maximum, absolute error <= 2^(e-21) otherwise (fp16 / bf16 carry 11 / 8
//    significant bits).  The three digit planes are three groups of 16 token columns of one MMA.
//
// Scales are applied after the MMA: with DD = D1 + D2 / 2^7 + D3 / 2^14 and SA the same combination
// of the digit sums over the scope's k, a scale group adds  (s / alpha) DD + (s (beta - zero) - zs) SA
// to the fp32 accumulators of the epilogue warps (zero = 8 for u4b8; zs = zero-point times scale as
// passed for u4).  The row factor 2^(e-6) is applied once at the end.
//
// Work split: persistent CTAs, one per SM, each owning a contiguous range of (256-column group,
// 128-k chunk) units.  Ranges that start or end inside a group leave fp32 partial sums in a scratch
// buffer which a small kernel adds in a fixed order (results repeat bit for bit).
//
// Warp roles (896 threads):  0 TMA producer | 1, 2 MMA issuers (one 128-column tile each; 1 owns the tensor
// memory) | 3 digit sums | 4-7 and 24-27 epilogue (tile, 32-lane quadrant) | 8-23 dequant (quadrant = warp % 4;
// warps 8-15 take the even chunks of the CTA's sequence, 16-23 the odd ones; a warp converts two of the chunk's four
// 32-k blocks).
// Every wait is bounded; a wait that gives up raises the CTA's abort flag, the kernel drains, frees
// its tensor memory and reports through g_dtc_status.

#include "codes.cuh"
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace mb200 {
namespace {

using codes::kHalf;

constexpr int GROUP_N = 256;
constexpr int THREADS = 896;
constexpr int KCH = 128;                  // k per chunk
constexpr int KB = KCH / 32;              // MMA k-blocks (32 k) per chunk
constexpr int KT16 = KCH / 16;            // 16-k rows of the packed tensor per chunk
constexpr int NDIG = 3;                   // digit planes of the activations
constexpr int NCOL = 16 * NDIG;           // token columns of an MMA
constexpr int STAGES = 8;                 // shared-memory ring
constexpr int TSTAGES = 4;                // tensor-memory operand ring
constexpr int RAW_BYTES = KCH * GROUP_N / 2;
constexpr int ACT_BYTES = NCOL * 128;     // digit rows of the chunk: 48 rows x 128 k
constexpr int META_BYTES = 2 * GROUP_N * 2;  // the chunk's scale row and zero row (16-bit each)
constexpr int OFF_ACT = RAW_BYTES;
constexpr int OFF_S = OFF_ACT + ACT_BYTES;
constexpr int OFF_Z = OFF_S + GROUP_N * 2;
constexpr int STAGE_BYTES = RAW_BYTES + ACT_BYTES + META_BYTES;
constexpr int TCOLS_STAGE = 2 * (KCH / 4);  // two 128-row tiles, one 32-bit column per four k
constexpr int DCOL = TSTAGES * TCOLS_STAGE;
constexpr int DBUF_COLS = 2 * NCOL;       // two tiles
constexpr int TMEM_COLS = 512;
constexpr int DQ_WARPS = 16;
constexpr int EPI_WARPS = 8;
constexpr int NUM_BARS = 3 * STAGES + TSTAGES + 4;
constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + NUM_BARS * 8 + 64;
static_assert(RAW_BYTES == 32 * 4 * 16 * KT16, "the weight box fills the raw part of a stage");
static_assert(DCOL + 2 * DBUF_COLS <= TMEM_COLS, "tensor memory budget");
static_assert(SMEM <= 227 * 1024, "shared memory budget");
static_assert(STAGE_BYTES % 1024 == 0 && OFF_ACT % 1024 == 0, "swizzled tiles stay 1024-byte aligned");

struct DtParams {
  void* c;
  const void* bias;
  const void* scales;
  const void* zeros;
  float* partials;
  const float* row_scale;   // 2^(e-6) per token row, written by act_digits_kernel
  int M, N, K;
  int num_groups;
  int cps;      // chunks per scale row (kc when there is one row)
  int kc, ng;
  uint32_t tx_bytes;
  int num_ctas;
};

__device__ int g_dtc_status = 0;


__device__ __forceinline__ int64_t range_start(int64_t p, int64_t U, int64_t P) { return p * U / P; }

// Programmatic dependent launch: the three kernels of a call are chained so that the next one may start
// (set up barriers, stream weights) while the previous one still runs; whoever consumes the previous
// kernel's output waits here first.
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The (group, chunk) units of a CTA in order, with the segment / scope boundaries every role needs.
// A segment is a run of chunks of one column group, a scope a run of chunks that share a scale row.
struct UnitWalk {
  int g, c, left, kc, cps, sp;  // sp = c % cps, kept incrementally
  bool first_unit;
  __device__ void init(int64_t u0, int64_t u1, int kc_, int cps_) {
    kc = kc_; cps = cps_;
    g = (int)(u0 / kc);
    c = (int)(u0 - (int64_t)g * kc);
    sp = c % cps;
    left = (int)(u1 - u0);
    first_unit = true;
  }
  __device__ bool valid() const { return left > 0; }
  __device__ bool seg_start() const { return first_unit || c == 0; }
  __device__ bool seg_end() const { return left == 1 || c == kc - 1; }
  __device__ bool scope_start() const { return first_unit || sp == 0; }
  __device__ bool scope_end() const { return left == 1 || c == kc - 1 || sp == cps - 1; }
  __device__ void next() {
    --left;
    first_unit = false;
    ++c;
    if (++sp == cps) sp = 0;
    if (c == kc) { c = 0; sp = 0; ++g; }
  }
};

template <typename T>
__device__ __forceinline__ T lds_as(uint32_t addr) {
  const unsigned short v = (unsigned short)lds16(addr);
  return *reinterpret_cast<const T*>(&v);
}

// kind::i8 instruction descriptor: s32 accumulate, signed 8-bit A and B, both K-major, M = 128, N = NCOL
__device__ __forceinline__ constexpr uint32_t instr_desc_i8() {
  uint32_t d = 0;
  d |= 2u << 4;                        // D format s32
  d |= 1u << 7;                        // A signed 8-bit
  d |= 1u << 10;                       // B signed 8-bit
  d |= (uint32_t)(NCOL >> 3) << 17;    // N
  d |= (uint32_t)(128 >> 4) << 24;     // M
  return d;
}
__device__ __forceinline__ void tc_mma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Order of k inside a block of 32: the digit (and the weight byte) of k sits at position
// 8t + (i ^ 2t) with t = k % 32 / 8, i = k % 8.  The eight k of a dequant thread are rotated that way so
// that its shared-memory reads of the packed words fall into 32 different banks; weights and digits use
// the same order, which is all a contraction needs.

// Weight column (inside the 256-column group) held by lane `lane` of quadrant `quad`, tile `tile`.
// The dequant thread (g, t) of that quadrant reads the packed words (nv = 2 quad + g / 4, sub = g % 4);
// byte j = 2 tile + half of a word holds the codes of columns order[2j] (low nibble, lanes 0-7 of the
// half) and order[2j + 1] (high nibble, lanes 8-15), order = 0,2,4,6,1,3,5,7.
__device__ __forceinline__ int lane_column(int quad, int tile, int lane) {
  const int h = lane >> 4, r = lane & 15, g = r & 7, hi = r >> 3;
  const int pos = 2 * (2 * tile + h) + hi;               // nibble position inside the word
  const int n_local = (pos & 3) * 2 + (pos >> 2);       // order[pos]
  return 64 * (g & 3) + 8 * (2 * quad + (g >> 2)) + n_local;
}

// ---- activations -> digit planes -----------------------------------------------------------------------
// One block per token row.  digits: int8 [NCOL][K], row d * 16 + m; rows of absent tokens are zero.
template <typename T>
__global__ void __launch_bounds__(256) act_digits_kernel(const T* __restrict__ a, int64_t a_stride, int M, int K,
                                                         int8_t* __restrict__ digits, float* __restrict__ row_scale) {
  const int m = blockIdx.x, tid = threadIdx.x;
  pdl_release_dependents();
  __shared__ float s_red[8];
  __shared__ float s_max;
  const int vecs = K / 8;
  if (m >= M) {
    for (int v = tid; v < vecs; v += 256)
#pragma unroll
      for (int d = 0; d < NDIG; ++d) *reinterpret_cast<uint2*>(digits + (int64_t)(d * 16 + m) * K + v * 8) = make_uint2(0, 0);
    if (tid == 0) row_scale[m] = 0.f;
    return;
  }
  const T* row = a + (int64_t)m * a_stride;
  float mx = 0.f;
  for (int v = tid; v < vecs; v += 256) {
    const uint4 q = *reinterpret_cast<const uint4*>(row + v * 8);
    const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(to_float<T>(e[i])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) s_red[tid >> 5] = mx;
  __syncthreads();
  if (tid == 0) {
    float t = s_red[0];
    for (int i = 1; i < 8; ++i) t = fmaxf(t, s_red[i]);
    s_max = t;
  }
  __syncthreads();
  mx = s_max;
  int e = 0;
  if (mx > 0.f && mx < 3.0e38f) (void)frexpf(mx, &e);   // mx = f * 2^e, f in [0.5, 1)
  // x64 = a * 2^(6 - e), |x64| < 64; done as two exact power-of-two multiplies to stay in range
  const float f1 = ldexpf(1.f, (6 - e) / 2), f2 = ldexpf(1.f, (6 - e) - (6 - e) / 2);
  if (tid == 0) row_scale[m] = (mx > 0.f && mx < 3.0e38f) ? ldexpf(1.f, e - 6) : 0.f;
  for (int v = tid; v < vecs; v += 256) {
    const uint4 q = *reinterpret_cast<const uint4*>(row + v * 8);
    const T* el = reinterpret_cast<const T*>(&q);
    const int t = v & 3;  // (k / 8) % 4
    uint32_t out[NDIG][2] = {};
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // natural order first
      const float x = to_float<T>(el[i]) * f1 * f2;
      const float d1 = rintf(x);
      const float r1 = (x - d1) * 128.f;
      const float d2 = rintf(r1);
      const float r2 = (r1 - d2) * 128.f;
      const float d3 = rintf(r2);
      const float dd[3] = {d1, d2, d3};
#pragma unroll
      for (int d = 0; d < NDIG; ++d) out[d][i >> 2] |= ((uint32_t)(int)dd[d] & 0xffu) << (8 * (i & 3));
    }
#pragma unroll
    for (int d = 0; d < NDIG; ++d) {
      // position i ^ 2t: bit 1 of t swaps the byte pairs of each word, bit 2 swaps the words
      uint32_t lo = out[d][0], hi = out[d][1];
      if (t & 1) { lo = prmt(lo, 0u, 0x1032u); hi = prmt(hi, 0u, 0x1032u); }
      if (t & 2) { const uint32_t x = lo; lo = hi; hi = x; }
      *reinterpret_cast<uint2*>(digits + (int64_t)(d * 16 + m) * K + v * 8) = make_uint2(lo, hi);
    }
  }
}

template <typename T, int FMT>
__global__ void __launch_bounds__(THREADS, 1)
decode_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
                 const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ, const DtParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = base + STAGES * STAGE_BYTES;
  // Chunk i of the CTA uses shared-memory stage i % STAGES (lap parity (i / STAGES) & 1) and operand
  // stage i % TSTAGES; scope j uses accumulator buffer j % 2.
  auto full = [&](int s) { return bar0 + 8u * s; };                       // TMA data landed
  auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };           // every shared-memory reader is done
  auto mma_done = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };    // the chunk's MMAs have completed
  auto a_ready = [&](int t) { return bar0 + 8u * (3 * STAGES + t); };     // operand bytes are in tensor memory
  auto d_free = [&](int b) { return bar0 + 8u * (3 * STAGES + TSTAGES + b); };
  auto sum_full = [&](int b) { return bar0 + 8u * (3 * STAGES + TSTAGES + 2 + b); };
  const uint32_t tmem_slot = bar0 + 8u * NUM_BARS;
  auto drain_bar = [&](int w) { return bar0 + 8u * NUM_BARS + 16u + 8u * w; };   // give-up path of the MMA issuers

  __shared__ int s_abort;
  __shared__ float s_asum[2][16];
  __shared__ int s_isum[NCOL];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), DQ_WARPS / 2 + 1 + EPI_WARPS);
      mbar_init(mma_done(s), 2);
    }
    for (int t = 0; t < TSTAGES; ++t) mbar_init(a_ready(t), DQ_WARPS / 2);
    for (int b = 0; b < 2; ++b) { mbar_init(d_free(b), EPI_WARPS); mbar_init(sum_full(b), 1); }
    mbar_init(drain_bar(0), 1);
    mbar_init(drain_bar(1), 1);
    fence_barrier_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmS);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = lds32(tmem_slot);

  const int64_t U = (int64_t)p.ng * p.kc;
  const int64_t u0 = range_start(blockIdx.x, U, p.num_ctas);
  const int64_t u1 = range_start(blockIdx.x + 1, U, p.num_ctas);
  UnitWalk w;
  w.init(u0, u1, p.kc, p.cps);
  pdl_release_dependents();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // Lanes 0-3 run the same loop side by side, lane l for the chunks l, l + 4, ...: one pass of the
    // loop puts four chunks in flight for the instruction count of one.
    if (lane < 4) {
      const int total = (int)(u1 - u0);
      int g = w.g, c = w.c + lane;
      while (c >= p.kc) { c -= p.kc; ++g; }
      auto issue = [&](int i, int gi, int ci, bool weights, bool digits) {
        const int s = i & (STAGES - 1);
        const uint32_t st = base + s * STAGE_BYTES;
        if (weights) {
          mbar_arrive_expect_tx(full(s), p.tx_bytes);
          tma_load_3d(st, &tmW, full(s), 0, gi * 16, ci * KT16);
          const int srow = (p.num_groups == 1) ? 0 : (ci / p.cps);
          tma_load_2d(st + OFF_S, &tmS, full(s), gi * GROUP_N, srow);
          if constexpr (format_has_zp(FMT)) tma_load_2d(st + OFF_Z, &tmZ, full(s), gi * GROUP_N, srow);
        }
        if (digits) tma_load_2d(st + OFF_ACT, &tmA, full(s), ci * KCH, 0);
      };
      // First lap of the ring: weights and scales go out at once, the digit planes only after the
      // kernel that writes them has finished (it may still be running when this kernel starts).
      const int g0 = g, c0 = c;
      c += 4;
      while (c >= p.kc) { c -= p.kc; ++g; }
      const int g1 = g, c1 = c;
      int last = -1;   // the last chunk this lane has issued copies for
      if (lane < total) { issue(lane, g0, c0, true, false); last = lane; }
      if (lane + 4 < total) { issue(lane + 4, g1, c1, true, false); last = lane + 4; }
      pdl_wait_prior_grid();
      if (lane < total) issue(lane, g0, c0, false, true);
      if (lane + 4 < total) issue(lane + 4, g1, c1, false, true);
      c += 4;
      while (c >= p.kc) { c -= p.kc; ++g; }
      for (int i = lane + 8; i < total; i += 4) {
        const int s = i & (STAGES - 1);
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        // weights and scales as soon as every shared-memory reader of the stage is done; the digit tile
        // (the MMA's B operand) only once the MMAs that read the old one have completed
        if (!mbar_wait(empty(s), ph ^ 1u, &s_abort)) { atomicExch(&g_dtc_status, 1); break; }
        issue(i, g, c, true, false);
        last = i;
        if (!mbar_wait(mma_done(s), ph ^ 1u, &s_abort)) { atomicExch(&g_dtc_status, 1); break; }
        issue(i, g, c, false, true);
        c += 4;
        while (c >= p.kc) { c -= p.kc; ++g; }
      }
      // no copy of this lane's is in flight when it leaves (a CTA must not exit with copies on their way into its
      // shared memory; after a give-up nobody else waits for them)
      if (s_abort != 0)
        for (int i = last; i >= 0 && i > last - STAGES; i -= 4) drain_barrier(full(i & (STAGES - 1)), (uint32_t)(i / STAGES) & 1u);
    }
  } else if (warp == 1 || warp == 2) {
    // ---------------- MMA issuers: warp 1 for the first 128-column tile, warp 2 for the second ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_i8();
      const int tile = warp - 1;
      const uint64_t desc0 = kmajor_sw128_desc(base + OFF_ACT);
      int i = 0, j = 0;
      for (; w.valid(); w.next(), ++i) {
        const bool sc_start = w.scope_start(), sc_end = w.scope_end();
        if (sc_start) {
          if (!mbar_wait(d_free(j & 1), (((uint32_t)j >> 1) & 1u) ^ 1u, &s_abort)) { atomicExch(&g_dtc_status, 2); break; }
        }
        if (!mbar_wait(a_ready(i & (TSTAGES - 1)), ((uint32_t)i / TSTAGES) & 1u, &s_abort)) { atomicExch(&g_dtc_status, 4); break; }
        tc_fence_after();
        const int s = i & (STAGES - 1);
        const uint64_t desc = desc0 + (uint64_t)((s * STAGE_BYTES) >> 4);
        const uint32_t a_addr = tmem + (i & (TSTAGES - 1)) * TCOLS_STAGE + tile * (KCH / 4);
        const uint32_t d_addr = tmem + DCOL + (j & 1) * DBUF_COLS + tile * NCOL;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tc_mma_i8_ts(d_addr, a_addr + kb * 8, desc + kb * 2, idesc, (sc_start && kb == 0) ? 0u : 1u);
        tc_commit(mma_done(s));
        if (sc_end) ++j;
      }
      // the tensor memory is freed only after this thread's MMAs have completed (after a give-up nobody else waits)
      if (s_abort != 0) {
        tc_commit(drain_bar(tile));
        drain_barrier(drain_bar(tile), 0);
      }
    }
  } else if (warp == 3) {
    // ---------------- digit sums per scope ----------------
    // lanes 0-23 add up two digit rows each (the 128 bytes of a row in whatever swizzled order);
    // at the end of a scope lanes 0-15 combine the three planes of their token.
    int i = 0, j = 0;
    int part0 = 0, part1 = 0;
    bool ok = true;
    for (; w.valid(); w.next(), ++i) {
      const int s = i & (STAGES - 1);
      if (ok && !mbar_wait(full(s), ((uint32_t)i / STAGES) & 1u, &s_abort)) { atomicExch(&g_dtc_status, 5); ok = false; }
      if (ok) {
        if (w.scope_start()) { part0 = 0; part1 = 0; }
        if (lane < NCOL / 2) {
          const uint32_t row = base + s * STAGE_BYTES + OFF_ACT + (2 * lane) * 128;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            // lane l starts at piece l of its rows: the 24 lanes of one load spread over all banks
            const uint32_t piece = (uint32_t)((q + lane) & 7) * 16;
            const uint4 v0 = lds128(row + piece), v1 = lds128(row + 128 + piece);
            part0 = __dp4a((int)v0.x, 0x01010101, part0); part0 = __dp4a((int)v0.y, 0x01010101, part0);
            part0 = __dp4a((int)v0.z, 0x01010101, part0); part0 = __dp4a((int)v0.w, 0x01010101, part0);
            part1 = __dp4a((int)v1.x, 0x01010101, part1); part1 = __dp4a((int)v1.y, 0x01010101, part1);
            part1 = __dp4a((int)v1.z, 0x01010101, part1); part1 = __dp4a((int)v1.w, 0x01010101, part1);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty(s));
      if (w.scope_end()) {
        const int db = j & 1;
        if (ok && !mbar_wait(d_free(db), (((uint32_t)j >> 1) & 1u) ^ 1u, &s_abort)) { atomicExch(&g_dtc_status, 6); ok = false; }
        if (lane < NCOL / 2) { s_isum[2 * lane] = part0; s_isum[2 * lane + 1] = part1; }
        __syncwarp();
        if (ok && lane < 16) {
          float v = (float)s_isum[lane];
          if (NDIG > 1) v = fmaf((float)s_isum[16 + lane], 1.f / 128.f, v);
          if (NDIG > 2) v = fmaf((float)s_isum[32 + lane], 1.f / 16384.f, v);
          s_asum[db][lane] = v;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(sum_full(db));
        ++j;
      }
    }
  } else if ((warp >= 4 && warp < 8) || warp >= 24) {
    // ---------------- epilogue: warps 4-7 own the first tile, warps 24-27 the second ----------------
    const int tile = (warp >= 24) ? 1 : 0;
    const int quad = warp & 3;
    const int ncol = lane_column(quad, tile, lane);
    // byte = alpha (q - beta): low-nibble lanes (1, 0), high-nibble lanes (16, 8)
    const bool hi_lane = (lane & 8) != 0;
    const float inv_alpha = hi_lane ? 1.f / 16.f : 1.f;
    const float beta_minus_zero = (hi_lane ? 8.f : 0.f) - (FMT == kU4B8 ? 8.f : 0.f);
    float acc[16];
    int i = 0, j = 0;
    bool ok = true;
    int seg_c0 = 0;
    bool first_segment = true;
    float sv = 0.f, zv = 0.f;
    for (; w.valid(); w.next(), ++i) {
      const int s = i & (STAGES - 1);
      const uint32_t ph = ((uint32_t)i / STAGES) & 1u;
      if (w.seg_start()) {
        seg_c0 = w.c;
#pragma unroll
        for (int m = 0; m < 16; ++m) acc[m] = 0.f;
      }
      // every chunk's stage carries the scale (and zero) row of its scope; the last chunk's copy is used
      if (ok && !mbar_wait(full(s), ph, &s_abort)) { atomicExch(&g_dtc_status, 11); ok = false; }
      const bool sc_end = w.scope_end();
      if (ok && sc_end) {
        const uint32_t st = base + s * STAGE_BYTES;
        sv = to_float<T>(lds_as<T>(st + OFF_S + ncol * 2));
        if constexpr (format_has_zp(FMT)) zv = to_float<T>(lds_as<T>(st + OFF_Z + ncol * 2));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty(s));
      if (sc_end) {
        const int db = j & 1;
        const uint32_t dph = ((uint32_t)j >> 1) & 1u;
        if (ok && !mbar_wait(mma_done(s), ph, &s_abort)) { atomicExch(&g_dtc_status, 7); ok = false; }
        if (ok && !mbar_wait(sum_full(db), dph, &s_abort)) { atomicExch(&g_dtc_status, 8); ok = false; }
        if (ok) {
          tc_fence_after();
          // three loads of 16 columns (one per digit plane); two in flight at a time
          const uint32_t dbase = tmem + ((uint32_t)(32 * quad) << 16) + DCOL + db * DBUF_COLS + tile * NCOL;
          uint32_t va[16], vb[16];
          tmem_ld16(dbase, va);
          tmem_ld16(dbase + 16, vb);
          tmem_ld_wait();
          const float t0 = sv * inv_alpha, t1 = t0 * (1.f / 128.f), t2 = t0 * (1.f / 16384.f);
#pragma unroll
          for (int m = 0; m < 16; ++m) acc[m] = fmaf(t0, (float)(int)va[m], acc[m]);
          if (NDIG > 2) tmem_ld16(dbase + 32, va);
#pragma unroll
          for (int m = 0; m < 16; ++m) acc[m] = fmaf(t1, (float)(int)vb[m], acc[m]);
          if (NDIG > 2) {
            tmem_ld_wait();
#pragma unroll
            for (int m = 0; m < 16; ++m) acc[m] = fmaf(t2, (float)(int)va[m], acc[m]);
          }
          const float cfix = sv * beta_minus_zero - zv;
#pragma unroll
          for (int m = 0; m < 16; ++m) acc[m] = fmaf(cfix, s_asum[db][m], acc[m]);
          tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(d_free(db));
        ++j;
      }
      if (w.seg_end()) {
        if (first_segment) pdl_wait_prior_grid();  // row factors come from the kernel in front
        if (ok && s_abort == 0) {
          const bool whole = (seg_c0 == 0) && (w.c == p.kc - 1);
          if (whole) {
            T* C = reinterpret_cast<T*>(p.c);
            const T* bias = reinterpret_cast<const T*>(p.bias);
            const int n = w.g * GROUP_N + ncol;
            const float b = (bias != nullptr) ? to_float<T>(bias[bias_index(n)]) : 0.f;
#pragma unroll
            for (int m = 0; m < 16; ++m)
              if (m < p.M) C[(int64_t)m * p.N + n] = from_float<T>(fmaf(acc[m], p.row_scale[m], b));
          } else {
            float* P = p.partials + ((int64_t)blockIdx.x * 2 + (first_segment ? 0 : 1)) * (16 * GROUP_N);
#pragma unroll
            for (int m = 0; m < 16; ++m) P[m * GROUP_N + ncol] = (m < p.M) ? acc[m] * p.row_scale[m] : 0.f;
          }
        }
        first_segment = false;
      }
    }
  } else {
    // ---------------- dequant (warps 8-23) ----------------
    // Two groups of eight warps take alternate chunks (a warp converts two of the chunk's four 32-k blocks), so that
    // one group's wait for its tensor-memory stores overlaps the other group's loads and byte transposes.
    const int quad = warp & 3, kb0 = 2 * (((warp - 8) >> 2) & 1), grp = (warp - 8) >> 3;
    const int g = lane >> 2, t = lane & 3;
    const int nv = 2 * quad + (g >> 2), sub = g & 3;
    // The thread's eight packed words of a 32-k block: k = 8t + (q ^ 2t), q = 0..7 (the rotation
    // spreads the 32 lanes over 32 banks); byte offsets inside the chunk, 128-byte swizzle folded in.
    int woff[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int kk = 8 * t + (q ^ (2 * t));       // k inside the 32-k block
      const int lk = kk & 15;
      woff[q] = (kb0 * 2 + (kk >> 4)) * 2048 + lk * 128 + ((nv ^ (lk & 7)) << 4) + sub * 4;
    }
    bool ok = true;
    int i = 0;
    for (; w.valid(); w.next(), ++i) {
      if ((i & 1) != grp) continue;
      const int s = i & (STAGES - 1), ts = i & (TSTAGES - 1);
      if (ok && !mbar_wait(full(s), ((uint32_t)i / STAGES) & 1u, &s_abort)) { atomicExch(&g_dtc_status, 9); ok = false; }
      uint32_t x[2][8];
      if (ok) {
        const uint32_t raw = base + s * STAGE_BYTES;
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
#pragma unroll
          for (int q = 0; q < 8; ++q) x[kk][q] = lds32(raw + woff[q] + kk * 4096);   // the next 32-k block is 4096 bytes on
      }
      // the operand stage is free once the MMAs of the chunk that used it last have completed
      if (ok && i >= TSTAGES) {
        const int ip = i - TSTAGES;
        if (!mbar_wait(mma_done(ip & (STAGES - 1)), ((uint32_t)ip / STAGES) & 1u, &s_abort)) { atomicExch(&g_dtc_status, 10); ok = false; }
      }
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
        const int kb = kb0 + kk;
        // 4 x 4 byte transposes: o[c][b] = byte b of the four words of column c (four consecutive k slots)
        uint32_t o[2][4];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint32_t a01 = prmt(x[kk][4 * c], x[kk][4 * c + 1], 0x5140u), a23 = prmt(x[kk][4 * c + 2], x[kk][4 * c + 3], 0x5140u);
          const uint32_t b01 = prmt(x[kk][4 * c], x[kk][4 * c + 1], 0x7362u), b23 = prmt(x[kk][4 * c + 2], x[kk][4 * c + 3], 0x7362u);
          o[c][0] = prmt(a01, a23, 0x5410u);
          o[c][1] = prmt(a01, a23, 0x7632u);
          o[c][2] = prmt(b01, b23, 0x5410u);
          o[c][3] = prmt(b01, b23, 0x7632u);
        }
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int b = 2 * tile + h;
            const uint32_t taddr = tmem + ((uint32_t)(32 * quad + 16 * h) << 16) + ts * TCOLS_STAGE + tile * (KCH / 4) + kb * 8;
            // lanes g: low nibbles as they are; lanes g + 8: high nibbles in place, top bit flipped
            tmem_st_16x256b(taddr, o[0][b] & 0x0f0f0f0fu, o[1][b] & 0x0f0f0f0fu,
                            (o[0][b] ^ 0x80808080u) & 0xf0f0f0f0u, (o[1][b] ^ 0x80808080u) & 0xf0f0f0f0u);
          }
        }
        tmem_st_wait();
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(a_ready(ts));
        mbar_arrive(empty(s));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// Adds the fp32 partials of every column group that was split across CTAs, in CTA order.  One thread
// per output element; grid = (groups, token rows).
template <typename T>
__global__ void __launch_bounds__(GROUP_N) decode_tc_reduce_kernel(const DtParams p) {
  const int g = blockIdx.x, tk = blockIdx.y;
  const int64_t U = (int64_t)p.ng * p.kc, P = p.num_ctas;
  const int64_t ua = (int64_t)g * p.kc, ub = ua + p.kc - 1;
  const int64_t pa = ((ua + 1) * P - 1) / U, pb = ((ub + 1) * P - 1) / U;
  pdl_wait_prior_grid();   // before any return: the grid never retires ahead of the kernel in front
  if (pa == pb) return;    // written directly by its only owner
  const int col = threadIdx.x;
  const int n = g * GROUP_N + col;
  constexpr int SLOT = 16 * GROUP_N;
  // the first owner's range either starts with this group (its first segment, slot 0) or reaches it
  // later (slot 1); every further owner starts inside the group (slot 0)
  const int first_slot = (range_start(pa, U, P) == ua) ? 0 : 1;
  const float* src = p.partials + tk * GROUP_N + col;
  float v = src[(pa * 2 + first_slot) * SLOT];
  for (int64_t q = pa + 1; q <= pb; ++q) v += src[(q * 2) * SLOT];
  float b = 0.f;
  if (p.bias != nullptr) b = to_float<T>(reinterpret_cast<const T*>(p.bias)[bias_index(n)]);
  reinterpret_cast<T*>(p.c)[(int64_t)tk * p.N + n] = from_float<T>(v + b);
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------
template <typename T, int FMT>
int launch_one(const GemmArgs& g, const void* a, void* c, int m) {
  const int64_t K = g.size_k, N = g.size_n;
  DtParams p{};
  p.c = c; p.bias = g.bias; p.scales = g.scales; p.zeros = g.zeros;
  // scratch: split-K partials | digit planes | row factors
  const int64_t part_bytes = (int64_t)sm_count() * 2 * 16 * GROUP_N * (int64_t)sizeof(float);
  p.partials = reinterpret_cast<float*>(g.scratch);
  int8_t* digits = reinterpret_cast<int8_t*>(g.scratch) + part_bytes;
  float* row_scale = reinterpret_cast<float*>(digits + (int64_t)NCOL * K);
  p.row_scale = row_scale;
  p.M = m; p.N = (int)N; p.K = (int)K;
  p.num_groups = (int)g.num_groups;
  p.kc = (int)(K / KCH);
  p.ng = (int)(N / GROUP_N);
  p.cps = (g.num_groups == 1) ? p.kc : (int)((K / g.num_groups) / KCH);
  const int64_t U = (int64_t)p.ng * p.kc;
  p.num_ctas = (int)(U < sm_count() ? U : sm_count());

  p.tx_bytes = RAW_BYTES + ACT_BYTES + GROUP_N * 2 * (format_has_zp(FMT) ? 2 : 1);
  act_digits_kernel<T><<<16, 256, 0, g.stream>>>(reinterpret_cast<const T*>(a), g.a_stride, m, (int)K, digits, row_scale);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  CUtensorMap tmW, tmA, tmS, tmZ;
  {
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)g.num_groups};
    const uint64_t strides[1] = {(uint64_t)N * 2};
    const uint32_t box[2] = {GROUP_N, 1};
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
    const uint64_t dims[3] = {32, (uint64_t)(16 * p.ng), (uint64_t)(K / 16)};
    const uint64_t strides[2] = {128, (uint64_t)(16 * p.ng) * 128};
    const uint32_t box[3] = {32, 16, KT16};
    if (int rc = cached_tensor_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, g.bq, dims, strides, box,
                                   CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)NCOL};
    const uint64_t strides[1] = {(uint64_t)K};
    const uint32_t box[2] = {KCH, NCOL};
    if (int rc = encode_tensor_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, digits, dims, strides, box,
                                   CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  static bool attr_set[64] = {};
  int dev = 0;
  MB_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    MB_CUDA(cudaFuncSetAttribute(decode_tc_kernel<T, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    attr_set[dev] = true;
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.num_ctas);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = g.stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MB_CUDA(cudaLaunchKernelEx(&cfg, decode_tc_kernel<T, FMT>, tmW, tmA, tmS, tmZ, p));
    count_launches(1);
  }
  // the reduce kernel is launched only when some column group really has more than one owner
  bool any_split = false;
  for (int64_t gi = 0; gi < p.ng && !any_split; ++gi) {
    const int64_t ua = gi * p.kc, ub = ua + p.kc - 1;
    any_split = ((ua + 1) * p.num_ctas - 1) / U != ((ub + 1) * p.num_ctas - 1) / U;
  }
  if (any_split) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.ng, m);
    cfg.blockDim = dim3(GROUP_N);
    cfg.stream = g.stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MB_CUDA(cudaLaunchKernelEx(&cfg, decode_tc_reduce_kernel<T>, p));
    count_launches(1);
  }
  return 0;
}

template <typename T, int FMT>
int launch_fmt(const GemmArgs& g) {
  const int64_t need = gemm_decode_scratch_bytes(g.size_m, g.size_n, g.size_k, FMT);
  if (g.scratch == nullptr || g.scratch_bytes < need) {
    set_error("scratch buffer too small: %lld bytes given, %lld needed", (long long)g.scratch_bytes, (long long)need);
    return MARLIN_B200_ESCRATCH;
  }
  const T* A = reinterpret_cast<const T*>(g.a);
  T* C = reinterpret_cast<T*>(g.c);
  for (int64_t m0 = 0; m0 < g.size_m; m0 += 16) {
    const int m = (int)(g.size_m - m0 < 16 ? g.size_m - m0 : 16);
    if (int rc = launch_one<T, FMT>(g, A + m0 * g.a_stride, C + m0 * g.size_n, m)) return rc;
  }
  return 0;
}

template <typename T>
int launch_dtype(const GemmArgs& g) {
  switch (g.format) {
    case kU4B8: return launch_fmt<T, kU4B8>(g);
    case kU4: return launch_fmt<T, kU4>(g);
  }
  return 1;
}

}  // namespace

// Returns 1 when the shape or format is left to the other kernels.
int launch_gemm_decode_tc(const GemmArgs& g) {
  if (g.sorted_ids != nullptr) return 1;
  if (g.format != kU4B8 && g.format != kU4) return 1;
  if (g.size_m <= 0 || g.size_n % GROUP_N != 0 || g.size_k % KCH != 0) return 1;
  if (g.num_groups > 1) {
    const int64_t gs = g.size_k / g.num_groups;
    if (gs % KCH != 0) return 1;
  }
  if (g.act_dtype == MARLIN_B200_F16) return launch_dtype<__half>(g);
  return launch_dtype<__nv_bfloat16>(g);
}

// Reads (and optionally clears) the word a kernel of this file sets when one of its bounded waits gave up.
int read_decode_tc_status(int* value, bool reset) {
  MB_CUDA(cudaMemcpyFromSymbol(value, g_dtc_status, sizeof(int)));
  if (reset && *value != 0) {
    const int zero = 0;
    MB_CUDA(cudaMemcpyToSymbol(g_dtc_status, &zero, sizeof(int)));
  }
  return 0;
}


}  // namespace mb200

