// Weight-streaming GEMM on the tcgen05 tensor cores for weights in the streaming layout
// (stream_layout.cuh): every size_m, all seven weight formats.
//
//   C[M, N] = A[M, K] * dequant(Wq)[K, N] (+ bias)      (reference operator: csrc/quantization/marlin/marlin.cu:83)
//
// The contraction runs transposed, D[n, m] = sum_k W[k, n] * A[m, k]: the 128 rows of an MMA are 128 weight
// columns, the MMA's N are MT token columns (16, 64 or 128; an MMA with M = 128 costs the same ~45 cycles for
// every N up to 64 and 64 cycles at N = 128).  Weights are decoded to the activation type in registers
// (scale and zero-point applied there, the reference's own dequantisation), written to tensor memory with
// tcgen05.st and used from there as the M-side operand of tcgen05.mma.kind::f16; decoded weights never touch
// shared memory.  Activations come straight from A by TMA (K-major, 128-byte swizzle) as the N-side operand.
// The accumulators stay in tensor memory for a whole run of k, so the epilogue runs once per column group,
// not once per scale group: the cost per weight byte does not depend on the group size or on M.
//
// Work split: persistent CTAs, one per SM, each owning a contiguous range of (256-column group, 128-k chunk)
// units, which in the streaming layout is one linear range of weight bytes.  A column group whose k range is
// shared by several CTAs leaves fp32 partial sums in scratch; the CTA that finishes last (a counter per column
// group, no waiting) adds them in CTA order and writes C, so results repeat bit for bit.
//
// Warps (736 threads): 0-3 epilogue (one per 32-lane quadrant of tensor memory) | 4-19 dequant (quadrant =
// warp % 4, (tile, chunk parity) = (warp - 4) / 4: two groups of eight warps on alternate chunks, a warp converts
// both 16-lane halves) | 20 TMA producer | 21, 22 MMA issuers (one 128-column tile each; 21 owns the tensor memory).
// Every wait is bounded; a wait that gives up raises the CTA's abort flag, the kernel drains, frees its
// tensor memory and reports through g_stream_status.
#pragma once

#include "codes.cuh"
#include "common.cuh"
#include "stream_layout.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace mb200 {
namespace stream {

using codes::kHalf;

constexpr int KCH = 128;   // k per chunk (two 64-k blocks of the streaming layout)
constexpr int THREADS = 736;
constexpr int EPI_WARPS = 4, DQ_WARP0 = 4, DQ_WARPS = 16, PROD_WARP = 20, MMA_WARP = 21, MMA_WARP2 = 22;
constexpr int TMEM_COLS = 512;
constexpr int A_COLS = 128;  // tensor-memory columns of one operand stage: 2 tiles x 64 (128 k as 16-bit pairs)

constexpr int round_up_c(int x, int a) { return (x + a - 1) / a * a; }

// SMODE 0: one scale row per chunk (group size a multiple of 128, or per-channel).
// SMODE 1: group size 16 / 32 / 64: 8 / 4 / 2 rows per chunk, picked per 16 k.
template <int FMT, int MT, int SMODE>
struct Cfg {
  static constexpr int BITS = format_bits(FMT);
  static constexpr int RAW_BYTES = KCH * kGroupN * BITS / 8;
  static constexpr int ACT_HALF = MT * 128;              // MT rows x 64 k x 2 bytes
  static constexpr int SROWS = SMODE ? 8 : 1;
  static constexpr int SELEM = format_scale_is_byte(FMT) ? 1 : 2;
  static constexpr int S_BYTES = SROWS * kGroupN * SELEM;
  static constexpr int OFF_ACT = RAW_BYTES;
  static constexpr int OFF_S = OFF_ACT + 2 * ACT_HALF;
  static constexpr int OFF_Z = OFF_S + S_BYTES;
  static constexpr int STAGE_BYTES = round_up_c(OFF_Z + (format_has_zp(FMT) ? S_BYTES : 0), 1024);
  static constexpr int STAGES_FIT = (227 * 1024 - 2048) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT < 8 ? STAGES_FIT : 8;
  static constexpr int TSTAGES = (MT <= 64) ? 3 : 2;
  static constexpr int NBUF = (TSTAGES * A_COLS + 4 * MT <= TMEM_COLS) ? 2 : 1;  // accumulator buffers
  static constexpr int DCOL = TSTAGES * A_COLS;
  static constexpr int NUM_BARS = 2 * STAGES + TSTAGES + 2 * NBUF;
  static constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + NUM_BARS * 8 + 64;
  static_assert(STAGES >= 3, "shared-memory ring too short");
  static_assert(DCOL + NBUF * 2 * MT <= TMEM_COLS, "tensor memory budget");
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

struct SParams {
  const uint8_t* w;      // streaming-layout weights
  void* c;
  const void* bias;
  const float* global_scale;
  float* partials;       // [CTA][2][MT][256] fp32
  int* counters;         // one per column group, zero on entry
  int M, N, K;
  int num_groups;
  int cps;        // SMODE 0: chunks per scale row
  int rpc;        // SMODE 1: scale rows per chunk
  int gs_shift;   // SMODE 1: log2(group size)
  int kc, ng;
  int num_ctas;
  int split;      // 1: ranges of units (column groups shared between CTAs); 0: whole column groups per CTA
  uint32_t tx_bytes;
};

// one copy per translation unit that instantiates the kernels (see read_status)
static __device__ int g_stream_status = 0;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ int64_t range_start(int64_t p, int64_t U, int64_t P) { return p * U / P; }
__device__ __forceinline__ int64_t unit_owner(int64_t u, int64_t U, int64_t P) { return ((u + 1) * P - 1) / U; }

template <typename T, int MT>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
  uint32_t d = 0;
  d |= 1u << 4;                        // D format f32
  d |= (kHalf<T> ? 0u : 1u) << 7;      // A format
  d |= (kHalf<T> ? 0u : 1u) << 10;     // B format
  d |= (uint32_t)(MT >> 3) << 17;      // N
  d |= (uint32_t)(128 >> 4) << 24;     // M
  return d;
}

// kind::f16 MMA, A operand in tensor memory, B descriptor given as its two 32-bit halves.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t desc_lo, uint32_t desc_hi,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 d;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 d, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_acc(uint32_t d_tmem, uint32_t a_tmem, uint32_t desc_lo, uint32_t desc_hi,
                                           uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .b64 d;\n\tmov.b64 d, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d, %4, 1;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(desc_lo), "r"(desc_hi), "r"(idesc)
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
__device__ __forceinline__ uint32_t pair16(uint32_t addr) {   // 16-bit value at addr, in both halves
  const uint32_t v = lds16(addr);
  return prmt(v, v, 0x1010u);
}

template <typename T, int FMT, int MT, int SMODE>
__global__ void __launch_bounds__(THREADS, 1)
stream_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmS,
                   const __grid_constant__ CUtensorMap tmZ, const SParams p) {
  using C = Cfg<FMT, MT, SMODE>;
  constexpr int STAGES = C::STAGES, TSTAGES = C::TSTAGES, NBUF = C::NBUF, BITS = C::BITS;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = base + STAGES * C::STAGE_BYTES;
  auto full = [&](int s) { return bar0 + 8u * s; };                           // the stage's copies have landed
  auto mma_done = [&](int s) { return bar0 + 8u * (STAGES + s); };            // the chunk's MMAs have completed
  auto a_ready = [&](int t) { return bar0 + 8u * (2 * STAGES + t); };         // operand stage written
  auto d_full = [&](int b) { return bar0 + 8u * (2 * STAGES + TSTAGES + b); };
  auto d_free = [&](int b) { return bar0 + 8u * (2 * STAGES + TSTAGES + NBUF + b); };
  const uint32_t tmem_slot = bar0 + 8u * C::NUM_BARS;
  auto drain_bar = [&](int w) { return bar0 + 8u * C::NUM_BARS + 16u + 8u * w; };   // give-up path of the MMA issuers

  __shared__ int s_abort;
  __shared__ int s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(full(s), 1); mbar_init(mma_done(s), 2); }
    for (int t = 0; t < TSTAGES; ++t) mbar_init(a_ready(t), DQ_WARPS / 2);
    for (int b = 0; b < NBUF; ++b) { mbar_init(d_full(b), 2); mbar_init(d_free(b), EPI_WARPS); }
    mbar_init(drain_bar(0), 1);
    mbar_init(drain_bar(1), 1);
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmS);
    if constexpr (format_has_zp(FMT)) prefetch_tensormap(&tmZ);
  }
  if (warp == MMA_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = lds32(tmem_slot);

  // this CTA's units [u0, u1): chunk c of column group g is unit g * kc + c
  const int64_t U = (int64_t)p.ng * p.kc;
  int64_t u0, u1;
  if (p.split) {
    u0 = range_start(blockIdx.x, U, p.num_ctas);
    u1 = range_start(blockIdx.x + 1, U, p.num_ctas);
  } else {
    u0 = range_start(blockIdx.x, p.ng, p.num_ctas) * p.kc;
    u1 = range_start(blockIdx.x + 1, p.ng, p.num_ctas) * p.kc;
  }
  const int total = (int)(u1 - u0);
  const int g_first = (int)(u0 / p.kc), c_first = (int)(u0 - (int64_t)g_first * p.kc);

  if (warp == PROD_WARP) {
    // ---------------- producer: one bulk copy of the chunk's weights, the activation tile, the scale rows --------
    if (lane == 0) {
      int g = g_first, c = c_first, s = 0, i = 0;
      uint32_t ph = 0;
      for (; i < total; ++i) {
        if (i >= STAGES && !mbar_wait_sleep(mma_done(s), ph ^ 1u, &s_abort, 100)) { atomicExch(&g_stream_status, 1); break; }
        const uint32_t st = base + s * C::STAGE_BYTES;
        mbar_arrive_expect_tx(full(s), p.tx_bytes);
        bulk_load(st, p.w + ((int64_t)g * p.kc + c) * C::RAW_BYTES, C::RAW_BYTES, full(s));
        tma_load_2d(st + C::OFF_ACT, &tmA, full(s), c * KCH, 0);
        tma_load_2d(st + C::OFF_ACT + C::ACT_HALF, &tmA, full(s), c * KCH + 64, 0);
        const int srow = SMODE ? c * p.rpc : ((p.num_groups == 1) ? 0 : c / p.cps);
        tma_load_2d(st + C::OFF_S, &tmS, full(s), g * kGroupN, srow);
        if constexpr (format_has_zp(FMT)) tma_load_2d(st + C::OFF_Z, &tmZ, full(s), g * kGroupN, srow);
        if (++c == p.kc) { c = 0; ++g; }
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
      // after a give-up nobody waits for the copies this thread issued last, and a CTA must not exit with copies on
      // their way into its shared memory
      if (s_abort != 0) drain_copies(full, STAGES, i);
    }
  } else if (warp == MMA_WARP || warp == MMA_WARP2) {
    // ---------------- MMA issuers: one 128-column tile each, on two SM partitions ----------------
    // (a traced run showed the single issuer as the limit: about 80 cycles per MMA, 16 MMAs per chunk)
    if (lane == 0) {
      const int tile = (warp == MMA_WARP) ? 0 : 1;
      constexpr uint32_t idesc = instr_desc<T, MT>();
      const uint64_t desc0 = kmajor_sw128_desc(base + C::OFF_ACT);
      const uint32_t desc_lo = (uint32_t)desc0, desc_hi = (uint32_t)(desc0 >> 32);
      int c = c_first, s = 0, t = 0, b = 0;
      uint32_t ph = 0, tph = 0, bph = 0;
      for (int i = 0; i < total; ++i) {
        const bool seg_start = (i == 0) || (c == 0);
        const bool seg_end = (i == total - 1) || (c == p.kc - 1);
        if (seg_start && !mbar_wait_sleep(d_free(b), bph ^ 1u, &s_abort, 100)) { atomicExch(&g_stream_status, 2); break; }
        // no wait for full(s): the dequant warps waited for it before they arrived at a_ready(t), and the copy of the
        // activation tile completes on the same barrier (each wait the lone issuing thread runs costs it 200 cycles)
        if (!mbar_wait_sleep(a_ready(t), tph, &s_abort, 20)) { atomicExch(&g_stream_status, 4); break; }
        tc_fence_after();
        // The issuing thread shares its scheduler with four dequant warps, so every instruction it needs
        // per MMA costs issue slots it has to wait for: operands are one add away from per-chunk bases
        // (the descriptor's address field is its low 14 bits, the rest of the 64 bits never changes).
        const uint32_t dlo = desc_lo + (uint32_t)((s * C::STAGE_BYTES) >> 4);
        const uint32_t a_base = tmem + t * A_COLS;
        const uint32_t d_base = tmem + C::DCOL + b * (2 * MT);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t lo = dlo + (uint32_t)(((ks >> 2) * C::ACT_HALF + (ks & 3) * 32) >> 4);
          if (ks == 0)
            mma_ts(d_base + tile * MT, a_base + tile * 64, lo, desc_hi, idesc, seg_start ? 0u : 1u);
          else
            mma_ts_acc(d_base + tile * MT, a_base + tile * 64 + ks * 8, lo, desc_hi, idesc);
        }
        tc_commit(mma_done(s));
        if (seg_end) {
          tc_commit(d_full(b));
          if (++b == NBUF) { b = 0; bph ^= 1u; }
        }
        if (++c == p.kc) c = 0;
        if (++s == STAGES) { s = 0; ph ^= 1u; }
        if (++t == TSTAGES) { t = 0; tph ^= 1u; }
      }
      // after a give-up nobody waits for this thread's MMAs: the tensor memory is freed only once they have completed
      if (s_abort != 0) {
        tc_commit(drain_bar(tile));
        drain_barrier(drain_bar(tile), 0);
      }
    }
  } else if (warp < EPI_WARPS) {
    // ---------------- epilogue: once per run of chunks of one column group ----------------
    const int quad = warp;
    T* Cout = reinterpret_cast<T*>(p.c);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const float gscale = (p.global_scale != nullptr) ? *p.global_scale : 1.f;
    int b = 0;
    uint32_t bph = 0;
    bool ok = true;
    bool first_segment = true;
    int64_t u = u0;
    while (u < u1) {
      const int g = (int)(u / p.kc), c0 = (int)(u - (int64_t)g * p.kc);
      const int len = (int)((u1 - u) < (int64_t)(p.kc - c0) ? (u1 - u) : (int64_t)(p.kc - c0));
      const bool whole = (c0 == 0) && (len == p.kc);
      if (ok && !mbar_wait_sleep(d_full(b), bph, &s_abort, 500)) { atomicExch(&g_stream_status, 5); ok = false; }
      if (ok) {
        tc_fence_after();
        float* P = p.partials + ((int64_t)blockIdx.x * 2 + (first_segment ? 0 : 1)) * (MT * kGroupN);
#pragma unroll
        for (int tile = 0; tile < 2; ++tile) {
          const int nl = tile * 128 + quad * 32 + lane;
          const int n = g * kGroupN + nl;
          const float bv = (whole && bias != nullptr) ? to_float<T>(bias[bias_index(n)]) : 0.f;
#pragma unroll
          for (int piece = 0; piece < MT / 16; ++piece) {
            uint32_t v[16];
            tmem_ld16(tmem + ((uint32_t)(32 * quad) << 16) + C::DCOL + b * (2 * MT) + tile * MT + piece * 16, v);
            tmem_ld_wait();
            if (whole) {
#pragma unroll
              for (int m = 0; m < 16; ++m)
                if (piece * 16 + m < p.M)
                  Cout[(int64_t)(piece * 16 + m) * p.N + n] = from_float<T>(fmaf(__uint_as_float(v[m]), gscale, bv));
            } else {
#pragma unroll
              for (int m = 0; m < 16; ++m)
                if (piece * 16 + m < p.M) P[(piece * 16 + m) * kGroupN + nl] = __uint_as_float(v[m]);
            }
          }
        }
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(d_free(b));
      if (++b == NBUF) { b = 0; bph ^= 1u; }
      if (!whole) {
        // Partial sums of this column group are complete once every CTA that owns a part of it has been
        // here; whoever comes last adds them up (always in CTA order).
        const int64_t ua = (int64_t)g * p.kc;
        const int64_t pa = unit_owner(ua, U, p.num_ctas), pb = unit_owner(ua + p.kc - 1, U, p.num_ctas);
        epi_barrier();
        if (tid == 0) {
          int last = 0;
          if (ok && s_abort == 0) {
            __threadfence();
            last = (atomicAdd(p.counters + g, 1) == (int)(pb - pa)) ? 1 : 0;
          }
          s_last = last;
        }
        epi_barrier();
        if (s_last) {
          __threadfence();
          const int first_slot = (range_start(pa, U, p.num_ctas) == ua) ? 0 : 1;
          // Thread -> four consecutive columns of a row; eight independent elements per round so that the
          // loads of a round are all in flight together (the partials come from L2 / DRAM).
          constexpr int64_t SLOT = (int64_t)MT * kGroupN;
          const float4* first = reinterpret_cast<const float4*>(p.partials + (pa * 2 + first_slot) * SLOT);
          const int total4 = p.M * (kGroupN / 4);
          for (int e0 = tid; e0 < total4; e0 += 128 * 8) {
            float4 acc[8];
#pragma unroll
            for (int uu = 0; uu < 8; ++uu) {
              const int e = e0 + 128 * uu;
              acc[uu] = (e < total4) ? __ldcg(first + e) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            for (int64_t q = pa + 1; q <= pb; ++q) {
              const float4* src = reinterpret_cast<const float4*>(p.partials + (q * 2) * SLOT);
              float4 v[8];
#pragma unroll
              for (int uu = 0; uu < 8; ++uu) {
                const int e = e0 + 128 * uu;
                v[uu] = (e < total4) ? __ldcg(src + e) : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int uu = 0; uu < 8; ++uu) {
                acc[uu].x += v[uu].x; acc[uu].y += v[uu].y; acc[uu].z += v[uu].z; acc[uu].w += v[uu].w;
              }
            }
#pragma unroll
            for (int uu = 0; uu < 8; ++uu) {
              const int e = e0 + 128 * uu;
              if (e < total4) {
                const int m = e / (kGroupN / 4), nl = (e % (kGroupN / 4)) * 4;
                const int n = g * kGroupN + nl;
                float bv[4] = {0.f, 0.f, 0.f, 0.f};
                if (bias != nullptr) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) bv[i] = to_float<T>(bias[bias_index(n + i)]);
                }
                T o[4];
                o[0] = from_float<T>(fmaf(acc[uu].x, gscale, bv[0]));
                o[1] = from_float<T>(fmaf(acc[uu].y, gscale, bv[1]));
                o[2] = from_float<T>(fmaf(acc[uu].z, gscale, bv[2]));
                o[3] = from_float<T>(fmaf(acc[uu].w, gscale, bv[3]));
                *reinterpret_cast<uint2*>(Cout + (int64_t)m * p.N + n) = *reinterpret_cast<const uint2*>(o);
              }
            }
          }
          if (tid == 0) p.counters[g] = 0;
        }
      }
      first_segment = false;
      u += len;
    }
  } else if (warp < DQ_WARP0 + DQ_WARPS) {
    // ---------------- dequant: packed words -> T pairs -> tensor memory ----------------
    // Two groups of eight warps take alternate chunks (a warp converts both 16-lane halves of its tile and lane
    // quarter), so that one group's wait for its tensor-memory stores overlaps the other group's loads and arithmetic.
    const int quad = warp & 3, idx = (warp - DQ_WARP0) >> 2;     // idx = tile * 2 + group
    const int tile = idx >> 1, grp = idx & 1;
    const int slab0 = (tile * 4 + quad) * 2;                      // the warp's slabs: slab0 (lanes 0-15 of the store), slab0 + 1
    const int g8 = lane >> 2;
    // byte offset of the thread's words inside a 64-k block, and of its scale entries inside a scale row
    uint32_t woff[2], soff_a[2], soff_b[2];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int slab = slab0 + hf;
      const int nl_a = slab * 16 + g8;                            // the thread's two columns: nl_a, nl_a + 8
      woff[hf] = (BITS == 4) ? (uint32_t)(slab * 512 + lane * 16) : (uint32_t)(slab * 1024 + lane * 16);
      if constexpr (FMT == kNVFP4) {
        soff_a[hf] = (uint32_t)nvfp4_scale_col(nl_a);
        soff_b[hf] = (uint32_t)nvfp4_scale_col(nl_a + 8);
      } else {
        soff_a[hf] = (uint32_t)nl_a * C::SELEM;
        soff_b[hf] = (uint32_t)(nl_a + 8) * C::SELEM;
      }
    }
    bool ok = true;
    int s = grp % STAGES, t = grp % TSTAGES, ms = (TSTAGES + grp) & 1;   // ms: stage of chunk i - TSTAGES, whose MMAs free operand stage t
    uint32_t ph = 0, mph = 0;
    for (int i = grp; i < total; i += 2) {
      if (ok && !mbar_wait(full(s), ph, &s_abort)) { atomicExch(&g_stream_status, 6); ok = false; }
      const uint32_t st = base + s * C::STAGE_BYTES;
      uint32_t x[2][2][BITS == 4 ? 4 : 8];
      uint32_t sa[2] = {0, 0}, sb[2] = {0, 0}, za[2] = {0, 0}, zb[2] = {0, 0};
      if (ok) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 v = lds128(st + h * (C::RAW_BYTES / 2) + woff[hf]);
            x[hf][h][0] = v.x; x[hf][h][1] = v.y; x[hf][h][2] = v.z; x[hf][h][3] = v.w;
            if constexpr (BITS == 8) {
              const uint4 v2 = lds128(st + h * (C::RAW_BYTES / 2) + woff[hf] + 512);
              x[hf][h][4] = v2.x; x[hf][h][5] = v2.y; x[hf][h][6] = v2.z; x[hf][h][7] = v2.w;
            }
          }
          if constexpr (SMODE == 0) {
            sa[hf] = pair16<T>(st + C::OFF_S + soff_a[hf]);
            sb[hf] = pair16<T>(st + C::OFF_S + soff_b[hf]);
            if constexpr (format_has_zp(FMT)) {
              za[hf] = pair16<T>(st + C::OFF_Z + soff_a[hf]) ^ 0x80008000u;   // -zero * scale
              zb[hf] = pair16<T>(st + C::OFF_Z + soff_b[hf]) ^ 0x80008000u;
            }
          }
        }
      }
      // the operand stage is free once the MMAs of the chunk that used it last have completed
      if (i >= TSTAGES) {
        if (ok && !mbar_wait(mma_done(ms), mph, &s_abort)) { atomicExch(&g_stream_status, 7); ok = false; }
        ms += 2;
        if (ms >= STAGES) { ms -= STAGES; mph ^= 1u; }
      }
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if constexpr (SMODE == 1) {
              const uint32_t row = (uint32_t)((h * 64 + j * 16) >> p.gs_shift) * (kGroupN * C::SELEM);
              if constexpr (format_scale_is_byte(FMT)) {
                sa[hf] = codes::fp4_scale_pair<T, FMT>(lds8(st + C::OFF_S + row + soff_a[hf]));
                sb[hf] = codes::fp4_scale_pair<T, FMT>(lds8(st + C::OFF_S + row + soff_b[hf]));
              } else {
                sa[hf] = pair16<T>(st + C::OFF_S + row + soff_a[hf]);
                sb[hf] = pair16<T>(st + C::OFF_S + row + soff_b[hf]);
                if constexpr (format_has_zp(FMT)) {
                  za[hf] = pair16<T>(st + C::OFF_Z + row + soff_a[hf]) ^ 0x80008000u;
                  zb[hf] = pair16<T>(st + C::OFF_Z + row + soff_b[hf]) ^ 0x80008000u;
                }
              }
            }
            // registers of the 16-lane x 8-column store: (lane g8: k 0-1, k 2-3), (lane g8 + 8: k 0-1, k 2-3)
            uint32_t va0, va1, vb0, vb1;
            if constexpr (BITS == 4) {
              const uint32_t z = x[hf][h][j];
              va0 = codes::value4<T, FMT>(z, 0); vb0 = codes::value4<T, FMT>(z, 1);
              va1 = codes::value4<T, FMT>(z, 2); vb1 = codes::value4<T, FMT>(z, 3);
            } else {
              const uint32_t y0 = x[hf][h][(j >> 1) * 4 + (j & 1) * 2], y1 = x[hf][h][(j >> 1) * 4 + (j & 1) * 2 + 1];
              va0 = codes::value8<T, FMT>(y0, 0); vb0 = codes::value8<T, FMT>(y0, 1);
              va1 = codes::value8<T, FMT>(y1, 0); vb1 = codes::value8<T, FMT>(y1, 1);
            }
            if constexpr (format_has_zp(FMT)) {
              r[4 * j + 0] = codes::pfma<T>(va0, sa[hf], za[hf]); r[4 * j + 1] = codes::pfma<T>(va1, sa[hf], za[hf]);
              r[4 * j + 2] = codes::pfma<T>(vb0, sb[hf], zb[hf]); r[4 * j + 3] = codes::pfma<T>(vb1, sb[hf], zb[hf]);
            } else {
              r[4 * j + 0] = codes::pmul<T>(va0, sa[hf]); r[4 * j + 1] = codes::pmul<T>(va1, sa[hf]);
              r[4 * j + 2] = codes::pmul<T>(vb0, sb[hf]); r[4 * j + 3] = codes::pmul<T>(vb1, sb[hf]);
            }
          }
          tmem_st_16x256b_x4(tmem + ((uint32_t)(32 * quad + 16 * hf) << 16) + t * A_COLS + tile * 64 + h * 32, r);
        }
        }
        tmem_st_wait();
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(a_ready(t));
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
inline int64_t counters_bytes(int64_t n) { return ((n / kGroupN) * 4 + 255) & ~(int64_t)255; }
inline int mt_for(int64_t m) { return m <= 16 ? 16 : (m <= 64 ? 64 : 128); }
// counters, then two partial slots of MT x 256 floats per CTA
inline int64_t scratch_bytes(int64_t m, int64_t n, int64_t k) {
  if (m <= 0 || !layout_accepts(k, n)) return 0;
  return counters_bytes(n) + (int64_t)sm_count() * 2 * mt_for(m) * kGroupN * (int64_t)sizeof(float);
}

template <typename T, int FMT, int MT, int SMODE>
int launch_one(const GemmArgs& g, const void* a, void* c, int m) {
  using C = Cfg<FMT, MT, SMODE>;
  const int64_t K = g.size_k, N = g.size_n;
  const int64_t gs = K / g.num_groups;
  SParams p{};
  p.w = reinterpret_cast<const uint8_t*>(g.bq);
  p.c = c; p.bias = g.bias; p.global_scale = g.global_scale;
  p.M = m; p.N = (int)N; p.K = (int)K;
  p.num_groups = (int)g.num_groups;
  p.kc = (int)(K / KCH);
  p.ng = (int)(N / kGroupN);
  p.cps = (g.num_groups == 1) ? p.kc : (int)(gs / KCH);
  p.rpc = SMODE ? (int)(KCH / gs) : 1;
  p.gs_shift = 0;
  while (SMODE && (1 << p.gs_shift) < gs) ++p.gs_shift;
  const int64_t U = (int64_t)p.ng * p.kc;
  const int64_t cb = counters_bytes(N);
  const int64_t part = (int64_t)sm_count() * 2 * MT * kGroupN * (int64_t)sizeof(float);
  p.split = (g.scratch != nullptr && g.scratch_bytes >= cb + part) ? 1 : 0;
  if (p.split) {
    p.num_ctas = (int)(U < sm_count() ? U : sm_count());
    p.counters = reinterpret_cast<int*>(g.scratch);
    p.partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(g.scratch) + cb);
    if (U % p.num_ctas != 0 || (U / p.num_ctas) % p.kc != 0)
      MB_CUDA(cudaMemsetAsync(p.counters, 0, (size_t)p.ng * 4, g.stream));
  } else {
    p.num_ctas = p.ng < sm_count() ? p.ng : sm_count();
  }
  p.tx_bytes = C::RAW_BYTES + 2 * C::ACT_HALF + p.rpc * kGroupN * C::SELEM * (format_has_zp(FMT) ? 2 : 1);

  CUtensorMap tmA, tmS, tmZ;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)m};
    const uint64_t strides[1] = {(uint64_t)g.a_stride * 2};
    const uint32_t box[2] = {64, MT};
    if (int rc = encode_tensor_map(&tmA, kHalf<T> ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                   2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const bool byte_scale = format_scale_is_byte(FMT);
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)g.num_groups};
    const uint64_t strides[1] = {(uint64_t)N * (byte_scale ? 1 : 2)};
    const uint32_t box[2] = {kGroupN, (uint32_t)p.rpc};
    const CUtensorMapDataType dt = byte_scale ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
    if (int rc = cached_tensor_map(&tmS, dt, 2, g.scales, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    tmZ = tmS;
    if (format_has_zp(FMT)) {
      if (int rc = cached_tensor_map(&tmZ, dt, 2, g.zeros, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    }
  }
  static bool attr_set[64] = {};
  int dev = 0;
  MB_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    MB_CUDA(cudaFuncSetAttribute(stream_gemm_kernel<T, FMT, MT, SMODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 C::SMEM));
    attr_set[dev] = true;
  }
  stream_gemm_kernel<T, FMT, MT, SMODE><<<p.num_ctas, THREADS, C::SMEM, g.stream>>>(tmA, tmS, tmZ, p);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

template <typename T, int FMT, int SMODE>
int launch_rows(const GemmArgs& g) {
  const T* A = reinterpret_cast<const T*>(g.a);
  T* Cc = reinterpret_cast<T*>(g.c);
  for (int64_t m0 = 0; m0 < g.size_m; m0 += 128) {
    const int m = (int)(g.size_m - m0 < 128 ? g.size_m - m0 : 128);
    const void* a = A + m0 * g.a_stride;
    void* c = Cc + m0 * g.size_n;
    int rc;
    if (m <= 16) rc = launch_one<T, FMT, 16, SMODE>(g, a, c, m);
    else if (m <= 64) rc = launch_one<T, FMT, 64, SMODE>(g, a, c, m);
    else rc = launch_one<T, FMT, 128, SMODE>(g, a, c, m);
    if (rc) return rc;
  }
  return 0;
}

template <typename T, int FMT>
int launch_fmt(const GemmArgs& g) {
  const int64_t gs = g.size_k / g.num_groups;
  if constexpr (FMT == kNVFP4 || FMT == kMXFP4) {
    return launch_rows<T, FMT, 1>(g);
  } else {
    if (g.num_groups == 1 || gs % KCH == 0) return launch_rows<T, FMT, 0>(g);
    if constexpr (FMT != kFP8) {
      if (gs == 16 || gs == 32 || gs == 64) return launch_rows<T, FMT, 1>(g);
    }
    set_error("weights in the streaming layout: group size %lld is not served (16, 32, 64, a multiple of 128, or "
              "per-channel)", (long long)gs);
    return MARLIN_B200_EINVAL;
  }
}

template <typename T>
int launch_dtype(const GemmArgs& g) {
  switch (g.format) {
    case kU4B8: return launch_fmt<T, kU4B8>(g);
    case kU4: return launch_fmt<T, kU4>(g);
    case kU8B128: return launch_fmt<T, kU8B128>(g);
    case kU8: return launch_fmt<T, kU8>(g);
    case kFP8: return launch_fmt<T, kFP8>(g);
    case kNVFP4: return launch_fmt<T, kNVFP4>(g);
    case kMXFP4: return launch_fmt<T, kMXFP4>(g);
  }
  set_error("unknown weight format %d", g.format);
  return MARLIN_B200_EINVAL;
}

inline int read_status(int* value, bool reset) {
  MB_CUDA(cudaMemcpyFromSymbol(value, g_stream_status, sizeof(int)));
  if (reset && *value != 0) {
    const int zero = 0;
    MB_CUDA(cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int)));
  }
  return 0;
}

}  // namespace stream
}  // namespace mb200
