// Weight-streaming GEMM for small M (decode): C[M<=16, N] = A * dequant(B), bounded by HBM bandwidth.
//
// One persistent CTA per SM.  The work is the list of (column group of 256, K chunk of 64) units in
// column-major order, cut into equal contiguous ranges, one per CTA (stream-K style), so every SM
// streams the same number of weight bytes whatever N and K are.  A producer thread feeds a ring of
// shared-memory stages with TMA: the packed weight chunk (3-D tensor map over the packed layout,
// 128-byte swizzle so that the fragment reads are bank-conflict free), the activation chunk (2-D
// map, rows beyond M read as zero) and the scale / zero-point rows of the chunk.
//
// Eight consumer warps form four pairs; pair j owns every fourth chunk of the CTA's range, the two
// warps of a pair split the 256 columns.  The packed words go from shared memory straight into
// mma.sync fragments: the weight tile is the 16-row operand (rows = output columns), the tokens are
// the 8-wide operand, so no tensor-core work is spent on padding M; a byte permute of the words of
// two k rows pairs two consecutive k of one column, which is what the fragments want.
//
// Integer and fp8 weights are NOT scaled before the MMA.  The operand is the raw code glued into
// a floating-point pattern (1024 + q, 64 + q or 128 + q: one logic instruction per pair), the
// products are accumulated per scale group in fp32, and at the end of the group
//     acc += s * tmp - (s * offset + zero_point * s) * sum_k(a)
// where sum_k(a) comes from one extra MMA against a fragment of ones.  This is exact in the codes
// (more accurate than rounding every scaled weight to 16 bits) and costs a few fp32 operations per
// output per group instead of two per weight.  The fp4 formats (groups of 16 / 32) scale before
// the MMA.
//
// A range that covers all of K for a column group writes C directly; a partial range stores fp32
// partial sums to scratch, and a second small kernel adds the partials of each split group in a
// fixed order (deterministic) and applies the epilogue (nvfp4 global scale, bias).
#include <mutex>

#include "common.cuh"
#include "tma.cuh"

namespace mb200 {
namespace {

constexpr int GROUP_N = 256;
constexpr int KCHUNK = 64;
constexpr int KT_PER_CHUNK = 4;
// Four consumer pairs plus one producer warp.  (Five pairs were measured for the 4-bit formats: no
// gain, the integer pipe that unpacks the codes is the shared limit.)
__host__ __device__ constexpr int pairs_of(int bits) { return bits == 4 ? 4 : 4; }
__host__ __device__ constexpr int threads_of(int bits) { return (2 * pairs_of(bits) + 1) * 32; }
constexpr int META_BYTES = 2048;  // scale rows of one chunk: up to 4 rows x 512 B
constexpr int A_BYTES = 2048;     // up to 16 token rows x 128 B

template <int BITS>
struct StageLayout {
  static constexpr int W_BYTES = KT_PER_CHUNK * 16 * GROUP_N * BITS / 8;  // 8 KiB / 16 KiB
  static constexpr int KT_BYTES = W_BYTES / KT_PER_CHUNK;
  static constexpr int OFF_A = W_BYTES;
  static constexpr int OFF_S = OFF_A + A_BYTES;
  static constexpr int OFF_Z = OFF_S + META_BYTES;
  static constexpr int BYTES = OFF_Z + META_BYTES;  // multiple of 1024
  // The ring depth is a multiple of PAIRS: a stage is then always consumed by the same pair.  With
  // any other depth two pairs alternate on a stage, the later one can reach its wait a whole phase
  // early, and an mbarrier parity wait cannot tell "one phase ahead" from "done" - it would read the
  // stage too soon and release it twice.
  static constexpr int PAIRS = pairs_of(BITS);
  static constexpr int STAGES = (BITS == 4 ? 3 : 2) * PAIRS;
  static_assert(STAGES % PAIRS == 0, "a stage must belong to one pair");
};

// How the scales are applied.  kPre: multiply before the MMA (fp4).  Otherwise after the MMA, once
// per `scope` k-tiles; kWhole applies them once per segment (per-channel scales).
constexpr int kPre = -1;
constexpr int kWhole = 0;

struct DecodeParams {
  void* c;
  const void* bias;
  const void* scales;  // global pointers, used by the per-channel fix-up
  const void* zeros;
  const float* global_scale;
  float* partials;
  int M, N, K;
  int num_groups;   // rows of the scale tensor
  int group_size;   // K / num_groups
  int rpc;          // scale rows per chunk (1 unless group_size < 64)
  int kc;           // chunks along K
  int ng;           // column groups
  int num_ctas;
  uint32_t tx_bytes;
};

__device__ int g_decode_status = 0;

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <typename T> constexpr bool kIsHalf = false;
template <> constexpr bool kIsHalf<__half> = true;

// D += A * B (ZERO_C: D = A * B)
template <typename T, bool ZERO_C>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kIsHalf<T>) {
    if constexpr (ZERO_C)
      asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                   : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                   : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    else
      asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                   : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                   : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    if constexpr (ZERO_C)
      asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                   : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                   : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    else
      asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                   : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                   : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <typename T>
__device__ __forceinline__ uint32_t pair_mul(uint32_t a, uint32_t b) {
  if constexpr (kIsHalf<T>) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
}

template <typename T>
__device__ __forceinline__ float lo_to_float(uint32_t w) {
  if constexpr (kIsHalf<T>) return __half2float(__ushort_as_half((unsigned short)(w & 0xffff)));
  else return __uint_as_float(w << 16);
}
template <typename T>
__device__ __forceinline__ float hi_to_float(uint32_t w) {
  if constexpr (kIsHalf<T>) return __half2float(__ushort_as_half((unsigned short)(w >> 16)));
  else return __uint_as_float(w & 0xffff0000u);
}

// ---- raw operand builders -----------------------------------------------------------------------------
// 4-bit: z holds, in each 16-bit half, four codes of one k (low half: first k of the pair, high half:
// the second); idx selects the code.  Returns the pair (k0, k1) as T x 2.
// Integer formats: value = code + raw_offset4<T>(idx) exactly.  e2m1: value = true * 2^-14 (fp16) or
// true * 2^-126 (bf16) exactly, subnormals included.
template <typename T, int FMT>
__device__ __forceinline__ uint32_t raw4(uint32_t z, int idx) {
  if constexpr (FMT == kU4B8 || FMT == kU4) {
    if constexpr (kIsHalf<T>) {
      const uint32_t sh = (idx >= 2) ? (z >> 8) : z;
      return (idx & 1) ? ((sh & 0x00f000f0u) | 0x54005400u)   // 64 + q
                       : ((sh & 0x000f000fu) | 0x64006400u);  // 1024 + q
    } else {
      return ((z >> (4 * idx)) & 0x000f000fu) | 0x43004300u;  // 128 + q
    }
  } else {
    const uint32_t t = z << (12 - 4 * idx);
    constexpr int sh = kIsHalf<T> ? 3 : 6;
    return ((t & 0x70007000u) >> sh) | (t & 0x80008000u);
  }
}
template <typename T>
__device__ __forceinline__ constexpr float raw_offset4(int idx) {
  return kIsHalf<T> ? ((idx & 1) ? 64.f : 1024.f) : 128.f;
}

// 8-bit: y holds bytes [k0 code a, k1 code a, k0 code b, k1 code b]; which picks a or b.
// u8 fp16: value = code + 1024.  u8 bf16: value = code - zero exactly (fp32 detour).  fp8: the e4m3
// bits moved into the 16-bit pattern, value = true * 2^-8 (fp16) / 2^-120 (bf16).
template <typename T, int FMT>
__device__ __forceinline__ uint32_t raw8(uint32_t y, int which) {
  if constexpr (FMT == kU8B128 || FMT == kU8) {
    if constexpr (kIsHalf<T>) {
      return prmt(y, 0x64646464u, which ? 0x4342u : 0x4140u);
    } else {
      constexpr float zero = (FMT == kU8B128) ? 128.f : 0.f;
      const uint32_t f0 = prmt(y, 0x4B000000u, which ? 0x7442u : 0x7440u);
      const uint32_t f1 = prmt(y, 0x4B000000u, which ? 0x7443u : 0x7441u);
      __nv_bfloat162 r = __floats2bfloat162_rn(__uint_as_float(f0) - (8388608.f + zero),
                                               __uint_as_float(f1) - (8388608.f + zero));
      return *reinterpret_cast<uint32_t*>(&r);
    }
  } else {
    const uint32_t r = prmt(y, 0u, which ? 0x3424u : 0x1404u);
    constexpr int sh = kIsHalf<T> ? 1 : 4;
    return ((r & 0x7f007f00u) >> sh) | (r & 0x80008000u);
  }
}

// value = code + raw_offset - zero  =>  what has to be subtracted (times sum of activations)
template <typename T, int FMT>
__device__ __forceinline__ constexpr float code_offset(int idx) {
  if (FMT == kU4B8) return raw_offset4<T>(idx) + 8.f;
  if (FMT == kU4) return raw_offset4<T>(idx);
  if (FMT == kU8B128) return kIsHalf<T> ? 1024.f + 128.f : 0.f;
  if (FMT == kU8) return kIsHalf<T> ? 1024.f : 0.f;
  return 0.f;
}
template <typename T, int FMT>
__host__ __device__ constexpr bool needs_act_sum() {
  return FMT == kU4B8 || FMT == kU4 || FMT == kU8 || (FMT == kU8B128 && kIsHalf<T>);
}

// slot -> first of its two columns inside the 256-column group
template <int BITS>
__device__ __forceinline__ int slot_col(int q, int p_lane, int gid) {
  if constexpr (BITS == 4) {
    const int s = q >> 2, m = q & 3;
    return (2 * p_lane + s) * 64 + gid * 8 + 2 * m;
  } else {
    const int h = q >> 2, s = (q >> 1) & 1, m = q & 1;
    return (2 * p_lane + s) * 64 + (gid + 8 * h) * 4 + 2 * m;
  }
}

// ---- scales for the multiply-before path (fp4) ---------------------------------------------------------
template <typename T, int FMT>
__device__ __forceinline__ void load_pre_scales(uint32_t srow, int nb, uint32_t (&s)[2]) {
  if constexpr (FMT == kNVFP4) {
    // bytes are interleaved [0,2,1,3] per 4 columns; value = fp16 with bits (byte << 7)
    const uint32_t w = lds32(srow + (nb & ~3));
    const uint32_t b0 = (nb & 2) ? ((w >> 8) & 0xff) : (w & 0xff);
    const uint32_t b1 = (nb & 2) ? (w >> 24) : ((w >> 16) & 0xff);
    if constexpr (kIsHalf<T>) {
      s[0] = b0 * 0x00800080u;
      s[1] = b1 * 0x00800080u;
    } else {
      // same value as bf16: exponent re-biased by 112 (valid for every normal scale; a zero scale
      // only ever multiplies zero codes)
      s[0] = b0 ? (b0 * 0x00100010u + 0x38003800u) : 0u;
      s[1] = b1 ? (b1 * 0x00100010u + 0x38003800u) : 0u;
    }
  } else {  // mxfp4: 2^(e-127) times the 2^14 / 2^126 that the e2m1 pattern leaves out
    const uint32_t w = lds16(srow + nb);
    const int e0 = (int)(w & 0xff), e1 = (int)(w >> 8);
    if constexpr (kIsHalf<T>) {
      const int f0 = min(max(e0 - 98, 0), 30), f1 = min(max(e1 - 98, 0), 30);
      s[0] = (uint32_t)f0 * 0x04000400u;
      s[1] = (uint32_t)f1 * 0x04000400u;
    } else {
      const int f0 = min(e0 + 126, 254), f1 = min(e1 + 126, 254);
      s[0] = (uint32_t)f0 * 0x00800080u;
      s[1] = (uint32_t)f1 * 0x00800080u;
    }
  }
}

// ---- scale-after-MMA fix-up -------------------------------------------------------------------------------
// dst (+)= s * src - (s * offset + zero) * actsum, for the 8 slots of a thread.  load_s / load_z
// return the 32-bit word holding the scale / zero pair of the slot's two columns.
template <typename T, int FMT, int MB, bool ACCUMULATE, typename LoadS, typename LoadZ>
__device__ __forceinline__ void fixup(float (&dst)[8][MB][4], const float (&src)[8][MB][4],
                                      const float (&asum)[MB][4], LoadS load_s, LoadZ load_z,
                                      int p_lane, int gid) {
  constexpr int BITS = format_bits(FMT);
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int nb = slot_col<BITS>(q, p_lane, gid);
    const uint32_t sw = load_s(nb);
    const float s0 = lo_to_float<T>(sw), s1 = hi_to_float<T>(sw);
    const float off = code_offset<T, FMT>(BITS == 4 ? (q & 3) : 0);
    float c0 = s0 * off, c1 = s1 * off;
    if constexpr (format_has_zp(FMT)) {
      const uint32_t zw = load_z(nb);
      c0 += lo_to_float<T>(zw);
      c1 += hi_to_float<T>(zw);
    }
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      const float sv[4] = {s0, s0, s1, s1};
      const float cv[4] = {c0, c0, c1, c1};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = ACCUMULATE ? fmaf(sv[i], src[q][mb][i], dst[q][mb][i]) : sv[i] * src[q][mb][i];
        if constexpr (needs_act_sum<T, FMT>()) v = fmaf(-cv[i], asum[mb][i & 1], v);
        dst[q][mb][i] = v;
      }
    }
  }
}

__device__ __forceinline__ int64_t range_start(int64_t p, int64_t U, int64_t P) { return p * U / P; }

// Programmatic dependent launch: the reduce kernel is allowed to become resident while the main kernel
// still runs (its launch latency disappears); it waits here before it reads the partial sums.
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (kIsHalf<T>) {
    __half2 r = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
  }
}

template <typename T, int FMT, int MB, int SCOPE>
__global__ void __launch_bounds__(threads_of(format_bits(FMT)), 1)
decode_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
              const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ,
              const DecodeParams p) {
  constexpr int BITS = format_bits(FMT);
  using L = StageLayout<BITS>;
  constexpr int STAGES = L::STAGES;
  constexpr int PAIRS = L::PAIRS;
  constexpr int CONSUMER_WARPS = 2 * PAIRS;
  constexpr int ACC = 8 * MB * 4;  // floats per thread
  constexpr int RED_BYTES = (PAIRS - 1) * 2 * 32 * ACC * 4;
  constexpr bool POST = SCOPE != kPre;
  constexpr bool STAGE_SCALES = SCOPE != kWhole;  // scale rows travel with the chunk
  constexpr uint32_t ONES = kIsHalf<T> ? 0x3C003C00u : 0x3F803F80u;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t red_base = base + STAGES * L::BYTES;
  const uint32_t bar_base = red_base + RED_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };

  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 2);  // the two warps of the owning pair
    }
    fence_barrier_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmA);
    if (STAGE_SCALES) prefetch_tensormap(&tmS);
  }
  __syncthreads();

  const int64_t U = (int64_t)p.ng * p.kc;
  const int64_t u0 = range_start(blockIdx.x, U, p.num_ctas);
  const int64_t u1 = range_start(blockIdx.x + 1, U, p.num_ctas);
  pdl_release_dependents();

  if (warp == CONSUMER_WARPS) {
    // ---------------- producers ----------------
    // Lane j feeds pair j: it owns the stages j, j + PAIRS, ... and every PAIRS-th chunk.  The lanes
    // run the same loop side by side, which multiplies the rate at which chunks can be issued.
    if (lane < PAIRS) {
      constexpr int ROWS_PER_KT = (BITS == 4) ? 16 : 32;  // 128-byte rows of one k-tile per group
      const int total = (int)(u1 - u0);
      int g = (int)(u0 / p.kc);
      int c = (int)(u0 - (int64_t)g * p.kc) + lane;
      while (c >= p.kc) { c -= p.kc; ++g; }
      int s = lane, issued = 0;
      uint32_t phase = 0;
      bool first_lap = true;
      for (int it = lane; it < total; it += PAIRS, ++issued) {
        if (!first_lap) {
          if (!mbar_wait(empty_bar(s), phase ^ 1u, &s_abort)) {
            atomicExch(&g_decode_status, 1);
            break;
          }
        }
        const uint32_t st = base + s * L::BYTES;
        mbar_arrive_expect_tx(full_bar(s), p.tx_bytes);
        tma_load_3d(st, &tmW, full_bar(s), 0, g * ROWS_PER_KT, c * KT_PER_CHUNK);
        tma_load_2d(st + L::OFF_A, &tmA, full_bar(s), c * KCHUNK, 0);
        if constexpr (STAGE_SCALES) {
          const int srow = (p.num_groups == 1) ? 0 : (c * KCHUNK) / p.group_size;
          tma_load_2d(st + L::OFF_S, &tmS, full_bar(s), g * GROUP_N, srow);
          if constexpr (format_has_zp(FMT)) tma_load_2d(st + L::OFF_Z, &tmZ, full_bar(s), g * GROUP_N, srow);
        }
        c += PAIRS;
        while (c >= p.kc) { c -= p.kc; ++g; }
        s += PAIRS;
        if (s >= STAGES) { s -= STAGES; phase ^= 1u; first_lap = false; }
      }
      // no copy of this lane's is in flight when it leaves (a CTA must not exit with copies on their way into its
      // shared memory; after a give-up nobody else waits for them): its stages are lane, lane + PAIRS, ...
      if (s_abort != 0) drain_copies([&](int idx) { return full_bar(lane + PAIRS * idx); }, STAGES / PAIRS, issued);
    }
    return;
  }

  // ---------------- consumers ----------------
  const int gid = lane >> 2, t = lane & 3;
  const int pair = warp >> 1, parity = warp & 1;
  const int p_lane = ((gid >> 1) & 1) ^ parity;
  constexpr int SROW_BYTES = format_scale_is_byte(FMT) ? GROUP_N : GROUP_N * 2;
  const uint8_t* const smem = smem_raw + (base - smem_u32(smem_raw));  // generic pointer to `base`

  // per-thread byte offsets inside a stage (the 128-byte swizzle folded in)
  int woff[BITS == 4 ? 4 : 8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lk = 2 * t + (i & 1) + ((i >> 1) << 3);
    if constexpr (BITS == 4) {
      woff[i] = lk * 128 + ((gid ^ (lk & 7)) << 4) + p_lane * 8;
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int R = lk * 2 + h;
        woff[h * 4 + i] = R * 128 + ((gid ^ (R & 7)) << 4) + p_lane * 8;
      }
    }
  }
  int aoff[MB];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb) aoff[mb] = L::OFF_A + (mb * 8 + gid) * 128 + t * 4;

  // k-tiles that share a row of block scales, minus one (group 16: 0, group 32: 1, >= 64: the whole chunk)
  const int pre_mask = min(max(p.group_size / 16, 1), KT_PER_CHUNK) - 1;
  float acc[8][MB][4];
  float tmp[(POST && SCOPE > 0) ? 8 : 1][MB][4];
  float asum[MB][4];
  bool alive = true;

  // walk the CTA's range segment by segment (a segment = consecutive chunks of one column group)
  int g = (int)(u0 / p.kc);
  int c0 = (int)(u0 - (int64_t)g * p.kc);
  const int total = (int)(u1 - u0);
  int it0 = 0;                       // index (inside the range) of the segment's first chunk
  int own = pair;                    // next chunk index this pair owns
  int stage = pair % STAGES;         // its stage and barrier phase
  uint32_t phase = 0;
  bool first_segment = true;

  while (it0 < total) {
    const int seg_len = min(p.kc - c0, total - it0);
#pragma unroll
    for (int q = 0; q < 8; ++q)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[q][mb][i] = 0.f;
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < 4; ++i) asum[mb][i] = 0.f;

    for (; own < it0 + seg_len; own += PAIRS) {
      // After a wait gave up the warp keeps walking its chunks (so that the CTA-wide barriers below
      // still meet) but no longer waits for, reads or writes any data.
      if (alive && !mbar_wait(full_bar(stage), phase, &s_abort)) {
        atomicExch(&g_decode_status, 2);
        alive = false;
      }
      const uint32_t st = base + stage * L::BYTES;
      const uint8_t* stp = smem + stage * L::BYTES;
      if (alive) {
        constexpr int NW = (BITS == 4) ? 4 : 8;
        uint32_t sc[POST ? 1 : 8][2];  // decoded block scales of the thread's eight column pairs (fp4 formats)
#pragma unroll
        for (int kt = 0; kt < KT_PER_CHUNK; ++kt) {
          uint2 xk[NW];
#pragma unroll
          for (int i = 0; i < NW; ++i) xk[i] = *reinterpret_cast<const uint2*>(stp + kt * L::KT_BYTES + woff[i]);
          uint32_t bfrag[MB][2];
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) {
            const int sw = (mb * 8 + gid) & 7;
            bfrag[mb][0] = *reinterpret_cast<const uint32_t*>(stp + aoff[mb] + (((kt * 2) ^ sw) << 4));
            bfrag[mb][1] = *reinterpret_cast<const uint32_t*>(stp + aoff[mb] + (((kt * 2 + 1) ^ sw) << 4));
          }
          // scope bookkeeping (compile time after unrolling)
          constexpr int SC = (POST && SCOPE > 0) ? SCOPE : KT_PER_CHUNK;
          const bool scope_first = (kt % SC) == 0;
          const bool scope_last = (kt % SC) == SC - 1;

          // ---- scales for the multiply-before path: decoded once per scale group ----
          if constexpr (!POST) {
            if (FMT == kNVFP4 || (kt & pre_mask) == 0) {  // nvfp4: a row of scales per k-tile
              const int srow_local = (p.rpc == 1) ? 0 : (kt * 16) / p.group_size;
              const uint32_t srow = st + L::OFF_S + srow_local * SROW_BYTES;
#pragma unroll
              for (int q = 0; q < 8; ++q) load_pre_scales<T, FMT>(srow, slot_col<BITS>(q, p_lane, gid), sc[q]);
            }
          }

          // ---- weights ----
          auto issue = [&](int q, const uint32_t (&a)[4]) {
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              if constexpr (POST && SCOPE > 0) {
                if (scope_first) mma16816<T, true>(tmp[q][mb], a, bfrag[mb][0], bfrag[mb][1]);
                else mma16816<T, false>(tmp[q][mb], a, bfrag[mb][0], bfrag[mb][1]);
              } else {
                mma16816<T, false>(acc[q][mb], a, bfrag[mb][0], bfrag[mb][1]);
              }
            }
          };
          if constexpr (BITS == 4) {
            const uint2 (&x)[NW] = xk;
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2) {
              const uint32_t x0 = s2 ? x[0].y : x[0].x, x1 = s2 ? x[1].y : x[1].x;
              const uint32_t x2 = s2 ? x[2].y : x[2].x, x3 = s2 ? x[3].y : x[3].x;
              const uint32_t zAl = prmt(x0, x1, 0x5410u), zAh = prmt(x0, x1, 0x7632u);
              const uint32_t zBl = prmt(x2, x3, 0x5410u), zBh = prmt(x2, x3, 0x7632u);
#pragma unroll
              for (int m = 0; m < 4; ++m) {
                const int q = s2 * 4 + m;
                uint32_t a[4] = {raw4<T, FMT>(zAl, m), raw4<T, FMT>(zAh, m), raw4<T, FMT>(zBl, m),
                                 raw4<T, FMT>(zBh, m)};
                if constexpr (!POST) {
                  a[0] = pair_mul<T>(a[0], sc[q][0]); a[1] = pair_mul<T>(a[1], sc[q][1]);
                  a[2] = pair_mul<T>(a[2], sc[q][0]); a[3] = pair_mul<T>(a[3], sc[q][1]);
                }
                issue(q, a);
              }
            }
          } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint2* x = &xk[h * 4];
#pragma unroll
              for (int s2 = 0; s2 < 2; ++s2) {
                const uint32_t x0 = s2 ? x[0].y : x[0].x, x1 = s2 ? x[1].y : x[1].x;
                const uint32_t x2 = s2 ? x[2].y : x[2].x, x3 = s2 ? x[3].y : x[3].x;
                // word bytes hold columns 0,2,1,3: bytes (0,2) are columns (0,1), bytes (1,3) columns (2,3)
                const uint32_t yA01 = prmt(x0, x1, 0x6240u), yA23 = prmt(x0, x1, 0x7351u);
                const uint32_t yB01 = prmt(x2, x3, 0x6240u), yB23 = prmt(x2, x3, 0x7351u);
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                  const int q = (h * 2 + s2) * 2 + m;
                  const uint32_t yA = m ? yA23 : yA01, yB = m ? yB23 : yB01;
                  const uint32_t a[4] = {raw8<T, FMT>(yA, 0), raw8<T, FMT>(yA, 1), raw8<T, FMT>(yB, 0),
                                         raw8<T, FMT>(yB, 1)};
                  issue(q, a);
                }
              }
            }
          }

          if constexpr (POST) {
            // sum of the activations of this k-tile per token: one MMA against ones
            if constexpr (needs_act_sum<T, FMT>()) {
              const uint32_t ones[4] = {ONES, ONES, ONES, ONES};
#pragma unroll
              for (int mb = 0; mb < MB; ++mb) {
                if (SCOPE > 0 && scope_first) mma16816<T, true>(asum[mb], ones, bfrag[mb][0], bfrag[mb][1]);
                else mma16816<T, false>(asum[mb], ones, bfrag[mb][0], bfrag[mb][1]);
              }
            }
            if constexpr (SCOPE > 0) {
              if (scope_last) {
                const int srow_local = (p.rpc == 1) ? 0 : (kt * 16) / p.group_size;
                const uint8_t* srow = stp + L::OFF_S + srow_local * SROW_BYTES;
                const uint8_t* zrow = stp + L::OFF_Z + srow_local * SROW_BYTES;
                auto ls = [&](int nb) { return *reinterpret_cast<const uint32_t*>(srow + nb * 2); };
                auto lz = [&](int nb) { return *reinterpret_cast<const uint32_t*>(zrow + nb * 2); };
                fixup<T, FMT, MB, true>(acc, tmp, asum, ls, lz, p_lane, gid);
              }
            }
          }
        }
      }  // alive
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(stage));
      stage += PAIRS;
      if (stage >= STAGES) { stage -= STAGES; phase ^= 1u; }
    }

    // ---- end of the segment: add the partials of the four pairs, write out ----
    {
      if constexpr (SCOPE == kWhole) {
        // per-channel scales: one fix-up for the whole segment, scales straight from global memory
        const uint32_t* sg = reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(p.scales) + (int64_t)g * GROUP_N);
        const uint32_t* zg = reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(p.zeros) + (int64_t)g * GROUP_N);
        auto ls = [&](int nb) { return sg[nb >> 1]; };
        auto lz = [&](int nb) { return zg[nb >> 1]; };
        fixup<T, FMT, MB, false>(acc, acc, asum, ls, lz, p_lane, gid);
      }
      if (pair > 0) {
        const uint32_t rb = red_base + ((((pair - 1) * 2 + parity) * ACC) * 32 + lane) * 4;
#pragma unroll
        for (int q = 0; q < 8; ++q)
#pragma unroll
          for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int i = 0; i < 4; ++i)
              asm volatile("st.shared.f32 [%0], %1;" ::"r"(rb + ((q * MB + mb) * 4 + i) * 128), "f"(acc[q][mb][i]) : "memory");
      }
      named_barrier_sync(1, CONSUMER_WARPS * 32);
      if (pair == 0 && alive && s_abort == 0) {
#pragma unroll
        for (int kk = 0; kk < PAIRS - 1; ++kk) {
          const uint32_t rb = red_base + (((kk * 2 + parity) * ACC) * 32 + lane) * 4;
#pragma unroll
          for (int q = 0; q < 8; ++q)
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                float v;
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(rb + ((q * MB + mb) * 4 + i) * 128));
                acc[q][mb][i] += v;
              }
        }
        const bool full = (c0 == 0) && (seg_len == p.kc);
        if (full) {
          float alpha = 1.f;
          if constexpr (FMT == kNVFP4) alpha = p.global_scale[0];
          T* C = reinterpret_cast<T*>(p.c);
          const T* bias = reinterpret_cast<const T*>(p.bias);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int n = g * GROUP_N + slot_col<BITS>(q, p_lane, gid);
            float b0 = 0.f, b1 = 0.f;
            if (bias != nullptr) {
              b0 = to_float<T>(bias[bias_index(n)]);
              b1 = to_float<T>(bias[bias_index(n + 1)]);
            }
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              const int tk = mb * 8 + 2 * t;
              if (tk < p.M)
                *reinterpret_cast<uint32_t*>(C + (int64_t)tk * p.N + n) =
                    pack2<T>(acc[q][mb][0] * alpha + b0, acc[q][mb][2] * alpha + b1);
              if (tk + 1 < p.M)
                *reinterpret_cast<uint32_t*>(C + (int64_t)(tk + 1) * p.N + n) =
                    pack2<T>(acc[q][mb][1] * alpha + b0, acc[q][mb][3] * alpha + b1);
            }
          }
        } else {
          const int slot = first_segment ? 0 : 1;
          float* P = p.partials + ((int64_t)blockIdx.x * 2 + slot) * (MB * 8 * GROUP_N);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int n = slot_col<BITS>(q, p_lane, gid);
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              const int tk = mb * 8 + 2 * t;
              *reinterpret_cast<float2*>(P + tk * GROUP_N + n) = make_float2(acc[q][mb][0], acc[q][mb][2]);
              *reinterpret_cast<float2*>(P + (tk + 1) * GROUP_N + n) = make_float2(acc[q][mb][1], acc[q][mb][3]);
            }
          }
        }
      }
      named_barrier_sync(1, CONSUMER_WARPS * 32);
    }
    it0 += seg_len;
    c0 = 0;
    ++g;
    first_segment = false;
  }
}

// Adds the fp32 partials of every column group that was split across CTAs, in CTA order (a fixed
// order, so results repeat bit for bit).  One thread per output element; grid = (groups, token rows).
template <typename T, int FMT, int MB>
__global__ void __launch_bounds__(GROUP_N) decode_reduce_kernel(const DecodeParams p) {
  const int g = blockIdx.x, tk = blockIdx.y;
  const int64_t U = (int64_t)p.ng * p.kc, P = p.num_ctas;
  const int64_t ua = (int64_t)g * p.kc, ub = ua + p.kc - 1;
  const int64_t pa = ((ua + 1) * P - 1) / U, pb = ((ub + 1) * P - 1) / U;
  pdl_wait_prior_grid();   // before any return: the grid never retires ahead of the kernel in front
  if (pa == pb) return;    // written directly by its only owner
  const int col = threadIdx.x;
  const int n = g * GROUP_N + col;
  constexpr int SLOT = MB * 8 * GROUP_N;
  // the first owner uses its second slot unless its range starts exactly at this group; every later
  // owner starts inside the group and uses its first slot
  const int first_slot = (range_start(pa, U, P) == ua) ? 0 : 1;
  const float* base = p.partials + tk * GROUP_N + col;
  float v = base[(pa * 2 + first_slot) * SLOT];
  int64_t q = pa + 1;
  for (; q + 3 <= pb; q += 4) {
    const float v0 = base[(q * 2) * SLOT], v1 = base[((q + 1) * 2) * SLOT];
    const float v2 = base[((q + 2) * 2) * SLOT], v3 = base[((q + 3) * 2) * SLOT];
    v = (((v + v0) + v1) + v2) + v3;
  }
  for (; q <= pb; ++q) v += base[(q * 2) * SLOT];
  float alpha = 1.f;
  if constexpr (FMT == kNVFP4) alpha = p.global_scale[0];
  float b = 0.f;
  if (p.bias != nullptr) b = to_float<T>(reinterpret_cast<const T*>(p.bias)[bias_index(n)]);
  reinterpret_cast<T*>(p.c)[(int64_t)tk * p.N + n] = from_float<T>(v * alpha + b);
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------
template <typename T, int FMT, int MB, int SCOPE>
int launch_one(const GemmArgs& g, const void* a, void* c, int m) {
  constexpr int BITS = format_bits(FMT);
  using L = StageLayout<BITS>;
  constexpr int ACC = 8 * MB * 4;
  constexpr int PAIRS = L::PAIRS;
  constexpr int THREADS = threads_of(BITS);
  constexpr int SMEM = 1024 + L::STAGES * L::BYTES + (PAIRS - 1) * 2 * 32 * ACC * 4 + 2 * L::STAGES * 8;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");

  const int64_t K = g.size_k, N = g.size_n;
  const int64_t gs = K / g.num_groups;
  DecodeParams p{};
  p.c = c; p.bias = g.bias; p.scales = g.scales; p.zeros = g.zeros; p.global_scale = g.global_scale;
  p.partials = reinterpret_cast<float*>(g.scratch);
  p.M = m; p.N = (int)N; p.K = (int)K;
  p.num_groups = (int)g.num_groups; p.group_size = (int)gs;
  p.rpc = (g.num_groups > 1 && gs < KCHUNK) ? (int)(KCHUNK / gs) : 1;
  p.kc = (int)((K + KCHUNK - 1) / KCHUNK);
  p.ng = (int)(N / GROUP_N);
  const int64_t U = (int64_t)p.ng * p.kc;
  p.num_ctas = (int)(U < sm_count() ? U : sm_count());
  const int srow_bytes = format_scale_is_byte(FMT) ? GROUP_N : GROUP_N * 2;
  p.tx_bytes = L::W_BYTES + MB * 8 * 128;
  if (SCOPE != kWhole) p.tx_bytes += p.rpc * srow_bytes * (format_has_zp(FMT) ? 2 : 1);

  CUtensorMap tmW, tmA, tmS, tmZ;
  {
    const int rows_per_kt = (BITS == 4 ? 16 : 32) * p.ng;
    const uint64_t dims[3] = {32, (uint64_t)rows_per_kt, (uint64_t)(K / 16)};
    const uint64_t strides[2] = {128, (uint64_t)rows_per_kt * 128};
    const uint32_t box[3] = {32, (uint32_t)(BITS == 4 ? 16 : 32), KT_PER_CHUNK};
    if (int rc = cached_tensor_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, g.bq, dims, strides,
                            box, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)m};
    const uint64_t strides[1] = {(uint64_t)g.a_stride * 2};
    const uint32_t box[2] = {KCHUNK, MB * 8};
    if (int rc = encode_tensor_map(&tmA, kIsHalf<T> ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                   2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const bool byte_scale = format_scale_is_byte(FMT);
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)g.num_groups};
    const uint64_t strides[1] = {(uint64_t)N * (byte_scale ? 1 : 2)};
    const uint32_t box[2] = {GROUP_N, (uint32_t)p.rpc};
    const CUtensorMapDataType dt = byte_scale ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
    if (int rc = cached_tensor_map(&tmS, dt, 2, g.scales, dims,
                            strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
    tmZ = tmS;
    if (format_has_zp(FMT)) {
      if (int rc = cached_tensor_map(&tmZ, dt, 2, g.zeros, dims,
                              strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
        return rc;
    }
  }

  static bool attr_set[64] = {};
  int dev = 0;
  MB_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    MB_CUDA(cudaFuncSetAttribute(decode_kernel<T, FMT, MB, SCOPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    attr_set[dev] = true;
  }
  decode_kernel<T, FMT, MB, SCOPE><<<p.num_ctas, THREADS, SMEM, g.stream>>>(tmW, tmA, tmS, tmZ, p);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  // the reduce kernel is launched only when some column group really has more than one owner
  bool any_split = false;
  for (int64_t gi = 0; gi < p.ng && !any_split; ++gi) {
    const int64_t ua = gi * p.kc, ub = ua + p.kc - 1;
    any_split = ((ua + 1) * p.num_ctas - 1) / U != ((ub + 1) * p.num_ctas - 1) / U;
  }
  if (any_split) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.ng, m);
    cfg.blockDim = dim3(GROUP_N);
    cfg.stream = g.stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MB_CUDA(cudaLaunchKernelEx(&cfg, decode_reduce_kernel<T, FMT, MB>, p));
    count_launches(1);
  }
  return 0;
}

template <typename T, int FMT, int SCOPE>
int launch_scope(const GemmArgs& g) {
  const T* A = reinterpret_cast<const T*>(g.a);
  T* C = reinterpret_cast<T*>(g.c);
  for (int64_t m0 = 0; m0 < g.size_m; m0 += 16) {
    const int m = (int)(g.size_m - m0 < 16 ? g.size_m - m0 : 16);
    int rc;
    if (m <= 8) rc = launch_one<T, FMT, 1, SCOPE>(g, A + m0 * g.a_stride, C + m0 * g.size_n, m);
    else rc = launch_one<T, FMT, 2, SCOPE>(g, A + m0 * g.a_stride, C + m0 * g.size_n, m);
    if (rc) return rc;
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
  if constexpr (FMT == kNVFP4 || FMT == kMXFP4) {
    return launch_scope<T, FMT, kPre>(g);
  } else {
    if (g.num_groups == 1) return launch_scope<T, FMT, kWhole>(g);
    const int64_t gs = g.size_k / g.num_groups;
    if (gs >= KCHUNK) return launch_scope<T, FMT, 4>(g);
    if constexpr (FMT != kFP8) {
      if (gs == 32) return launch_scope<T, FMT, 2>(g);
      if (gs == 16) return launch_scope<T, FMT, 1>(g);
    }
    return 1;
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
  return 1;
}

bool decode_accepts(int64_t m, int64_t n, int64_t k, int64_t num_groups) {
  if (m <= 0 || n % GROUP_N != 0 || k % 32 != 0) return false;
  if (num_groups > 1) {
    const int64_t gs = k / num_groups;
    if (!(gs == 16 || gs == 32 || gs % KCHUNK == 0)) return false;
  }
  return true;
}

}  // namespace

int64_t gemm_decode_scratch_bytes(int64_t m, int64_t n, int64_t k, int format) {
  (void)format;
  if (m <= 0 || n % GROUP_N != 0) return 0;
  // two partial slots of 16 x 256 floats per persistent CTA, then (tensor-memory decode kernel) the
  // three 8-bit digit planes of 16 token rows and their 16 row factors
  return (int64_t)sm_count() * 2 * 16 * GROUP_N * (int64_t)sizeof(float) + 48 * k + 256;
}

int launch_gemm_decode(const GemmArgs& g) {
  if (g.sorted_ids != nullptr) return 1;
  if (!decode_accepts(g.size_m, g.size_n, g.size_k, g.num_groups)) return 1;
  if (g.act_dtype == MARLIN_B200_F16) return launch_dtype<__half>(g);
  return launch_dtype<__nv_bfloat16>(g);
}

// Reads (and optionally clears) the word a kernel of this file sets when one of its bounded waits gave up.
int read_decode_status(int* value, bool reset) {
  MB_CUDA(cudaMemcpyFromSymbol(value, g_decode_status, sizeof(int)));
  if (reset && *value != 0) {
    const int zero = 0;
    MB_CUDA(cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int)));
  }
  return 0;
}


}  // namespace mb200

// ---------------------------------------------------------------------------------------------------
// Dense GEMM with built-in scratch
// ---------------------------------------------------------------------------------------------------
namespace {
// 6 MiB.  What the M <= 16 kernels need is SMs * 32 KiB of split-K partial sums (two slots of 16 x 256
// floats per persistent CTA) plus 48 * size_k + 256 bytes for the digit planes of the integer-MMA kernel:
// on a 148-SM device that fits for size_k up to 30 016.  For M > 16 the tensor-memory kernel plans its
// k cut inside whatever room it is given, so 6 MiB only limits how finely K is cut.
constexpr int64_t kStaticScratchBytes = 6ll << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
std::mutex g_static_mutex;
void* g_static_ptr[64] = {};
}  // namespace

// marlin_b200_gemm for callers that must not allocate device memory around the call (a host runtime
// with a fixed memory plan, a plugin that gets no allocator, code running between the capture calls
// of someone else's stream): the split-K partial sums live in a 6 MiB array that is part of the
// loaded library image on every GPU.  The first call on a device looks the array's device address
// up (the name of the array is only a host-side handle, not an address a kernel could use); make
// that first call before any stream capture starts on that device.
extern "C" int marlin_b200_gemm_static_scratch(const void* a, void* c, const int32_t* b_q_weight,
                                               const void* b_scales, const void* b_zeros, const void* b_bias,
                                               const float* global_scale, int act_dtype, int format,
                                               int64_t size_m, int64_t size_n, int64_t size_k, int64_t a_stride,
                                               int64_t num_groups, void* stream) {
  using namespace mb200;
  int dev = 0;
  MB_CUDA(cudaGetDevice(&dev));
  MB_CHECK(dev >= 0 && dev < 64, "device ordinal %d is out of range for the built-in scratch table", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_ptr[dev] == nullptr) {
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || p == nullptr) {
        set_error("cudaGetSymbolAddress failed for the built-in scratch: %s", cudaGetErrorString(e));
        return MARLIN_B200_ECUDA;
      }
      g_static_ptr[dev] = p;
    }
    scratch = g_static_ptr[dev];
  }
  // The same routing as marlin_b200_gemm with a 6 MiB buffer: the M > 16 kernel fits its k cut into the
  // room, the M <= 16 kernels have a fixed need and refuse when it is larger.
  const int rc = marlin_b200_gemm(a, c, b_q_weight, b_scales, b_zeros, b_bias, global_scale, act_dtype, format,
                                  size_m, size_n, size_k, a_stride, num_groups, scratch, kStaticScratchBytes, stream);
  if (rc == MARLIN_B200_ESCRATCH) {
    set_error("the built-in scratch holds %lld bytes; this problem needs %lld (SMs * 32768 + 48 * size_k + 256 "
              "with %d SMs, size_k = %lld): use marlin_b200_gemm with a caller-provided buffer",
              (long long)kStaticScratchBytes, (long long)gemm_decode_scratch_bytes(size_m, size_n, size_k, format),
              sm_count(), (long long)size_k);
  }
  return rc;
}
