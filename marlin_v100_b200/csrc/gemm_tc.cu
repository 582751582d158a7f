// Tensor-memory GEMM for M > 16: C[M, N] = A[M, K] * dequant(B)[K, N] on the 5th-generation tensor
// cores (tcgen05.mma, accumulators in TMEM).
//
// One persistent CTA per SM, 768 threads, warp-specialised:
//   warp 0      TMA producer of the packed weight chunks (+ their scale / zero-point rows)
//   warp 1      TMA producer of the activation tiles
//   warp 2      allocates tensor memory, issues the MMAs (one thread)
//   warps 4-7   epilogue: tcgen05.ld the accumulator, bias / nvfp4 global scale, store C
//   warps 8-23  dequantise: packed codes (shared memory) -> K-major 128-byte-swizzled operand tile
//               of the activation type, scaled per group, in shared memory
// Output tile: (128 * MT) rows x 256 columns (one packed column group), K walked in chunks of 64.
// Per chunk the tensor core runs 4 * MT MMAs of 128 x 256 x 16; the two 128-row halves share the
// dequantised weight tile, which halves the dequantisation work and the operand-write traffic per
// flop (MT = 2).  The accumulators use 256 * MT of the 512 TMEM columns.
//
// Pipelines (all mbarrier based, every wait bounded):
//   raw ring   : TMA -> dequant warps                (raw_full / raw_empty)
//   A ring     : TMA -> MMA                          (a_full / a_empty via tcgen05.commit)
//   B ring     : dequant warps -> MMA                (b_full / b_empty via tcgen05.commit)
//   accumulator: MMA -> epilogue -> MMA              (acc_full via tcgen05.commit / acc_empty)
//

#include <cstdint>
#include "codes.cuh"
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"

namespace mb200 {
namespace {

using namespace codes;

constexpr int BN = 256;
constexpr int BK = 64;
constexpr int KT = 4;            // k-tiles of 16 per chunk
constexpr int META = 2048;       // bytes reserved for the scale rows of a chunk (and again for zeros)
constexpr int THREADS = 768;
constexpr int DQ_WARPS = 16;
constexpr int MOE_A_STAGES = 4;  // gathered activation ring of the grouped kernel

template <int BITS, int MT, int AST = 3>
struct TcLayout {
  static constexpr int RAW_W = KT * 16 * BN * BITS / 8;  // 8 KiB / 16 KiB
  static constexpr int RAW_BYTES = RAW_W + 2 * META;
  // as deep as shared memory allows: with few row tiles the kernel streams weights and the ring
  // depth is what hides the HBM latency
  static constexpr int RAW_STAGES = (AST != 3) ? (BITS == 4 ? (MT == 1 ? 4 : 6) : 4)   // grouped kernel
                                    : (MT == 1 ? (BITS == 4 ? 6 : 4) : (BITS == 4 ? 5 : 3));
  static constexpr int A_BYTES = MT * 128 * 128;
  static constexpr int A_STAGES = AST;
  static constexpr int B_BYTES = BN * 128;
  // three operand stages where they fit: the dense kernel then runs its dequant warps in two groups
  static constexpr int B_STAGES = (MT == 1 && (BITS == 4 || AST == 3)) ? 3 : 2;
  static constexpr int OFF_RAW = 0;
  static constexpr int OFF_A = OFF_RAW + RAW_STAGES * RAW_BYTES;
  static constexpr int OFF_B = OFF_A + A_STAGES * A_BYTES;
  static constexpr int OFF_BAR = OFF_B + B_STAGES * B_BYTES;
  static constexpr int NUM_BARS = 2 * RAW_STAGES + 2 * A_STAGES + 2 * B_STAGES + 2;
  static constexpr int TOTAL = OFF_BAR + NUM_BARS * 8 + 16;   // + tensor-memory slot, + the issuer's drain barrier
};

struct TcParams {
  void* c;
  const void* bias;
  const float* global_scale;
  int M, N, K;
  int num_groups, group_size, rpc;
  int kc;       // chunks along K
  int m_tiles, n_tiles;
  uint32_t raw_tx, a_tx;
  int splits;        // k slices per tile; > 1: fp32 partials [slice][M][N], summed by tc_splitk_reduce_kernel
  int sk;            // > 0: stream-K over (tile, chunk) units with this many CTAs; fp32 partials
                     // [CTA][2][tile rows][256], summed by tc_streamk_reduce_kernel
  float* partials;
};

__device__ int g_tc_status = 0;

// A work item of the dense kernel: the chunks [c0, c1) of one tile.  Whole tiles write C; k slices and
// stream-K segments write fp32 partial sums at partials[pbase + row * pstride + pcol + column].
struct TcItem {
  int mt, nt, c0, c1;
  bool partial;
  int64_t pbase;
  int pstride, pcol;
};

// The work items of a CTA.  Tile / k-slice mode: items blockIdx.x, blockIdx.x + gridDim.x, ...  Stream-K
// mode: the (tile, chunk) units are cut into gridDim.x equal ranges, a CTA's range touches at most two
// tiles (the launch has fewer tiles than CTAs) and each touched tile is one item (segment 0, then 1).
struct TcWalk {
  int item, num_items;
  int64_t u, u1;
  int seg;
  __device__ explicit TcWalk(const TcParams& p) {
    item = blockIdx.x;
    num_items = p.m_tiles * p.n_tiles * p.splits;
    const int64_t U = (int64_t)p.m_tiles * p.n_tiles * p.kc;
    u = (int64_t)blockIdx.x * U / gridDim.x;
    u1 = (int64_t)(blockIdx.x + 1) * U / gridDim.x;
    seg = 0;
  }
  __device__ bool next(const TcParams& p, int slot_elems, TcItem& it) {
    if (p.sk > 0) {
      if (u >= u1) return false;
      const int tile = (int)(u / p.kc);
      it.mt = tile % p.m_tiles;
      it.nt = tile / p.m_tiles;
      it.c0 = (int)(u - (int64_t)tile * p.kc);
      const int64_t left = u1 - u;
      it.c1 = (int)((int64_t)it.c0 + left < (int64_t)p.kc ? (int64_t)it.c0 + left : (int64_t)p.kc);
      it.partial = !(it.c0 == 0 && it.c1 == p.kc);
      it.pbase = ((int64_t)blockIdx.x * 2 + seg) * slot_elems - (int64_t)it.mt * (slot_elems / BN) * BN;
      it.pstride = BN;
      it.pcol = 0;
      u += it.c1 - it.c0;
      ++seg;
      return true;
    }
    if (item >= num_items) return false;
    const int tile = item / p.splits;
    const int slice = item - tile * p.splits;
    it.mt = tile % p.m_tiles;
    it.nt = tile / p.m_tiles;
    it.c0 = (int)((int64_t)p.kc * slice / p.splits);
    it.c1 = (int)((int64_t)p.kc * (slice + 1) / p.splits);
    it.partial = p.splits > 1;
    it.pbase = (int64_t)slice * p.M * p.N;
    it.pstride = p.N;
    it.pcol = it.nt * BN;
    item += gridDim.x;
    return true;
  }
};


// kind::f16 instruction descriptor: fp32 accumulate, A and B both T, both K-major, M = 128, N = 256.
template <typename T>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
  uint32_t d = 0;
  d |= 1u << 4;                                  // D format f32
  d |= (kHalf<T> ? 0u : 1u) << 7;                // A format
  d |= (kHalf<T> ? 0u : 1u) << 10;               // B format
  d |= (uint32_t)(BN >> 3) << 17;                // N
  d |= (uint32_t)(128 >> 4) << 24;               // M
  return d;
}

// ---- dequantisation of one chunk (256 columns x 64 k) by the eight dequant warps ------------------------
// Warp d handles the 8 k of 16-byte chunk index d of every row (k-tile d >> 1, half d & 1); lane ->
// (64-column tile sub = lane >> 3, 8-column vector nv = lane & 7).  The thread reads the 8 (16) packed
// words of its columns (conflict-free: the 32 lanes read one 128-byte line), pairs consecutive k with
// byte permutes, decodes, applies scale / zero and writes, per column, the 16 bytes (8 k) of the
// operand row at its swizzled position.
//
// Store order: in step s a lane does not write its column s but column s ^ nv (4-bit) resp.
// s ^ (nv >> 1) (8-bit).  The eight lanes of a quarter warp then hit eight different rows mod 8,
// i.e. eight different 16-byte positions of the swizzled 128-byte lines, and the 16-byte stores
// are bank-conflict free.  The column index is a run-time value, so codes are picked with run-time
// shifts / permute selectors and the scale of the column is fetched from shared memory.
template <typename T>
__device__ __forceinline__ uint32_t scale_pair_at(uint32_t row, int n) {
  const uint32_t w = lds16(row + n * 2);
  return prmt(w, w, 0x1010u);
}

template <typename T, int FMT>
__device__ __forceinline__ void dequant_chunk(uint32_t raw, uint32_t btile, int dw, int lane, int rpc, int group_size) {
  // 16 warps: warp dw -> 16-byte k chunk d = dw & 7 and the pair of 64-column tiles dw >> 3;
  // lane -> tile of the pair (bit 4), half of the store steps (bit 3), 8-column vector nv (bits 0-2).
  constexpr int BITS = format_bits(FMT);
  constexpr int RAW_W = KT * 16 * BN * BITS / 8;
  constexpr int SROW = format_scale_is_byte(FMT) ? BN : BN * 2;
  const int d = dw & 7;
  const int kt = d >> 1, half = d & 1;
  const int sub = (dw >> 3) * 2 + (lane >> 4), nv = lane & 7, sh = (lane >> 3) & 1;
  const int row_local = (rpc == 1) ? 0 : (kt * 16 + half * 8) / group_size;
  const uint32_t srow = raw + RAW_W + row_local * SROW;
  const uint32_t zrow = raw + RAW_W + META + row_local * SROW;

  if constexpr (BITS == 4) {
    const int n8 = sub * 64 + nv * 8;
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int lk = half * 8 + i;
      w[i] = lds32(raw + kt * 2048 + lk * 128 + ((nv ^ (lk & 7)) << 4) + sub * 4);
    }
    // scales / zeros of this thread's four columns, fetched before any arithmetic
    uint32_t sp[4], zp[4];
#pragma unroll
    for (int s4 = 0; s4 < 4; ++s4) {
      const int j = (sh * 4 + s4) ^ nv;
      const int n = n8 + j;
      zp[s4] = 0;
      if constexpr (FMT == kNVFP4) {
        const int pos = (j & 4) + ((j & 3) == 1 ? 2 : (j & 3) == 2 ? 1 : (j & 3));
        sp[s4] = fp4_scale_pair<T, FMT>((lds16(srow + ((n8 + pos) & ~1)) >> (8 * (pos & 1))) & 0xffu);
      } else if constexpr (FMT == kMXFP4) {
        sp[s4] = fp4_scale_pair<T, FMT>((lds16(srow + (n & ~1)) >> (8 * (n & 1))) & 0xffu);
      } else {
        sp[s4] = scale_pair_at<T>(srow, n);
        if constexpr (format_has_zp(FMT)) zp[s4] = scale_pair_at<T>(zrow, n) ^ 0x80008000u;
      }
    }
    // za: codes of the columns whose parity equals this lane's nv parity; zb: the other parity
    // (low 16 bits of a word = even columns 0,2,4,6; high 16 bits = odd columns 1,3,5,7)
    const uint32_t sel_a = (nv & 1) ? 0x7632u : 0x5410u, sel_b = (nv & 1) ? 0x5410u : 0x7632u;
    uint32_t za[4], zb[4];
#pragma unroll
    for (int kp = 0; kp < 4; ++kp) {
      za[kp] = prmt(w[2 * kp], w[2 * kp + 1], sel_a);
      zb[kp] = prmt(w[2 * kp], w[2 * kp + 1], sel_b);
    }
#pragma unroll
    for (int s4 = 0; s4 < 4; ++s4) {
      const int s = sh * 4 + s4;
      const int j = s ^ nv;  // column handled in this step
      const int m = j >> 1;  // its code index inside the 16-bit half
      const int n = n8 + j;
      uint32_t v[4];
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {
        const uint32_t z = (s4 & 1) ? zb[kp] : za[kp];  // s and s4 have the same parity
        uint32_t q;
        if constexpr (FMT == kU4B8 || FMT == kU4) {
          constexpr uint32_t zero = (FMT == kU4B8) ? 8 : 0;
          constexpr uint32_t magic = kHalf<T> ? 0x6400u : 0x4300u;  // 1024 / 128: one unit per code step
          constexpr uint32_t c = magic + zero;
          q = psub<T>(((z >> (4 * m)) & 0x000f000fu) | (magic | (magic << 16)), c | (c << 16));
        } else {
          const uint32_t t = z << (12 - 4 * m);
          constexpr int shf = kHalf<T> ? 3 : 6;
          q = ((t & 0x70007000u) >> shf) | (t & 0x80008000u);
        }
        if constexpr (format_has_zp(FMT)) v[kp] = pfma<T>(q, sp[s4], zp[s4]);
        else v[kp] = pmul<T>(q, sp[s4]);
      }
      sts128(btile + n * 128 + ((d ^ j) << 4), v[0], v[1], v[2], v[3]);
    }
  } else {
    // 8-bit: the two lanes that differ in bit 3 take the two 128-byte half lines (columns nv*4 and
    // (nv + 8)*4 of the tile); each writes its four columns, rotated by nv >> 1.
    const int rot = (nv >> 1) & 3;
    const int hh = sh;
    const int n4 = sub * 64 + (nv + 8 * hh) * 4;
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int R = (half * 8 + i) * 2 + hh;
      w[i] = lds32(raw + kt * 4096 + R * 128 + ((nv ^ (R & 7)) << 4) + sub * 4);
    }
    uint32_t sp[4], zp[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int n = n4 + (s ^ rot);
      sp[s] = scale_pair_at<T>(srow, n);
      zp[s] = 0;
      if constexpr (format_has_zp(FMT)) zp[s] = scale_pair_at<T>(zrow, n) ^ 0x80008000u;
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int j = s ^ rot;                         // column handled in this step
      const int bp = (j & 1) * 2 + (j >> 1);         // its byte inside the word
      const uint32_t sel = (uint32_t)bp | ((uint32_t)(4 + bp) << 4);
      const int n = n4 + j;
      uint32_t v[4];
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {
        const uint32_t y = prmt(w[2 * kp], w[2 * kp + 1], sel);  // bytes 0,1 = the code at k0, k1
        const uint32_t q = value8<T, FMT>(y, 0);
        if constexpr (format_has_zp(FMT)) v[kp] = pfma<T>(q, sp[s], zp[s]);
        else v[kp] = pmul<T>(q, sp[s]);
      }
      sts128(btile + n * 128 + ((d ^ (n & 7)) << 4), v[0], v[1], v[2], v[3]);
    }
  }
}

template <typename T>
__device__ __forceinline__ uint32_t pack_out(float a, float b) {
  if constexpr (kHalf<T>) {
    __half2 r = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
  }
}

template <typename T, int FMT, int MT>
__global__ void __launch_bounds__(THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
               const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ, const TcParams p) {
  constexpr int BITS = format_bits(FMT);
  using L = TcLayout<BITS, MT>;
  constexpr int RS = L::RAW_STAGES, AS = L::A_STAGES, BS = L::B_STAGES;
  constexpr uint32_t NCOLS = 256 * MT;
  // With three operand stages the dequant warps work in two groups of eight on alternate chunks (a warp takes both
  // column halves of its 8-k slice): one group's barrier round trips overlap the other group's conversion.
  constexpr bool DQ_SPLIT = (BS == 3) && (RS % 2 == 0);
  constexpr int DQ_ARRIVALS = DQ_SPLIT ? DQ_WARPS / 2 : DQ_WARPS;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = base + L::OFF_BAR;
  auto raw_full = [&](int s) { return bar0 + 8u * s; };
  auto raw_empty = [&](int s) { return bar0 + 8u * (RS + s); };
  auto a_full = [&](int s) { return bar0 + 8u * (2 * RS + s); };
  auto a_empty = [&](int s) { return bar0 + 8u * (2 * RS + AS + s); };
  auto b_full = [&](int s) { return bar0 + 8u * (2 * RS + 2 * AS + s); };
  auto b_empty = [&](int s) { return bar0 + 8u * (2 * RS + 2 * AS + BS + s); };
  const uint32_t acc_full = bar0 + 8u * (2 * RS + 2 * AS + 2 * BS);
  const uint32_t acc_empty = acc_full + 8u;
  const uint32_t tmem_slot = acc_empty + 8u;
  const uint32_t drain_bar = tmem_slot + 8u;   // the MMA issuer's own commit before the tensor memory is freed

  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < RS; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), DQ_ARRIVALS); }
    for (int s = 0; s < AS; ++s) { mbar_init(a_full(s), 1); mbar_init(a_empty(s), 1); }
    for (int s = 0; s < BS; ++s) { mbar_init(b_full(s), DQ_ARRIVALS); mbar_init(b_empty(s), 1); }
    mbar_init(drain_bar, 1);
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 4);
    fence_barrier_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmS);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, NCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  constexpr int ROWS_PER_KT = (BITS == 4) ? 16 : 32;
  constexpr int SLOT_ELEMS = 128 * MT * BN;  // a stream-K partial: the rows of a tile x 256 columns
  // the reduce kernel of a split launch may be scheduled now; it waits for this grid's completion itself
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ---------------- packed-weight producer ----------------
    if (lane == 0) {
      int s = 0, issued = 0;
      uint32_t ph = 0;
      bool ok = true;
      TcWalk wk(p);
      TcItem it;
      while (ok && wk.next(p, SLOT_ELEMS, it)) {
        const int nt = it.nt;
        for (int c = it.c0; c < it.c1; ++c) {
          if (!mbar_wait(raw_empty(s), ph ^ 1u, &s_abort)) { atomicExch(&g_tc_status, 1); ok = false; break; }
          const uint32_t st = base + L::OFF_RAW + s * L::RAW_BYTES;
          mbar_arrive_expect_tx(raw_full(s), p.raw_tx);
          tma_load_3d(st, &tmW, raw_full(s), 0, nt * ROWS_PER_KT, c * KT);
          const int srow = (p.num_groups == 1) ? 0 : (c * BK) / p.group_size;
          tma_load_2d(st + L::RAW_W, &tmS, raw_full(s), nt * BN, srow);
          if constexpr (format_has_zp(FMT)) tma_load_2d(st + L::RAW_W + META, &tmZ, raw_full(s), nt * BN, srow);
          if (++s == RS) { s = 0; ph ^= 1u; }
          ++issued;
        }
      }
      if (s_abort != 0) drain_copies(raw_full, RS, issued);   // no copy of this thread's is in flight when it leaves
    }
  } else if (warp == 1) {
    // ---------------- activation producer ----------------
    if (lane == 0) {
      int s = 0, issued = 0;
      uint32_t ph = 0;
      bool ok = true;
      TcWalk wk(p);
      TcItem it;
      while (ok && wk.next(p, SLOT_ELEMS, it)) {
        const int mt = it.mt;
        for (int c = it.c0; c < it.c1; ++c) {
          if (!mbar_wait(a_empty(s), ph ^ 1u, &s_abort)) { atomicExch(&g_tc_status, 2); ok = false; break; }
          mbar_arrive_expect_tx(a_full(s), p.a_tx);
          tma_load_2d(base + L::OFF_A + s * L::A_BYTES, &tmA, a_full(s), c * BK, mt * 128 * MT);
          if (++s == AS) { s = 0; ph ^= 1u; }
          ++issued;
        }
      }
      if (s_abort != 0) drain_copies(a_full, AS, issued);
    }
  } else if (warp == 2) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc<T>();
      int sa = 0, sb = 0;
      uint32_t pha = 0, phb = 0, phacc = 0;
      bool ok = true;
      TcWalk wk(p);
      TcItem it;
      while (ok && wk.next(p, SLOT_ELEMS, it)) {
        if (!mbar_wait(acc_empty, phacc ^ 1u, &s_abort)) { atomicExch(&g_tc_status, 3); ok = false; break; }
        tc_fence_after();
        for (int c = it.c0; c < it.c1; ++c) {
          if (!mbar_wait(a_full(sa), pha, &s_abort) || !mbar_wait(b_full(sb), phb, &s_abort)) {
            atomicExch(&g_tc_status, 4);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = base + L::OFF_A + sa * L::A_BYTES;
          const uint32_t b_addr = base + L::OFF_B + sb * L::B_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t bdesc = kmajor_sw128_desc(b_addr + kk * 32);
#pragma unroll
            for (int h = 0; h < MT; ++h) {
              const uint64_t adesc = kmajor_sw128_desc(a_addr + h * (128 * 128) + kk * 32);
              tc_mma_f16(tmem_base + h * 256, adesc, bdesc, idesc, (c > it.c0 || kk > 0) ? 1u : 0u);
            }
          }
          tc_commit(a_empty(sa));
          tc_commit(b_empty(sb));
          if (++sa == AS) { sa = 0; pha ^= 1u; }
          if (++sb == BS) { sb = 0; phb ^= 1u; }
        }
        if (ok) tc_commit(acc_full);
        phacc ^= 1u;
      }
      // the tensor memory is freed only after this thread's MMAs have completed (after a give-up nobody else waits)
      if (s_abort != 0) {
        tc_commit(drain_bar);
        drain_barrier(drain_bar, 0);
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ---------------- epilogue ----------------
    const int q = warp - 4;
    uint32_t ph = 0;
    float alpha = 1.f;
    if constexpr (FMT == kNVFP4) alpha = p.global_scale[0];
    T* C = reinterpret_cast<T*>(p.c);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    TcWalk wk(p);
    TcItem it;
    while (wk.next(p, SLOT_ELEMS, it)) {
      const int mt = it.mt, nt = it.nt;
      if (!mbar_wait(acc_full, ph, &s_abort)) { atomicExch(&g_tc_status, 5); break; }
      ph ^= 1u;
      tc_fence_after();
#pragma unroll 1
      for (int h = 0; h < MT; ++h) {
        const int row = mt * 128 * MT + h * 128 + q * 32 + lane;
#pragma unroll 1
        for (int cb = 0; cb < BN / 16; ++cb) {
          uint32_t v[16];
          tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + h * 256 + cb * 16, v);
          tmem_ld_wait();
          const int col0 = nt * BN + cb * 16;
          if (it.partial) {
            // part of a tile's K range: raw fp32 sums; scale, bias and rounding happen once, in the reduce kernel
            if (row < p.M) {
              uint4* dst = reinterpret_cast<uint4*>(p.partials + it.pbase + (int64_t)row * it.pstride + it.pcol + cb * 16);
#pragma unroll
              for (int i = 0; i < 4; ++i) dst[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            }
          } else if (row < p.M) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float x0 = __uint_as_float(v[2 * i]) * alpha, x1 = __uint_as_float(v[2 * i + 1]) * alpha;
              if (bias != nullptr) {
                x0 += to_float<T>(bias[bias_index(col0 + 2 * i)]);
                x1 += to_float<T>(bias[bias_index(col0 + 2 * i + 1)]);
              }
              o[i] = pack_out<T>(x0, x1);
            }
            uint4* dst = reinterpret_cast<uint4*>(C + (int64_t)row * p.N + col0);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
    }
  } else if (warp >= 8) {
    // ---------------- dequantisation ----------------
    const int d = warp - 8;
    bool ok = true;
    TcWalk wk(p);
    TcItem it;
    if constexpr (DQ_SPLIT) {
      const int grp = d >> 3, d8 = d & 7;
      int sr = grp % RS, sb = grp % BS, j = 0;
      uint32_t phr = 0, phb = 0;
      while (ok && wk.next(p, SLOT_ELEMS, it)) {
        for (int c = it.c0; c < it.c1; ++c, ++j) {
          if ((j & 1) != grp) continue;
          if (!mbar_wait(raw_full(sr), phr, &s_abort) || !mbar_wait(b_empty(sb), phb ^ 1u, &s_abort)) {
            atomicExch(&g_tc_status, 6);
            ok = false;
            break;
          }
          const uint32_t raw = base + L::OFF_RAW + sr * L::RAW_BYTES, bt = base + L::OFF_B + sb * L::B_BYTES;
          dequant_chunk<T, FMT>(raw, bt, d8, lane, p.rpc, p.group_size);
          dequant_chunk<T, FMT>(raw, bt, d8 + 8, lane, p.rpc, p.group_size);
          fence_proxy_async();  // the tensor core reads the tile through the async proxy
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(b_full(sb));
            mbar_arrive(raw_empty(sr));
          }
          sr += 2;
          if (sr >= RS) { sr -= RS; phr ^= 1u; }
          sb += 2;
          if (sb >= BS) { sb -= BS; phb ^= 1u; }
        }
      }
    } else {
    int sr = 0, sb = 0;
    uint32_t phr = 0, phb = 0;
    while (ok && wk.next(p, SLOT_ELEMS, it)) {
      for (int c = it.c0; c < it.c1; ++c) {
        if (!mbar_wait(raw_full(sr), phr, &s_abort) || !mbar_wait(b_empty(sb), phb ^ 1u, &s_abort)) {
          atomicExch(&g_tc_status, 6);
          ok = false;
          break;
        }
        dequant_chunk<T, FMT>(base + L::OFF_RAW + sr * L::RAW_BYTES, base + L::OFF_B + sb * L::B_BYTES, d, lane,
                              p.rpc, p.group_size);
        fence_proxy_async();  // the tensor core reads the tile through the async proxy
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(b_full(sb));
          mbar_arrive(raw_empty(sr));
        }
        if (++sr == RS) { sr = 0; phr ^= 1u; }
        if (++sb == BS) { sb = 0; phb ^= 1u; }
      }
    }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, NCOLS);
  }
}

// Sums the k slices of a split launch in slice order (the same order every run), then applies the
// nvfp4 global scale and the bias and rounds once.  One thread per four consecutive columns; the loads of
// four slices are issued before their sums so that their latencies overlap.  Launched as a programmatic
// dependent of the GEMM kernel: it may start early and waits here for the partials.
template <typename T>
__global__ void __launch_bounds__(256) tc_splitk_reduce_kernel(const TcParams p, bool has_alpha) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t vecs = (int64_t)p.M * p.N / 4;
  const int64_t slice_stride = (int64_t)p.M * p.N;
  const float alpha = has_alpha ? p.global_scale[0] : 1.f;
  const T* bias = reinterpret_cast<const T*>(p.bias);
  T* C = reinterpret_cast<T*>(p.c);
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = v * 4;
    const int col0 = (int)(e % p.N);
    const float* src = p.partials + e;
    float4 a = *reinterpret_cast<const float4*>(src);
    int sl = 1;
    for (; sl + 3 < p.splits; sl += 4) {
      const float4 x0 = *reinterpret_cast<const float4*>(src + sl * slice_stride);
      const float4 x1 = *reinterpret_cast<const float4*>(src + (sl + 1) * slice_stride);
      const float4 x2 = *reinterpret_cast<const float4*>(src + (sl + 2) * slice_stride);
      const float4 x3 = *reinterpret_cast<const float4*>(src + (sl + 3) * slice_stride);
      a.x = (((a.x + x0.x) + x1.x) + x2.x) + x3.x;
      a.y = (((a.y + x0.y) + x1.y) + x2.y) + x3.y;
      a.z = (((a.z + x0.z) + x1.z) + x2.z) + x3.z;
      a.w = (((a.w + x0.w) + x1.w) + x2.w) + x3.w;
    }
    for (; sl < p.splits; ++sl) {
      const float4 x = *reinterpret_cast<const float4*>(src + sl * slice_stride);
      a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
    }
    float r[4] = {a.x * alpha, a.y * alpha, a.z * alpha, a.w * alpha};
    if (bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 4; ++i) r[i] += to_float<T>(bias[bias_index(col0 + i)]);
    }
    *reinterpret_cast<uint2*>(C + e) = make_uint2(pack_out<T>(r[0], r[1]), pack_out<T>(r[2], r[3]));
  }
}

// Stream-K: adds, for every tile that more than one CTA worked on, the owners' partial tiles in CTA order,
// then scale, bias and rounding as above.  CTA q owns the units [q U / P, (q + 1) U / P); the first owner
// of a tile wrote its second slot unless its range starts with the tile, every later owner its first.
template <typename T>
__global__ void __launch_bounds__(256) tc_streamk_reduce_kernel(const TcParams p, int tile_rows, bool has_alpha) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t vecs = (int64_t)p.M * p.N / 4;
  const int64_t P = p.sk, U = (int64_t)p.m_tiles * p.n_tiles * p.kc;
  const int64_t slot_elems = (int64_t)tile_rows * BN;
  const float alpha = has_alpha ? p.global_scale[0] : 1.f;
  const T* bias = reinterpret_cast<const T*>(p.bias);
  T* C = reinterpret_cast<T*>(p.c);
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = v * 4;
    const int row = (int)(e / p.N), col = (int)(e % p.N);
    const int nt = col / BN, mt = row / tile_rows;
    const int64_t tile = (int64_t)nt * p.m_tiles + mt;
    const int64_t ua = tile * p.kc, ub = ua + p.kc - 1;
    const int64_t pa = ((ua + 1) * P - 1) / U, pb = ((ub + 1) * P - 1) / U;
    if (pa == pb) continue;  // one owner: it wrote C itself
    const int first_slot = (pa * U / P == ua) ? 0 : 1;
    const float* src = p.partials + (int64_t)(row - mt * tile_rows) * BN + (col - nt * BN);
    float4 a = *reinterpret_cast<const float4*>(src + (pa * 2 + first_slot) * slot_elems);
    int64_t q = pa + 1;
    for (; q + 3 <= pb; q += 4) {
      const float4 x0 = *reinterpret_cast<const float4*>(src + (q * 2) * slot_elems);
      const float4 x1 = *reinterpret_cast<const float4*>(src + ((q + 1) * 2) * slot_elems);
      const float4 x2 = *reinterpret_cast<const float4*>(src + ((q + 2) * 2) * slot_elems);
      const float4 x3 = *reinterpret_cast<const float4*>(src + ((q + 3) * 2) * slot_elems);
      a.x = (((a.x + x0.x) + x1.x) + x2.x) + x3.x;
      a.y = (((a.y + x0.y) + x1.y) + x2.y) + x3.y;
      a.z = (((a.z + x0.z) + x1.z) + x2.z) + x3.z;
      a.w = (((a.w + x0.w) + x1.w) + x2.w) + x3.w;
    }
    for (; q <= pb; ++q) {
      const float4 x = *reinterpret_cast<const float4*>(src + (q * 2) * slot_elems);
      a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
    }
    float r[4] = {a.x * alpha, a.y * alpha, a.z * alpha, a.w * alpha};
    if (bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 4; ++i) r[i] += to_float<T>(bias[bias_index(col + i)]);
    }
    *reinterpret_cast<uint2*>(C + e) = make_uint2(pack_out<T>(r[0], r[1]), pack_out<T>(r[2], r[3]));
  }
}

// ---------------------------------------------------------------------------------------------------
// Grouped (MoE) variant
// ---------------------------------------------------------------------------------------------------
// Rows come from `sorted_token_ids`: blocks of `bs` routes, each block belonging to one expert, the
// blocks of an expert next to each other.  moe_gather_rows_kernel first copies the activation rows into
// that order, moe_tile_list_kernel lists the tiles: up to 128 * MT / bs consecutive blocks of ONE
// expert, starting at the expert's first block.  A work item is (tile, column group): the whole K loop
// with that expert's weights on rows loaded by plain TMA boxes, after which the epilogue scatters the
// rows of the tile (C row = route id, times the router weight when asked).
struct MoeParams {
  const void* a;
  void* c;
  const void* bias;
  const float* global_scale;
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post_pad;
  const float* topk_weights;
  int64_t size_m;
  int N, K;
  int num_groups, group_size, rpc;
  int kc, n_tiles, num_tiles;
  int num_sorted, num_experts;
  int bs, blocks_per_tile, top_k, mul_topk;
  uint32_t raw_tx;
  const int32_t* tile_start;  // first block of every tile (written by moe_tile_list_kernel)
  const int32_t* tile_count;  // number of tiles
};

// Copies the activation rows into the order of sorted_token_ids (row pos <- A[sid / top_k], zeros for
// padding entries), 16 bytes per thread step, for the padded length only.
template <typename T>
__global__ void __launch_bounds__(256) moe_gather_rows_kernel(const T* __restrict__ a, T* __restrict__ out,
                                                              const int32_t* __restrict__ sorted_ids,
                                                              const int32_t* __restrict__ num_post_pad,
                                                              int num_sorted, int64_t size_m, int top_k, int K) {
  const int vec_per_row = K / 8;
  const int rows = min(num_post_pad[0], num_sorted);
  const int64_t total = (int64_t)rows * vec_per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int pos = (int)(idx / vec_per_row), v = (int)(idx % vec_per_row);
    const int sid = sorted_ids[pos];
    uint4 val = make_uint4(0, 0, 0, 0);
    if (sid >= 0 && (int64_t)sid < size_m * top_k)
      val = *reinterpret_cast<const uint4*>(a + (int64_t)(sid / top_k) * K + v * 8);
    *reinterpret_cast<uint4*>(out + (int64_t)pos * K + v * 8) = val;
  }
}

// Cuts the sorted route list into tiles that never mix experts: a tile starts at the first block of an
// expert's run and then every blocks_per_tile blocks inside the run.  One CTA of 1024 threads; blocks are
// scanned 1024 at a time (a max-scan of run starts, then a sum-scan to compact the tile starts).
__global__ void __launch_bounds__(1024) moe_tile_list_kernel(const int32_t* __restrict__ expert_ids,
                                                            const int32_t* __restrict__ num_post_pad, int num_sorted,
                                                            int bs, int blocks_per_tile, int num_experts,
                                                            int32_t* __restrict__ tile_start,
                                                            int32_t* __restrict__ tile_count) {
  __shared__ int s_scan[1024];
  __shared__ int s_carry_start, s_carry_count;
  const int tid = threadIdx.x;
  const int nb = min(num_post_pad[0], num_sorted) / bs;
  if (tid == 0) { s_carry_start = 0; s_carry_count = 0; }
  __syncthreads();
  for (int b0 = 0; b0 < nb; b0 += 1024) {
    const int b = b0 + tid;
    int e = -1, run_start = -1;
    if (b < nb) {
      e = expert_ids[b];
      if (b == 0 || expert_ids[b - 1] != e) run_start = b;
    }
    // inclusive max-scan of the run starts, seeded with the run that reaches into this batch
    s_scan[tid] = (tid == 0 && run_start < 0) ? s_carry_start : run_start;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const int v = (tid >= off) ? s_scan[tid - off] : -1;
      __syncthreads();
      s_scan[tid] = max(s_scan[tid], v);
      __syncthreads();
    }
    run_start = s_scan[tid];
    const int carry_start = s_scan[1023];
    const bool is_start = b < nb && e >= 0 && e < num_experts && ((b - run_start) % blocks_per_tile) == 0;
    __syncthreads();
    s_scan[tid] = is_start ? 1 : 0;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const int v = (tid >= off) ? s_scan[tid - off] : 0;
      __syncthreads();
      s_scan[tid] += v;
      __syncthreads();
    }
    const int base = s_carry_count;
    if (is_start) tile_start[base + s_scan[tid] - 1] = b;
    const int batch_total = s_scan[1023];
    __syncthreads();
    if (tid == 0) { s_carry_start = carry_start; s_carry_count = base + batch_total; }
    __syncthreads();
  }
  if (tid == 0) tile_count[0] = s_carry_count;
}

// Work items of a CTA: (tile, column group) pairs, tile-major, strided by the grid.
struct ItemIter {
  int w, total, stride, n_tiles, blocks_per_tile, bs, num_blocks;
  int nt, blk;
  const int32_t* expert_ids;
  const int32_t* tile_start;
  __device__ void init(const MoeParams& p) {
    stride = gridDim.x;
    w = (int)blockIdx.x - stride;
    total = p.tile_count[0] * p.n_tiles;
    n_tiles = p.n_tiles;
    blocks_per_tile = p.blocks_per_tile;
    bs = p.bs;
    num_blocks = min(p.num_post_pad[0], p.num_sorted) / p.bs;
    expert_ids = p.expert_ids;
    tile_start = p.tile_start;
    blk = nt = 0;
  }
  // Advances to the next item; rows [0, row_hi) of the tile that starts at block `blk` belong to expert e.
  __device__ bool next(int& e, int& row_lo, int& row_hi) {
    w += stride;
    if (w >= total) return false;
    const int ti = w / n_tiles;
    nt = w - ti * n_tiles;
    blk = tile_start[ti];
    e = expert_ids[blk];
    int count = 1;
    while (count < blocks_per_tile && blk + count < num_blocks && expert_ids[blk + count] == e) ++count;
    row_lo = 0;
    row_hi = count * bs;
    return true;
  }
  __device__ int row0() const { return blk * bs; }
};

template <typename T, int FMT, int MT>
__global__ void __launch_bounds__(THREADS, 1)
tc_moe_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
              const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ, const MoeParams p) {
  constexpr int BITS = format_bits(FMT);
  // MT = 2: 256-row tiles whose two halves share every dequantised B tile (ring depths of the dense kernel)
  using L = TcLayout<BITS, MT, MT == 1 ? MOE_A_STAGES : 3>;
  constexpr int RS = L::RAW_STAGES, AS = L::A_STAGES, BS = L::B_STAGES;
  constexpr uint32_t NCOLS = 256 * MT;
  // with three operand stages the dequant warps work in two groups of eight on alternate chunks (see tc_gemm_kernel)
  constexpr bool DQ_SPLIT = (BS == 3) && (RS % 2 == 0);
  constexpr int DQ_ARRIVALS = DQ_SPLIT ? DQ_WARPS / 2 : DQ_WARPS;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = base + L::OFF_BAR;
  auto raw_full = [&](int s) { return bar0 + 8u * s; };
  auto raw_empty = [&](int s) { return bar0 + 8u * (RS + s); };
  auto a_full = [&](int s) { return bar0 + 8u * (2 * RS + s); };
  auto a_empty = [&](int s) { return bar0 + 8u * (2 * RS + AS + s); };
  auto b_full = [&](int s) { return bar0 + 8u * (2 * RS + 2 * AS + s); };
  auto b_empty = [&](int s) { return bar0 + 8u * (2 * RS + 2 * AS + BS + s); };
  const uint32_t acc_full = bar0 + 8u * (2 * RS + 2 * AS + 2 * BS);
  const uint32_t acc_empty = acc_full + 8u;
  const uint32_t tmem_slot = acc_empty + 8u;
  const uint32_t drain_bar = tmem_slot + 8u;   // the MMA issuer's own commit before the tensor memory is freed

  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < RS; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), DQ_ARRIVALS); }
    for (int s = 0; s < AS; ++s) { mbar_init(a_full(s), 1); mbar_init(a_empty(s), 1); }
    for (int s = 0; s < BS; ++s) { mbar_init(b_full(s), DQ_ARRIVALS); mbar_init(b_empty(s), 1); }
    mbar_init(drain_bar, 1);
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 4);
    fence_barrier_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmS);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, NCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  constexpr int ROWS_PER_KT = (BITS == 4) ? 16 : 32;
  ItemIter iter;
  iter.init(p);
  int e = 0, row_lo = 0, row_hi = 0;

  if (warp == 0) {
    // ---------------- packed-weight producer ----------------
    if (lane == 0) {
      int s = 0, issued = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && iter.next(e, row_lo, row_hi)) {
        for (int c = 0; c < p.kc; ++c) {
          if (!mbar_wait(raw_empty(s), ph ^ 1u, &s_abort)) { atomicExch(&g_tc_status, 11); ok = false; break; }
          const uint32_t st = base + L::OFF_RAW + s * L::RAW_BYTES;
          mbar_arrive_expect_tx(raw_full(s), p.raw_tx);
          // experts are stacked along the k-tile rows (weights) and along the group rows (scales)
          tma_load_3d(st, &tmW, raw_full(s), 0, iter.nt * ROWS_PER_KT, e * (p.K / 16) + c * KT);
          const int srow = e * p.num_groups + ((p.num_groups == 1) ? 0 : (c * BK) / p.group_size);
          tma_load_2d(st + L::RAW_W, &tmS, raw_full(s), iter.nt * BN, srow);
          if constexpr (format_has_zp(FMT)) tma_load_2d(st + L::RAW_W + META, &tmZ, raw_full(s), iter.nt * BN, srow);
          if (++s == RS) { s = 0; ph ^= 1u; }
          ++issued;
        }
      }
      if (s_abort != 0) drain_copies(raw_full, RS, issued);   // no copy of this thread's is in flight when it leaves
    }
  } else if (warp == 1) {
    // ---------------- activation producer ----------------
    // The rows were copied into sorted order by moe_gather_rows_kernel, so a tile's rows are
    // contiguous and one TMA box load per chunk feeds the MMA, exactly as in the dense kernel.
    // (Gathering inside this kernel was measured and rejected: cp.async copies are capped by the
    // number of copies the load/store unit keeps in flight - about 128 cycles per warp instruction -
    // and TMA gather4 loads cost about 100 cycles of issue time per 4 rows; both starve the MMA.)
    if (lane == 0) {
      int s = 0, issued = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && iter.next(e, row_lo, row_hi)) {
        const int row0 = iter.row0();
        for (int c = 0; c < p.kc; ++c) {
          if (!mbar_wait(a_empty(s), ph ^ 1u, &s_abort)) { atomicExch(&g_tc_status, 12); ok = false; break; }
          mbar_arrive_expect_tx(a_full(s), L::A_BYTES);
          tma_load_2d(base + L::OFF_A + s * L::A_BYTES, &tmA, a_full(s), c * BK, row0);
          if (++s == AS) { s = 0; ph ^= 1u; }
          ++issued;
        }
      }
      if (s_abort != 0) drain_copies(a_full, AS, issued);
    }
  } else if (warp == 2) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc<T>();
      int sa = 0, sb = 0;
      uint32_t pha = 0, phb = 0, phacc = 0;
      bool ok = true;
      while (ok && iter.next(e, row_lo, row_hi)) {
        if (!mbar_wait(acc_empty, phacc ^ 1u, &s_abort)) { atomicExch(&g_tc_status, 13); ok = false; break; }
        tc_fence_after();
        for (int c = 0; c < p.kc; ++c) {
          if (!mbar_wait(a_full(sa), pha, &s_abort)) { atomicExch(&g_tc_status, 14); ok = false; break; }
          if (!mbar_wait(b_full(sb), phb, &s_abort)) { atomicExch(&g_tc_status, 14); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = base + L::OFF_A + sa * L::A_BYTES;
          const uint32_t b_addr = base + L::OFF_B + sb * L::B_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t bdesc = kmajor_sw128_desc(b_addr + kk * 32);
#pragma unroll
            for (int h = 0; h < MT; ++h)
              tc_mma_f16(tmem_base + h * 256, kmajor_sw128_desc(a_addr + h * (128 * 128) + kk * 32), bdesc, idesc,
                         (c > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(a_empty(sa));
          tc_commit(b_empty(sb));
          if (++sa == AS) { sa = 0; pha ^= 1u; }
          if (++sb == BS) { sb = 0; phb ^= 1u; }
        }
        if (ok) tc_commit(acc_full);
        phacc ^= 1u;
      }
      // the tensor memory is freed only after this thread's MMAs have completed (after a give-up nobody else waits)
      if (s_abort != 0) {
        tc_commit(drain_bar);
        drain_barrier(drain_bar, 0);
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ---------------- epilogue: scatter the rows of the run ----------------
    const int q = warp - 4;
    uint32_t ph = 0;
    T* C = reinterpret_cast<T*>(p.c);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    while (iter.next(e, row_lo, row_hi)) {
      if (!mbar_wait(acc_full, ph, &s_abort)) { atomicExch(&g_tc_status, 15); break; }
      ph ^= 1u;
      tc_fence_after();
      float gs = 1.f;
      if constexpr (FMT == kNVFP4) gs = p.global_scale[e];
      const float bias_mul = (FMT == kNVFP4 && p.mul_topk) ? gs : 1.f;
#pragma unroll 1
      for (int h = 0; h < MT; ++h) {
        const int r = h * 128 + q * 32 + lane;
        // a warp whose 32 rows lie outside the run has nothing to store (warp-uniform test)
        if (h * 128 + q * 32 >= row_hi || h * 128 + q * 32 + 32 <= row_lo) continue;
        int sid = -1;
        if (r >= row_lo && r < row_hi) {
          const int64_t pos = (int64_t)iter.row0() + r;
          if (pos < p.num_sorted) sid = p.sorted_ids[pos];
          if (sid < 0 || (int64_t)sid >= p.size_m * p.top_k) sid = -1;
        }
        const float tw = (sid >= 0 && p.mul_topk) ? p.topk_weights[sid] : 1.f;
#pragma unroll 1
        for (int cb = 0; cb < BN / 16; ++cb) {
          uint32_t v[16];
          tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + h * 256 + cb * 16, v);
          tmem_ld_wait();
          const int col0 = iter.nt * BN + cb * 16;
          if (sid >= 0) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float x0 = __uint_as_float(v[2 * i]) * gs, x1 = __uint_as_float(v[2 * i + 1]) * gs;
              if (bias != nullptr) {
                x0 += to_float<T>(bias[(int64_t)e * p.N + bias_index(col0 + 2 * i)]) * bias_mul;
                x1 += to_float<T>(bias[(int64_t)e * p.N + bias_index(col0 + 2 * i + 1)]) * bias_mul;
              }
              o[i] = pack_out<T>(x0 * tw, x1 * tw);
            }
            uint4* dst = reinterpret_cast<uint4*>(C + (int64_t)sid * p.N + col0);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
    }
  } else if (warp >= 8) {
    // ---------------- dequantisation ----------------
    const int d = warp - 8;
    bool ok = true;
    if constexpr (DQ_SPLIT) {
      const int grp = d >> 3, d8 = d & 7;
      int sr = grp % RS, sb = grp % BS, j = 0;
      uint32_t phr = 0, phb = 0;
      while (ok && iter.next(e, row_lo, row_hi)) {
        for (int c = 0; c < p.kc; ++c, ++j) {
          if ((j & 1) != grp) continue;
          if (!mbar_wait(raw_full(sr), phr, &s_abort) || !mbar_wait(b_empty(sb), phb ^ 1u, &s_abort)) {
            atomicExch(&g_tc_status, 16);
            ok = false;
            break;
          }
          const uint32_t raw = base + L::OFF_RAW + sr * L::RAW_BYTES, bt = base + L::OFF_B + sb * L::B_BYTES;
          dequant_chunk<T, FMT>(raw, bt, d8, lane, p.rpc, p.group_size);
          dequant_chunk<T, FMT>(raw, bt, d8 + 8, lane, p.rpc, p.group_size);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(b_full(sb));
            mbar_arrive(raw_empty(sr));
          }
          sr += 2;
          if (sr >= RS) { sr -= RS; phr ^= 1u; }
          sb += 2;
          if (sb >= BS) { sb -= BS; phb ^= 1u; }
        }
      }
    } else {
    int sr = 0, sb = 0;
    uint32_t phr = 0, phb = 0;
    while (ok && iter.next(e, row_lo, row_hi)) {
      for (int c = 0; c < p.kc; ++c) {
        if (!mbar_wait(raw_full(sr), phr, &s_abort)) { atomicExch(&g_tc_status, 16); ok = false; break; }
        if (!mbar_wait(b_empty(sb), phb ^ 1u, &s_abort)) { atomicExch(&g_tc_status, 16); ok = false; break; }
        dequant_chunk<T, FMT>(base + L::OFF_RAW + sr * L::RAW_BYTES, base + L::OFF_B + sb * L::B_BYTES, d, lane,
                              p.rpc, p.group_size);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(b_full(sb));
          mbar_arrive(raw_empty(sr));
        }
        if (++sr == RS) { sr = 0; phr ^= 1u; }
        if (++sb == BS) { sb = 0; phb ^= 1u; }
      }
    }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, NCOLS);
  }
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------
// How the dense kernel cuts its work.  A CTA turns one chunk of packed weights into an operand tile in
// about 0.75 us (0.93 us with 256-row tiles) whatever else the GPU does, so a launch with fewer tiles than
// SMs, or a few more, is as slow as its longest CTA.  Three ways: whole tiles; k slices (every tile cut
// into the same number of slices, fp32 partials [slice][M][N]); stream-K (fewer tiles than SMs: the (tile,
// chunk) units cut into one equal range per SM, fp32 partial tiles per CTA).  The estimates below
// (microseconds) weigh the chunks of the longest CTA against the partials written and read back and the
// second launch; a split is used when it wins by a tenth.  A slice keeps at least four chunks.
struct TcPlan {
  int splits = 1;
  int sk = 0;
  int64_t scratch = 0;
};

TcPlan tc_plan(int64_t M, int64_t N, int64_t K, int64_t scratch_avail) {
  TcPlan plan;
  if (M <= 16 || N % BN != 0) return plan;
  const int mt_rows = (M <= 128) ? 128 : 256;
  const int64_t tiles = ((M + mt_rows - 1) / mt_rows) * (N / BN);
  const int64_t kc = (K + BK - 1) / BK;
  const int64_t sms = sm_count();
  if (tiles <= 0 || sms <= 0) return plan;
  const double chunk_us = (mt_rows == 128 ? 0.75 : 0.93);
  const double whole = (double)kc * chunk_us;
  double best = (double)((tiles + sms - 1) / sms) * whole * 0.9;
  for (int64_t s = 2; s <= 16 && s <= kc / 4; ++s) {
    const int64_t bytes = s * M * N * (int64_t)sizeof(float);
    if (bytes > (128ll << 20) || bytes > scratch_avail) break;
    const double rounds = (double)((tiles * s + sms - 1) / sms);
    const double t = rounds * whole / (double)s + 4.0 + 2.0 * (double)bytes / 5.0e6;
    if (t < best) { best = t; plan.splits = (int)s; plan.sk = 0; plan.scratch = bytes; }
  }
  if (tiles < sms && tiles * kc >= 4 * sms) {
    const int64_t ctas = sms;
    const int64_t bytes = ctas * 2 * mt_rows * BN * (int64_t)sizeof(float);
    // partial tiles actually written: about one per CTA plus one per tile, the valid rows of each
    const int64_t rows = M < mt_rows ? M : mt_rows;
    const double moved = (double)(ctas + tiles) * (double)rows * BN * sizeof(float);
    const double t = (double)((tiles * kc + ctas - 1) / ctas) * chunk_us + 4.0 + 2.0 * moved / 5.0e6;
    if (bytes <= scratch_avail && t < best) { best = t; plan.splits = 1; plan.sk = (int)ctas; plan.scratch = bytes; }
  }
  return plan;
}

template <typename T, int FMT, int MT>
int launch_tc(const GemmArgs& g) {
  constexpr int BITS = format_bits(FMT);
  using L = TcLayout<BITS, MT>;
  constexpr int SMEM = 1024 + L::TOTAL;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
  const int64_t K = g.size_k, N = g.size_n, M = g.size_m;
  const int64_t gs = K / g.num_groups;
  TcParams p{};
  p.c = g.c; p.bias = g.bias; p.global_scale = g.global_scale;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.num_groups = (int)g.num_groups; p.group_size = (int)gs;
  p.rpc = (g.num_groups > 1 && gs < BK) ? (int)(BK / gs) : 1;
  p.kc = (int)((K + BK - 1) / BK);
  p.m_tiles = (int)((M + 128 * MT - 1) / (128 * MT));
  p.n_tiles = (int)(N / BN);
  const int srow_bytes = format_scale_is_byte(FMT) ? BN : BN * 2;
  p.raw_tx = L::RAW_W + p.rpc * srow_bytes * (format_has_zp(FMT) ? 2 : 1);
  p.a_tx = L::A_BYTES;

  CUtensorMap tmW, tmA, tmS, tmZ;
  {
    const int rows_per_kt = (BITS == 4 ? 16 : 32) * p.n_tiles;
    const uint64_t dims[3] = {32, (uint64_t)rows_per_kt, (uint64_t)(K / 16)};
    const uint64_t strides[2] = {128, (uint64_t)rows_per_kt * 128};
    const uint32_t box[3] = {32, (uint32_t)(BITS == 4 ? 16 : 32), KT};
    if (int rc = cached_tensor_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, g.bq, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t strides[1] = {(uint64_t)g.a_stride * 2};
    const uint32_t box[2] = {BK, 128 * MT};
    if (int rc = encode_tensor_map(&tmA, kHalf<T> ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                   g.a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const bool byte_scale = format_scale_is_byte(FMT);
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)g.num_groups};
    const uint64_t strides[1] = {(uint64_t)N * (byte_scale ? 1 : 2)};
    const uint32_t box[2] = {BN, (uint32_t)p.rpc};
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
    MB_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<T, FMT, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    attr_set[dev] = true;
  }
  const int tiles = p.m_tiles * p.n_tiles;
  // Tiles that would leave SMs idle are cut along K, as far as the caller's scratch has room (tc_plan).
  const TcPlan plan = tc_plan(M, N, K, g.scratch != nullptr ? g.scratch_bytes : 0);
  p.splits = plan.splits;
  p.sk = plan.sk;
  p.partials = reinterpret_cast<float*>(g.scratch);
  const int64_t items = p.sk > 0 ? p.sk : (int64_t)tiles * p.splits;
  const int grid = (int)(items < sm_count() ? items : sm_count());
  tc_gemm_kernel<T, FMT, MT><<<grid, THREADS, SMEM, g.stream>>>(tmW, tmA, tmS, tmZ, p);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  if (p.splits > 1 || p.sk > 0) {
    const int64_t vecs = M * N / 4;
    const int64_t want = (vecs + 255) / 256;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(want < 8 * (int64_t)sm_count() ? want : 8 * (int64_t)sm_count()));
    cfg.blockDim = dim3(256);
    cfg.stream = g.stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (p.sk > 0) MB_CUDA(cudaLaunchKernelEx(&cfg, tc_streamk_reduce_kernel<T>, p, 128 * MT, FMT == kNVFP4));
    else MB_CUDA(cudaLaunchKernelEx(&cfg, tc_splitk_reduce_kernel<T>, p, FMT == kNVFP4));
    count_launches(1);
  }
  return 0;
}

template <typename T, int FMT>
int launch_fmt(const GemmArgs& g) {
  if (g.size_m <= 128) return launch_tc<T, FMT, 1>(g);
  return launch_tc<T, FMT, 2>(g);
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


template <typename T, int FMT, int MT>
int launch_moe(const GemmArgs& g) {
  constexpr int BITS = format_bits(FMT);
  using L = TcLayout<BITS, MT, MT == 1 ? MOE_A_STAGES : 3>;
  constexpr int SMEM = 1024 + L::TOTAL;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
  const int64_t K = g.size_k, N = g.size_n, E = g.num_experts;
  const int64_t gs = K / g.num_groups;
  MoeParams p{};
  p.a = g.a; p.c = g.c; p.bias = g.bias; p.global_scale = g.global_scale;
  p.sorted_ids = g.sorted_ids; p.expert_ids = g.expert_ids; p.num_post_pad = g.num_post_pad;
  p.topk_weights = g.topk_weights;
  p.size_m = g.size_m; p.N = (int)N; p.K = (int)K;
  p.num_groups = (int)g.num_groups; p.group_size = (int)gs;
  p.rpc = (g.num_groups > 1 && gs < BK) ? (int)(BK / gs) : 1;
  p.kc = (int)((K + BK - 1) / BK);
  p.n_tiles = (int)(N / BN);
  p.bs = g.block_size;
  // A tile holds up to 128 * MT rows of one expert (blocks of different experts cannot share an MMA);
  // the tiles are listed on the device from expert_ids, so none of them straddles two experts.
  p.blocks_per_tile = (128 * MT) / g.block_size;
  p.num_sorted = (int)g.num_sorted;
  const int64_t blocks = g.num_sorted / g.block_size;
  p.num_tiles = (int)blocks;  // upper bound; the device-side count is what the kernel walks
  p.num_experts = (int)E; p.top_k = g.top_k; p.mul_topk = g.mul_topk;
  const int srow_bytes = format_scale_is_byte(FMT) ? BN : BN * 2;
  p.raw_tx = L::RAW_W + p.rpc * srow_bytes * (format_has_zp(FMT) ? 2 : 1);
  if (p.num_tiles == 0) return 0;

  CUtensorMap tmW, tmA, tmS, tmZ;
  {
    // activation rows in sorted order live in the scratch buffer
    const int64_t rows_bytes = ((int64_t)g.num_sorted * K * 2 + 255) & ~(int64_t)255;
    const int64_t need = rows_bytes + (blocks + 64) * 4;
    if (g.scratch == nullptr || g.scratch_bytes < need) {
      set_error("moe scratch buffer too small: %lld bytes given, %lld needed", (long long)g.scratch_bytes, (long long)need);
      return MARLIN_B200_ESCRATCH;
    }
    const int64_t vecs = (int64_t)g.num_sorted * (K / 8);
    const int64_t want = (vecs + 255) / 256;
    const int gblocks = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
    moe_gather_rows_kernel<T><<<gblocks, 256, 0, g.stream>>>(reinterpret_cast<const T*>(g.a), reinterpret_cast<T*>(g.scratch),
                                                            g.sorted_ids, g.num_post_pad, (int)g.num_sorted, g.size_m,
                                                            g.top_k, (int)K);
    MB_CUDA(cudaGetLastError());
    int32_t* tile_count = reinterpret_cast<int32_t*>(reinterpret_cast<char*>(g.scratch) + rows_bytes);
    int32_t* tile_start = tile_count + 64;
    moe_tile_list_kernel<<<1, 1024, 0, g.stream>>>(g.expert_ids, g.num_post_pad, (int)g.num_sorted, g.block_size,
                                                   p.blocks_per_tile, (int)E, tile_start, tile_count);
    MB_CUDA(cudaGetLastError());
    p.tile_start = tile_start;
    p.tile_count = tile_count;
    count_launches(2);
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)g.num_sorted};
    const uint64_t strides[1] = {(uint64_t)K * 2};
    const uint32_t box[2] = {BK, 128 * MT};
    if (int rc = encode_tensor_map(&tmA, kHalf<T> ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                   g.scratch, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const int rows_per_kt = (BITS == 4 ? 16 : 32) * p.n_tiles;
    const uint64_t dims[3] = {32, (uint64_t)rows_per_kt, (uint64_t)(K / 16) * (uint64_t)E};
    const uint64_t strides[2] = {128, (uint64_t)rows_per_kt * 128};
    const uint32_t box[3] = {32, (uint32_t)(BITS == 4 ? 16 : 32), KT};
    if (int rc = cached_tensor_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, g.bq, dims, strides,
                            box, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const bool byte_scale = format_scale_is_byte(FMT);
    const uint64_t es = byte_scale ? 1 : 2;
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)g.num_groups * (uint64_t)E};
    const uint64_t strides[1] = {(uint64_t)N * es};
    const uint32_t box[2] = {BN, (uint32_t)p.rpc};
    const CUtensorMapDataType dt = byte_scale ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
    if (int rc = cached_tensor_map(&tmS, dt, 2, g.scales,
                            dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
    tmZ = tmS;
    if (format_has_zp(FMT)) {
      if (int rc = cached_tensor_map(&tmZ, dt, 2, g.zeros,
                              dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
        return rc;
    }
  }
  static bool attr_set[64] = {};
  int dev = 0;
  MB_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    MB_CUDA(cudaFuncSetAttribute(tc_moe_kernel<T, FMT, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    attr_set[dev] = true;
  }
  const int64_t work = (int64_t)p.num_tiles * p.n_tiles;
  const int grid = (int)(work < sm_count() ? work : sm_count());
  tc_moe_kernel<T, FMT, MT><<<grid, THREADS, SMEM, g.stream>>>(tmW, tmA, tmS, tmZ, p);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

template <typename T, int FMT>
int launch_moe_mt(const GemmArgs& g) {
  // 256-row tiles pay off once an expert's run of rows spans most of a tile: from about 192 routes per
  // expert on average; below that the second half of a tile would mostly multiply rows of other experts.
  const int64_t routes = g.size_m * g.top_k;
  if (routes / g.num_experts >= 192) return launch_moe<T, FMT, 2>(g);
  return launch_moe<T, FMT, 1>(g);
}

template <typename T>
int launch_moe_dtype(const GemmArgs& g) {
  switch (g.format) {
    case kU4B8: return launch_moe_mt<T, kU4B8>(g);
    case kU4: return launch_moe_mt<T, kU4>(g);
    case kU8B128: return launch_moe_mt<T, kU8B128>(g);
    case kU8: return launch_moe_mt<T, kU8>(g);
    case kFP8: return launch_moe_mt<T, kFP8>(g);
    case kNVFP4: return launch_moe_mt<T, kNVFP4>(g);
    case kMXFP4: return launch_moe_mt<T, kMXFP4>(g);
  }
  return 1;
}
}  // namespace

// Room for the fp32 partials of the k slices the dense kernel would like to use for this shape.
int64_t gemm_tc_scratch_bytes(int64_t m, int64_t n, int64_t k) {
  if (m <= 16 || n <= 0 || k <= 0) return 0;
  return tc_plan(m, n, k, INT64_MAX).scratch;
}

// Returns 1 when the problem is not one this kernel takes.
int launch_gemm_tc(const GemmArgs& g) {
  if (g.size_n % BN != 0 || g.size_k % 32 != 0) return 1;
  if (g.sorted_ids != nullptr) {
    if (g.num_groups > 1) {
      const int64_t gs = g.size_k / g.num_groups;
      if (!(gs == 16 || gs == 32 || gs % BK == 0)) return 1;
    }
    // experts are stacked along K in the tensor maps, so a K tail would read the next expert
    if (g.size_k % BK != 0 || (reinterpret_cast<uintptr_t>(g.a) & 15) != 0) return 1;
    if (g.act_dtype == MARLIN_B200_F16) return launch_moe_dtype<__half>(g);
    return launch_moe_dtype<__nv_bfloat16>(g);
  }
  if (g.size_m <= 0 || g.size_n % BN != 0 || g.size_k % 32 != 0) return 1;
  if (g.num_groups > 1) {
    const int64_t gs = g.size_k / g.num_groups;
    if (!(gs == 16 || gs == 32 || gs % BK == 0)) return 1;
  }
  if (g.act_dtype == MARLIN_B200_F16) return launch_dtype<__half>(g);
  return launch_dtype<__nv_bfloat16>(g);
}

// Reads (and optionally clears) the word a kernel of this file sets when one of its bounded waits gave up.
int read_tc_status(int* value, bool reset) {
  MB_CUDA(cudaMemcpyFromSymbol(value, g_tc_status, sizeof(int)));
  if (reset && *value != 0) {
    const int zero = 0;
    MB_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
  }
  return 0;
}


}  // namespace mb200
