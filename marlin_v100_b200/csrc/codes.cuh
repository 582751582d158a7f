// Register-level decoders for packed weight codes, shared by the tensor-memory GEMM kernel.
//
// All functions work on "k pairs": a 32-bit register holding the values of one column at two
// consecutive k as T x 2 (T = __half or __nv_bfloat16), which is the element order of a K-major
// operand tile.
#pragma once

#include "common.cuh"
#include "tma.cuh"

namespace mb200 {
namespace codes {

template <typename T> constexpr bool kHalf = false;
template <> constexpr bool kHalf<__half> = true;

// a - b as a fused multiply-add, a * 1 + (-b): the same result (one rounding), but issued to the FMA pipe.
// The packed 16-bit add / subtract was measured to occupy the half-rate ALU pipe that the shifts and logic
// operations of the decoders already fill.
template <typename T>
__device__ __forceinline__ uint32_t psub(uint32_t a, uint32_t b) {
  const uint32_t nb = b ^ 0x80008000u;
  if constexpr (kHalf<T>) {
    const uint32_t one = 0x3C003C00u;
    __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<const __half2*>(&one),
                        *reinterpret_cast<const __half2*>(&nb));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    const uint32_t one = 0x3F803F80u;
    __nv_bfloat162 r = __hfma2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&one),
                               *reinterpret_cast<const __nv_bfloat162*>(&nb));
    return *reinterpret_cast<uint32_t*>(&r);
  }
}
template <typename T>
__device__ __forceinline__ uint32_t pmul(uint32_t a, uint32_t b) {
  if constexpr (kHalf<T>) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
}
template <typename T>
__device__ __forceinline__ uint32_t pfma(uint32_t a, uint32_t b, uint32_t c) {
  if constexpr (kHalf<T>) {
    __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b),
                        *reinterpret_cast<__half2*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __nv_bfloat162 r = __hfma2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b),
                               *reinterpret_cast<__nv_bfloat162*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
  }
}

// 4-bit: z holds four codes of k0 in its low half and the same four columns at k1 in its high half;
// idx picks the code.  Integer formats return the exact integer value minus `zero` (8 for u4b8, 0 for
// u4).  e2m1 returns true * 2^-14 (fp16) / 2^-126 (bf16), exactly.
template <typename T, int FMT>
__device__ __forceinline__ uint32_t value4(uint32_t z, int idx) {
  if constexpr (FMT == kU4B8 || FMT == kU4) {
    constexpr uint32_t zero = (FMT == kU4B8) ? 8 : 0;
    if constexpr (kHalf<T>) {
      const uint32_t sh = (idx >= 2) ? (z >> 8) : z;
      if ((idx & 1) == 0) {
        constexpr uint32_t c = 0x6400u + zero;  // 1024 + zero
        return psub<T>((sh & 0x000f000fu) | 0x64006400u, c | (c << 16));
      } else {
        constexpr uint32_t c = 0x5400u + (zero << 4);  // 64 + zero
        return psub<T>((sh & 0x00f000f0u) | 0x54005400u, c | (c << 16));
      }
    } else {
      constexpr uint32_t c = 0x4300u + zero;  // 128 + zero
      return psub<T>(((z >> (4 * idx)) & 0x000f000fu) | 0x43004300u, c | (c << 16));
    }
  } else {
    const uint32_t t = z << (12 - 4 * idx);
    constexpr int sh = kHalf<T> ? 3 : 6;
    return ((t & 0x70007000u) >> sh) | (t & 0x80008000u);
  }
}

// 8-bit: y holds bytes [k0 code a, k1 code a, k0 code b, k1 code b]; which picks a (0) or b (1).
// Integer formats return the exact value minus `zero` (128 for u8b128); fp8 returns
// true * 2^-8 (fp16) / 2^-120 (bf16).
template <typename T, int FMT>
__device__ __forceinline__ uint32_t value8(uint32_t y, int which) {
  if constexpr (FMT == kU8B128 || FMT == kU8) {
    constexpr int zero = (FMT == kU8B128) ? 128 : 0;
    if constexpr (kHalf<T>) {
      constexpr uint32_t c = 0x6400u + zero;
      return psub<T>(prmt(y, 0x64646464u, which ? 0x4342u : 0x4140u), c | (c << 16));
    } else {
      const uint32_t f0 = prmt(y, 0x4B000000u, which ? 0x7442u : 0x7440u);
      const uint32_t f1 = prmt(y, 0x4B000000u, which ? 0x7443u : 0x7441u);
      __nv_bfloat162 r = __floats2bfloat162_rn(__uint_as_float(f0) - (8388608.f + zero),
                                               __uint_as_float(f1) - (8388608.f + zero));
      return *reinterpret_cast<uint32_t*>(&r);
    }
  } else {
    const uint32_t r = prmt(y, 0u, which ? 0x3424u : 0x1404u);
    constexpr int sh = kHalf<T> ? 1 : 4;
    return ((r & 0x7f007f00u) >> sh) | (r & 0x80008000u);
  }
}

// One byte of an fp4 block scale -> multiplier pair (T x 2, both halves equal).
// nvfp4: the byte is the high byte of an fp16 pattern shifted left by one (value = bits << 7).
// mxfp4: e8m0 exponent; the 2^14 / 2^126 left out by value4 for e2m1 is folded in.
template <typename T, int FMT>
__device__ __forceinline__ uint32_t fp4_scale_pair(uint32_t b) {
  if constexpr (FMT == kNVFP4) {
    if constexpr (kHalf<T>) return b * 0x00800080u;
    else return b ? (b * 0x00100010u + 0x38003800u) : 0u;
  } else {
    if constexpr (kHalf<T>) return (uint32_t)min(max((int)b - 98, 0), 30) * 0x04000400u;
    else return (uint32_t)min((int)b + 126, 254) * 0x00800080u;
  }
}

}  // namespace codes
}  // namespace mb200
