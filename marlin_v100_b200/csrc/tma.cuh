// Thin wrappers over the sm_100a TMA / mbarrier PTX used by the GEMM kernels, plus host-side
// tensor-map encoding through the driver entry point (no link-time dependency on libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb200 {

// ---- host: tensor maps ---------------------------------------------------------------------------
// Encodes a tiled tensor map.  dims/box are innermost first; strides (bytes) has rank-1 entries for
// dims 1.. .  Returns 0 on success (sets the library error otherwise).
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                      CUtensorMapSwizzle swizzle);

// Same, through a process-wide cache keyed by (base pointer, element type, rank, dims, strides, box,
// swizzle): encoding a map costs a few microseconds of host time, weights and scales are encoded once.
int cached_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                      CUtensorMapSwizzle swizzle);

#ifdef __CUDACC__
// ---- device --------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// (A suspend-time hint on try_wait and a nanosleep between polls were both measured on the decode
// kernel: the first cost 10 %, the second changed nothing.)
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: polls the barrier; every 256 polls it looks at the CTA's abort flag (set by whoever
// gave up first) and at the clock, and gives up after about two seconds.  Returns false on give-up
// so the caller can record an error and run to the end without touching the data.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (global_timer_ns() - t0 > 2000000000ull) {
      *abort_flag = 1;
      return false;
    }
  }
}

// The same bounded wait for warps that expect to wait long (an epilogue waiting for a whole run of chunks, a
// producer or MMA issuer that is ahead of the other warps): between polls the warp sleeps `ns` nanoseconds,
// so it does not take issue slots from the warps that do the arithmetic.
__device__ __forceinline__ bool mbar_wait_sleep(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      __nanosleep(ns);
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag != 0) return false;
    if (global_timer_ns() - t0 > 2000000000ull) {
      *abort_flag = 1;
      return false;
    }
  }
}

// Bounded wait that lets the hardware park the thread: try_wait with a suspend-time hint returns when the phase
// completes or when the hint (nanoseconds) runs out, and a parked thread takes no issue slots.  For waits that
// are expected to last from a fraction of a microsecond to many microseconds.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_park(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t hint_ns) {
  if (mbar_try_wait_hint(bar, parity, hint_ns)) return true;
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait_hint(bar, parity, hint_ns)) return true;
    if (*abort_flag != 0) return false;
    if (global_timer_ns() - t0 > 2000000000ull) {
      *abort_flag = 1;
      return false;
    }
  }
}

// For the give-up path of a producer thread: a CTA must not exit while copies into its shared memory are in
// flight.  Waits (bounded by about 50 ms, not by the abort flag, which is set by then) until the copy issued last
// into every stage of a ring has landed: `issued` copies went to stages 0, 1, ... round robin, and `bar_of(s)` is the
// barrier a copy into stage s completes on.  In a run without a give-up every copy has been consumed before the
// kernel ends, and a producer that finished its loop long before a give-up has nothing in flight either (a wait
// gives up after two seconds), so callers use this when they leave their loop with the abort flag up.
template <class BarOf>
__device__ __forceinline__ void drain_copies(BarOf bar_of, int stages, int issued) {
  const uint64_t t0 = global_timer_ns();
  for (int j = (issued > stages) ? issued - stages : 0; j < issued; ++j) {
    const uint32_t bar = bar_of(j % stages), parity = (uint32_t)((j / stages) & 1);
#pragma unroll 1
    while (!mbar_try_wait_hint(bar, parity, 1000)) {
      if (global_timer_ns() - t0 > 50000000ull) return;
    }
  }
}
// The same for one barrier (an MMA issuer's own tcgen05.commit before the tensor memory is freed).
__device__ __forceinline__ void drain_barrier(uint32_t bar, uint32_t parity) {
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  while (!mbar_try_wait_hint(bar, parity, 1000)) {
    if (global_timer_ns() - t0 > 50000000ull) return;
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
#endif  // __CUDACC__

}  // namespace mb200
