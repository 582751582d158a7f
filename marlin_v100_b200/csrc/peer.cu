// Multi-GPU steps of the Marlin path over peer-mapped memory (NVLink / NVSwitch): every rank owns one
// "arena" of device memory that all ranks of the node map (CUDA IPC), and the kernels here move data with
// plain loads and stores to peer addresses and order it with per-rank flags.  No multicast, no TMA and no
// library kernel ever touches a peer address.
//
//  * peer_allgather_kernel: the column-parallel dense layer.  Every rank stores its [M, N/world] slice into
//    every rank's gather buffer with the step number inside every stored unit, polls the units the other
//    ranks store into its own buffer and writes the assembled rows out.
//  * the expert-parallel layer, one step:
//      ep_plan_kernel      rows per destination rank from the sorted route list; the counts go to every
//                          rank's count table (signal A)
//      ep_dispatch_kernel  waits for all count rows (A); every route's hidden row, local expert id and router
//                          weight are stored straight into the owning rank's receive buffer at the position
//                          the count table implies (signal B); the row total goes to the host through a
//                          mapped word, so the host can size the expert GEMMs without a stream synchronise
//      ep_wait_kernel      (B) in front of the expert layer
//      ep_signal_kernel    (C) behind it
//      ep_combine_kernel   waits for all (C); every token reads its top-k contributions from the owning ranks'
//                          output buffers and sums them in fp32
//    The reference has no multi-GPU code; the hooks this stands on are its `expert_map` and independent
//    output columns (fused_marlin_moe.py:170-171, csrc/quantization/marlin/marlin.cu:356-359 there).
//
// Flags only grow: a step's epoch is the arena's step counter + 1, kept on the device so a captured graph
// can replay.  Every wait is bounded (two seconds of %globaltimer); a wait that gives up records its phase in
// the arena's status word and the kernel returns without touching the data it waited for.
#include <string.h>
#include <time.h>

#include "common.cuh"

namespace mb200 {
namespace {

constexpr int MAX_RANKS = 16;
constexpr unsigned long long WAIT_NS = 2000000000ull;

enum Phase : int { kGather = 0, kCounts = 1, kRows = 2, kOutputs = 3, kPhases = 4 };

struct PeerHeader {                                  // offset 0 of every arena
  unsigned int epoch;                                // steps completed by this rank
  unsigned int status;                               // 0, or 1 + phase of a wait that gave up; 16 = row capacity
  unsigned int done[4];                              // CTA arrival counters of the running kernel
  unsigned int pad[2];
  unsigned int flags[kPhases][MAX_RANKS];            // written by peers: flags[phase][source rank] = epoch
  int counts[2][MAX_RANKS][MAX_RANKS + 1];           // [epoch parity][source][destination | invalid routes]
  int seg_start[MAX_RANKS + 2];                      // this rank's sorted routes: first route per destination
};
static_assert(sizeof(PeerHeader) <= 4096, "header must fit the reserved page");

struct PeerTable {
  char* base[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint4 ld_cg(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ PeerHeader* header(const PeerTable& tab, int r) {
  return reinterpret_cast<PeerHeader*>(tab.base[r]);
}

// Called by every thread of a CTA.  Warp 0 polls this rank's flags of `phase` (lane = source rank) until all
// have reached `epoch`; false after WAIT_NS or when the arena already carries a status.
__device__ bool wait_phase(PeerHeader* me, int world, int phase, unsigned int epoch) {
  __shared__ int s_ok;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    bool ok = false;
    const unsigned long long t0 = global_ns();
    for (;;) {
      bool mine = true;
      if (lane < world) mine = (int)(ld_acquire_sys(&me->flags[phase][lane]) - epoch) >= 0;
      ok = __all_sync(0xffffffffu, mine);
      if (ok) break;
      if (global_ns() - t0 > WAIT_NS) break;
      __nanosleep(200);
    }
    if (lane == 0) {
      if (!ok) atomicCAS(&me->status, 0u, 1u + (unsigned)phase);
      s_ok = ok && (*(volatile unsigned int*)&me->status == 0u);
    }
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  __syncthreads();
  return ok;
}

// All threads call it after their stores to peers.  The last CTA to arrive raises this rank's flag of `phase`
// on every rank.
__device__ void signal_phase(const PeerTable& tab, int rank, int world, int phase, unsigned int epoch,
                             unsigned int* done) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done, 1u);
    if (prev == gridDim.x - 1) {
      *done = 0;
      __threadfence_system();
      for (int p = 0; p < world; ++p) st_release_sys(&header(tab, p)->flags[phase][rank], epoch);
    }
  }
}

// The last CTA through here closes the step.
__device__ void finish_step(PeerHeader* me, unsigned int epoch, unsigned int* done) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done, 1u);
    if (prev == gridDim.x - 1) {
      *done = 0;
      __threadfence();
      *(volatile unsigned int*)&me->epoch = epoch;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// dense column-parallel layer: all-gather of [M, N/world] slices
// ---------------------------------------------------------------------------------------------------------
// The slices are small (decode sizes), so the step is bound by latency, not by bytes: data and flag travel in
// the same store (every 16-byte unit is {4 data bytes, epoch, 4 data bytes, epoch}, each 8-byte half atomic on
// its own), the receiver polls the units themselves, and no fence, separate flag or arrival counter sits on
// the path.  Every thread issues all its stores before it polls, so no CTA waits for another CTA of its own
// grid.  gather buffers: arena + buf_off, [2 (epoch parity)][world][2 * vecs] of 16 bytes.
__device__ __forceinline__ uint4 ld_volatile(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__global__ void __launch_bounds__(256) peer_allgather_kernel(PeerTable tab, int rank, int world,
                                                             const uint4* __restrict__ src, int64_t vecs,
                                                             int64_t buf_off, uint4* __restrict__ out,
                                                             int64_t slice_rows) {
  PeerHeader* me = header(tab, rank);
  const unsigned int epoch = *(volatile unsigned int*)&me->epoch + 1;
  const int64_t par = epoch & 1;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // slice_rows > 0: the slices are [slice_rows, cols] row blocks and out is [slice_rows, world * cols]
  const int64_t row_vecs = slice_rows > 0 ? vecs / slice_rows : vecs;
  auto out_index = [&](int64_t r, int64_t v) {
    return slice_rows > 0 ? ((v / row_vecs) * world + r) * row_vecs + v % row_vecs : r * vecs + v;
  };
  for (int64_t idx = first; idx < vecs * world; idx += stride) {
    const int p = (int)(idx / vecs);
    const int64_t v = idx % vecs;
    const uint4 x = src[v];
    if (p == rank) {
      out[out_index(rank, v)] = x;
    } else {
      uint4* dst = reinterpret_cast<uint4*>(tab.base[p] + buf_off) + ((par * world + rank) * vecs + v) * 2;
      dst[0] = make_uint4(x.x, epoch, x.y, epoch);
      dst[1] = make_uint4(x.z, epoch, x.w, epoch);
    }
  }
  bool gave_up = (*(volatile unsigned int*)&me->status != 0u);
  const uint4* buf = reinterpret_cast<const uint4*>(tab.base[rank] + buf_off) + par * world * vecs * 2;
  for (int64_t idx = first; idx < vecs * world && !gave_up; idx += stride) {
    const int r = (int)(idx / vecs);
    const int64_t v = idx % vecs;
    if (r == rank) continue;
    const uint4* slot = buf + idx * 2;
    uint4 a = ld_volatile(slot), b = ld_volatile(slot + 1);
    unsigned long long t0 = 0;
    for (unsigned int spin = 0; a.y != epoch || a.w != epoch || b.y != epoch || b.w != epoch; ++spin) {
      if ((spin & 255u) == 255u) {
        const unsigned long long now = global_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > WAIT_NS) {
          atomicCAS(&me->status, 0u, 1u + (unsigned)kGather);
          gave_up = true;
          break;
        }
      }
      a = ld_volatile(slot);
      b = ld_volatile(slot + 1);
    }
    if (!gave_up) out[out_index(r, v)] = make_uint4(a.x, a.z, b.x, b.z);
  }
  finish_step(me, epoch, &me->done[1]);
}

// ---------------------------------------------------------------------------------------------------------
// expert-parallel layer
// ---------------------------------------------------------------------------------------------------------
struct EpLayout {          // arena offsets (bytes), the same on every rank
  int64_t rows;            // received hidden rows  [capacity][row_bytes]
  int64_t expert;          // int32 [capacity]: expert index on this rank
  int64_t weight;          // float [capacity]: router weight
  int64_t outputs;         // expert outputs        [capacity][row_bytes]
  int64_t capacity;        // rows
  int64_t row_bytes;       // multiple of 16
};

// destination rank of sorted route i from the segment starts (world + 1 entries, ascending)
__device__ __forceinline__ int dest_of(const int* seg, int world, int i) {
  int d = 0;
  while (d + 1 < world && i >= seg[d + 1]) ++d;
  return d;
}

// slot_sorted: slot (rank * experts_per_rank + index on the rank) of every sorted route, ascending; routes
// whose expert id was outside the table sit at the end as -1.
__global__ void __launch_bounds__(64) ep_plan_kernel(PeerTable tab, int rank, int world,
                                                     const int32_t* __restrict__ slot_sorted, int numel,
                                                     int experts_per_rank) {
  PeerHeader* me = header(tab, rank);
  const unsigned int epoch = *(volatile unsigned int*)&me->epoch + 1;
  const int par = epoch & 1;
  __shared__ int s_seg[MAX_RANKS + 2];
  const int d = threadIdx.x;
  if (d <= world) {
    // first route whose slot is >= d * experts_per_rank (d == world: the first invalid route)
    const int key = d * experts_per_rank;
    int lo = 0, hi = numel;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      const int s = slot_sorted[mid];
      if (s >= 0 && s < key) lo = mid + 1; else hi = mid;
    }
    s_seg[d] = lo;
    me->seg_start[d] = lo;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < world * (world + 1); i += blockDim.x) {
    const int p = i / (world + 1), c = i % (world + 1);
    const int value = c < world ? s_seg[c + 1] - s_seg[c] : numel - s_seg[world];
    header(tab, p)->counts[par][rank][c] = value;
  }
  signal_phase(tab, rank, world, kCounts, epoch, &me->done[0]);
}

// host_word (mapped host memory): [0] rows this rank receives, [1] invalid routes anywhere, [2] arena status,
// [3] epoch (written last)
__global__ void __launch_bounds__(512) ep_dispatch_kernel(PeerTable tab, int rank, int world, EpLayout lay,
                                                          const uint4* __restrict__ hidden,
                                                          const int32_t* __restrict__ order,
                                                          const int32_t* __restrict__ slot_sorted,
                                                          const float* __restrict__ topk_weights,
                                                          int32_t* __restrict__ position_of_route, int top_k,
                                                          int experts_per_rank, volatile int* host_word) {
  PeerHeader* me = header(tab, rank);
  const unsigned int epoch = *(volatile unsigned int*)&me->epoch + 1;
  const int par = epoch & 1;
  __shared__ int s_seg[MAX_RANKS + 2], s_base[MAX_RANKS];
  __shared__ int s_total, s_invalid;
  const bool ok = wait_phase(me, world, kCounts, epoch);
  if (ok) {
    if (threadIdx.x <= world) s_seg[threadIdx.x] = me->seg_start[threadIdx.x];
    if (threadIdx.x < world) {
      int base = 0;
      for (int s = 0; s < rank; ++s) base += me->counts[par][s][threadIdx.x];   // rows of lower ranks come first
      s_base[threadIdx.x] = base;
    }
    if (threadIdx.x == 32) {
      int total = 0, invalid = 0;
      for (int s = 0; s < world; ++s) {
        total += me->counts[par][s][rank];
        invalid += me->counts[par][s][world];
      }
      s_total = total;
      s_invalid = invalid;
      if (total > lay.capacity) atomicCAS(&me->status, 0u, 16u);
    }
  }
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    host_word[0] = ok ? s_total : 0;
    host_word[1] = ok ? s_invalid : 0;
    host_word[2] = (int)*(volatile unsigned int*)&me->status;
    __threadfence_system();
    host_word[3] = (int)epoch;
  }
  if (ok && s_total <= lay.capacity) {
    const int nvalid = s_seg[world];
    const int vec_per_row = (int)(lay.row_bytes / 16);
    const int warps = blockDim.x / 32, lane = threadIdx.x & 31;
    for (int i = blockIdx.x * warps + threadIdx.x / 32; i < nvalid; i += gridDim.x * warps) {
      const int d = dest_of(s_seg, world, i);
      const int64_t pos = s_base[d] + (i - s_seg[d]);
      const int route = order[i];
      if (pos >= lay.capacity) {   // the receiver's buffer is full: it reports the same condition itself
        if (lane == 0) atomicCAS(&me->status, 0u, 16u);
        continue;
      }
      const uint4* src = hidden + (int64_t)(route / top_k) * vec_per_row;
      uint4* dst = reinterpret_cast<uint4*>(tab.base[d] + lay.rows) + pos * vec_per_row;
      // all loads of a batch are issued before its first store: a row costs one trip to memory, not one per
      // 512 bytes (rows of up to 8 KiB in one batch)
      for (int v0 = 0; v0 < vec_per_row; v0 += 32 * 16) {
        uint4 buf[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int v = v0 + u * 32 + lane;
          if (v < vec_per_row) buf[u] = src[v];
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int v = v0 + u * 32 + lane;
          if (v < vec_per_row) dst[v] = buf[u];
        }
      }
      if (lane == 0) {
        reinterpret_cast<int32_t*>(tab.base[d] + lay.expert)[pos] = slot_sorted[i] % experts_per_rank;
        reinterpret_cast<float*>(tab.base[d] + lay.weight)[pos] = topk_weights[route];
        position_of_route[route] = i;
      }
    }
  }
  signal_phase(tab, rank, world, kRows, epoch, &me->done[1]);
}

__global__ void ep_wait_kernel(PeerTable tab, int rank, int world, int phase) {
  PeerHeader* me = header(tab, rank);
  const unsigned int epoch = *(volatile unsigned int*)&me->epoch + 1;
  wait_phase(me, world, phase, epoch);
}

__global__ void ep_signal_kernel(PeerTable tab, int rank, int world, int phase) {
  PeerHeader* me = header(tab, rank);
  const unsigned int epoch = *(volatile unsigned int*)&me->epoch + 1;
  signal_phase(tab, rank, world, phase, epoch, &me->done[2]);
}

// out[t] = sum over the token's routes of the owning rank's output row, fp32 accumulation in route order.
// skip != 0: only close the step (the host found invalid routes and raises).
template <typename T>
__global__ void __launch_bounds__(256) ep_combine_kernel(PeerTable tab, int rank, int world, EpLayout lay,
                                                         const int32_t* __restrict__ position_of_route,
                                                         int top_k, int64_t tokens, T* __restrict__ out, int skip) {
  PeerHeader* me = header(tab, rank);
  const unsigned int epoch = *(volatile unsigned int*)&me->epoch + 1;
  const int par = epoch & 1;
  __shared__ int s_seg[MAX_RANKS + 2], s_base[MAX_RANKS];
  __shared__ const uint4* s_row[32];
  const bool ok = wait_phase(me, world, kOutputs, epoch) && !skip;
  if (ok) {
    if (threadIdx.x <= world) s_seg[threadIdx.x] = me->seg_start[threadIdx.x];
    if (threadIdx.x < world) {
      int base = 0;
      for (int s = 0; s < rank; ++s) base += me->counts[par][s][threadIdx.x];
      s_base[threadIdx.x] = base;
    }
    __syncthreads();
    const int vec_per_row = (int)(lay.row_bytes / 16);
    for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
      if (threadIdx.x < top_k) {
        const int i = position_of_route[t * top_k + threadIdx.x];
        const int d = dest_of(s_seg, world, i);
        const int64_t pos = s_base[d] + (i - s_seg[d]);
        s_row[threadIdx.x] = reinterpret_cast<const uint4*>(tab.base[d] + lay.outputs) + pos * vec_per_row;
      }
      __syncthreads();
      for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
        float acc[8] = {};
        // the loads of up to eight routes are in flight together (peer loads cost microseconds each); the adds
        // keep the route order
        for (int j0 = 0; j0 < top_k; j0 += 8) {
          uint4 x4[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (j0 + u < top_k) x4[u] = ld_cg(s_row[j0 + u] + v);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (j0 + u < top_k) {
              const T* xp = reinterpret_cast<const T*>(&x4[u]);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[e] += to_float<T>(xp[e]);
            }
          }
        }
        uint4 o4;
        T* op = reinterpret_cast<T*>(&o4);
#pragma unroll
        for (int e = 0; e < 8; ++e) op[e] = from_float<T>(acc[e]);
        reinterpret_cast<uint4*>(out)[t * vec_per_row + v] = o4;
      }
      __syncthreads();
    }
  }
  finish_step(me, epoch, &me->done[3]);
}

int fill_table(PeerTable& tab, const void* const* bases, int rank, int world) {
  MB_CHECK(world >= 1 && world <= MAX_RANKS, "world size %d out of range (1..%d)", world, MAX_RANKS);
  MB_CHECK(rank >= 0 && rank < world, "rank %d outside the world of %d", rank, world);
  MB_CHECK(bases != nullptr, "null arena table");
  for (int r = 0; r < world; ++r) {
    MB_CHECK(bases[r] != nullptr && ((uintptr_t)bases[r] & 255) == 0, "arena %d is null or not 256-byte aligned", r);
    tab.base[r] = (char*)bases[r];
  }
  return 0;
}

int fill_layout(EpLayout& lay, const int64_t* layout) {
  MB_CHECK(layout != nullptr, "null layout");
  lay.rows = layout[0]; lay.expert = layout[1]; lay.weight = layout[2]; lay.outputs = layout[3];
  lay.capacity = layout[4]; lay.row_bytes = layout[5];
  MB_CHECK(lay.row_bytes > 0 && lay.row_bytes % 16 == 0, "row size must be a positive multiple of 16 bytes");
  MB_CHECK(lay.rows >= 4096 && lay.rows % 256 == 0 && lay.outputs % 256 == 0 && lay.expert % 256 == 0 &&
               lay.weight % 256 == 0, "arena offsets must be multiples of 256 bytes behind the 4096-byte header");
  MB_CHECK(lay.capacity > 0, "row capacity must be positive");
  return 0;
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" int marlin_b200_peer_header_bytes() { return 4096; }

extern "C" int marlin_b200_peer_alloc(int64_t bytes, void** ptr) {
  MB_CHECK(bytes >= 4096 && ptr != nullptr, "an arena needs at least its 4096-byte header");
  MB_CUDA(cudaMalloc(ptr, (size_t)bytes));
  MB_CUDA(cudaMemset(*ptr, 0, (size_t)bytes));
  MB_CUDA(cudaDeviceSynchronize());
  return 0;
}

extern "C" int marlin_b200_peer_free(void* ptr) {
  if (ptr != nullptr) MB_CUDA(cudaFree(ptr));
  return 0;
}

extern "C" int marlin_b200_peer_export(void* ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  MB_CHECK(ptr != nullptr && handle64 != nullptr, "null pointer");
  MB_CUDA(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64), ptr));
  return 0;
}

extern "C" int marlin_b200_peer_open(const void* handle64, void** ptr) {
  MB_CHECK(ptr != nullptr && handle64 != nullptr, "null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  MB_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}

extern "C" int marlin_b200_peer_close(void* ptr) {
  if (ptr != nullptr) MB_CUDA(cudaIpcCloseMemHandle(ptr));
  return 0;
}

extern "C" int marlin_b200_peer_host_word_alloc(void** host_ptr, void** device_ptr) {
  MB_CHECK(host_ptr != nullptr && device_ptr != nullptr, "null pointer");
  MB_CUDA(cudaHostAlloc(host_ptr, 64, cudaHostAllocMapped));
  memset(*host_ptr, 0, 64);
  MB_CUDA(cudaHostGetDevicePointer(device_ptr, *host_ptr, 0));
  return 0;
}

extern "C" int marlin_b200_peer_host_word_free(void* host_ptr) {
  if (host_ptr != nullptr) MB_CUDA(cudaFreeHost(host_ptr));
  return 0;
}

extern "C" int marlin_b200_peer_status(const void* arena, int* status, int* epoch) {
  MB_CHECK(arena != nullptr && status != nullptr && epoch != nullptr, "null pointer");
  PeerHeader h;
  MB_CUDA(cudaMemcpy(&h, arena, sizeof(unsigned int) * 2, cudaMemcpyDeviceToHost));
  *status = (int)h.status;
  *epoch = (int)h.epoch;
  return 0;
}

extern "C" int marlin_b200_peer_allgather(const void* const* arenas, int rank, int world, const void* src,
                                          int64_t bytes_per_rank, int64_t buffer_offset, void* out,
                                          int64_t slice_rows, void* stream) {
  PeerTable tab;
  if (int rc = fill_table(tab, arenas, rank, world)) return rc;
  MB_CHECK(bytes_per_rank > 0 && bytes_per_rank % 16 == 0, "slice size must be a positive multiple of 16 bytes");
  MB_CHECK(buffer_offset >= 4096 && buffer_offset % 256 == 0, "gather buffers start behind the 4096-byte header");
  MB_CHECK(src != nullptr && out != nullptr && ((uintptr_t)src & 15) == 0 && ((uintptr_t)out & 15) == 0,
           "source and output must be 16-byte aligned");
  const int64_t vecs = bytes_per_rank / 16;
  MB_CHECK(slice_rows >= 0 && (slice_rows == 0 || vecs % slice_rows == 0),
           "a slice of %lld bytes does not split into %lld rows of whole 16-byte units", (long long)bytes_per_rank,
           (long long)slice_rows);
  const int64_t want = (vecs * world + 255) / 256, cap = (int64_t)sm_count() * 4;
  const int grid = (int)(want < cap ? (want > 0 ? want : 1) : cap);
  peer_allgather_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(tab, rank, world, (const uint4*)src, vecs,
                                                                buffer_offset, (uint4*)out, slice_rows);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

extern "C" int marlin_b200_ep_plan(const void* const* arenas, int rank, int world, const int32_t* slot_sorted,
                                   int64_t numel, int experts_per_rank, void* stream) {
  PeerTable tab;
  if (int rc = fill_table(tab, arenas, rank, world)) return rc;
  MB_CHECK(numel >= 0 && numel < (1ll << 31) && experts_per_rank > 0, "route count or experts per rank out of range");
  MB_CHECK(slot_sorted != nullptr || numel == 0, "null slot list");
  ep_plan_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(tab, rank, world, slot_sorted, (int)numel, experts_per_rank);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

extern "C" int marlin_b200_ep_dispatch(const void* const* arenas, int rank, int world, const int64_t* layout,
                                       const void* hidden, const int32_t* order, const int32_t* slot_sorted,
                                       const float* topk_weights, int32_t* position_of_route, int top_k,
                                       int experts_per_rank, void* host_word_device, void* stream) {
  PeerTable tab;
  EpLayout lay;
  if (int rc = fill_table(tab, arenas, rank, world)) return rc;
  if (int rc = fill_layout(lay, layout)) return rc;
  MB_CHECK(top_k >= 1 && top_k <= 32 && experts_per_rank > 0, "top_k or experts per rank out of range");
  MB_CHECK(host_word_device != nullptr && position_of_route != nullptr, "null pointer");
  MB_CHECK(((uintptr_t)hidden & 15) == 0, "hidden must be 16-byte aligned");
  ep_dispatch_kernel<<<sm_count(), 512, 0, (cudaStream_t)stream>>>(
      tab, rank, world, lay, (const uint4*)hidden, order, slot_sorted, topk_weights, position_of_route, top_k,
      experts_per_rank, (volatile int*)host_word_device);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

// Host side of the dispatch: spins on the mapped word until the dispatch kernel of step `epoch` has written
// the row total.  Returns EINVAL with a message after `timeout_ms`.
extern "C" int marlin_b200_ep_poll_rows(const void* host_word, int epoch, int timeout_ms, int64_t* rows,
                                        int* invalid_routes, int* status) {
  MB_CHECK(host_word != nullptr && rows != nullptr && invalid_routes != nullptr && status != nullptr, "null pointer");
  volatile const int* w = reinterpret_cast<volatile const int*>(host_word);
  timespec t0, t1;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  for (unsigned spin = 0;; ++spin) {
    if (w[3] == epoch) break;
    if ((spin & 1023) == 1023) {
      clock_gettime(CLOCK_MONOTONIC, &t1);
      const double ms = (t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6;
      MB_CHECK(ms < timeout_ms, "expert-parallel dispatch of step %d did not report within %d ms (last step seen %d)",
               epoch, timeout_ms, (int)w[3]);
    }
  }
  __sync_synchronize();
  *rows = w[0];
  *invalid_routes = w[1];
  *status = w[2];
  return 0;
}

extern "C" int marlin_b200_ep_wait(const void* const* arenas, int rank, int world, int phase, void* stream) {
  PeerTable tab;
  if (int rc = fill_table(tab, arenas, rank, world)) return rc;
  MB_CHECK(phase >= 0 && phase < kPhases, "phase %d out of range", phase);
  ep_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(tab, rank, world, phase);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

extern "C" int marlin_b200_ep_signal(const void* const* arenas, int rank, int world, int phase, void* stream) {
  PeerTable tab;
  if (int rc = fill_table(tab, arenas, rank, world)) return rc;
  MB_CHECK(phase >= 0 && phase < kPhases, "phase %d out of range", phase);
  ep_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(tab, rank, world, phase);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

extern "C" int marlin_b200_ep_combine(const void* const* arenas, int rank, int world, const int64_t* layout,
                                      const int32_t* position_of_route, int top_k, int64_t tokens, void* out,
                                      int act_dtype, int skip, void* stream) {
  PeerTable tab;
  EpLayout lay;
  if (int rc = fill_table(tab, arenas, rank, world)) return rc;
  if (int rc = fill_layout(lay, layout)) return rc;
  MB_CHECK(top_k >= 1 && top_k <= 32 && tokens >= 0, "top_k or token count out of range");
  MB_CHECK(act_dtype == MARLIN_B200_F16 || act_dtype == MARLIN_B200_BF16, "activation dtype must be fp16 or bf16");
  // every CTA waits for the other ranks: the grid stays within one wave
  const int64_t cap = (int64_t)sm_count() * 4;
  const int grid = (int)(tokens < cap ? (tokens > 0 ? tokens : 1) : cap);
  auto s = (cudaStream_t)stream;
  if (act_dtype == MARLIN_B200_F16)
    ep_combine_kernel<__half><<<grid, 256, 0, s>>>(tab, rank, world, lay, position_of_route, top_k, tokens,
                                                   (__half*)out, skip);
  else
    ep_combine_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(tab, rank, world, lay, position_of_route, top_k, tokens,
                                                          (__nv_bfloat16*)out, skip);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}
