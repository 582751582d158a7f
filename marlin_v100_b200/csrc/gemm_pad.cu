// Dense GEMM for size_n % 256 != 0 (size_n % 64 == 0) through the tensor-core kernels.
//
// The reference's packed layout interleaves the 64-column tiles of a 256-, 128- or 64-column group word by word
// (common.cuh: macro_n_of), so a matrix whose N is not a multiple of 256 is laid out differently from one whose N
// is, and the fast kernels only read the 256-column form.  This path copies the operands once per call into the
// 256-column form of a matrix with N' = N rounded up to 256 columns (a pure permutation of packed words; the
// padding columns get zero codes, zero scales, zero zero-points and zero bias), runs the regular selector on that
// matrix with a [M, N'] output in scratch, and copies the first N columns of every row back.  It costs one extra
// read and write of the weights per call, which the GEMM kernels win back many times over against the CUDA-core
// kernel that served these shapes before (reference shapes: the alignment matrix of
// tests/writeback_marlin_cases.py, N = 192 ... 1152, and column shards such as 25600 / 8 = 3200).
// Everything lives in the caller's scratch buffer; with a buffer that is too small the shape-agnostic kernel is
// used as before.
#include "common.cuh"

namespace mb200 {
namespace {

constexpr int64_t kAlign = 1024;
int64_t align_up(int64_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

// one thread per packed word of the padded matrix
template <int BITS>
__global__ void __launch_bounds__(256) pad_weights_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst,
                                                          int64_t rows, int n, int n_pad, int g_src) {
  constexpr int pf = 32 / BITS;
  constexpr int W = 1024 / pf;          // words of a 64-column tile in one packed row
  const int64_t row_len_dst = (int64_t)n_pad * 16 / pf, row_len_src = (int64_t)n * 16 / pf;
  const int64_t total = rows * row_len_dst;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = idx / row_len_dst;
    const int col = (int)(idx - row * row_len_dst);
    // 256-column form: col = grp * 4 W + (lk * (64 / pf) + nv) * 4 + sub
    const int grp = col / (4 * W), rem = col % (4 * W);
    const int sub = rem & 3, t = rem >> 2;
    const int lk = t / (64 / pf), nv = t % (64 / pf);
    const int n0 = grp * 256 + sub * 64 + nv * pf;   // first of the pf columns the word holds
    uint32_t w = 0;
    if (n0 < n) w = src[row * row_len_src + packed_col<BITS>(lk, n0, g_src)];
    dst[idx] = w;
  }
}

// rows of `elem` bytes per column: [rows, n] -> [rows, n_pad], zero behind column n
__global__ void __launch_bounds__(256) pad_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                       int64_t rows, int64_t row_bytes, int64_t row_bytes_pad) {
  const int64_t total = rows * row_bytes_pad;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / row_bytes_pad, b = idx - r * row_bytes_pad;
    dst[idx] = (b < row_bytes) ? src[r * row_bytes + b] : (uint8_t)0;
  }
}

// C[m, 0 .. n) = C'[m, 0 .. n), 16-bit elements, eight at a time (n % 64 == 0, both bases 16-byte aligned)
__global__ void __launch_bounds__(256) unpad_output_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                           int64_t m, int n, int n_pad) {
  const int v = n / 8, v_pad = n_pad / 8;
  const int64_t total = m * v;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / v;
    const int c = (int)(idx - r * v);
    dst[idx] = src[r * v_pad + c];
  }
}

int grid_for(int64_t items) {
  const int64_t blocks = (items + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

struct PadPlan {
  int64_t n_pad, w_bytes, s_bytes, z_bytes, b_bytes, c_bytes, total;
};

PadPlan plan_of(int64_t m, int64_t n, int64_t k, int format, int64_t num_groups, bool has_zeros, bool has_bias) {
  PadPlan p{};
  p.n_pad = (n + 255) / 256 * 256;
  const int selem = format_scale_is_byte(format) ? 1 : 2;
  p.w_bytes = align_up(k * p.n_pad * format_bits(format) / 8);
  p.s_bytes = align_up(num_groups * p.n_pad * selem);
  p.z_bytes = has_zeros ? p.s_bytes : 0;
  p.b_bytes = has_bias ? align_up(p.n_pad * 2) : 0;
  p.c_bytes = align_up(m * p.n_pad * 2);
  p.total = p.w_bytes + p.s_bytes + p.z_bytes + p.b_bytes + p.c_bytes;
  return p;
}

}  // namespace

bool gemm_pad_applies(const GemmArgs& g) {
  return g.sorted_ids == nullptr && !g.prepared && g.size_n % 256 != 0 && g.size_n % 64 == 0 && g.size_k % 64 == 0 &&
         g.size_m > 0;
}

// scratch for the padded operands, the padded output and the kernels that then run on N' columns (`inner` bytes);
// scale rows are bounded by one per 16 k, the finest group any format has
int64_t gemm_pad_scratch_bytes(int64_t m, int64_t n, int64_t k, int format, int64_t inner) {
  const PadPlan p = plan_of(m, n, k, format, k / 16 > 0 ? k / 16 : 1, true, true);
  return p.total + align_up(inner);
}

// Fills `out` with the arguments of the padded problem and enqueues the copies; returns 1 when the scratch
// buffer cannot hold it (the caller then keeps the shape-agnostic kernel).
int gemm_pad_prepare(const GemmArgs& g, GemmArgs* out) {
  const PadPlan p = plan_of(g.size_m, g.size_n, g.size_k, g.format, g.num_groups, g.zeros != nullptr, g.bias != nullptr);
  if (g.scratch == nullptr || ((uintptr_t)g.scratch & 255) != 0 || g.scratch_bytes < p.total) return 1;
  uint8_t* base = reinterpret_cast<uint8_t*>(g.scratch);
  uint8_t* w = base;
  uint8_t* s = w + p.w_bytes;
  uint8_t* z = s + p.s_bytes;
  uint8_t* b = z + p.z_bytes;
  uint8_t* c = b + p.b_bytes;
  uint8_t* inner = c + p.c_bytes;
  const int n = (int)g.size_n, n_pad = (int)p.n_pad;
  const int g_src = macro_n_of(g.size_n) / 64;
  const int64_t rows = g.size_k / 16;
  const int bits = format_bits(g.format);
  {
    const int64_t words = rows * ((int64_t)n_pad * 16 / (32 / bits));
    if (bits == 4)
      pad_weights_kernel<4><<<grid_for(words), 256, 0, g.stream>>>(reinterpret_cast<const uint32_t*>(g.bq),
                                                                    reinterpret_cast<uint32_t*>(w), rows, n, n_pad, g_src);
    else
      pad_weights_kernel<8><<<grid_for(words), 256, 0, g.stream>>>(reinterpret_cast<const uint32_t*>(g.bq),
                                                                    reinterpret_cast<uint32_t*>(w), rows, n, n_pad, g_src);
    MB_CUDA(cudaGetLastError());
    count_launches(1);
  }
  const int selem = format_scale_is_byte(g.format) ? 1 : 2;
  {
    const int64_t bytes = g.num_groups * (int64_t)n_pad * selem;
    pad_rows_kernel<<<grid_for(bytes), 256, 0, g.stream>>>(reinterpret_cast<const uint8_t*>(g.scales), s, g.num_groups,
                                                           (int64_t)n * selem, (int64_t)n_pad * selem);
    MB_CUDA(cudaGetLastError());
    count_launches(1);
    if (g.zeros != nullptr) {
      pad_rows_kernel<<<grid_for(bytes), 256, 0, g.stream>>>(reinterpret_cast<const uint8_t*>(g.zeros), z, g.num_groups,
                                                             (int64_t)n * selem, (int64_t)n_pad * selem);
      MB_CUDA(cudaGetLastError());
      count_launches(1);
    }
  }
  if (g.bias != nullptr) {
    pad_rows_kernel<<<grid_for((int64_t)n_pad * 2), 256, 0, g.stream>>>(reinterpret_cast<const uint8_t*>(g.bias), b, 1,
                                                                        (int64_t)n * 2, (int64_t)n_pad * 2);
    MB_CUDA(cudaGetLastError());
    count_launches(1);
  }
  *out = g;
  out->bq = reinterpret_cast<const int32_t*>(w);
  out->scales = s;
  out->zeros = (g.zeros != nullptr) ? z : nullptr;
  out->bias = (g.bias != nullptr) ? b : nullptr;
  out->c = c;
  out->size_n = p.n_pad;
  out->scratch = inner;
  out->scratch_bytes = g.scratch_bytes - p.total;
  if (out->scratch_bytes <= 0) {
    out->scratch = nullptr;
    out->scratch_bytes = 0;
  }
  return 0;
}

// copies the first size_n columns of the padded output back into the caller's C
int gemm_pad_finish(const GemmArgs& g, const GemmArgs& padded) {
  const int64_t vecs = g.size_m * (g.size_n / 8);
  unpad_output_kernel<<<grid_for(vecs), 256, 0, g.stream>>>(reinterpret_cast<const uint4*>(padded.c),
                                                            reinterpret_cast<uint4*>(g.c), g.size_m, (int)g.size_n,
                                                            (int)padded.size_n);
  MB_CUDA(cudaGetLastError());
  count_launches(1);
  return 0;
}

}  // namespace mb200
