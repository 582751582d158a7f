// C ABI entry points of the GEMM paths: argument checks (the conditions the reference enforces with
// TORCH_CHECK in marlin.cu / ops.cu, restated for raw pointers) and kernel selection.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "stream_layout.cuh"

namespace mb200 {

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

namespace {
std::atomic<int64_t> g_launches{0};
}
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace {

// ScalarType id: exponent(8) | mantissa(8) | signed(1) | bias(32) | finite_only(1) | nan_repr(8)
constexpr int64_t type_id(int64_t e, int64_t m, int64_t s, int64_t bias, int64_t fin, int64_t nan) {
  return e | (m << 8) | (s << 16) | (bias << 17) | (fin << 49) | (nan << 50);
}
constexpr int64_t kIdU4 = type_id(0, 4, 0, 0, 0, 1);
constexpr int64_t kIdU4B8 = type_id(0, 4, 0, 8, 0, 1);
constexpr int64_t kIdU8 = type_id(0, 8, 0, 0, 0, 1);
constexpr int64_t kIdU8B128 = type_id(0, 8, 0, 128, 0, 1);
constexpr int64_t kIdFE2M1 = type_id(2, 1, 1, 0, 1, 0);
constexpr int64_t kIdFE4M3 = type_id(4, 3, 1, 0, 1, 2);

int check_common(const GemmArgs& g) {
  MB_CHECK(g.act_dtype == MARLIN_B200_F16 || g.act_dtype == MARLIN_B200_BF16,
           "unsupported `a` scalar_type (code %d): float16 or bfloat16 expected", g.act_dtype);
  MB_CHECK(g.format >= kU4B8 && g.format <= kMXFP4,
           "Marlin currently implements only uint4, uint4b8, uint8, uint8b128, fp8_e4m3fn, nvfp4, "
           "and mxfp4 weights (format code %d)", g.format);
  MB_CHECK(g.size_m >= 0 && g.size_n >= 0 && g.size_k >= 0, "negative problem size");
  MB_CHECK(g.size_k % 16 == 0, "size_k = %lld is not divisible by tile_size = 16", (long long)g.size_k);
  MB_CHECK(g.size_n % 64 == 0, "Marlin requires size_n % 64 == 0. size_n = %lld, min_thread_n = 64",
           (long long)g.size_n);
  MB_CHECK(g.size_k % 32 == 0, "Marlin requires size_k % 32 == 0. size_k = %lld", (long long)g.size_k);
  MB_CHECK(g.num_groups >= 1, "b_scales has no rows");
  MB_CHECK(g.size_k % g.num_groups == 0, "size_k = %lld, is not divisible by b_scales.size(0) = %lld",
           (long long)g.size_k, (long long)g.num_groups);
  const int64_t group_size = g.num_groups > 1 ? g.size_k / g.num_groups : -1;
  const bool has_zp = g.zeros != nullptr;
  MB_CHECK(!has_zp || format_has_zp(g.format),
           "Marlin does not support zero-point metadata for this quant type.");
  if (format_has_zp(g.format))
    MB_CHECK(has_zp, "Marlin uint4/uint8 path requires float zero points (b_zeros = zero_point * scale).");
  if (g.format == kFP8)
    MB_CHECK(group_size == -1 || group_size == 128,
             "Marlin fp8_e4m3 supports only group_size -1 or 128. Got %lld", (long long)group_size);
  if (g.format == kNVFP4) {
    MB_CHECK(g.global_scale != nullptr, "the global_scale parameter must be passed for nvfp4 format.");
    MB_CHECK(group_size == 16, "Marlin nvfp4 supports only group_size 16. Got %lld", (long long)group_size);
  } else {
    MB_CHECK(g.global_scale == nullptr, "Marlin supports global_scale only for nvfp4 format.");
  }
  if (g.format == kMXFP4)
    MB_CHECK(group_size == 32,
             "Marlin mxfp4 supports only group_size 32 when global_scale is not provided. Got %lld",
             (long long)group_size);
  if (g.size_m > 0 && g.size_n > 0) {
    MB_CHECK(g.a != nullptr && g.c != nullptr && g.bq != nullptr && g.scales != nullptr,
             "null tensor pointer");
    MB_CHECK(((uintptr_t)g.a) % 16 == 0, "A must aligned to 16 bytes");
    MB_CHECK(((uintptr_t)g.c) % 16 == 0, "C must aligned to 16 bytes");
    MB_CHECK(((uintptr_t)g.bq) % 16 == 0, "b_q_weight must aligned to 16 bytes");
  }
  return 0;
}

int dispatch(const GemmArgs& g) {
  if (g.size_m == 0 || g.size_n == 0) return 0;
  if (g.size_k == 0) {
    set_error("size_k must be positive");
    return MARLIN_B200_EINVAL;
  }
  if (g.prepared) {
    // weights in the streaming layout: one kernel family for every size_m
    MB_CHECK(stream::layout_accepts(g.size_k, g.size_n),
             "weights in the streaming layout need size_k %% 128 == 0 and size_n %% 256 == 0");
    if (gemm_stream_i8_accepts(g)) return launch_gemm_stream_i8(g);
    return g.act_dtype == MARLIN_B200_F16 ? launch_gemm_stream_f16(g) : launch_gemm_stream_bf16(g);
  }
  // size_n % 256 != 0: the same kernels on a copy padded to the next multiple of 256 columns, when the scratch
  // buffer holds it
  if (gemm_pad_applies(g) && g.scratch != nullptr &&
      g.scratch_bytes >= marlin_b200_gemm_scratch_bytes(g.size_m, g.size_n, g.size_k, g.format)) {
    GemmArgs padded;
    int rc = gemm_pad_prepare(g, &padded);
    if (rc < 0) return rc;
    if (rc == 0) {
      rc = dispatch(padded);
      if (rc != 0) return rc;
      return gemm_pad_finish(g, padded);
    }
  }
  // M <= 16: weight-streaming kernel.  Larger M: tensor-memory kernel; shapes it does not take fall
  // back to passes of the streaming kernel, and anything else to the shape-agnostic kernel.
  if (g.size_m > 16) {
    const int rc = launch_gemm_tc(g);
    if (rc <= 0) return rc;  // handled (0) or failed (<0)
  }
  // Integer-MMA decode kernel (4-bit integer formats, weights through tensor memory): measured ahead of
  // the register-fragment kernel only for 9-16 rows on large matrices (54 vs 57 us at K = 8192,
  // N = 28672), behind it for fewer rows and for small matrices, where its two helper launches weigh.
  if (g.size_m > 8 && g.size_m <= 16 && g.size_k * g.size_n >= (1ll << 27)) {
    const int rc = launch_gemm_decode_tc(g);
    if (rc <= 0) return rc;
  }
  const int rc = launch_gemm_decode(g);
  if (rc <= 0) return rc;
  return launch_gemm_generic(g);
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" const char* marlin_b200_last_error(void) { return g_error; }
extern "C" const char* marlin_b200_version(void) { return "0.1"; }
extern "C" int64_t marlin_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int marlin_b200_kernel_status(int* status, int reset) {
  MB_CHECK(status != nullptr, "null status pointer");
  int a = 0, b = 0, c = 0, d = 0, e = 0;
  if (int rc = read_decode_status(&a, reset != 0)) return rc;
  if (int rc = read_tc_status(&b, reset != 0)) return rc;
  if (int rc = read_decode_tc_status(&c, reset != 0)) return rc;
  if (int rc = read_stream_status_f16(&d, reset != 0)) return rc;
  if (int rc = read_stream_status_bf16(&e, reset != 0)) return rc;
  if (d == 0) d = e;
  if (d == 0) {
    if (int rc = read_stream_i8_status(&d, reset != 0)) return rc;
    if (d != 0) d |= 0x80;
  }
  *status = (a & 0xff) | ((b & 0xff) << 8) | ((c & 0xff) << 16) | ((d & 0xff) << 24);
  return 0;
}

extern "C" int marlin_b200_format_from_type_id(int64_t id, int scale_kind) {
  if (id == kIdU4B8) return kU4B8;
  if (id == kIdU4) return kU4;
  if (id == kIdU8B128) return kU8B128;
  if (id == kIdU8) return kU8;
  if (id == kIdFE4M3) return kFP8;
  if (id == kIdFE2M1) {
    if (scale_kind == MARLIN_B200_SCALE_E4M3) return kNVFP4;
    if (scale_kind == MARLIN_B200_SCALE_E8M0) return kMXFP4;
  }
  return -1;
}

extern "C" int64_t marlin_b200_gemm_scratch_bytes(int64_t size_m, int64_t size_n, int64_t size_k,
                                                  int format) {
  if (format & MARLIN_B200_FMT_PREPARED) {
    const int64_t a = gemm_stream_scratch_bytes(size_m, size_n, size_k);
    const int f = format & ~MARLIN_B200_FMT_PREPARED;
    const int64_t b = (size_m <= 32 && (f == kU4B8 || f == kU4)) ? gemm_stream_i8_scratch_bytes(size_m, size_n, size_k) : 0;
    return a > b ? a : b;
  }
  if (size_n % 256 != 0 && size_n % 64 == 0 && size_k % 64 == 0 && size_m > 0) {
    // the padded copy of the operands and of the output, then what the kernels need on N' columns
    const int64_t n_pad = (size_n + 255) / 256 * 256;
    const int64_t a = gemm_decode_scratch_bytes(size_m, n_pad, size_k, format);
    const int64_t b = gemm_tc_scratch_bytes(size_m, n_pad, size_k);
    return gemm_pad_scratch_bytes(size_m, size_n, size_k, format, a > b ? a : b);
  }
  const int64_t a = gemm_decode_scratch_bytes(size_m, size_n, size_k, format);
  const int64_t b = gemm_tc_scratch_bytes(size_m, size_n, size_k);
  return a > b ? a : b;
}

extern "C" int marlin_b200_gemm(const void* a, void* c, const int32_t* b_q_weight, const void* b_scales,
                                const void* b_zeros, const void* b_bias, const float* global_scale,
                                int act_dtype, int format, int64_t size_m, int64_t size_n,
                                int64_t size_k, int64_t a_stride, int64_t num_groups, void* scratch,
                                int64_t scratch_bytes, void* stream) {
  GemmArgs g{};
  g.a = a; g.c = c; g.bq = b_q_weight; g.scales = b_scales; g.zeros = b_zeros; g.bias = b_bias;
  g.global_scale = global_scale; g.act_dtype = act_dtype; g.format = format & ~MARLIN_B200_FMT_PREPARED;
  g.prepared = (format & MARLIN_B200_FMT_PREPARED) != 0;
  g.size_m = size_m; g.size_n = size_n; g.size_k = size_k; g.a_stride = a_stride;
  g.num_groups = num_groups; g.num_experts = 1; g.top_k = 1;
  g.scratch = scratch; g.scratch_bytes = scratch_bytes; g.stream = (cudaStream_t)stream;
  if (int rc = check_common(g)) return rc;
  MB_CHECK(scratch == nullptr || ((uintptr_t)scratch & 255) == 0, "scratch must be aligned to 256 bytes");
  MB_CHECK(a_stride % 8 == 0, "A.stride(0) must divisible by 8");
  MB_CHECK(a_stride >= size_k, "A.stride(0) = %lld is smaller than size_k = %lld", (long long)a_stride,
           (long long)size_k);
  return dispatch(g);
}

extern "C" int64_t marlin_b200_moe_gemm_scratch_bytes(int64_t num_sorted, int64_t size_n, int64_t size_k, int format) {
  if (format & MARLIN_B200_FMT_PREPARED) return gemm_stream_i8_grouped_scratch_bytes(num_sorted, size_n, size_k);
  if (size_n % 256 != 0 || size_k % 64 != 0) return 0;  // served by the shape-agnostic kernel
  // the routed rows in sorted order, then the tile list (one entry per block of at least 8 routes)
  return ((num_sorted * size_k * 2 + 255) & ~(int64_t)255) + (num_sorted / 8 + 64) * 4;
}

extern "C" int marlin_b200_moe_gemm(const void* a, void* c, const int32_t* b_q_weight,
                                    const void* b_scales, const void* b_zeros, const void* b_bias,
                                    const float* global_scale, const int32_t* sorted_token_ids,
                                    const int32_t* expert_ids, const int32_t* num_tokens_past_padded,
                                    const float* topk_weights, int64_t num_sorted, int64_t num_experts,
                                    int moe_block_size, int top_k, int mul_topk_weights, int act_dtype,
                                    int format, int64_t size_m, int64_t size_n, int64_t size_k,
                                    int64_t num_groups, void* scratch, int64_t scratch_bytes,
                                    void* stream) {
  GemmArgs g{};
  g.a = a; g.c = c; g.bq = b_q_weight; g.scales = b_scales; g.zeros = b_zeros; g.bias = b_bias;
  g.global_scale = global_scale; g.act_dtype = act_dtype; g.format = format;
  g.size_m = size_m; g.size_n = size_n; g.size_k = size_k; g.a_stride = size_k;
  g.num_groups = num_groups;
  g.sorted_ids = sorted_token_ids; g.expert_ids = expert_ids; g.num_post_pad = num_tokens_past_padded;
  g.topk_weights = topk_weights; g.num_sorted = num_sorted; g.num_experts = num_experts;
  g.block_size = moe_block_size; g.top_k = top_k; g.mul_topk = mul_topk_weights;
  g.scratch = scratch; g.scratch_bytes = scratch_bytes; g.stream = (cudaStream_t)stream;
  g.prepared = (format & MARLIN_B200_FMT_PREPARED) != 0;
  g.silu_input = (format & MARLIN_B200_FMT_SILU_INPUT) != 0;
  g.format = format & ~(MARLIN_B200_FMT_PREPARED | MARLIN_B200_FMT_SILU_INPUT);
  MB_CHECK(!g.silu_input || g.prepared, "SiLU-and-mul on load is served for expert weights in the streaming layout only");
  if (g.silu_input) g.a_stride = 2 * size_k;
  if (moe_block_size != 8) {
    MB_CHECK(moe_block_size % 16 == 0 && moe_block_size >= 16 && moe_block_size <= 64,
             "unsupported moe_block_size=%d", moe_block_size);
  }
  MB_CHECK(top_k >= 1, "top_k must be positive, got %d", top_k);
  MB_CHECK(num_experts >= 1, "b_q_weight has no experts");
  if (int rc = check_common(g)) return rc;
  MB_CHECK(scratch == nullptr || ((uintptr_t)scratch & 255) == 0, "scratch must be aligned to 256 bytes");
  MB_CHECK(sorted_token_ids != nullptr && expert_ids != nullptr && num_tokens_past_padded != nullptr,
           "null routing tensor pointer");
  MB_CHECK(!mul_topk_weights || topk_weights != nullptr, "mul_topk_weights needs topk_weights");
  MB_CHECK(size_m * top_k < (1ll << 31), "size_m * top_k does not fit 32-bit route ids");
  if (g.size_m == 0 || g.size_n == 0 || num_sorted == 0) return 0;
  if (g.prepared) {
    // expert weights in the streaming layout: served by the decode-sized integer-MMA kernel only
    MB_CHECK(gemm_stream_i8_grouped_accepts(g),
             "expert weights in the streaming layout are served for uint4 / uint4b8, moe_block_size 8, 16 or 32, "
             "size_k %% 128 == 0, size_n %% 256 == 0, group size a multiple of 128 (or per channel) and a scratch "
             "buffer of marlin_b200_moe_gemm_scratch_bytes; pass the reference layout otherwise");
    return launch_gemm_stream_i8_grouped(g);
  }
  const int rc = launch_gemm_tc(g);  // tensor-memory grouped kernel when the shape qualifies
  if (rc <= 0) return rc;
  return launch_gemm_generic(g);
}
