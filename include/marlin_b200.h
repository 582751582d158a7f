/*
 * marlin_b200.h - C ABI of the B200 (sm_100a) Marlin weight-only GEMM / fused-MoE library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*, a
 * cudaStream_t).  Nothing here allocates device memory unless stated; work is enqueued on the given
 * stream and the call returns without synchronising.  Return value: 0 on success, a negative
 * MARLIN_B200_E* code otherwise; marlin_b200_last_error() then returns a message for the calling
 * thread.  The library is stateless apart from per-device caches (SM count, TMA descriptors keyed
 * by weight pointer) and is safe to call from several host threads.
 *
 * Each declaration names the interface of the reference project (zhinianqin/marlin_v100) that it
 * stands in for, as file:line inside that project.
 */
#ifndef MARLIN_B200_H_
#define MARLIN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MARLIN_B200_OK 0
#define MARLIN_B200_EINVAL (-1)   /* argument check failed (the reference raises through TORCH_CHECK) */
#define MARLIN_B200_ECUDA (-2)    /* a CUDA runtime / driver call failed */
#define MARLIN_B200_ESCRATCH (-3) /* scratch buffer too small */

/* Activation / output / scale element type. */
#define MARLIN_B200_F16 0
#define MARLIN_B200_BF16 1

/* Weight formats.  The integer is what marlin_b200_format_from_type_id() returns for the
 * reference's 58-bit ScalarType id (csrc/core/scalar_type.hpp:124-157, vllm/scalar_type.py:26-43)
 * together with the scale element kind (float4_e2m1f is nvfp4 with e4m3 scales, mxfp4 with e8m0). */
#define MARLIN_B200_FMT_U4B8 0
#define MARLIN_B200_FMT_U4 1
#define MARLIN_B200_FMT_U8B128 2
#define MARLIN_B200_FMT_U8 3
#define MARLIN_B200_FMT_FP8 4
#define MARLIN_B200_FMT_NVFP4 5
#define MARLIN_B200_FMT_MXFP4 6

/* Flag, or-ed into the `format` argument of marlin_b200_gemm / marlin_b200_moe_gemm and their scratch-size
 * functions: b_q_weight is in the library's streaming layout (made by marlin_b200_prepare_weights), not in the
 * reference layout.  The grouped GEMM serves such weights for uint4 / uint4b8 with moe_block_size 8, 16 or 32 (the
 * decode regime); marlin_b200_moe_gemm_scratch_bytes then returns the room for digit planes in sorted order. */
#define MARLIN_B200_FMT_PREPARED 0x100
/* Flag for marlin_b200_moe_gemm together with MARLIN_B200_FMT_PREPARED: `a` is the [size_m, 2 * size_k]
 * gate | up output of the expert layer's first GEMM, and silu(gate) * up (rounded to the activation type where
 * marlin_b200_silu_and_mul rounds) is what the GEMM multiplies: the second GEMM of the layer without the
 * separate SiLU-and-mul pass (eager PyTorch in the reference, fused_marlin_moe.py:161-165). */
#define MARLIN_B200_FMT_SILU_INPUT 0x200

/* Scale element kinds for marlin_b200_format_from_type_id(). */
#define MARLIN_B200_SCALE_ACT 0  /* same 16-bit type as the activations */
#define MARLIN_B200_SCALE_E4M3 1 /* nvfp4 block scales */
#define MARLIN_B200_SCALE_E8M0 2 /* mxfp4 block scales */

/* Message of the last failed call on this host thread (never NULL). */
const char* marlin_b200_last_error(void);

/* Library version, "major.minor". */
const char* marlin_b200_version(void);

/* Number of kernels this library has launched in this process so far (all entry points, all
 * threads).  Diagnostics only; it has no counterpart in the reference. */
int64_t marlin_b200_launch_count(void);
/* Diagnostic (no reference counterpart): every wait inside the pipelined kernels is bounded (about two
 * seconds); a kernel whose wait gave up drains without touching its output and leaves a code here.
 * *status = 0 when no kernel on the current device gave up since the last reset; otherwise byte 0 /
 * 1 / 2 / 3 hold the code of the register-fragment decode kernel / the tensor-memory kernels / the
 * integer-MMA decode kernel / the weight-streaming kernel.  Synchronises with the device: call it outside the hot path. */
int marlin_b200_kernel_status(int* status, int reset);

/* Maps (b_type_id, scale kind) to a MARLIN_B200_FMT_* value, or -1.
 * Stands in for the b_type routing of csrc/quantization/marlin/marlin.cu:142-183,385-505. */
int marlin_b200_format_from_type_id(int64_t b_type_id, int scale_kind);

/* ----------------------------------------------------------------------------------------------
 * Weight repack.  Stand in for
 *   gptq_marlin_repack  csrc/quantization/marlin/gptq_marlin_repack.cu:399-469
 *   awq_marlin_repack   csrc/quantization/marlin/awq_marlin_repack.cu:319-381
 * in : GPTQ int32 [size_k / pf, size_n] (packed along K) or AWQ int32 [size_k, size_n / pf]
 *      (packed along N with the AWQ nibble interleave), pf = 32 / num_bits, num_bits in {4, 8};
 *      perm: int32 [size_k] source row for each destination row (act-order) or NULL.
 * out: int32 [size_k / 16, size_n * 16 / pf], bit-identical to the reference's packed layout.
 * Requires size_k % 16 == 0 and size_n % 64 == 0.
 * -------------------------------------------------------------------------------------------- */
int marlin_b200_gptq_repack(const int32_t* b_q_weight, const int32_t* perm, int32_t* out,
                            int64_t size_k, int64_t size_n, int num_bits, void* stream);
int marlin_b200_awq_repack(const int32_t* b_q_weight, int32_t* out, int64_t size_k, int64_t size_n,
                           int num_bits, void* stream);

/* ----------------------------------------------------------------------------------------------
 * Streaming layout (opt-in).  The reference's packed layout stores a 256-column group of 16 k as a run of
 * 2 KiB (4 KiB for 8-bit codes) and the next 16 k size_n * 8 bytes further on; read as a stream that
 * pattern reaches about two thirds of the DRAM bandwidth of a linear read, and its nibble order forces byte
 * transposes in the kernel.  marlin_b200_prepare_weights writes the SAME codes in another order (every
 * 256-column x 64-k block contiguous, blocks of a column group consecutive along k, codes placed where the
 * GEMM kernel's threads consume them); marlin_b200_restore_weights is its exact inverse, so
 * restore(prepare(w)) == w bit for bit and both tensors have size_k * size_n * num_bits / 8 bytes per expert.
 * This is the "TMA-friendly packed layout that stays bit-identical in unpacked semantics"; what
 * gptq_marlin_repack / awq_marlin_repack return is unchanged (csrc/quantization/marlin/
 * gptq_marlin_repack.cu:399-469 defines it), a caller converts once after repacking and then passes
 * `format | MARLIN_B200_FMT_PREPARED` to marlin_b200_gemm.  The reference has no counterpart of the two
 * entry points.  b_q_weight / out: int32 [num_experts, size_k / 16, size_n * 16 / pf]; out must not alias
 * the input.  Requires size_k % 128 == 0 and size_n % 256 == 0 (other shapes stay in the reference layout).
 * -------------------------------------------------------------------------------------------- */
int marlin_b200_prepare_weights(const int32_t* b_q_weight, int32_t* out, int64_t size_k, int64_t size_n,
                                int num_bits, int64_t num_experts, void* stream);
int marlin_b200_restore_weights(const int32_t* prepared, int32_t* out, int64_t size_k, int64_t size_n,
                                int num_bits, int64_t num_experts, void* stream);

/* ----------------------------------------------------------------------------------------------
 * Dense GEMM  C[M,N] = A[M,K] * dequant(B)[K,N] (+ bias).  Stands in for
 *   marlin_gemm  csrc/quantization/marlin/marlin.cu:83-506
 * a           : f16/bf16 [size_m, size_k], row stride a_stride elements (multiple of 8), 16-byte
 *               aligned.
 * c           : same type, [size_m, size_n], contiguous.
 * b_q_weight  : int32 [size_k / 16, size_n * 16 / pf] as produced by the repack entry points.
 * b_scales    : [num_groups, size_n]; element type = activation type for the integer formats and
 *               fp8, one byte for nvfp4 (special S0E5M3 bytes) and mxfp4 (e8m0), exactly as the
 *               reference's Python wrappers prepare them.  group size = size_k / num_groups
 *               (num_groups == 1: per-channel).
 * b_zeros     : NULL, or [num_groups, size_n] of the activation type holding zero_point * scale
 *               (u4 / u8 only: w = q * s - zeros).
 * b_bias      : NULL, or [size_n] of the activation type in the reference's permuted order.
 * global_scale: NULL, or fp32 [1] (nvfp4 only).
 * scratch     : device buffer of at least marlin_b200_gemm_scratch_bytes() bytes (may be NULL when
 *               that is 0): fp32 split-K partial sums and, for the integer-MMA kernel, the 8-bit
 *               digit planes of the activation rows.  Contents on entry are irrelevant; it is
 *               overwritten.  For size_m > 16 on matrices whose 256-column tiles would leave SMs idle
 *               the K range of the tiles is cut and the buffer holds fp32 partial sums ([k slices]
 *               [size_m][size_n], or two partial tiles per SM); a smaller buffer is accepted there and
 *               selects a cheaper cut or none (results stay within rounding of each other, and are
 *               bit-identical from run to run for one buffer size).
 *               For size_n % 256 != 0 (size_n % 64 == 0, size_k % 64 == 0) the buffer also holds a copy of
 *               the weights, scales, zero-points, bias and output padded to the next multiple of 256
 *               columns, made on every call (the reference's packed layout differs for such widths and
 *               the tensor-core kernels read the 256-column form); with a smaller buffer a slower
 *               shape-agnostic kernel serves the call, same results within rounding.
 * With MARLIN_B200_FMT_PREPARED in `format`, b_q_weight is the streaming layout and one kernel family serves
 * every size_m (passes of up to 128 rows); scratch then holds one counter per 256-column group and two fp32
 * partial tiles per SM, and a buffer that is too small (or NULL) makes every CTA take whole column groups
 * instead of equal shares of the weight stream (slower when size_n / 256 does not fill the SMs, same results
 * up to the order of the fp32 sums).
 * Requires size_k % 32 == 0 and size_n % 64 == 0.  size_m == 0 is a no-op.
 * -------------------------------------------------------------------------------------------- */
int64_t marlin_b200_gemm_scratch_bytes(int64_t size_m, int64_t size_n, int64_t size_k, int format);

int marlin_b200_gemm(const void* a, void* c, const int32_t* b_q_weight, const void* b_scales,
                     const void* b_zeros, const void* b_bias, const float* global_scale,
                     int act_dtype, int format, int64_t size_m, int64_t size_n, int64_t size_k,
                     int64_t a_stride, int64_t num_groups, void* scratch, int64_t scratch_bytes,
                     void* stream);

/* Same computation as marlin_b200_gemm, for callers that cannot hand over a scratch buffer because
 * they are not allowed to allocate device memory where the call happens (a serving runtime whose memory
 * plan is fixed at start-up, a plugin that is given tensors but no allocator, host code that runs while
 * another component captures the stream).  The scratch is a 6 MiB array inside the library image instead
 * (present on every GPU that loads the library, until the process exits).  For size_m <= 16 the kernels
 * need SMs * 32 KiB + 48 * size_k + 256 bytes of it (a 148-SM B200: size_k up to 30 016); a problem beyond
 * that gets MARLIN_B200_ESCRATCH and a message.  For size_m > 16 the K cut is planned inside the 6 MiB, as
 * marlin_b200_gemm does with a buffer of that size (results equal that call's bit for bit).  The call
 * allocates nothing.  Its first use on a device resolves the array's device address: do that first
 * call outside any stream capture.  All calls on a device share the array; nothing in it has to start
 * at zero (every partial is written before it is read within one call), but two calls whose kernels
 * overlap on the GPU (different streams) would overwrite each other's partial sums: keep calls to this
 * entry point on one stream per device, or order them with events.
 * This entry point has no counterpart in the reference. */
int marlin_b200_gemm_static_scratch(const void* a, void* c, const int32_t* b_q_weight,
                                    const void* b_scales, const void* b_zeros, const void* b_bias,
                                    const float* global_scale, int act_dtype, int format,
                                    int64_t size_m, int64_t size_n, int64_t size_k, int64_t a_stride,
                                    int64_t num_groups, void* stream);

/* ----------------------------------------------------------------------------------------------
 * Grouped expert GEMM.  Stands in for
 *   moe_wna16_marlin_gemm  csrc/moe/marlin_moe_wna16/ops.cu:102-529
 * Row r of block b is sid = sorted_token_ids[b * moe_block_size + r]; it is valid when
 * 0 <= sid < size_m * top_k.  It reads A row sid / top_k, uses the weights of expert
 * expert_ids[b] (a block with a negative id, or at or beyond num_tokens_past_padded[0], is skipped)
 * and writes C row sid:
 *   value = acc * global_scale[e]; value += bias[e][n] * (mul_topk_weights ? global_scale[e] : 1)
 *   value *= mul_topk_weights ? topk_weights[sid] : 1
 * (csrc/moe/marlin_moe_wna16/sm70_marlin_gemm.cuh:3472-3509).
 * a [size_m, size_k] contiguous; c [size_m * top_k, size_n]; b_q_weight [E, size_k/16, size_n*16/pf];
 * b_scales [E, num_groups, size_n]; b_zeros / b_bias / global_scale per expert ([E,G,N], [E,N], [E]).
 * sorted_token_ids int32 [num_sorted]; expert_ids int32 [>= num_sorted / moe_block_size];
 * num_tokens_past_padded int32 [1], read on the device; topk_weights fp32 [size_m * top_k].
 * moe_block_size in {8, 16, 32, 48, 64}.
 * -------------------------------------------------------------------------------------------- */
/* Scratch for marlin_b200_moe_gemm: room for the activation rows copied into sorted order
 * (num_sorted * size_k * 2 bytes) and the list of row tiles (0 when the shape is served by the kernel
 * that needs none). */
int64_t marlin_b200_moe_gemm_scratch_bytes(int64_t num_sorted, int64_t size_n, int64_t size_k, int format);

int marlin_b200_moe_gemm(const void* a, void* c, const int32_t* b_q_weight, const void* b_scales,
                         const void* b_zeros, const void* b_bias, const float* global_scale,
                         const int32_t* sorted_token_ids, const int32_t* expert_ids,
                         const int32_t* num_tokens_past_padded, const float* topk_weights,
                         int64_t num_sorted, int64_t num_experts, int moe_block_size, int top_k,
                         int mul_topk_weights, int act_dtype, int format, int64_t size_m,
                         int64_t size_n, int64_t size_k, int64_t num_groups, void* scratch,
                         int64_t scratch_bytes, void* stream);

/* ----------------------------------------------------------------------------------------------
 * Token sorting for the grouped GEMM.  Stands in for
 *   moe_align_block_size  csrc/moe/moe_align_sum_kernels.cu:477-569
 * topk_ids int32 [numel] (flattened [tokens, top_k]); expert_map NULL or int32 [num_global_experts]
 * (global -> local id, -1 = not on this rank; ids are looked up before counting).
 * sorted_token_ids int32 [sorted_capacity] with sorted_capacity >= numel + num_experts*(block-1):
 * per expert in ascending id its flat route indices in ascending order, padded with `numel` to a
 * multiple of block_size; the tail is filled with `numel`.  expert_ids int32 [expert_ids_capacity]:
 * expert of every block, tail -1.  num_tokens_post_pad int32 [1].
 * The in-expert order is the stable ascending order of the reference's test oracle
 * (tests/test_marlin_moe.py:194-213), deterministic for every size.
 * scratch: at least marlin_b200_moe_align_scratch_bytes() bytes.
 * -------------------------------------------------------------------------------------------- */
int64_t marlin_b200_moe_align_scratch_bytes(int64_t numel, int64_t num_experts);

int marlin_b200_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int64_t num_experts,
                                     int64_t num_global_experts, int block_size,
                                     const int32_t* expert_map, int32_t* sorted_token_ids,
                                     int64_t sorted_capacity, int32_t* expert_ids,
                                     int64_t expert_ids_capacity, int32_t* num_tokens_post_pad,
                                     void* scratch, int64_t scratch_bytes, void* stream);

/* ----------------------------------------------------------------------------------------------
 * Fused softmax + top-k gating.  Stands in for
 *   topk_softmax  csrc/moe/topk_softmax_kernels.cu:773-809
 * gating [num_tokens, num_experts] of gating_dtype (MARLIN_B200_F16 / _BF16, or 2 = fp32);
 * bias NULL or fp32 [num_experts], added to the probabilities for selection only.
 * topk_weights fp32 [num_tokens, topk]; topk_indices int32 [num_tokens, topk];
 * token_expert_indices int32 [num_tokens, topk] = j * num_tokens + t.  Ties pick the lower index.
 * -------------------------------------------------------------------------------------------- */
int marlin_b200_topk_softmax(const void* gating, int gating_dtype, const float* bias,
                             float* topk_weights, int32_t* topk_indices,
                             int32_t* token_expert_indices, int64_t num_tokens, int64_t num_experts,
                             int topk, int renormalize, void* stream);

/* The same selection on per-expert sigmoid scores 1 / (1 + exp(-x)) instead of the row softmax.  Stands in for
 *   topk_sigmoid  csrc/moe/topk_softmax_kernels.cu:811-850 (scores: :436-441) */
int marlin_b200_topk_sigmoid(const void* gating, int gating_dtype, const float* bias,
                             float* topk_weights, int32_t* topk_indices,
                             int32_t* token_expert_indices, int64_t num_tokens, int64_t num_experts,
                             int topk, int renormalize, void* stream);

/* ----------------------------------------------------------------------------------------------
 * Block lists for tokens that are already grouped by expert (the "batched experts" format: expert e owns rows
 * [e * max_tokens_per_batch, e * max_tokens_per_batch + expert_num_tokens[e])).  Stands in for
 *   batched_moe_align_block_size  csrc/moe/moe_align_sum_kernels.cu:22-78,571-596
 * sorted_token_ids int32 [num_batches * ceil(max_tokens_per_batch / block) * block]: per expert its row ids,
 * padded to a multiple of block_size, experts back to back; everything else = num_batches *
 * max_tokens_per_batch.  block_ids int32 [sorted_size / block]: expert of every used block, -1 elsewhere.
 * num_tokens_post_pad int32 [1].
 * -------------------------------------------------------------------------------------------- */
int marlin_b200_batched_moe_align_block_size(int64_t max_tokens_per_batch, int block_size,
                                             const int32_t* expert_num_tokens, int64_t num_batches,
                                             int32_t* sorted_token_ids, int64_t sorted_size,
                                             int32_t* block_ids, int64_t num_blocks,
                                             int32_t* num_tokens_post_pad, void* stream);

/* ----------------------------------------------------------------------------------------------
 * Re-coding of 4-bit codes for the int4 -> fp8 path: per code v, v >= z ? v - z : 15 - v with z = 8
 * (qzeros == NULL; any word count) or z = the code's AWQ zero-point (qweight int32 [rows, words_per_row],
 * qzeros int32 [zero_rows, words_per_row], rows / zero_rows = group size, a multiple of 8).  out may be
 * qweight itself.  Stands in for
 *   marlin_int4_fp8_preprocess  csrc/quantization/marlin/marlin_int4_fp8_preprocess.cu:8-102
 * -------------------------------------------------------------------------------------------- */
int marlin_b200_int4_fp8_preprocess(const int32_t* qweight, const int32_t* qzeros, int32_t* out,
                                    int64_t rows, int64_t words_per_row, int64_t zero_rows, void* stream);

/* ----------------------------------------------------------------------------------------------
 * Glue of the two-GEMM expert layer (eager PyTorch in the reference,
 * vllm/model_executor/layers/fused_moe/fused_marlin_moe.py:161-165,379-382).
 * silu_and_mul: out[r, i] = silu(in[r, i]) * in[r, inter + i], in [rows, 2*inter], out [rows, inter].
 * moe_sum     : out[t, :] = sum_j in[t * top_k + j, :], in [tokens * top_k, hidden].
 * -------------------------------------------------------------------------------------------- */
int marlin_b200_silu_and_mul(const void* in, void* out, int64_t rows, int64_t inter, int act_dtype,
                             void* stream);
int marlin_b200_moe_sum(const void* in, void* out, int64_t tokens, int top_k, int64_t hidden,
                        int act_dtype, void* stream);
/* The same sum over rows picked by an index: out[t] = sum_j in[rows[t * top_k + j]] (no counterpart in
 * the reference: the combine step of the expert-parallel layer, whose contributions come back from
 * the all-to-all in sender order). */
int marlin_b200_moe_sum_rows(const void* in, const int32_t* rows, void* out, int64_t tokens, int top_k,
                             int64_t hidden, int act_dtype, void* stream);

/* ----------------------------------------------------------------------------------------------
 * Load-time helpers for expert layers and fp4 / fp8 checkpoints.
 * gptq_moe_repack / awq_moe_repack: all experts of a layer in one launch (b_q_weight [E][...], perm [E][size_k]
 *   or NULL, out [E][size_k / 16][size_n * 16 / pack_factor]); stand in for the per-expert Python loops
 *   gptq_marlin_moe_repack / awq_marlin_moe_repack   vllm/_custom_ops.py:1228-1269
 * nvfp4_scale_min + nvfp4_process_scales: block scales (fp16 values of the e4m3 scales, [rows][cols]) -> the
 *   interleaved S0E5M3 bytes; scale_min leaves min(scale * 2^7 over non-zero scales) in *min_out (a device float)
 *   from which the caller derives the power-of-two rescale (2^ceil(log2(2 / min)) if min < 2, bf16 activations only)
 *   nvfp4_marlin_process_scales   .../quantization/utils/marlin_utils_fp4.py:30-112
 * interleave_scale_bytes: the [0,2,1,3] interleave per four columns of one-byte (e8m0) scales
 *   mxfp4_marlin_process_scales   .../marlin_utils_fp4.py:115-129 (marlin_b200_gemm itself takes mxfp4 scales in
 *   natural column order: this is for callers that hold the reference's own form)
 * fp8_fuse_exponent_bias: scales * 2^8 (fp16) / 2^120 (bf16)
 *   fp8_fused_exponent_bias_into_scales   .../marlin_utils_fp8.py:28-39
 * -------------------------------------------------------------------------------------------- */
int marlin_b200_gptq_moe_repack(const int32_t* b_q_weight, const int32_t* perm, int32_t* out, int64_t num_experts,
                                int64_t size_k, int64_t size_n, int num_bits, void* stream);
int marlin_b200_awq_moe_repack(const int32_t* b_q_weight, int32_t* out, int64_t num_experts, int64_t size_k,
                               int64_t size_n, int num_bits, void* stream);
int marlin_b200_nvfp4_scale_min(const void* scales_half, int64_t count, float* min_out, void* stream);
int marlin_b200_nvfp4_process_scales(const void* scales_half, uint8_t* out, int64_t rows, int64_t cols,
                                     float scale_factor, void* stream);
int marlin_b200_interleave_scale_bytes(const uint8_t* in, uint8_t* out, int64_t rows, int64_t cols, void* stream);
int marlin_b200_fp8_fuse_exponent_bias(const void* in, void* out, int64_t count, int act_dtype, void* stream);

/* ----------------------------------------------------------------------------------------------
 * Multi-GPU steps over peer-mapped memory.  No counterpart in the reference, whose distributed layer is a
 * world-size-1 stub (vllm/distributed/__init__.py:4-25); the layouts stand on its `expert_map` hook
 * (fused_marlin_moe.py:170-171) and on output columns being independent (marlin.cu:356-359).
 *
 * Every rank (one process per GPU of one node) allocates an arena, exports it, and opens the arenas of
 * all other ranks; `arenas[r]` is rank r's arena as mapped in THIS process (arenas[rank] is the local
 * allocation).  The first marlin_b200_peer_header_bytes() bytes of an arena belong to the library (step
 * counter, status, flags, count tables); the caller lays out the rest, identically on every rank.  The
 * kernels move data with plain loads and stores to peer addresses and order it with flags; every wait is
 * bounded (two seconds), after which the arena's status word is set and the kernels of that arena stop
 * moving data: read it with marlin_b200_peer_status (0 = fine, 1 + phase = a wait of that phase gave up,
 * 16 = receive capacity exceeded).  All ranks must issue the same sequence of steps on an arena.
 * -------------------------------------------------------------------------------------------- */
int marlin_b200_peer_header_bytes(void);
int marlin_b200_peer_alloc(int64_t bytes, void** ptr);            /* zero-filled device memory           */
int marlin_b200_peer_free(void* ptr);
int marlin_b200_peer_export(void* ptr, void* handle64);           /* 64-byte handle for other processes  */
int marlin_b200_peer_open(const void* handle64, void** ptr);      /* map another rank's arena            */
int marlin_b200_peer_close(void* ptr);
int marlin_b200_peer_status(const void* arena, int* status, int* steps_done);   /* synchronous read     */
int marlin_b200_peer_host_word_alloc(void** host_ptr, void** device_ptr);       /* 64 mapped host bytes */
int marlin_b200_peer_host_word_free(void* host_ptr);

/* Column-parallel dense layer: every rank's `src` (bytes_per_rank bytes, a multiple of 16) gathered into
 * `out`.  slice_rows == 0: out is [world][bytes_per_rank].  slice_rows == M: src is an [M, cols] row block and
 * out is [M, world * cols] (rank r's columns at r * cols).  The arena holds two gather buffers of
 * 2 * world * bytes_per_rank bytes at buffer_offset (every 8 data bytes travel with 8 bytes of step number).  No host synchronisation: the call can be captured. */
int marlin_b200_peer_allgather(const void* const* arenas, int rank, int world, const void* src,
                               int64_t bytes_per_rank, int64_t buffer_offset, void* out, int64_t slice_rows,
                               void* stream);

/* Expert-parallel layer, one step = plan, dispatch, [poll_rows on the host], wait(2), the expert layer on
 * the received rows, signal(3), combine.
 *   layout[6] = arena offsets of {received rows, int32 expert index per row, float router weight per row,
 *               expert outputs}, row capacity, bytes per row (hidden * 2).
 *   slot_sorted / order: the expert_ids / sorted_token_ids outputs of marlin_b200_moe_align_block_size with
 *               block_size 1 and the expert -> slot table as expert_map (slot = rank * experts_per_rank +
 *               index on that rank; routes with ids outside the table sit at the end as -1).
 *   position_of_route: int32 [tokens * top_k] scratch written by dispatch and read by combine.
 *   poll_rows returns the rows this rank received, the number of routes with invalid ids on any rank (the
 *               caller then issues signal + combine with skip = 1 and raises on every rank) and the status. */
int marlin_b200_ep_plan(const void* const* arenas, int rank, int world, const int32_t* slot_sorted, int64_t numel,
                        int experts_per_rank, void* stream);
int marlin_b200_ep_dispatch(const void* const* arenas, int rank, int world, const int64_t* layout,
                            const void* hidden, const int32_t* order, const int32_t* slot_sorted,
                            const float* topk_weights, int32_t* position_of_route, int top_k,
                            int experts_per_rank, void* host_word_device, void* stream);
int marlin_b200_ep_poll_rows(const void* host_word, int step, int timeout_ms, int64_t* rows,
                             int* invalid_routes, int* status);
int marlin_b200_ep_wait(const void* const* arenas, int rank, int world, int phase, void* stream);
int marlin_b200_ep_signal(const void* const* arenas, int rank, int world, int phase, void* stream);
int marlin_b200_ep_combine(const void* const* arenas, int rank, int world, const int64_t* layout,
                           const int32_t* position_of_route, int top_k, int64_t tokens, void* out,
                           int act_dtype, int skip, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MARLIN_B200_H_ */
