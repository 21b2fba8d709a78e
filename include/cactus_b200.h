/*
 * cactus_b200 -- C ABI of the B200 (sm_100a) kernels behind the ggml backend plug-in.
 *
 * This is the boundary between host code (the ggml-backend plug-in in C++, or any FFI binding) and the
 * hand-written CUDA kernels.  Plain pointers, sizes and byte strides only; no C++ or framework types.
 * Unless said otherwise every pointer is a DEVICE pointer, every call is asynchronous on `stream`
 * (a cudaStream_t passed as void*, NULL = the legacy default stream) and returns 0 on success or a
 * negative B200_E_* code; b200_last_error() gives the message for the calling thread.
 *
 * Each entry point names the routine of the reference (cactus's vendored ggml, paths relative to the
 * reference project root) whose work it takes over when the plug-in's graph_compute
 * (cactus/ggml-backend-impl.h:110) dispatches a node.
 *
 * Tensor conventions are ggml's: ne[0] is the contiguous dimension.  A mul_mat computes
 * dst[n][m] = sum_k W[m][k] * x[n][k]   with W = src0 [K, M], x = src1 [K, N], dst [M, N].
 */
#ifndef CACTUS_B200_H
#define CACTUS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define B200_API __declspec(dllexport)
#else
#define B200_API __attribute__((visibility("default")))
#endif

#define B200_ABI_VERSION 1

/* error codes */
#define B200_OK 0
#define B200_E_INVALID (-1)   /* bad argument (shape, alignment, type) */
#define B200_E_CUDA (-2)      /* a CUDA runtime call or launch failed */
#define B200_E_SCRATCH (-3)   /* scratch buffer too small */
#define B200_E_NODEVICE (-4)  /* no sm_100 device */

/* weight types: the ids of the reference's enum lm_ggml_type (cactus/ggml.h:351-360) */
#define B200_TYPE_F32 0
#define B200_TYPE_F16 1
#define B200_TYPE_Q4_0 2
#define B200_TYPE_Q8_0 8

/* Q8_0 activation quantiser arithmetic (cactus/ggml-cpu/ggml-cpu-quants.c:732-1045) */
#define B200_Q8_AVX2 0   /* id = 127/max, round to nearest even: the x86 AVX/AVX2 branch (:802-885) */
#define B200_Q8_SCALAR 1 /* id = 1/d, roundf: quantize_row_q8_0_ref (cactus/ggml-quants.c:188-211) */

typedef void *b200_stream_t;

B200_API int b200_abi_version(void);
B200_API const char *b200_last_error(void);
/* number of sm_100 devices visible; fills name/total memory of `device` when the pointers are non-NULL */
B200_API int b200_device_count(void);
B200_API int b200_device_info(int device, char *name, size_t name_len, size_t *free_bytes, size_t *total_bytes, int *sm_count);
/* kernels launched by this library in the calling process since load (for launch accounting) */
B200_API uint64_t b200_launch_count(void);
/* 0, or non-zero once a kernel on the current device gave up a bounded wait on one of its own barriers (its result
 * is then invalid; the context stays usable).  No reference counterpart: the CPU kernels have no such waits. */
B200_API int b200_kernel_status(void);
/* How many polling rounds such a wait makes before it gives up (0 restores the default, which amounts to seconds), and
 * clears b200_kernel_status.  A monitoring or test hook: a kernel that gave up has waited for its own copies and tensor
 * core work in flight (that wait keeps its own, fixed limit) and returned normally. */
B200_API void b200_kernel_set_wait_limit(unsigned rounds);

/* ------------------------------------------------------------------------------------------------
 * Weight storage.
 *
 * Quantised weights live on the device in a tiled layout ("T16": 16-row x 4-block tiles in the
 * register order of the int8 tensor-core fragments, nibbles stored as two's-complement, scales in a
 * separate plane).  b200_weight_bytes gives the device size for a [K, M] tensor; b200_weight_upload
 * converts from the reference's row-major block_q4_0 / block_q8_0 stream (cactus/ggml-common.h:167-172,
 * :209-214), as a backend buffer's set_tensor (cactus/ggml-backend-impl.h:51) does at model load;
 * b200_weight_download is the exact inverse (get_tensor, :52).  `src`/`dst` of upload/download are
 * DEVICE pointers to the row-major stream (the plug-in stages host data through a device bounce
 * buffer); `rows_begin/rows_count` select a range of rows (multiple of 16 unless it ends at M) so that
 * a loader may upload in pieces.
 * ---------------------------------------------------------------------------------------------- */
B200_API size_t b200_weight_bytes(int wtype, int64_t K, int64_t M);
B200_API int b200_weight_upload(int wtype, int64_t K, int64_t M, const void *src_rowmajor, void *dst_tiled,
                                int64_t rows_begin, int64_t rows_count, b200_stream_t stream);
B200_API int b200_weight_download(int wtype, int64_t K, int64_t M, const void *src_tiled, void *dst_rowmajor,
                                  int64_t rows_begin, int64_t rows_count, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * quantize_row_q8_0 (cactus/ggml-cpu/ggml-cpu-quants.c:732) over N rows of K floats.
 * Output in the reference's block_q8_0 layout (34-byte blocks, row after row): bit-exact with the
 * selected variant.  Used for parity checks; mul_mat quantises internally with the same device code.
 * ---------------------------------------------------------------------------------------------- */
B200_API int b200_quantize_q8_0(const float *x, int64_t x_row_stride_bytes, int64_t K, int64_t N, void *dst_blocks,
                                int variant, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * MUL_MAT with quantised weights: lm_ggml_compute_forward_mul_mat (cactus/ggml-cpu/ggml-cpu.c:1257-1449)
 * = quantize_row_q8_0 on every src1 row, then lm_ggml_vec_dot_q4_0_q8_0 / _q8_0_q8_0
 * (ggml-cpu-quants.c:1906 / :3591) for every (row, column).
 *   w        tiled weights from b200_weight_upload, [K, M]
 *   x        f32 activations, N rows of K, row stride in bytes
 *   dst      f32, N rows of M, row stride in bytes
 *   scratch  b200_mul_mat_scratch_bytes(wtype, K, M, N) bytes of device memory, 256-byte aligned,
 *            private to the call until it completes: the quantised activations (b200_act_bytes) followed
 *            by the kernel workspace (b200_mul_mat_workspace_bytes: split-K partial sums or the parked tiles and
 *            arrival counters of the stream-K work split)
 * N <= 2 uses the HBM-bound dp4a kernel, larger N the int8 tensor-core kernel (B200_MMVQ_MAX_N moves the border up to 8).
 * ---------------------------------------------------------------------------------------------- */
B200_API size_t b200_act_bytes(int64_t K, int64_t N);
B200_API size_t b200_mul_mat_workspace_bytes(int wtype, int64_t K, int64_t M, int64_t N);
B200_API size_t b200_mul_mat_scratch_bytes(int wtype, int64_t K, int64_t M, int64_t N);
B200_API int b200_mul_mat_q(int wtype, const void *w, int64_t K, int64_t M, const float *x, int64_t x_row_stride_bytes,
                            int64_t N, float *dst, int64_t dst_row_stride_bytes, void *scratch, size_t scratch_bytes,
                            int variant, b200_stream_t stream);
/* The two halves of b200_mul_mat_q, so one quantised activation tensor can feed several weights
 * (wq/wk/wv, gate/up): quantise once into `act` (b200_act_bytes), then multiply; `workspace`
 * (b200_mul_mat_workspace_bytes, may be 0 -> NULL) is private to each multiply. */
B200_API int b200_quantize_activations(const float *x, int64_t x_row_stride_bytes, int64_t K, int64_t N, void *act,
                                       size_t act_bytes, int variant, b200_stream_t stream);
B200_API int b200_mul_mat_q_prequant(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N,
                                     float *dst, int64_t dst_row_stride_bytes, void *workspace, size_t workspace_bytes,
                                     b200_stream_t stream);
/* Up to three weights of one type and K (a layer's gate and up projections, or q, k and v) against the same quantised
 * activations in ONE launch: dst[i] = mul_mat(w[i], x) as by b200_mul_mat_q_prequant on each, for separate weight and
 * destination tensors (what a graph_compute sees: ggml allocates them one by one), with the work of all of them dealt
 * out together.  All destinations share dst_row_stride_bytes; `workspace` as for one product of M[0] + M[1] + ... rows.
 * Weights but the last must hold a multiple of 128 rows, else (and for the GEMV widths) the products run one by one. */
B200_API int b200_mul_mat_q_prequant_multi(int wtype, int n_weights, const void *const *w, const int64_t *M, int64_t K, const void *act,
                                           int64_t N, float *const *dst, int64_t dst_row_stride_bytes, void *workspace,
                                           size_t workspace_bytes, b200_stream_t stream);
/* No counterpart in the reference: b200_mul_mat_q for callers that must not allocate device memory.
 *
 * Some hosts cannot hand this library a scratch buffer: code running under a memory budget that was fixed at
 * start-up, a plug-in loaded into a process whose allocator owns all device memory, or a caller inside a region
 * where cudaMalloc is forbidden.  For them the quantised activations go into an array that is built into the
 * library image (320 KiB of device memory on every GPU that loads the library, held until the process exits), so
 * the call takes inputs and outputs only and performs no cudaMalloc / cudaFree of its own.
 *
 * Limits: N <= B200_NOALLOC_MAX_N columns (the decode kernel) and K <= B200_NOALLOC_MAX_K; larger sizes are
 * refused with B200_E_INVALID.  Results are within the mul_mat tolerance of b200_mul_mat_q, and bit-identical to it
 * whenever both calls split K the same way (for 3 to 8 columns b200_mul_mat_q may split K across CTAs through its
 * workspace; this entry point has no workspace and never does).  The first call on a device looks up the
 * array's device address (a one-off set-up step): make that first call outside any stream capture.  All calls
 * share the one array, which keeps whatever the last call left in it: two calls that overlap on the GPU (different
 * streams, or different threads without ordering between them) race; calls ordered on one stream are fine. */
#define B200_NOALLOC_MAX_N 8
#define B200_NOALLOC_MAX_K 32768
B200_API int b200_mul_mat_q_noalloc(int wtype, const void *w, int64_t K, int64_t M, const float *x, int64_t x_row_stride_bytes,
                                    int64_t N, float *dst, int64_t dst_row_stride_bytes, int variant, b200_stream_t stream);
/* Exact per-block integer dots of the same kernel inputs (debug/parity): out int32 [N][M][K/32]. */
B200_API int b200_block_dots(int wtype, const void *w, int64_t K, int64_t M, const float *x, int64_t x_row_stride_bytes,
                             int64_t N, int32_t *out, void *act, size_t act_bytes, int variant, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * FLASH_ATTN_EXT: lm_ggml_compute_forward_flash_attn_ext_f16 (cactus/ggml-cpu/ops.cpp:6948-7165) for
 * f32 Q, f16 K/V (the unified KV cache, cactus/llama-kv-cache.cpp:583-656) and an f16 mask.
 *   q     f32, element (d, token t, head h) at byte offset t*q_nb_tok + h*q_nb_head + 4*d
 *   k, v  f16, element (d, cell c, kv-head g) at byte offset c*k_nb_cell + g*k_nb_head + 2*d
 *   mask  f16 [n_kv] per token row, row stride mask_nb_row bytes; a cell is skipped iff its mask is -inf
 *         (:7078-7081); may be NULL (no masking)
 *   dst   f32 [D, H, Nq] contiguous: row (t*H + h)
 *   scale, max_bias, logit_softcap: op_params of the node (cactus/ggml.c:4405-4444)
 *   scratch b200_flash_attn_scratch_bytes(...) bytes, 256-byte aligned
 * D in {64, 128}; H a multiple of Hkv (grouped-query attention).
 * ---------------------------------------------------------------------------------------------- */
B200_API size_t b200_flash_attn_scratch_bytes(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv);
B200_API int b200_flash_attn_ext(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv,
                                 const float *q, int64_t q_nb_tok, int64_t q_nb_head,
                                 const void *k, int64_t k_nb_cell, int64_t k_nb_head,
                                 const void *v, int64_t v_nb_cell, int64_t v_nb_head,
                                 const void *mask, int64_t mask_nb_row,
                                 float scale, float max_bias, float logit_softcap,
                                 float *dst, void *scratch, size_t scratch_bytes, b200_stream_t stream);
/* The mask scan alone: per token row, the list of cells whose mask is not -inf.  A plug-in runs it
 * once per graph and shares the result between all layers (the mask tensor is the same node).
 * b200_flash_attn_ext_indexed then skips its own scan. */
B200_API size_t b200_mask_index_bytes(int64_t Nq, int64_t n_kv);
B200_API int b200_mask_index_build(const void *mask, int64_t mask_nb_row, int64_t Nq, int64_t n_kv, void *index,
                                   size_t index_bytes, b200_stream_t stream);
B200_API int b200_flash_attn_ext_indexed(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv,
                                         const float *q, int64_t q_nb_tok, int64_t q_nb_head,
                                         const void *k, int64_t k_nb_cell, int64_t k_nb_head,
                                         const void *v, int64_t v_nb_cell, int64_t v_nb_head,
                                         const void *mask, int64_t mask_nb_row, const void *index,
                                         float scale, float max_bias, float logit_softcap,
                                         float *dst, void *scratch, size_t scratch_bytes, b200_stream_t stream);
/* b200_flash_attn_ext_indexed whose result is (also) left as the Q8_0-quantised activations of the mul_mat that
 * consumes it (attention output -> wo in llm_build_llama, cactus/llama-model.cpp:4517-4671): what
 * b200_quantize_activations(dst, ..., K = H * D, N = Nq, act, ...) would write, bit for bit, without the extra
 * launch.  dst may be NULL when only the quantised form is wanted.  H * D must be a multiple of 128.  Measured on B200
 * at 64 tokens x 32 heads x 128 over 57k cells it is slower than the two launches (70.5 us against 57.5 + 2.5: the
 * attention kernel sits at its register limit), so it pays only where launches, not kernel time, are the cost. */
B200_API int b200_flash_attn_ext_quant(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv,
                                       const float *q, int64_t q_nb_tok, int64_t q_nb_head,
                                       const void *k, int64_t k_nb_cell, int64_t k_nb_head,
                                       const void *v, int64_t v_nb_cell, int64_t v_nb_head,
                                       const void *mask, int64_t mask_nb_row, const void *index,
                                       float scale, float max_bias, float logit_softcap,
                                       float *dst, void *act, size_t act_bytes, int variant,
                                       void *scratch, size_t scratch_bytes, b200_stream_t stream);
/* Validation variant: one warp per (token, head) walks the unmasked cells in ascending order with the
 * reference's exact sequence of roundings (fp16 Q, the AVX2 lane order of the K.Q dot, the fp16 output
 * accumulator of cactus/ggml-cpu/ops.cpp:7103-7117).  Slow; it exists to show that the distance between the
 * fast kernel and the reference is the reference's fp16 accumulator.  Needs no scratch. */
B200_API int b200_flash_attn_ext_parity(int64_t D, int64_t H, int64_t Hkv, int64_t Nq, int64_t n_kv,
                                        const float *q, int64_t q_nb_tok, int64_t q_nb_head,
                                        const void *k, int64_t k_nb_cell, int64_t k_nb_head,
                                        const void *v, int64_t v_nb_cell, int64_t v_nb_head,
                                        const void *mask, int64_t mask_nb_row, const void *index,
                                        float scale, float max_bias, float logit_softcap,
                                        float *dst, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * The small ops that keep a llama layer on the device (cactus/ggml-cpu/ops.cpp, binary-ops.cpp).
 * All rows are f32 with the given byte strides unless noted.
 * ---------------------------------------------------------------------------------------------- */
/* RMS_NORM (ops.cpp:3268-3316); w may be NULL; with w it also applies the following MUL by a weight row
 * (binary-ops.cpp:152-154), which is how llama builds every norm (cactus/llama-graph.cpp:527-560) */
B200_API int b200_rms_norm(const float *x, int64_t x_nb_row, const float *w, float *dst, int64_t dst_nb_row, int64_t d,
                           int64_t rows, float eps, b200_stream_t stream);
/* ADD / MUL of same-shape contiguous tensors, or with b broadcast along rows when b_rows == 1 */
B200_API int b200_add(const float *a, const float *b, float *dst, int64_t d, int64_t rows, int64_t b_rows, b200_stream_t stream);
B200_API int b200_mul(const float *a, const float *b, float *dst, int64_t d, int64_t rows, int64_t b_rows, b200_stream_t stream);
/* UNARY SILU (ops.cpp:2902-2981); with b != NULL also the following MUL (llama-graph.cpp:619-664) */
B200_API int b200_silu(const float *a, const float *b, float *dst, int64_t n, b200_stream_t stream);
/* ROPE, mode 0 ("norm", adjacent pairs), no YaRN extrapolation (ops.cpp:5080-5118, 5178-5362):
 * x [D, H, T] with byte strides, int32 pos[T]; freq_factors may be NULL; n_dims <= D */
B200_API int b200_rope_norm(const float *x, int64_t x_nb_head, int64_t x_nb_tok, float *dst, int64_t dst_nb_head,
                            int64_t dst_nb_tok, int64_t D, int64_t H, int64_t T, int n_dims, const int32_t *pos,
                            const float *freq_factors, float freq_base, float freq_scale, float attn_factor,
                            b200_stream_t stream);
/* KV-cache maintenance graphs (cactus/llama-kv-cache.cpp:822-926, :928-1210).
 * K-shift: ROPE mode 0 applied in place to the cached f16 keys viewed as [D, Hkv, cells], with the per-cell position
 * shift as `pos` (lm_ggml_compute_forward_rope_f16, cactus/ggml-cpu/ops.cpp:5364-5520: widen to f32, rotate, round to f16).
 * Defragmentation: CPY f16 -> f16 of row ranges of the cache from one run of cells to another. */
B200_API int b200_rope_norm_f16(const void *x, int64_t x_nb_head, int64_t x_nb_tok, void *dst, int64_t dst_nb_head, int64_t dst_nb_tok,
                                int64_t D, int64_t H, int64_t T, int n_dims, const int32_t *pos, const float *freq_factors, float freq_base,
                                float freq_scale, float attn_factor, b200_stream_t stream);
B200_API int b200_cpy_f16_f16(const void *x, int64_t x_nb_row, void *dst, int64_t dst_nb_row, int64_t d, int64_t rows, b200_stream_t stream);
/* CPY f32 -> f16 / f32 -> f32 (ops.cpp:657, :4180): rows of d elements with byte strides on both sides */
B200_API int b200_cpy_f32_f16(const float *x, int64_t x_nb_row, void *dst, int64_t dst_nb_row, int64_t d, int64_t rows,
                              b200_stream_t stream);
B200_API int b200_cpy_f32_f32(const float *x, int64_t x_nb_row, float *dst, int64_t dst_nb_row, int64_t d, int64_t rows,
                              b200_stream_t stream);
/* GET_ROWS (ops.cpp:4236-4403): table f32 (row stride bytes) or tiled quantised weights [d, n_table_rows] */
B200_API int b200_get_rows_f32(const float *table, int64_t table_nb_row, const int32_t *ids, float *dst, int64_t dst_nb_row,
                               int64_t d, int64_t n_ids, b200_stream_t stream);
B200_API int b200_get_rows_q(int wtype, const void *table_tiled, int64_t d, int64_t n_table_rows, const int32_t *ids,
                             float *dst, int64_t dst_nb_row, int64_t n_ids, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * KV-cache bookkeeping on the device (what the reference does on the host around the graph).
 * ---------------------------------------------------------------------------------------------- */
/* llama_kv_cache_unified::set_input_kq_mask (cactus/llama-kv-cache.cpp:696-761), one sequence id per cell,
 * no sliding window: mask f16 [pad64(n_tokens)][n_kv], 0 where cell_seq == tok_seq and cell_pos <= tok_pos,
 * -inf elsewhere and in the padding rows. */
B200_API int b200_kq_mask_build(const int32_t *cell_pos, const int32_t *cell_seq, int64_t n_kv, const int32_t *tok_pos,
                                const int32_t *tok_seq, int64_t n_tokens, void *mask, int64_t mask_nb_row, b200_stream_t stream);
/* dst[idx[i]] = src[i]: records the (pos, seq) of the cells find_slot (llama-kv-cache.cpp:476-569) hands to a ubatch */
B200_API int b200_scatter_i32(int32_t *dst, const int32_t *idx, const int32_t *src, int64_t n, b200_stream_t stream);
/* cpy_k / cpy_v (llama-kv-cache.cpp:617-656): f32 rows -> f16 cache rows slots[r] */
B200_API int b200_set_rows_f16(const float *x, int64_t x_nb_row, const int32_t *slots, void *dst, int64_t dst_nb_row,
                               int64_t d, int64_t rows, b200_stream_t stream);
/* greedy sampling of each logits row (the argmax a caller runs after llama_get_logits,
 * cactus/cactus_completion.cpp:210); ties go to the lowest index */
B200_API int b200_argmax_rows(const float *x, int64_t x_nb_row, int64_t d, int64_t rows, int32_t *out, b200_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Fused forms of the ops between the mul_mats of a llama layer (llm_build_llama, cactus/llama-model.cpp:4517-4671).
 * Each computes bit for bit what the chain of the separate entry points computes; the f32 intermediates that only the
 * next mul_mat would read are not written.
 *
 * b200_add_rms_norm_quantize: x += residual (ADD, cactus/ggml-cpu/ops.cpp:1283-1300; skipped when residual is NULL),
 *   h = rms_norm(x) * w (ops.cpp:3268-3316 + MUL; w may be NULL), h quantised into `scratch` as
 *   b200_quantize_activations would; h itself is stored only when `h` is not NULL.
 * b200_silu_mul_quantize: silu(gate) * up (ops.cpp:2902-2981 + MUL) quantised into `scratch`; the f32 product is stored
 *   only when `dst` is not NULL.
 * b200_rope_store: ROPE (mode 0, as b200_rope_norm) of q in place and of k, with k and v stored as f16 into the cache
 *   rows slots[t] (cpy_k / cpy_v, cactus/llama-kv-cache.cpp:617-656); the f32 k is left as it was.  With slots NULL
 *   token t goes to row t of the k_cache / v_cache pointers given (a ubatch occupies consecutive cells from `head` on).
 * ------------------------------------------------------------------------------------------------ */
B200_API int b200_add_rms_norm_quantize(float *x, int64_t x_nb_row, const float *residual, int64_t residual_nb_row, const float *w, float *h,
                                        int64_t h_nb_row, int64_t d, int64_t rows, float eps, void *scratch, size_t scratch_bytes,
                                        int variant, b200_stream_t stream);
B200_API int b200_silu_mul_quantize(const float *gate, const float *up, int64_t nb_row, float *dst, int64_t dst_nb_row, int64_t K, int64_t N,
                                    void *scratch, size_t scratch_bytes, int variant, b200_stream_t stream);
B200_API int b200_rope_store(float *q, int64_t q_nb_head, int64_t q_nb_tok, const float *k, int64_t k_nb_head, int64_t k_nb_tok,
                             const float *v, int64_t v_nb_tok, int64_t D, int64_t H, int64_t Hkv, int64_t T, int n_dims, const int32_t *pos,
                             const float *freq_factors, float freq_base, float freq_scale, float attn_factor, const int32_t *slots,
                             void *k_cache, int64_t k_cache_nb_row, void *v_cache, int64_t v_cache_nb_row, b200_stream_t stream);
/* the same with the rotated q written to q_dst (same strides as q; q_dst == q is the call above): the ROPE node of a
 * graph whose allocator did not place the result over its source.  H = 0 (q, q_dst NULL) leaves q out, v NULL leaves
 * the V store out: ROPE(k) + K store alone, what a graph_compute can run in the place of the ROPE(k) node. */
B200_API int b200_rope_store_to(const float *q, float *q_dst, int64_t q_nb_head, int64_t q_nb_tok, const float *k, int64_t k_nb_head,
                                int64_t k_nb_tok, const float *v, int64_t v_nb_tok, int64_t D, int64_t H, int64_t Hkv, int64_t T, int n_dims,
                                const int32_t *pos, const float *freq_factors, float freq_base, float freq_scale, float attn_factor,
                                const int32_t *slots, void *k_cache, int64_t k_cache_nb_row, void *v_cache, int64_t v_cache_nb_row,
                                b200_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Row-split mul_mat over the GPUs of one node (one process per GPU).
 *
 * The reference splits the rows of mul_mat weights over devices with a split buffer type
 * (lm_ggml_backend_split_buffer_type, cactus/ggml-backend.h:188; requested by the loader for
 * LLAMA_SPLIT_MODE_ROW, cactus/llama-model.cpp:339-351) and leaves the join to the backend.  Here each process
 * computes its row range with b200_mul_mat_q* on a row slice of the weight (a slice on 16-row boundaries of a tiled
 * weight is two byte ranges: quants, scales) and b200_allgather_rows joins the slices: it stores the caller's
 * [T, M/g] slice at column rank*M/g of every rank's [T, M] buffer over NVLink and returns (in stream order) once
 * every rank's slice has arrived in the caller's buffer.
 *
 * b200_peer_alloc allocates (zeroed) device memory that other processes can map: the 64-byte handle is passed to them
 * by any host channel and opened with b200_peer_open.  Every rank allocates one dst region and one 64-byte flag block
 * this way; dst_of_rank[r] / flags_of_rank[r] are rank r's dst buffer and flag block as mapped in the calling process
 * (the caller's own allocation at index `rank`).  All ranks must issue the same sequence of b200_allgather_rows calls.
 * The wait for the peers is bounded (seconds); b200_peer_status(own flag block) returns 0, or 1 + the first rank whose
 * slice did not arrive.
 * ------------------------------------------------------------------------------------------------ */
B200_API int b200_peer_alloc(size_t bytes, void **ptr, unsigned char handle[64]);
B200_API int b200_peer_open(const unsigned char handle[64], void **ptr);
B200_API int b200_peer_close(void *ptr);
B200_API int b200_peer_free(void *ptr);
B200_API int b200_allgather_rows(const float *src, int64_t src_nb_row, int64_t T, int64_t Mg, int rank, int g, void *const *dst_of_rank,
                                 int64_t dst_nb_row, void *const *flags_of_rank, b200_stream_t stream);
B200_API int b200_peer_status(const void *flags);
/* The number of polls (about 100 ns each) after which the wait for a peer gives up; 0 restores the default (seconds).
 * Also clears the status of the flag block.  A rank that left between steps is noticed this way: the next collective of
 * the others returns after the limit with b200_peer_status = 1 + that rank, and their contexts stay usable. */
B200_API int b200_peer_set_wait_limit(void *flags, unsigned polls);
/* mul_mat and join in one step: b200_mul_mat_q_prequant on this rank's row slice (M rows, the columns first_column ..
 * first_column + M - 1 of the full product), with the kernel's own write-back storing every value into dst_of_rank[r]
 * of all g ranks, followed by the flag exchange of b200_allgather_rows.  dst_of_rank[r] is rank r's full [N, *] buffer. */
B200_API int b200_mul_mat_q_rowsplit(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N, int rank, int g,
                                     void *const *dst_of_rank, int64_t dst_row_stride_bytes, int64_t first_column, void *workspace,
                                     size_t workspace_bytes, void *const *flags_of_rank, b200_stream_t stream);
/* The same for a stacked weight of this rank (its rows of wq, wk, wv one after the other, or of gate and up): part i
 * holds part_rows[i] rows (a multiple of 16 but for the last) that belong at columns part_first_column[i] ... of the
 * joined output; one product and one flag exchange instead of one per tensor. */
B200_API int b200_mul_mat_q_rowsplit_stacked(int wtype, const void *w, int64_t K, int64_t M, const void *act, int64_t N, int rank, int g,
                                             void *const *dst_of_rank, int64_t dst_row_stride_bytes, int n_parts, const int64_t *part_rows,
                                             const int64_t *part_first_column, void *workspace, size_t workspace_bytes,
                                             void *const *flags_of_rank, b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
