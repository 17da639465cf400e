/*
 * rnb_b200 — C ABI of the sm_100a batch-1 decode/prefill operator library.
 *
 * Drop-in boundary: runNburn has no C ABI for its CUDA operators; what `rnb-runtime` and
 * `rnb-llm` call is the set of Rust free functions that `rnb_backend_cuda` re-exports
 * (crates/rnb-backend/cuda/src/lib.rs:44-175).  Each entry point below replaces one of
 * those functions (cited per declaration, paths relative to the reference project):
 * slices become (pointer, length), `Result<_, String>` becomes an int status plus
 * rnb_b200_last_error(), and `Vec<f32>` results become caller-provided buffers.
 *
 * Conventions kept from the reference:
 *  - weight slices are borrowed host memory (the GGUF mmap) that outlives the call; the
 *    library owns every device copy and keys it by (host address, length);
 *  - shape errors are reported before any CUDA call, with the reference's messages;
 *  - host-returning calls synchronise their stream before returning; `_dev` calls do not;
 *  - callable from any thread; calls are serialised on one process-wide lock;
 *  - device selection by the RNB_CUDA_DEVICE environment variable (default 0);
 *  - there is no CPU fallback: without a usable CUDA device every compute call fails.
 */
#ifndef RNB_B200_H
#define RNB_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes — DeviceOpStatus, crates/rnb-backend/api/src/lib.rs:205-211, plus CUDA errors */
#define RNB_B200_OK 0
#define RNB_B200_UNSUPPORTED 1
#define RNB_B200_VALIDATION_FAILED 2
#define RNB_B200_OUT_OF_MEMORY 3
#define RNB_B200_CUDA_ERROR 4
#define RNB_B200_DEVICE_FAULT_FLAG 5 /* a kernel reported a bounded wait that gave up */

/* GGML type ids used by `down_quant: u32` arguments */
#define RNB_B200_TYPE_Q8_0 8u
#define RNB_B200_TYPE_Q4_K 12u
#define RNB_B200_TYPE_Q6_K 14u

/* Message of the last failing call on this thread (never NULL). */
const char *rnb_b200_last_error(void);

/* CudaState::open — crates/rnb-backend/cuda/src/runtime/state/init.rs:86-139.  Every compute
 * call opens the state lazily; calling this first only moves the cost. */
int rnb_b200_open(void);
/* Drop for CudaState — state/init.rs:446-857: frees every device allocation. */
void rnb_b200_close(void);
/* cuda_memory_info — api/cache_api.rs:97 */
int rnb_b200_cuda_memory_info(size_t *free_bytes, size_t *total_bytes);
int rnb_b200_device_sm_count(int *sm_count);

/* ---- resident weight cache -------------------------------------------------------------- */
/* cuda_cache_snapshot / cuda_weight_residency_counters — api/cache_api.rs:114,147;
 * DeviceTransferCounters — crates/rnb-backend/api/src/lib.rs:213-242 */
typedef struct {
    uint64_t lookups, hits, misses, evictions, uploads, upload_bytes, transient_uploads;
    uint64_t resident_entries, resident_bytes, resident_limit_bytes;
    uint64_t h2d_bytes, d2h_bytes;
} rnb_b200_cache_snapshot;
int rnb_b200_cuda_cache_snapshot(rnb_b200_cache_snapshot *out);
/* clear_q4k_cache — api/cache_api.rs:18 */
int rnb_b200_clear_q4k_cache(void);
/* reset_state_for_engine_init — api/cache_api.rs:83 */
int rnb_b200_reset_state_for_engine_init(void);
/* prewarm_q4k_weights(&[&[u8]]) -> usize — api/quant_api.rs:952-971 */
int rnb_b200_prewarm_q4k_weights(const uint8_t *const *slices, const size_t *lens, size_t n,
                                 size_t *n_resident);
/* Residency budget override in bytes (0 = derive from free memory as
 * DeviceResidencyPlan does — crates/rnb-memory/src/device_residency.rs:40-91). */
int rnb_b200_set_resident_limit(size_t bytes);
/* inject_qwen35_resident_alloc_ooms_for_test — crates/rnb-backend/cuda/src/runtime/state/
 * q4k_cache.rs:1040-1053: the next `count` device allocations of the resident cache report
 * out-of-memory without touching the driver, so the evict-and-retry ladder
 * (q4k_cache.rs:757-851) can be driven from a test.  Host-side fault injection only. */
int rnb_b200_inject_resident_alloc_ooms_for_test(size_t count);
/* host_register.rs:45-190 — pin the page-aligned interior of a host range for async DMA;
 * clear_host_registered_ranges — api/cache_api.rs */
int rnb_b200_register_host_range(const void *ptr, size_t len);
int rnb_b200_clear_host_registered_ranges(void);

/* ---- Q8_K activation quantisation --------------------------------------------------------
 * quantize_input_q8k_into — crates/rnb-cpu/src/gemm/activation_q8.rs:122-139 (the reference
 * quantises activations on the host; this path does it on the device, bit-exactly).
 * `blocks_out` receives n/256 blocks of 292 bytes (f32 d, i8 qs[256], i16 bsums[16]). */
int rnb_b200_quantize_q8k(const float *input, size_t n, void *blocks_out);

/* ---- quantised matvec -------------------------------------------------------------------- */
/* q4k_gemv / q4k_gemv_into — api/quant_api.rs:183-218,220 */
int rnb_b200_q4k_gemv(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                      const float *input, size_t input_len, float *output, size_t output_len);
/* Q5_K (GGML type 13, 176-byte blocks) beside the Q4_K_M set: the CPU's dispatch
 * (crates/rnb-cpu/src/gemm/quant_gemv.rs:94-101, QuantGemvType::Q5K -> dot_q5k_q8k_avx2,
 * crates/rnb-cpu/src/gemm/avx2_dot.rs:698-789), bit-exact; `down_quant` 13 of
 * rnb_b200_dense_q4k_silu_ffn_batch takes the same kernel.  _batch: input [seq][cols], output
 * seq-major. */
/* Q2_K (GGML type 10, 84-byte blocks): QuantGemvType::Q2K -> dot_q2k_q8k_avx2
 * (crates/rnb-cpu/src/gemm/avx2_dot.rs:169-245), bit-exact */
int rnb_b200_q2k_gemv(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                      const float *input, size_t input_len, float *output, size_t output_len);
int rnb_b200_q2k_gemv_batch(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                            const float *input, size_t input_len, float *output, size_t output_len);
/* Q3_K (GGML type 11, 110-byte blocks, 2-byte aligned): QuantGemvType::Q3K -> dot_q3k_q8k_avx2
 * (crates/rnb-cpu/src/gemm/avx2_dot.rs:247-378), bit-exact */
int rnb_b200_q3k_gemv(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                      const float *input, size_t input_len, float *output, size_t output_len);
int rnb_b200_q3k_gemv_batch(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                            const float *input, size_t input_len, float *output, size_t output_len);
int rnb_b200_q5k_gemv(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                      const float *input, size_t input_len, float *output, size_t output_len);
int rnb_b200_q5k_gemv_batch(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                            const float *input, size_t input_len, float *output, size_t output_len);
/* q6k_gemv — api/quant_api.rs:2071-2106 */
int rnb_b200_q6k_gemv(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                      const float *input, size_t input_len, float *output, size_t output_len);
/* q8_0_gemv — api/quant_api.rs:498-505 (f32 activations, as rnb-cpu's x86 path) */
int rnb_b200_q8_0_gemv(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                       const float *input, size_t input_len, float *output, size_t output_len);
/* q4k_gemv_with_device_input — api/quant_api.rs:288; q6k_… — :242.  `input_dev` is a device
 * address of `cols` f32 values. */
int rnb_b200_q4k_gemv_with_device_input(const uint8_t *weights, size_t weights_len, size_t rows,
                                        size_t cols, uint64_t input_dev, float *output,
                                        size_t output_len);
int rnb_b200_q6k_gemv_with_device_input(const uint8_t *weights, size_t weights_len, size_t rows,
                                        size_t cols, uint64_t input_dev, float *output,
                                        size_t output_len);
/* q6k_gemv_argmax -> (u32, f32) — api/quant_api.rs:2170.  Ties resolve to the LAST index, the
 * rule of the reference's CPU sampler (crates/rnb-llm/src/sampler/greedy.rs:4-11). */
int rnb_b200_q6k_gemv_argmax(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                             const float *input, size_t input_len, uint32_t *index_out,
                             float *value_out);
/* q8_0_gemv_argmax -> (u32, f32) and q8_0_gemv_batch — api/quant_api.rs:733,807: the Q8_0 LM head
 * and the batched Q8_0 matvec (input [seq][cols], output [seq][rows]); same tie rule. */
int rnb_b200_q8_0_gemv_argmax(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                              const float *input, size_t input_len, uint32_t *index_out,
                              float *value_out);
int rnb_b200_q8_0_gemv_batch(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                             const float *input, size_t input_len, float *output, size_t output_len);
/* q4k_gemv_batch / q6k_gemv_batch — api/quant_api.rs:2283,3919: input [seq][cols], output
 * seq-major [seq][rows]. */
int rnb_b200_q4k_gemv_batch(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                            const float *input, size_t input_len, float *output,
                            size_t output_len);
int rnb_b200_q6k_gemv_batch(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                            const float *input, size_t input_len, float *output,
                            size_t output_len);
/* q4k_f16_qkv_gemm_batch(q_weights, k_weights, v_weights, q_rows, kv_rows, cols, input) ->
 * (q, k, v) — api/quant_api.rs:2405-2463: the three Q4_K projections of a token batch behind one
 * token matrix; here one tcgen05 launch (bf16 x bf16, f32 accumulate).  Outputs [seq][q_rows],
 * [seq][kv_rows], [seq][kv_rows]. */
int rnb_b200_q4k_bf16_qkv_gemm_batch(const uint8_t *q_weights, size_t q_weights_len,
                                     const uint8_t *k_weights, size_t k_weights_len,
                                     const uint8_t *v_weights, size_t v_weights_len, size_t q_rows,
                                     size_t kv_rows, size_t cols, const float *input,
                                     size_t input_len, float *q_out, size_t q_out_len,
                                     float *k_out, size_t k_out_len, float *v_out,
                                     size_t v_out_len);
/* q4k_f16_gemm_batch — api/quant_api.rs:2364 (runtime/gemv.rs:2335-2421: dequant -> f16 +
 * cublasGemmEx with f32 accumulation).  Here: weights dequantised tile-wise to bf16 inside a
 * tcgen05 kernel, tokens rounded to bf16, f32 accumulators in tensor memory.  Same argument
 * meaning and [seq][rows] output as the batch matvecs; a Q6_K twin for attn_v / ffn_down /
 * output weights. */
int rnb_b200_q4k_bf16_gemm_batch(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                                 const float *input, size_t input_len, float *output,
                                 size_t output_len);
int rnb_b200_q6k_bf16_gemm_batch(const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                                 const float *input, size_t input_len, float *output,
                                 size_t output_len);

/* quant_embedding_gather(quant, weights, rows, cols, token_ids) — api/quant_api.rs:1827-1905:
 * out [n_tokens][cols] f32 = the dequantised rows token_ids[i] of a quantised embedding table
 * (bit-identical to the CPU dequantisers).  quant: RNB_B200_TYPE_Q8_0 / Q4_K / Q6_K, cols a multiple
 * of 256; other types RNB_B200_UNSUPPORTED; an id >= rows RNB_B200_VALIDATION_FAILED; no tokens:
 * nothing written. */
int rnb_b200_quant_embedding_gather(uint32_t quant, const uint8_t *weights, size_t weights_len,
                                    size_t rows, size_t cols, const uint32_t *token_ids,
                                    size_t n_tokens, float *out, size_t out_len);

/* ---- attention ---------------------------------------------------------------------------- */
/* attention_decode_hd128 — api/attention_api.rs:1943-1978.  q f32[heads*128]; k, v f16 bits
 * [kv_len][kv_heads][128]; out f32[heads*128]. */
int rnb_b200_attention_decode_hd128(const float *q, size_t q_len, const uint16_t *k,
                                    const uint16_t *v, size_t kv_elems, size_t kv_len,
                                    size_t num_heads, size_t num_kv_heads, float scale,
                                    float *out, size_t out_len);
/* attention_decode_hd256 / attention_decode_hd512 — api/attention_api.rs:1906-1941,1980-2015: the
 * same call for head_dim 256 and 512 (q f32[heads*D]; k, v f16 bits [kv_len][kv_heads][D]).  fp32
 * split-KV on CUDA cores: within 1e-3 of the CPU routine, not tuned. */
int rnb_b200_attention_decode_hd256(const float *q, size_t q_len, const uint16_t *k,
                                    const uint16_t *v, size_t kv_elems, size_t kv_len,
                                    size_t num_heads, size_t num_kv_heads, float scale,
                                    float *out, size_t out_len);
int rnb_b200_attention_decode_hd512(const float *q, size_t q_len, const uint16_t *k,
                                    const uint16_t *v, size_t kv_elems, size_t kv_len,
                                    size_t num_heads, size_t num_kv_heads, float scale,
                                    float *out, size_t out_len);
/* attention_decode_cached — api/attention_api.rs:2055-2102 (runtime/attention.rs:3913-4291):
 * per-layer device KV mirror keyed by the host K/V base addresses; only rows the mirror does
 * not hold yet are uploaded. */
int rnb_b200_attention_decode_cached(size_t layer_index, const float *q, size_t q_len,
                                     const uint16_t *k, const uint16_t *v, size_t kv_elems,
                                     size_t kv_len, size_t num_heads, size_t num_kv_heads,
                                     size_t head_dim, float scale, float *out, size_t out_len);
/* attention_decode_cached_window(layer_index, q, k, v, kv_len, window_start, window_len, num_heads,
 * num_kv_heads, head_dim, scale) — api/attention_api.rs:2105-2163: sliding-window decode; attention
 * over positions [window_start, window_start + window_len) of the mirrored cache.  With
 * window_start + window_len == kv_len the result equals the CPU routine's with
 * sliding_window = window_len (crates/rnb-cpu/src/kernels/attention/decode_flash.rs:139-146: masked
 * positions score -inf and contribute exact zeros).  An empty or out-of-range window is
 * RNB_B200_VALIDATION_FAILED. */
int rnb_b200_attention_decode_cached_window(size_t layer_index, const float *q, size_t q_len,
                                            const uint16_t *k, const uint16_t *v, size_t kv_elems,
                                            size_t kv_len, size_t window_start, size_t window_len,
                                            size_t num_heads, size_t num_kv_heads, size_t head_dim,
                                            float scale, float *out, size_t out_len);
/* clear_decode_attention_kv_cache — api/cache_api.rs:136 */
int rnb_b200_clear_decode_attention_kv_cache(void);
/* attention_prefill_flash_hd128 — api/attention_api.rs:661-700: causal, query i sees keys
 * 0..(kv_len - seq_len + i); q f32 [seq][heads][128]; k, v f32 [kv_len][kv_heads][128]. */
int rnb_b200_attention_prefill_flash_hd128(const float *q, const float *k, const float *v,
                                           size_t seq_len, size_t kv_len, size_t num_heads,
                                           size_t num_kv_heads, float scale, float *out);
/* The same with an f16 cache (bit patterns), k, v [kv_len][kv_heads][128] — the layout and
 * argument order of the reference's f16-KV prefill operators (attention_prefill_flash_hd512_f16kv,
 * api/attention_api.rs:43-89) at head dimension 128.  Runs the query-tiled tensor-core kernel. */
int rnb_b200_attention_prefill_flash_hd128_f16kv(const float *q, const uint16_t *k, const uint16_t *v,
                                                 size_t seq_len, size_t kv_len, size_t num_heads,
                                                 size_t num_kv_heads, float scale, float *out);
/* dense_q4k_attention_qkv(q_weights, k_weights, v_weights, q_rows, kv_rows, n_embd, input, q, k, v)
 * — api/dense_api.rs:916-986: the three projections of one token in one launch, no RoPE; each
 * output equals the single-matrix matvec's bit for bit.  A GGML type id per matrix (Q4_K_M keeps
 * attn_v in Q6_K). */
int rnb_b200_dense_attention_qkv(const uint8_t *q_w, size_t q_w_len, uint32_t q_type,
                                 const uint8_t *k_w, size_t k_w_len, uint32_t k_type,
                                 const uint8_t *v_w, size_t v_w_len, uint32_t v_type, size_t q_rows,
                                 size_t kv_rows, size_t n_embd, const float *input,
                                 size_t input_len, float *q, size_t q_len, float *k, size_t k_len,
                                 float *v, size_t v_len);
/* dense_q4k_attention_qkv_rope_hd128_decode — api/dense_api.rs:988-1074: q/k/v matvec,
 * adjacent-pair RoPE on q and k at position pos_start, K/V rounded to f16.  Weight types are
 * given per matrix (the reference's name says Q4_K; Q4_K_M files carry Q6_K in attn_v). */
int rnb_b200_dense_attention_qkv_rope_hd128_decode(
    const uint8_t *q_w, size_t q_w_len, uint32_t q_type, const uint8_t *k_w, size_t k_w_len,
    uint32_t k_type, const uint8_t *v_w, size_t v_w_len, uint32_t v_type, size_t q_rows,
    size_t kv_rows, size_t n_embd, size_t num_heads, size_t num_kv_heads, float rope_theta,
    size_t pos_start, const float *input, float *q_rope, uint16_t *k_bits, uint16_t *v_bits);
/* dense_q4k_silu_ffn_batch — api/dense_api.rs:297-339: down(silu(gate x) * (up x)),
 * seq-major [seq][n_embd] */
int rnb_b200_dense_q4k_silu_ffn_batch(const uint8_t *gate, size_t gate_len, const uint8_t *up,
                                      size_t up_len, const uint8_t *down, size_t down_len,
                                      uint32_t down_quant, size_t n_ff, size_t n_embd,
                                      size_t seq_len, const float *input, float *output);

/* ---- MoE ---------------------------------------------------------------------------------- */
/* moe_route_topk_f32 — api/dense_api.rs:1834 (kernel quant_batch_and_ops.cuh:4782-4912).
 * Softmax mode only (sigmoid_mode != 0 → RNB_B200_UNSUPPORTED).  ids/weights: [seq][top_k],
 * retained_counts: [seq]. */
int rnb_b200_moe_route_topk_f32(const float *logits, size_t logits_len,
                                const float *selection_bias, size_t seq_len, size_t n_expert,
                                size_t top_k, int sigmoid_mode, int normalize_selected,
                                float scale, float adaptive_top_p, uint32_t *ids_out,
                                float *weights_out, uint32_t *retained_counts_out);
/* Router logits f32 [n_expert][hidden] x h, in the summation order of the reference's host
 * gemv_f32 (crates/rnb-cpu/src/gemm/f32_gemv.rs:215-237), bit-exact. */
int rnb_b200_router_logits_f32(const float *router_w, size_t n_expert, size_t hidden,
                               const float *h, float *logits_out);
/* qwen35_expert(gate, up, down, down_quant, n_ff, n_embd, input) — api/qwen_moe_api.rs:1566: one
 * expert's FFN, down(silu(gate x) * (up x)). */
int rnb_b200_qwen35_expert(const uint8_t *gate, size_t gate_len, const uint8_t *up, size_t up_len,
                           const uint8_t *down, size_t down_len, uint32_t down_quant, size_t n_ff,
                           size_t n_embd, const float *input, size_t input_len, float *output,
                           size_t output_len);
/* qwen35_sparse_experts_by_token(gate, up, down, route_weights, token_ids, token_count, down_quant,
 * n_ff, n_embd, input) — api/qwen_moe_api.rs:2477: a batch of tokens; slot s applies its expert to
 * token token_ids[s] with weight route_weights[s]; output [token_count][n_embd], a token's slots
 * summed in slot order, zero for a token without slots (and for no slots at all). */
int rnb_b200_qwen35_sparse_experts_by_token(const uint8_t *const *gate, const uint8_t *const *up,
                                            const uint8_t *const *down, size_t gate_slice_len,
                                            size_t down_slice_len, const float *route_weights,
                                            const uint32_t *token_ids, size_t n_slots,
                                            size_t token_count, uint32_t down_quant, size_t n_ff,
                                            size_t n_embd, const float *input, size_t input_len,
                                            float *output, size_t output_len);
/* qwen35_sparse_experts — api/qwen_moe_api.rs:1712-1803: out = sum_e w_e * Down_e(silu(Gate_e
 * x) * (Up_e x)) over the routed experts, summed in selection order.  gate/up are Q4_K,
 * down is `down_quant`. */
int rnb_b200_qwen35_sparse_experts(const uint8_t *const *gate, const uint8_t *const *up,
                                   const uint8_t *const *down, size_t gate_slice_len,
                                   size_t down_slice_len, const float *route_weights,
                                   size_t n_selected, uint32_t down_quant, size_t n_ff,
                                   size_t n_embd, const float *input, float *output);
/* qwen35_register_moe_layer — api/qwen_moe_api.rs:1502-1553: uploads one layer's stacked
 * expert tensors without evicting; *fitted = 0 when it did not fit. */
int rnb_b200_qwen35_register_moe_layer(const uint8_t *gate_all, size_t gate_len,
                                       const uint8_t *up_all, size_t up_len,
                                       const uint8_t *down_all, size_t down_len,
                                       uint32_t down_quant, size_t n_ff, size_t n_embd,
                                       int *fitted);

/* ---- glue ops ------------------------------------------------------------------------------ */
/* rms_norm_rows_f32 — api/dense_api.rs:2527 (CPU formula: f64 mean square, (x/rms)*w) */
int rnb_b200_rms_norm_rows_f32(const float *input, const float *weight, size_t hidden,
                               size_t rows, float eps, float *output);
/* rope_f32_inplace — api/dense_api.rs:2001 (adjacent pairs; neox != 0 → half-split) */
int rnb_b200_rope_f32_inplace(float *data, size_t n, size_t pos_start, size_t head_dim,
                              size_t dim, float theta, int neox);
/* activation_mul_f32_inplace — api/dense_api.rs:1331: gate = silu(gate) * up */
int rnb_b200_activation_mul_f32_inplace(float *gate, const float *up, size_t n);

/* ---- expert-cache bookkeeping (host only; crates/rnb-memory/src/sparse_expert_cache.rs) ---- */
typedef struct {
    uint64_t missing_bytes, eviction_reload_bytes;
    uint32_t predicted_future_reuses, replaces_temp_upload;
} rnb_b200_bundle_admission;
/* evaluate_expert_bundle_admission — sparse_expert_cache.rs:221-245: 1 = admit */
int rnb_b200_evaluate_expert_bundle_admission(const rnb_b200_bundle_admission *a);
/* ---- expert-bundle cache bookkeeping (host accounting only) ---------------------------------------
 * crates/rnb-memory/src/sparse_expert_cache.rs.  Keys are (layer, expert), ordered layer first. */
/* ExpertBundleReuseHistory — :272-393.  observe() returns the decayed frequency before this
 * lookup; frequency halves once per `decay_interval` (default = capacity, at least 1) epochs
 * spent unobserved; over capacity the minimum of (effective frequency, last-seen epoch, key)
 * goes.  decay_interval 0 on create selects the default. */
typedef struct rnb_b200_expert_history rnb_b200_expert_history;
typedef struct {
    uint64_t capacity, decay_interval, epoch, len;
} rnb_b200_expert_history_info;
int rnb_b200_expert_history_create(size_t capacity, uint64_t decay_interval, rnb_b200_expert_history **out);
void rnb_b200_expert_history_destroy(rnb_b200_expert_history *h);
uint64_t rnb_b200_expert_history_observe(rnb_b200_expert_history *h, uint32_t layer, uint32_t expert);
void rnb_b200_expert_history_set_capacity(rnb_b200_expert_history *h, size_t capacity);
int rnb_b200_expert_history_contains(const rnb_b200_expert_history *h, uint32_t layer, uint32_t expert);
void rnb_b200_expert_history_get_info(const rnb_b200_expert_history *h, rnb_b200_expert_history_info *out);
void rnb_b200_expert_history_set_epoch_for_test(rnb_b200_expert_history *h, uint64_t epoch);
/* SparseExpertCacheBudget over ByteLruPolicy — :505-530, crates/rnb-memory/src/byte_lru.rs:17-116:
 * byte-budgeted LRU accounting; touch() returns the keys to reclaim as (layer << 32) | expert. */
typedef struct rnb_b200_expert_budget rnb_b200_expert_budget;
int rnb_b200_expert_budget_create(uint64_t max_bytes, rnb_b200_expert_budget **out);
void rnb_b200_expert_budget_destroy(rnb_b200_expert_budget *b);
int rnb_b200_expert_budget_touch(rnb_b200_expert_budget *b, uint32_t layer, uint32_t expert, uint64_t bytes,
                                 uint64_t *evicted, size_t cap, size_t *n_evicted);
int rnb_b200_expert_budget_remove(rnb_b200_expert_budget *b, uint32_t layer, uint32_t expert);
uint64_t rnb_b200_expert_budget_resident_bytes(const rnb_b200_expert_budget *b);
/* evaluate_expert_bundle_admission with its whole cost record — :221-270.  The 128-bit fields of
 * ExpertBundleAdmissionCost come back as (lo, hi) pairs; residency: 0 full, 1 partial, 2 miss. */
typedef struct {
    uint64_t gate_bytes, up_bytes, down_bytes;
    uint32_t gate_resident, up_resident, down_resident, replaces_temp_upload;
    uint64_t predicted_future_reuses, eviction_reload_bytes;
} rnb_b200_bundle_candidate;
typedef struct {
    uint32_t admit, profitable, residency, reserved;
    uint64_t missing_admission_bytes, eviction_reload_bytes, predicted_future_reuses;
    uint64_t predicted_saved_lo, predicted_saved_hi;
    uint64_t net_saved_lo;
    int64_t net_saved_hi;
} rnb_b200_bundle_decision;
int rnb_b200_evaluate_expert_bundle(const rnb_b200_bundle_candidate *c, rnb_b200_bundle_decision *out);
/* ExpertBundleCacheStats, ExpertBundleObservationReceipt — :395-500 (saturating counters) */
typedef struct {
    uint64_t bundle_lookups, bundle_hits, bundle_partial_hits, bundle_misses, bundle_admissions,
        bundle_evictions, admitted_bytes, evicted_bytes, h2d_bytes, temp_h2d_bytes;
} rnb_b200_expert_bundle_stats;
typedef struct {
    uint32_t consumed, reserved;
    rnb_b200_expert_bundle_stats pending_stats;
} rnb_b200_expert_bundle_receipt;
void rnb_b200_expert_stats_record_lookup(rnb_b200_expert_bundle_stats *s, int gate_resident, int up_resident, int down_resident);
void rnb_b200_expert_stats_delta(const rnb_b200_expert_bundle_stats *after, const rnb_b200_expert_bundle_stats *before,
                                 rnb_b200_expert_bundle_stats *out);
void rnb_b200_expert_stats_add(rnb_b200_expert_bundle_stats *acc, const rnb_b200_expert_bundle_stats *delta);
void rnb_b200_expert_receipt_record(rnb_b200_expert_bundle_receipt *r, const rnb_b200_expert_bundle_stats *stats);
void rnb_b200_expert_receipt_mark_consumed(rnb_b200_expert_bundle_receipt *r);
void rnb_b200_expert_receipt_clear_stats(rnb_b200_expert_bundle_receipt *r);
/* qwen35_moe_layer_cache_limit / qwen35_moe_transient_reserve_bytes —
 * crates/rnb-backend/cuda/src/runtime/state/moe_cache.rs:6-29 */
uint64_t rnb_b200_qwen35_moe_layer_cache_limit(uint64_t model_moe_bytes, uint64_t free_bytes,
                                               uint64_t device_resident_limit_bytes, uint64_t requested_bytes,
                                               uint64_t runtime_headroom_bytes);
uint64_t rnb_b200_qwen35_moe_transient_reserve_bytes(uint64_t dynamic_reserve_bytes, uint64_t model_moe_bytes,
                                                     uint64_t resident_moe_bytes, uint64_t min_layer_bytes);
/* DeviceResidencyPlan::from_snapshot — crates/rnb-memory/src/device_residency.rs:40-91:
 * resident_limit = free - reserve, reserve = clamp(ceil_256MiB(total/16), 512 MiB, 2 GiB) */
uint64_t rnb_b200_resident_limit_for(uint64_t total_bytes, uint64_t free_bytes);

/* ---- the rest of the operator boundary ---------------------------------------------------------
 * add_f32_inplace(dst, src) — api/dense_api.rs:1389 (same messages: shape mismatch, u32 overflow) */
int rnb_b200_add_f32_inplace(float *dst, size_t dst_len, const float *src, size_t src_len);
/* upload_device_tensor_f32(desc, input) -> DeviceTensorId, download_device_tensor_f32(id),
 * download_device_tensor_f32_row(id, row), release_device_tensor(id) -> bool —
 * api/sequence_api.rs:4-56; DeviceTensorDesc{rows, cols, dtype f32, role} and DeviceTensorId{backend,
 * raw} of crates/rnb-backend/api/src/lib.rs:132-203: `id` is the raw handle, `role` the
 * DeviceTensorRole discriminant (kept, not interpreted).  device_tensor_ptr exposes the device
 * address for calls that take `*_dev` arguments. */
int rnb_b200_upload_device_tensor_f32(size_t rows, size_t cols, uint32_t role, const float *data, size_t len, uint64_t *id_out);
int rnb_b200_download_device_tensor_f32(uint64_t id, float *out, size_t out_len);
int rnb_b200_download_device_tensor_f32_row(uint64_t id, size_t row, float *out, size_t out_len);
int rnb_b200_release_device_tensor(uint64_t id, int *released);
int rnb_b200_device_tensor_ptr(uint64_t id, uint64_t *dev_ptr, size_t *rows, size_t *cols);
/* acquire_decode_{hidden,norm_buf,k,v,k_f16,v_f16,attn_out}_carrier(bytes) -> u64,
 * upload_to_decode_hidden_carrier(host, dev), download_from_decode_hidden_carrier(dev, host),
 * sync_decode_stream() — api/dense_api.rs:1176-1330,2428.  One entry point with the carrier kind;
 * uploads and downloads are asynchronous on the decode stream as the reference's are (the host buffer
 * stays the caller's until rnb_b200_sync_decode_stream). */
enum {
    RNB_B200_CARRIER_HIDDEN = 0, RNB_B200_CARRIER_NORM_BUF = 1, RNB_B200_CARRIER_K = 2, RNB_B200_CARRIER_V = 3,
    RNB_B200_CARRIER_K_F16 = 4, RNB_B200_CARRIER_V_F16 = 5, RNB_B200_CARRIER_ATTN_OUT = 6, RNB_B200_CARRIER_KINDS = 7
};
int rnb_b200_acquire_decode_carrier(uint32_t kind, size_t bytes, uint64_t *dev_out);
int rnb_b200_upload_to_decode_carrier(const void *host, size_t bytes, uint64_t dev);
int rnb_b200_download_from_decode_carrier(uint64_t dev, void *host, size_t bytes);
int rnb_b200_sync_decode_stream(void);
/* attention_decode_cached_to_device(layer_index, q, k, v, kv_len, num_heads, num_kv_heads, head_dim,
 * scale, output_dev_target, last_token_k_dev: Option<u64>, last_token_v_dev, q_dev_override) —
 * api/attention_api.rs:1776: the result stays at `output_dev` (f32 [heads][128]) and the call does
 * not synchronise; 0 stands for None.  With last-token device rows the newest K/V row is copied
 * device to device into the layer's mirror instead of uploaded. */
int rnb_b200_attention_decode_cached_to_device(size_t layer, const float *q, size_t q_len, const uint16_t *k, const uint16_t *v, size_t kv_elems,
                                               size_t kv_len, size_t heads, size_t kv_heads, size_t head_dim, float scale, uint64_t output_dev,
                                               uint64_t last_token_k_dev, uint64_t last_token_v_dev, uint64_t q_dev_override);
/* dense_q4k_attention_qkv_rope_hd128_prefill(.., seq_len, ..) — api/dense_api.rs:1075: input
 * [seq][n_embd], q_rope [seq][q_rows], k_bits / v_bits [seq][kv_rows]; token s sits at position
 * pos_start + s. */
int rnb_b200_dense_attention_qkv_rope_hd128_prefill(const uint8_t *q_w, size_t q_w_len, uint32_t q_type, const uint8_t *k_w, size_t k_w_len,
                                                    uint32_t k_type, const uint8_t *v_w, size_t v_w_len, uint32_t v_type, size_t q_rows,
                                                    size_t kv_rows, size_t n_embd, size_t num_heads, size_t num_kv_heads, float rope_theta,
                                                    size_t pos_start, size_t seq_len, const float *input, size_t input_len, float *q_rope,
                                                    uint16_t *k_bits, uint16_t *v_bits);
/* qwen35_sparse_experts_into / qwen35_sparse_experts_add_residual_into(gate, up, down, route_weights,
 * layer_idx: Option<usize>, selected_expert_ids, receipt: &mut ExpertBundleObservationReceipt,
 * down_quant, n_ff, n_embd, input, output | residual) — api/qwen_moe_api.rs:1918,2163.  layer_idx < 0
 * is None.  Every selected bundle is looked up (full / partial / miss), observed in the reuse history
 * and, on a miss, put to the admission test of sparse_expert_cache.rs:221-270; the stats delta of the
 * call is recorded in `receipt` (may be null). */
int rnb_b200_qwen35_sparse_experts_into(const uint8_t *const *gate, const uint8_t *const *up, const uint8_t *const *down, size_t gate_slice_len,
                                        size_t down_slice_len, const float *route_weights, size_t n_selected, int64_t layer_idx,
                                        const size_t *selected_expert_ids, rnb_b200_expert_bundle_receipt *receipt, uint32_t down_quant,
                                        size_t n_ff, size_t n_embd, const float *input, float *output, size_t output_len);
int rnb_b200_qwen35_sparse_experts_add_residual_into(const uint8_t *const *gate, const uint8_t *const *up, const uint8_t *const *down,
                                                     size_t gate_slice_len, size_t down_slice_len, const float *route_weights, size_t n_selected,
                                                     int64_t layer_idx, const size_t *selected_expert_ids, rnb_b200_expert_bundle_receipt *receipt,
                                                     uint32_t down_quant, size_t n_ff, size_t n_embd, const float *input, float *residual_inout,
                                                     size_t residual_len);
/* running totals of the accounting above (ExpertBundleCacheStats) */
int rnb_b200_qwen35_expert_cache_stats(rnb_b200_expert_bundle_stats *out);
/* qwen35_configure_moe_layer_cache(model_moe_bytes, runtime_headroom_bytes, min_layer_bytes) -> usize
 * — api/qwen_moe_api.rs:1483: the byte limit chosen for resident expert layers */
int rnb_b200_qwen35_configure_moe_layer_cache(size_t model_moe_bytes, size_t runtime_headroom_bytes, size_t min_layer_bytes, size_t *limit_out);
/* qwen35_admit_expert_misses_async — api/qwen_moe_api.rs:2082: uploads the given weight slices into
 * the residency cache on the stream without synchronising and without evicting anything */
int rnb_b200_qwen35_admit_expert_misses_async(const uint8_t *const *slices, const size_t *lens, size_t n, size_t *n_admitted);
/* qwen35_prefill_device_topk_route_slots(router_w, n_expert, hidden_dim, norm_all, seq_len,
 * n_expert_used) -> (ids, weights, token_ids) — api/qwen_moe_api.rs:1521: router matvec on the
 * device, then the softmax top-k of moe_route_topk_f32; slot s * n_expert_used + j belongs to token s */
int rnb_b200_qwen35_prefill_device_topk_route_slots(const float *router_w, size_t n_expert, size_t hidden_dim, const float *norm_all, size_t seq_len,
                                                    size_t n_expert_used, uint32_t *ids_out, float *weights_out, uint32_t *token_ids_out);
/* cuda_weight_residency_counters() -> CudaWeightResidencyCounters — api/cache_api.rs:97,
 * runtime/types.rs:68-82.  This library keeps weights as raw GGUF quant bytes only, so the expanded
 * f16 / f32 and packed fields are always 0. */
typedef struct {
    uint64_t expanded_diag_bytes, native_f32_bytes, packed_q8dot_bytes, raw_quant_bytes, transient_quant_upload_bytes;
    uint64_t q4_expanded_f16_bytes, q4_expanded_f32_bytes, q6_expanded_f16_bytes, q6_expanded_f32_bytes;
    uint64_t q4_raw_quant_bytes, q6_raw_quant_bytes, q4_transient_quant_upload_bytes, q6_transient_quant_upload_bytes;
} rnb_b200_weight_residency_counters;
int rnb_b200_cuda_weight_residency_counters(rnb_b200_weight_residency_counters *out);
/* prewarm_quant_resident_weights — api/quant_api.rs:977 (any quant type; same cache as prewarm_q4k_weights) */
int rnb_b200_prewarm_quant_resident_weights(const uint8_t *const *slices, const size_t *lens, size_t n, size_t *n_resident);

/* ---- token-level decoder: the device-resident chain ------------------------------------------
 * The reference drives one operator call (and usually one stream sync) per projection; its
 * "carrier" variants (api/dense_api.rs:1176-1311, 2098-2400) were moving toward keeping
 * activations on the device.  The decoder is that chain finished: weights are registered
 * once, a decode step is one CUDA graph launch, and only the token id crosses PCIe.
 * Mirrors Engine::forward_decode — crates/rnb-llm/src/engine/decode_inference.rs:175-208,
 * decode.rs:199-564, decode_ffn.rs:294-366, logits.rs. */
typedef struct {
    int32_t n_layer, hidden, n_head, n_kv_head, head_dim, n_ff, vocab;
    int32_t rope_neox;
    float rms_eps, rope_theta;
    int32_t n_expert, n_expert_used, n_ff_expert;
    int32_t max_ctx;
    /* row sharding across GPUs (1 = single GPU) */
    int32_t world_size, rank;
} rnb_b200_model_cfg;
typedef struct {
    uint32_t type;
    const uint8_t *data; /* host bytes (copied to the device) */
    size_t len;
} rnb_b200_qweight;
typedef struct {
    const float *attn_norm, *ffn_norm;
    rnb_b200_qweight wq, wk, wv, wo, gate, up, down;
    const float *router;
    rnb_b200_qweight gate_exps, up_exps, down_exps;
} rnb_b200_layer_weights;
typedef struct rnb_b200_decoder rnb_b200_decoder;

int rnb_b200_decoder_create(const rnb_b200_model_cfg *cfg, rnb_b200_decoder **out);
void rnb_b200_decoder_destroy(rnb_b200_decoder *d);
/* Copies one layer's weights to the device (row-sharded when world_size > 1). */
int rnb_b200_decoder_set_layer(rnb_b200_decoder *d, int layer, const rnb_b200_layer_weights *w);
int rnb_b200_decoder_set_globals(rnb_b200_decoder *d, rnb_b200_qweight token_embd,
                                 const float *out_norm, rnb_b200_qweight output);
/* Fills every weight with synthetic data generated on the device (bench only): N(0, sigma)
 * values quantised per block with a min/max fit; norms = 1. */
int rnb_b200_decoder_fill_synthetic(rnb_b200_decoder *d, uint64_t seed, float sigma);
/* Fills the KV cache rows [0, n_pos) with synthetic f16 values (bench only). */
int rnb_b200_decoder_fill_kv_synthetic(rnb_b200_decoder *d, int n_pos, uint64_t seed);
/* One decode step at position `pos`: token in, greedy next token out (host buffers).
 * logits_out may be NULL; otherwise receives `vocab` floats. */
int rnb_b200_decoder_step(rnb_b200_decoder *d, uint32_t token, int pos, uint32_t *next_token,
                          float *logits_out);
/* Enqueue-only variant for device-resident timing: consumes the token already on the device
 * (the previous step's argmax when `chain` != 0), no host copy, no synchronisation.
 * pos >= 0 sets the position; pos < 0 continues at the position after the previous step. */
int rnb_b200_decoder_step_dev(rnb_b200_decoder *d, int pos, int chain);
int rnb_b200_decoder_sync(rnb_b200_decoder *d);
/* Device stream handle (cudaStream_t) the decoder launches on, for event timing. */
void *rnb_b200_decoder_stream(rnb_b200_decoder *d);
int rnb_b200_decoder_read_kv(rnb_b200_decoder *d, int layer, int n_pos, uint16_t *k_out,
                             uint16_t *v_out);
int rnb_b200_decoder_read_hidden(rnb_b200_decoder *d, float *hidden_out);
int rnb_b200_decoder_read_expert_ids(rnb_b200_decoder *d, int layer, uint32_t *ids_out);
/* kernels launched per decode step, bytes of weights resident, per-step algorithmic bytes */
int rnb_b200_decoder_stats(rnb_b200_decoder *d, uint64_t *launches_per_step,
                           uint64_t *weight_bytes, uint64_t *kv_bytes_per_pos);
/* Measurement helpers (CUDA events on the decoder's stream).  time_steps: `steps` chained
 * device-resident decode steps from position `pos`.  time_matvecs: only the weight-streaming
 * matvec launches of a step, `iters` times, with their algorithmic bytes and launch count. */
int rnb_b200_decoder_time_steps(rnb_b200_decoder *d, int pos, int steps, float *ms_out);
int rnb_b200_decoder_time_matvecs(rnb_b200_decoder *d, int iters, float *ms_out,
                                  uint64_t *bytes_per_iter, uint64_t *launches_per_iter);
/* Multi-GPU: attach an NCCL communicator built from a 128-byte unique id that rank 0 made
 * with rnb_b200_nccl_unique_id and the host side distributed to every rank. */
int rnb_b200_nccl_unique_id(uint8_t id_out[128]);
int rnb_b200_decoder_attach_nccl(rnb_b200_decoder *d, const uint8_t id[128]);
/* Prefill of n prompt tokens at positions pos0..pos0+n-1 (Engine::forward_prefill,
 * crates/rnb-llm/src/engine/prefill.rs; CUDA path crates/rnb-runtime/src/cuda_inference/cuda/
 * prefill.rs:1104-1166): all matmuls on the tcgen05 kernel (bf16 x bf16 -> f32), RoPE + f16 KV
 * append for every position, causal attention over the cache, then the last token's logits ->
 * greedy token.  Leaves the decoder ready to decode at position pos0+n.  ms_out (optional):
 * device time between two events on the decoder's stream.  The tensor-core path serves single-GPU
 * dense stacks in Q4_K / Q6_K; MoE stacks, sharded decoders (every rank calls) and other weight
 * types take the prompt token by token through the decode step (ms_out: host wall time). */
int rnb_b200_decoder_prefill(rnb_b200_decoder *d, const uint32_t *tokens, int n, int pos0,
                             uint32_t *next_token, float *ms_out);
/* Logits of the last step or prefill (this rank's vocab slice), for tests. */
int rnb_b200_decoder_read_logits(rnb_b200_decoder *d, float *out, size_t n);

/* Multi-GPU exchange over peer memory (the alternative to the NCCL communicator above, which
 * measured 3-10 % faster per token on 2-8 GPUs): every rank exports the CUDA IPC handle of its exchange arena, the host side
 * all-gathers the 64-byte handles, every rank attaches the full list (rank order).  After
 * that the slices of the four per-layer all-gathers travel as peer stores with a flag per
 * exchange and rank; a slice that does not arrive within about a second sets the device error
 * flag instead of hanging.  No counterpart in the reference (its CUDA path is single-GPU). */
int rnb_b200_decoder_exchange_handle(rnb_b200_decoder *d, uint8_t handle_out[64]);
int rnb_b200_decoder_attach_peers(rnb_b200_decoder *d, const uint8_t *handles /* world x 64 */);
/* Single-GPU check of the exchange's failure path: waits for a peer flag that nobody raises; the
 * bounded wait gives up after about a second and *status_out receives the device error code
 * (4 = peer timeout).  The context stays usable. */
int rnb_b200_peer_exchange_timeout_selftest(int *status_out);

/* Shape the decoder was created with. */
int rnb_b200_decoder_config(const rnb_b200_decoder *d, rnb_b200_model_cfg *out);
/* Longest context (positions, 0..4096) that decode steps serve with the reference-order attention
 * kernel, whose output is bit-identical to rnb-cpu's four-pass decode attention
 * (crates/rnb-cpu/src/kernels/attention/decode_flash.rs:91-212); longer contexts use the chunked
 * tensor-core kernel (same result to ~1e-6).  0 turns the reference-order kernel off.  Default:
 * environment RNB_B200_EXACT_ATTN_MAX, else 512 (its in-order sums cost about 6 us per layer at
 * 128 positions and 26 us at 512 over the chunked kernel).  Only before the first step. */
int rnb_b200_decoder_set_exact_attention_max(rnb_b200_decoder *d, int max_positions);

/* ---- GGUF container and file loader ------------------------------------------------------------
 * GGUFFile::parse — crates/rnb-loader/src/gguf/parser.rs:244-404 (magic "GGUF", versions 2 and 3,
 * little-endian only, u64 counts, KV metadata, tensor infos with dims stored innermost first,
 * `general.alignment` (default 32, a power of two), data section at the next aligned offset;
 * limits and messages as the reference's); type ids — gguf/types.rs:5-40.  `open` maps the file
 * read-only; `parse` reads a buffer the caller keeps alive.  Tensor data is never copied on the
 * host. */
typedef struct rnb_b200_gguf rnb_b200_gguf;
typedef struct {
    char name[64];
    uint32_t n_dims, ggml_type;
    uint64_t dims[4];      /* row-major: outermost first, as the reference normalises them */
    uint64_t offset;       /* from the start of the data section */
    uint64_t n_elements;
    uint64_t n_bytes;      /* 0 when the type's block size is not tabulated */
    const uint8_t *data;   /* inside the mapped file */
} rnb_b200_gguf_tensor_info;
int rnb_b200_gguf_open(const char *path, rnb_b200_gguf **out);
int rnb_b200_gguf_parse(const void *data, size_t len, rnb_b200_gguf **out);
void rnb_b200_gguf_close(rnb_b200_gguf *g);
int rnb_b200_gguf_info(const rnb_b200_gguf *g, uint32_t *version, uint64_t *alignment,
                       uint64_t *data_start, uint64_t *n_tensors, uint64_t *n_metadata);
/* Metadata getters (get_u32 / get_f32 / get_string / get_u32_array of arch/mod.rs): a missing key
 * returns RNB_B200_UNSUPPORTED, a value of another kind RNB_B200_VALIDATION_FAILED. */
int rnb_b200_gguf_get_u64(const rnb_b200_gguf *g, const char *key, uint64_t *out);
int rnb_b200_gguf_get_f64(const rnb_b200_gguf *g, const char *key, double *out);
int rnb_b200_gguf_get_str(const rnb_b200_gguf *g, const char *key, char *buf, size_t cap,
                          size_t *len_out);
int rnb_b200_gguf_get_array_u64(const rnb_b200_gguf *g, const char *key, uint64_t *out,
                                size_t cap, size_t *len_out);
int rnb_b200_gguf_tensor(const rnb_b200_gguf *g, const char *name, rnb_b200_gguf_tensor_info *out);
int rnb_b200_gguf_tensor_at(const rnb_b200_gguf *g, size_t index, rnb_b200_gguf_tensor_info *out);
/* extract_metadata — crates/rnb-loader/src/arch/mod.rs:304-560, for the Llama-style families the
 * decoder runs: `<arch>.embedding_length`, `.block_count`, `.attention.head_count[_kv]`,
 * `.feed_forward_length`, `.rope.freq_base` (default 10000), `.attention.layer_norm_rms_epsilon`
 * (default 1e-5), `.expert_count`, `.expert_used_count`, `.expert_feed_forward_length`;
 * max_ctx <= 0 takes `<arch>.context_length` (default 4096). */
int rnb_b200_gguf_model_config(const rnb_b200_gguf *g, int max_ctx, rnb_b200_model_cfg *cfg);
/* Tensor names of crates/rnb-loader/src/arch/llama.rs:33-155 (`token_embd`, `blk.N.attn_q`, ...,
 * `output_norm`, `output`; a file without `output.weight` ties the LM head to the embedding)
 * uploaded from the mapped pages; register_pages != 0 pins the data section first
 * (rnb_b200_register_host_range) where the mapping can be pinned: best effort. */
int rnb_b200_decoder_load_gguf(rnb_b200_decoder *d, const rnb_b200_gguf *g, int register_pages);

/* ---- device-pointer tier (no host copies, no synchronisation; for callers that keep
 * activations on the device and for kernel timing).  `stream` is a cudaStream_t or NULL. */
int rnb_b200_dev_quantize_q8k(const float *x_dev, size_t cols, size_t seq, void *xq_dev,
                              void *ref_blocks_dev, void *stream);
size_t rnb_b200_dev_q8k_bytes(size_t cols);
int rnb_b200_dev_gemv(uint32_t type, const uint8_t *w_dev, size_t rows, size_t cols,
                      const void *x_dev /* Q8K-dev layout, or f32 for Q8_0 */, float *y_dev,
                      int rows_per_tile /* 0 = auto */, void *stream);
/* Tensor-core prefill matmul on device-resident operands: x_dev f32 [seq][cols], xb_dev scratch
 * of seq*cols bf16, y_dev f32 [seq][rows]; type = GGML type id (12 Q4_K, 14 Q6_K). */
int rnb_b200_dev_prefill_gemm(int type, const uint8_t *w_dev, size_t rows, size_t cols,
                              const float *x_dev, size_t seq, uint16_t *xb_dev, float *y_dev,
                              void *stream);
/* Up to three matrices that share the tokens (q/k/v, gate/up) in one launch; arrays of length n. */
int rnb_b200_dev_prefill_gemm_multi(int n, const int *types, const uint8_t *const *w_dev,
                                    const size_t *rows, float *const *y_dev, size_t cols,
                                    const float *x_dev, size_t seq, uint16_t *xb_dev, void *stream);
/* gate + up of a token batch with silu(gate) * up computed in the matmul's epilogue: act_dev bf16
 * [seq][rows] (the token matrix of the down matmul); gate and up share the GGML type; act_dev must
 * not alias xb_dev. */
int rnb_b200_dev_prefill_gemm_silu(int type, const uint8_t *gate_dev, const uint8_t *up_dev,
                                   size_t rows, size_t cols, const float *x_dev, size_t seq,
                                   uint16_t *xb_dev, uint16_t *act_dev, void *stream);
int rnb_b200_dev_flash_decode(const float *q_dev, const uint16_t *k_dev, const uint16_t *v_dev,
                              size_t kv_len, size_t num_heads, size_t num_kv_heads, float scale,
                              float *partials_dev, size_t partials_bytes, int n_chunks,
                              float *out_dev, void *stream);
size_t rnb_b200_flash_decode_scratch_bytes(size_t num_heads, int n_chunks);
int rnb_b200_flash_decode_default_chunks(size_t kv_len, size_t num_kv_heads);
/* Decode attention for hosts that must not allocate device memory after start-up (a plug-in
 * inside a server with a frozen memory pool, a sandbox whose allocator hooks abort on late
 * allocations, a real-time loop that may not take the driver's allocation locks).  This entry
 * point has no counterpart in the reference.  Same arithmetic as
 * rnb_b200_dev_flash_decode, but the per-chunk partial results live in a fixed array inside
 * the library (1 064 960 bytes per device that loads it, held until the process exits), so the
 * call performs no cudaMalloc, cudaFree or allocating library call.  All pointers are device
 * pointers owned by the caller; `stream` is a cudaStream_t or NULL; the call does not
 * synchronise.  Limits: at most 64 query heads (more is rejected with
 * RNB_B200_VALIDATION_FAILED); head_dim 128; long contexts are split into at most 32 chunks.
 * The first call on each device looks up the array's device address (one
 * cudaGetSymbolAddress); make that first call before starting any stream capture.
 * Every call on a device uses the same array: calls that overlap on the GPU (different
 * streams, or this entry point from two threads) race on it and must be serialised by the
 * caller.  Nothing in the array needs clearing between calls: each call rewrites every record
 * it later reads.  Alignment: q_dev on a 16-byte boundary, k_dev and v_dev on 8 bytes (16 bytes
 * selects the faster tensor-core kernel), out_dev on 4 bytes; anything else is rejected with
 * RNB_B200_VALIDATION_FAILED rather than left to fault on the device. */
int rnb_b200_attention_decode_hd128_noalloc(const float *q_dev, const uint16_t *k_dev,
                                            const uint16_t *v_dev, size_t kv_len,
                                            size_t num_heads, size_t num_kv_heads, float scale,
                                            float *out_dev, void *stream);
/* Companion of the call above, also without a counterpart in the reference and also free of
 * allocations: waits for `stream`, then reads (and clears) the entry point's own status word on
 * the current device, a second fixed word beside the scratch array.  0 = every launch since the
 * last read completed; non-zero = a bounded wait inside a kernel gave up and the outputs written
 * since then are not to be trusted (the codes are those of rnb_b200_dev_error_flag). */
int rnb_b200_attention_decode_hd128_noalloc_status(int *status_out, void *stream);
/* Reads and clears the device error word set by kernels whose bounded waits gave up. */
int rnb_b200_dev_error_flag(int *flag_out);

#ifdef __cplusplus
}
#endif
#endif /* RNB_B200_H */
