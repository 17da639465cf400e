/*
 * CPU oracle: a plain-C restatement of the x86 path of runNburn's `rnb-cpu` crate
 * (plus the few `rnb-llm` host routines the batch-1 decode path uses).
 *
 * THIS IS TEST INFRASTRUCTURE.  It is the checker the CUDA path is compared against
 * and the timed CPU baseline; nothing in the shipped library links, loads or calls it.
 * Every function names the reference file:line whose behaviour it restates (paths are
 * relative to the reference project root).
 *
 * Parity pin: the reference is Rust and cannot be compiled where this was written, so
 * the oracle is pinned by re-stating the reference's own unit-test fixtures
 * (tests/test_oracle_kats.py) and by an independent dequantiser (the `gguf` Python
 * package) through committed fixtures under tests/golden/.
 */
#ifndef RNB_ORACLE_H
#define RNB_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORC_QK_K 256
#define ORC_Q2K_BYTES 84
#define ORC_Q3K_BYTES 110
#define ORC_Q4K_BYTES 144
#define ORC_Q5K_BYTES 176
#define ORC_Q6K_BYTES 210
#define ORC_Q8_0_BYTES 34
#define ORC_Q8K_BYTES 292

/* GGML type ids as the reference passes them (`down_quant: u32`). */
#define ORC_TYPE_Q8_0 8
#define ORC_TYPE_Q2_K 10
#define ORC_TYPE_Q3_K 11
#define ORC_TYPE_Q4_K 12
#define ORC_TYPE_Q5_K 13
#define ORC_TYPE_Q6_K 14

/* crates/rnb-cpu/src/gemm/activation_q8.rs:66-72 — repr(C) { f32 d; i8 qs[256]; i16 bsums[16]; } */
typedef struct {
    float d;
    int8_t qs[256];
    int16_t bsums[16];
} orc_q8k_block;

/* ---- scalar conversions (half crate semantics: IEEE round-to-nearest-even) ---- */
float orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float f);
void orc_f32_to_f16_row(const float *src, uint16_t *dst, size_t n);

/* ---- activation quantisation ---- */
void orc_quantize_q8k(const float *x, size_t n, orc_q8k_block *out);

/* ---- dequantisation of one block / of a row of blocks ---- */
void orc_dequantize_q4k_block(const uint8_t *block, float *out256);
void orc_dequantize_q2k_block(const uint8_t *block, float *out256);
void orc_dequantize_q3k_block(const uint8_t *block, float *out256);
void orc_dequantize_q5k_block(const uint8_t *block, float *out256);
void orc_dequantize_q6k_block(const uint8_t *block, float *out256);
void orc_dequantize_q8_0_block(const uint8_t *block, float *out32);
int orc_dequantize_row(int ggml_type, const uint8_t *row, size_t cols, float *out);

/* ---- weight quantisers (harness utilities for building synthetic models) ---- */
void orc_quantize_row_q4k(const float *x, size_t n, uint8_t *out);
void orc_quantize_row_q2k(const float *x, size_t n, uint8_t *out);   /* harness utility */
void orc_quantize_row_q3k(const float *x, size_t n, uint8_t *out);   /* harness utility */
void orc_quantize_row_q5k(const float *x, size_t n, uint8_t *out);   /* harness utility */
void orc_quantize_row_q6k(const float *x, size_t n, uint8_t *out);
void orc_quantize_row_q8_0(const float *x, size_t n, uint8_t *out);
int orc_quantize_matrix(int ggml_type, const float *x, size_t rows, size_t cols, uint8_t *out,
                        int threads);
/* harness utility: seeded N(0, sigma) weights quantised with a plain per-block fit (fast) */
int orc_synth_matrix(int ggml_type, size_t rows, size_t cols, uint64_t seed, float sigma, uint8_t *out,
                     int threads);

/* ---- row dots ---- */
float orc_dot_q4k_q8k(const uint8_t *row, const orc_q8k_block *y, size_t nb);
float orc_dot_q2k_q8k(const uint8_t *row, const orc_q8k_block *y, size_t nb);
float orc_dot_q3k_q8k(const uint8_t *row, const orc_q8k_block *y, size_t nb);
float orc_dot_q5k_q8k(const uint8_t *row, const orc_q8k_block *y, size_t nb);
float orc_dot_q6k_q8k(const uint8_t *row, const orc_q8k_block *y, size_t nb);
float orc_dot_q4k_q8k_lanes(const uint8_t *row, const orc_q8k_block *y, size_t nb);
float orc_dot_q6k_q8k_lanes(const uint8_t *row, const orc_q8k_block *y, size_t nb);
float orc_dot_q8_0_row(const uint8_t *row, const float *x, size_t blocks_per_row);
float orc_dot_dequant_row(int ggml_type, const uint8_t *row, const float *x, size_t cols);
int orc_have_avx2(void);
void orc_force_scalar(int on);

/* ---- GEMV / batched GEMV, seq-major output ---- */
int orc_gemv(int ggml_type, const uint8_t *w, const float *x, float *out, size_t rows,
             size_t cols, size_t seq_len, int threads);
size_t orc_row_bytes(int ggml_type, size_t cols);

/* ---- attention ---- */
void orc_attention_decode(const float *q, const uint16_t *k, const uint16_t *v, float *out,
                          size_t num_heads, size_t num_kv_heads, size_t head_dim, size_t kv_len,
                          float scale);
void orc_attention_decode_window(const float *q, const uint16_t *k, const uint16_t *v, float *out,
                                 size_t num_heads, size_t num_kv_heads, size_t head_dim, size_t kv_len,
                                 float scale, size_t window);
void orc_attention_decode_mt(const float *q, const uint16_t *k, const uint16_t *v, float *out,
                             size_t num_heads, size_t num_kv_heads, size_t head_dim, size_t kv_len,
                             float scale, int threads);
void orc_attention_decode_online(const float *q, const uint16_t *k, const uint16_t *v, float *out,
                                 size_t num_heads, size_t num_kv_heads, size_t head_dim,
                                 size_t kv_len, float scale);
void orc_attention_prefill(const float *q, const float *k, const float *v, float *out,
                           size_t seq_len, size_t kv_len, size_t num_heads, size_t num_kv_heads,
                           size_t head_dim, float scale);
void orc_attention_prefill_f16kv(const float *q, const uint16_t *k, const uint16_t *v, float *out,
                                 size_t seq_len, size_t kv_len, size_t num_heads,
                                 size_t num_kv_heads, size_t head_dim, float scale);

/* ---- MoE routing ---- */
size_t orc_moe_route_topk(const float *logits, size_t n_expert, size_t top_k, uint32_t *ids,
                          float *weights);
void orc_gemv_f32(const float *w, const float *x, float *out, size_t rows, size_t cols);
int orc_moe_experts(const uint8_t *const *gate, const uint8_t *const *up,
                    const uint8_t *const *down, const float *route_weights, size_t n_selected,
                    int down_type, size_t n_ff, size_t n_embd, const float *x, float *out,
                    int threads);

/* ---- glue ---- */
void orc_rms_norm(const float *x, const float *w, float eps, float *out, size_t hidden,
                  size_t seq_len);
void orc_rope_inplace(float *data, size_t n, size_t pos_start, size_t head_dim, size_t dim,
                      float theta);
void orc_rope_neox_inplace(float *data, size_t n, size_t pos_start, size_t head_dim, size_t dim,
                           float theta);
void orc_rope_table(size_t pos, size_t head_dim, float theta, float *cos_out, float *sin_out);
void orc_silu_mul_inplace(float *gate, const float *up, size_t n);
uint32_t orc_argmax_last(const float *x, size_t n);

/* ---- token-level decode of a Llama-style model (test driver) ---- */
typedef struct {
    int32_t n_layer, hidden, n_head, n_kv_head, head_dim, n_ff, vocab;
    int32_t rope_neox; /* 0 = adjacent pairs (Llama), 1 = half-split */
    float rms_eps, rope_theta;
    /* MoE (n_expert == 0 → dense FFN) */
    int32_t n_expert, n_expert_used, n_ff_expert;
} orc_model_cfg;

typedef struct {
    int32_t type;        /* GGML type id */
    const uint8_t *data; /* rows × row_bytes */
} orc_qweight;

typedef struct {
    const float *attn_norm, *ffn_norm;
    orc_qweight wq, wk, wv, wo;
    orc_qweight gate, up, down;           /* dense FFN */
    const float *router;                  /* [n_expert][hidden] f32 (MoE) */
    orc_qweight gate_exps, up_exps, down_exps; /* stacked [n_expert] (MoE) */
} orc_layer;

typedef struct orc_model orc_model;
orc_model *orc_model_create(const orc_model_cfg *cfg, const orc_layer *layers,
                            orc_qweight token_embd, const float *out_norm, orc_qweight output,
                            size_t max_ctx, int threads);
void orc_model_free(orc_model *m);
void orc_model_reset(orc_model *m);
/* feeds one token at position `pos`; returns logits pointer (vocab floats) */
const float *orc_model_decode(orc_model *m, uint32_t token, size_t pos);
const uint16_t *orc_model_k_cache(const orc_model *m, int layer);
const uint16_t *orc_model_v_cache(const orc_model *m, int layer);
const float *orc_model_hidden(const orc_model *m);
const uint32_t *orc_model_last_expert_ids(const orc_model *m, int layer);

#ifdef __cplusplus
}
#endif
#endif
