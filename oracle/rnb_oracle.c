/*
 * CPU oracle — see rnb_oracle.h.  TEST INFRASTRUCTURE ONLY: the CUDA library never
 * links or calls this file; tests and the bench's CPU-baseline leg do.
 *
 * Build: see oracle/Makefile (gcc -O2 -mavx2 -mfma -mf16c -ffp-contract=off).
 * `-ffp-contract=off` matters: the reference's scalar Rust never fuses a*b+c, and
 * its AVX2 code fuses exactly where it writes `_mm256_fmadd_ps`.
 */
#include "rnb_oracle.h"

#include <immintrin.h>
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------
 * f16 <-> f32.  The reference uses the `half` crate (IEEE binary16, round-to-nearest-even on
 * narrowing: crates/rnb-llm/src/kv_cache.rs:126-141, crates/rnb-cpu/src/quantize/blocks.rs).
 * Software conversion so the oracle does not depend on F16C being present.
 * ---------------------------------------------------------------------------------------- */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                e++;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + (127 - 15)) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t orc_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) { /* inf / nan */
        uint32_t man = absx & 0x7fffffu;
        return (uint16_t)(sign | 0x7c00u | (man ? (0x200u | (man >> 13)) : 0));
    }
    if (absx >= 0x477ff000u) { /* rounds to >= 65520 → inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x38800000u) { /* subnormal half or zero */
        if (absx < 0x33000000u) return (uint16_t)sign; /* < 2^-25 → 0 */
        int e = (int)(absx >> 23);
        uint32_t man = (absx & 0x7fffffu) | 0x800000u;
        int shift = 126 - e; /* 14..24: man >> shift lands on the subnormal grid */
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t e = (absx >> 23) - 112u;
    uint32_t man = absx & 0x7fffffu;
    uint32_t h = (e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)(sign | h);
}

void orc_f32_to_f16_row(const float *src, uint16_t *dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = orc_f32_to_f16(src[i]);
}

static inline uint16_t rd_u16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static inline uint32_t rd_u32(const uint8_t *p) {
    uint32_t v;
    memcpy(&v, p, 4);
    return v;
}

/* ------------------------------------------------------------------------------------------
 * Tiny parallel-for: contiguous chunks of ceil(n / threads), one pthread per chunk — the
 * same partition as rayon's par_chunks_mut(ceil(rows / threads))
 * (crates/rnb-cpu/src/gemm/quant_gemv.rs:1128-1144).
 * ---------------------------------------------------------------------------------------- */
typedef void (*orc_range_fn)(size_t begin, size_t end, void *ctx);
typedef struct {
    orc_range_fn fn;
    void *ctx;
    size_t begin, end;
} orc_task;
static void *orc_task_main(void *p) {
    orc_task *t = (orc_task *)p;
    t->fn(t->begin, t->end, t->ctx);
    return NULL;
}
static void orc_parallel_for(size_t n, int threads, orc_range_fn fn, void *ctx) {
    if (threads <= 1 || n <= 64) {
        fn(0, n, ctx);
        return;
    }
    if (threads > 256) threads = 256;
    size_t chunk = (n + (size_t)threads - 1) / (size_t)threads;
    pthread_t tid[256];
    orc_task task[256];
    int nt = 0;
    for (size_t b = 0; b < n; b += chunk) {
        task[nt].fn = fn;
        task[nt].ctx = ctx;
        task[nt].begin = b;
        task[nt].end = b + chunk < n ? b + chunk : n;
        nt++;
    }
    for (int i = 1; i < nt; i++) pthread_create(&tid[i], NULL, orc_task_main, &task[i]);
    orc_task_main(&task[0]);
    for (int i = 1; i < nt; i++) pthread_join(tid[i], NULL);
}

/* ------------------------------------------------------------------------------------------
 * Q8_K activation quantisation.
 * crates/rnb-cpu/src/gemm/activation_q8.rs:149-173 (quantize_q8k_block_ggml):
 *   max_val = first element with the strictly largest |x|; iscale = -127/max_val;
 *   d = 1/iscale; q = min(127, round_ties_even(iscale*x)); bsums per 16 elements.
 * ---------------------------------------------------------------------------------------- */
static void quantize_q8k_block(const float *x, orc_q8k_block *out) {
    float amax = 0.0f, max_val = 0.0f;
    for (int i = 0; i < 256; i++) {
        float ax = fabsf(x[i]);
        if (ax > amax) {
            amax = ax;
            max_val = x[i];
        }
    }
    memset(out, 0, sizeof(*out));
    if (amax == 0.0f) return;
    volatile float iscale = -127.0f / max_val;
    out->d = 1.0f / iscale;
    for (int i = 0; i < 256; i++) {
        volatile float prod = iscale * x[i];
        int v = (int)nearbyintf(prod); /* default rounding mode = ties-to-even */
        if (v > 127) v = 127;
        int8_t q = (int8_t)v;
        out->qs[i] = q;
        out->bsums[i / 16] = (int16_t)(out->bsums[i / 16] + q);
    }
}

void orc_quantize_q8k(const float *x, size_t n, orc_q8k_block *out) {
    size_t nb = n / 256;
    for (size_t b = 0; b < nb; b++) quantize_q8k_block(x + b * 256, out + b);
}

/* ------------------------------------------------------------------------------------------
 * Block dequantisation.
 * Q4_K: crates/rnb-cpu/src/quantize/dequant.rs:302-381 (+ get_scale_min_k4, quant.rs:590-599)
 * Q6_K: crates/rnb-cpu/src/quantize/dequant.rs:780-807
 * Q8_0: crates/rnb-cpu/src/quantize/dequant.rs:55-60
 * ---------------------------------------------------------------------------------------- */
static inline void get_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

void orc_dequantize_q4k_block(const uint8_t *block, float *out) {
    float d = orc_f16_to_f32(rd_u16(block));
    float dmin = orc_f16_to_f32(rd_u16(block + 2));
    const uint8_t *scales = block + 4;
    const uint8_t *q = block + 16;
    int is = 0;
    for (int grp = 0; grp < 4; grp++) {
        uint8_t sc1, m1, sc2, m2;
        get_scale_min_k4(is, scales, &sc1, &m1);
        get_scale_min_k4(is + 1, scales, &sc2, &m2);
        float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
        float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
        for (int l = 0; l < 32; l++) out[64 * grp + l] = d1 * (float)(q[32 * grp + l] & 0xF) - mm1;
        for (int l = 0; l < 32; l++)
            out[64 * grp + 32 + l] = d2 * (float)(q[32 * grp + l] >> 4) - mm2;
        is += 2;
    }
}

/* Q2_K: crates/rnb-cpu/src/quantize/dequant.rs:66-86; block = scales[16] (low nibble scale, high
 * nibble min) | qs[64] | d f16 | dmin f16 (crates/rnb-cpu/src/quantize/blocks.rs:63-69, 84 bytes).
 * Each 128-element half interleaves four 32-element groups in its 32 bytes, two bits apiece. */
void orc_dequantize_q2k_block(const uint8_t *block, float *out) {
    float d = orc_f16_to_f32(rd_u16(block + 80));
    float dmin = orc_f16_to_f32(rd_u16(block + 82));
    const uint8_t *qs = block + 16;
    for (int j = 0; j < 16; j++) {
        uint8_t sc = block[j];
        float scale = d * (float)(sc & 0x0F), mn = dmin * (float)(sc >> 4);
        int half = j / 8, group = j % 8;
        int q_base = half * 32 + (group % 2) * 16, shift = (group / 2) * 2;
        for (int l = 0; l < 16; l++) out[j * 16 + l] = (float)((qs[q_base + l] >> shift) & 3) * scale - mn;
    }
}

/* Q3_K: crates/rnb-cpu/src/quantize/dequant.rs:237-297; block = hmask[32] | qs[64] | scales[12] | d f16
 * (crates/rnb-cpu/src/quantize/blocks.rs:72-78, 110 bytes).  16 six-bit scales (bias 32); element =
 * 2 low bits minus 4 where its hmask bit is CLEAR. */
static void q3k_scales(const uint8_t *sb, int8_t scales[16]) {
    const uint32_t kmask1 = 0x03030303u, kmask2 = 0x0f0f0f0fu;
    uint32_t aux[4];
    aux[0] = rd_u32(sb);
    aux[1] = rd_u32(sb + 4);
    aux[2] = rd_u32(sb + 8);
    uint32_t tmp = aux[2];
    aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
    aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
    aux[0] = (aux[0] & kmask2) | (((tmp >> 0) & kmask1) << 4);
    aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
    for (int i = 0; i < 4; i++)
        for (int j = 0; j < 4; j++) scales[i * 4 + j] = (int8_t)((aux[i] >> (8 * j)) & 0xff);
}
void orc_dequantize_q3k_block(const uint8_t *block, float *out) {
    float d_all = orc_f16_to_f32(rd_u16(block + 108));
    int8_t scales[16];
    q3k_scales(block + 96, scales);
    const uint8_t *hm = block, *q = block + 32;
    int is = 0, y_idx = 0, q_off = 0;
    uint8_t m = 1;
    for (int half = 0; half < 2; half++) {
        int shift = 0;
        for (int k = 0; k < 4; k++) {
            for (int part = 0; part < 2; part++) {
                float dl = d_all * ((float)scales[is++] - 32.0f);
                for (int l = 0; l < 16; l++) {
                    int qv = (q[q_off + l + 16 * part] >> shift) & 3;
                    int hv = (hm[l + 16 * part] & m) ? 0 : 4;
                    out[y_idx++] = dl * (float)(qv - hv);
                }
            }
            shift += 2;
            m = (uint8_t)(m << 1);
        }
        q_off += 32;
    }
}

/* Q5_K: crates/rnb-cpu/src/quantize/dequant.rs:729-770; block = d f16 | dmin f16 | scales[12] |
 * qh[32] | qs[128] (crates/rnb-cpu/src/quantize/blocks.rs:90-98, 176 bytes) */
void orc_dequantize_q5k_block(const uint8_t *block, float *out) {
    float d = orc_f16_to_f32(rd_u16(block));
    float dmin = orc_f16_to_f32(rd_u16(block + 2));
    const uint8_t *scales = block + 4, *qh = block + 16, *ql = block + 48;
    int is = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int grp = 0; grp < 4; grp++) {
        uint8_t sc1, m1, sc2, m2;
        get_scale_min_k4(is, scales, &sc1, &m1);
        get_scale_min_k4(is + 1, scales, &sc2, &m2);
        float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
        float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
        for (int l = 0; l < 32; l++)
            out[64 * grp + l] = d1 * (float)((ql[32 * grp + l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - mm1;
        for (int l = 0; l < 32; l++)
            out[64 * grp + 32 + l] = d2 * (float)((ql[32 * grp + l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - mm2;
        is += 2;
        u1 = (uint8_t)(u1 << 2);
        u2 = (uint8_t)(u2 << 2);
    }
}

void orc_dequantize_q6k_block(const uint8_t *block, float *out) {
    const uint8_t *ql = block, *qh = block + 128;
    const int8_t *sc = (const int8_t *)(block + 192);
    float d = orc_f16_to_f32(rd_u16(block + 208));
    for (int n = 0; n < 2; n++) {
        const uint8_t *l4 = ql + 64 * n, *h2 = qh + 32 * n;
        const int8_t *s = sc + 8 * n;
        float *y = out + 128 * n;
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int q1 = (l4[l] & 0x0F) | (((h2[l] >> 0) & 3) << 4);
            int q2 = (l4[l + 32] & 0x0F) | (((h2[l] >> 2) & 3) << 4);
            int q3 = (l4[l] >> 4) | (((h2[l] >> 4) & 3) << 4);
            int q4 = (l4[l + 32] >> 4) | (((h2[l] >> 6) & 3) << 4);
            y[l] = d * (float)s[is] * (float)(q1 - 32);
            y[l + 32] = d * (float)s[is + 2] * (float)(q2 - 32);
            y[l + 64] = d * (float)s[is + 4] * (float)(q3 - 32);
            y[l + 96] = d * (float)s[is + 6] * (float)(q4 - 32);
        }
    }
}

void orc_dequantize_q8_0_block(const uint8_t *block, float *out) {
    float d = orc_f16_to_f32(rd_u16(block));
    for (int i = 0; i < 32; i++) out[i] = (float)(int8_t)block[2 + i] * d;
}

size_t orc_row_bytes(int t, size_t cols) {
    switch (t) {
    case ORC_TYPE_Q2_K: return cols / 256 * ORC_Q2K_BYTES;
    case ORC_TYPE_Q3_K: return cols / 256 * ORC_Q3K_BYTES;
    case ORC_TYPE_Q4_K: return cols / 256 * ORC_Q4K_BYTES;
    case ORC_TYPE_Q5_K: return cols / 256 * ORC_Q5K_BYTES;
    case ORC_TYPE_Q6_K: return cols / 256 * ORC_Q6K_BYTES;
    case ORC_TYPE_Q8_0: return cols / 32 * ORC_Q8_0_BYTES;
    default: return 0;
    }
}

int orc_dequantize_row(int t, const uint8_t *row, size_t cols, float *out) {
    switch (t) {
    case ORC_TYPE_Q4_K:
        for (size_t b = 0; b < cols / 256; b++)
            orc_dequantize_q4k_block(row + b * ORC_Q4K_BYTES, out + b * 256);
        return 0;
    case ORC_TYPE_Q2_K:
        for (size_t b = 0; b < cols / 256; b++)
            orc_dequantize_q2k_block(row + b * ORC_Q2K_BYTES, out + b * 256);
        return 0;
    case ORC_TYPE_Q3_K:
        for (size_t b = 0; b < cols / 256; b++)
            orc_dequantize_q3k_block(row + b * ORC_Q3K_BYTES, out + b * 256);
        return 0;
    case ORC_TYPE_Q5_K:
        for (size_t b = 0; b < cols / 256; b++)
            orc_dequantize_q5k_block(row + b * ORC_Q5K_BYTES, out + b * 256);
        return 0;
    case ORC_TYPE_Q6_K:
        for (size_t b = 0; b < cols / 256; b++)
            orc_dequantize_q6k_block(row + b * ORC_Q6K_BYTES, out + b * 256);
        return 0;
    case ORC_TYPE_Q8_0:
        for (size_t b = 0; b < cols / 32; b++)
            orc_dequantize_q8_0_block(row + b * ORC_Q8_0_BYTES, out + b * 32);
        return 0;
    default: return -1;
    }
}

/* ------------------------------------------------------------------------------------------
 * Weight quantisers.
 * Q4_K: crates/rnb-cpu/src/quantize/quant.rs:173-178 (nearest_int), :189-280
 *       (make_qkx2_quants), :289-413 (quantize_row_q4_k).
 * Q6_K / Q8_0: the reference ships no quantiser for these; the two below are harness
 *       utilities validated only through the reference's dequantisers (round trip).
 * ---------------------------------------------------------------------------------------- */
static inline int nearest_int(float fval) {
    float val = fval + 12582912.0f;
    uint32_t bits;
    memcpy(&bits, &val, 4);
    return (int)(bits & 0x007fffffu) - 0x00400000;
}
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

static float make_qkx2_quants(int n, int nmax, const float *x, const float *weights, uint8_t *L,
                              float *the_min, uint8_t *Laux, float rmin, float rdelta, int nstep) {
    float min = x[0], max = x[0];
    float sum_w = weights[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; i++) {
        if (x[i] < min) min = x[i];
        if (x[i] > max) max = x[i];
        float w = weights[i];
        sum_w += w;
        sum_x += w * x[i];
    }
    if (min > 0.0f) min = 0.0f;
    if (max == min) {
        for (int i = 0; i < n; i++) L[i] = 0;
        *the_min = -min;
        return 0.0f;
    }
    float iscale = (float)nmax / (max - min);
    float scale = 1.0f / iscale;
    float best_error = 0.0f;
    for (int i = 0; i < n; i++) {
        int li = clampi(nearest_int(iscale * (x[i] - min)), 0, nmax);
        L[i] = (uint8_t)li;
        float diff = scale * (float)li + min - x[i];
        diff = diff * diff;
        best_error += weights[i] * diff;
    }
    if (nstep < 1) {
        *the_min = -min;
        return scale;
    }
    for (int is = 0; is <= nstep; is++) {
        iscale = (rmin + rdelta * (float)is + (float)nmax) / (max - min);
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; i++) {
            int li = clampi(nearest_int(iscale * (x[i] - min)), 0, nmax);
            Laux[i] = (uint8_t)li;
            float w = weights[i];
            sum_l += w * (float)li;
            sum_l2 += w * (float)li * (float)li;
            sum_xl += w * (float)li * x[i];
        }
        float d_det = sum_w * sum_l2 - sum_l * sum_l;
        if (d_det > 0.0f) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / d_det;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / d_det;
            if (this_min > 0.0f) {
                this_min = 0.0f;
                this_scale = sum_xl / sum_l2;
            }
            float cur_error = 0.0f;
            for (int i = 0; i < n; i++) {
                float diff = this_scale * (float)Laux[i] + this_min - x[i];
                diff = diff * diff;
                cur_error += weights[i] * diff;
            }
            if (cur_error < best_error) {
                memcpy(L, Laux, (size_t)n);
                best_error = cur_error;
                scale = this_scale;
                min = this_min;
            }
        }
    }
    *the_min = -min;
    return scale;
}

void orc_quantize_row_q4k(const float *input, size_t n, uint8_t *output) {
    size_t nb = n / 256;
    uint8_t el[256], laux[32];
    float mins[8], scales[8], weights[32];
    for (size_t i = 0; i < nb; i++) {
        const float *x = input + i * 256;
        float max_scale = 0.0f, max_min = 0.0f;
        for (int j = 0; j < 8; j++) {
            const float *xs = x + 32 * j;
            float sum_x2 = 0.0f;
            for (int l = 0; l < 32; l++) sum_x2 += xs[l] * xs[l];
            float av_x = sqrtf(sum_x2 / 32.0f);
            for (int l = 0; l < 32; l++) weights[l] = av_x + fabsf(xs[l]);
            float sub_min = 0.0f;
            float s = make_qkx2_quants(32, 15, xs, weights, el + 32 * j, &sub_min, laux, -0.5f,
                                       0.1f, 15);
            scales[j] = s;
            mins[j] = sub_min;
            if (s > max_scale) max_scale = s;
            if (sub_min > max_min) max_min = sub_min;
        }
        float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
        float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
        uint8_t ys[12];
        memset(ys, 0, 12);
        for (int j = 0; j < 8; j++) {
            uint8_t ls = (uint8_t)clampi(nearest_int(inv_scale * scales[j]), 0, 63);
            uint8_t lm = (uint8_t)clampi(nearest_int(inv_min * mins[j]), 0, 63);
            if (j < 4) {
                ys[j] = ls;
                ys[j + 4] = lm;
            } else {
                ys[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                ys[j - 4] |= (uint8_t)((ls >> 4) << 6);
                ys[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        uint16_t d16 = orc_f32_to_f16(max_scale / 63.0f);
        uint16_t dmin16 = orc_f32_to_f16(max_min / 63.0f);
        float d_round = orc_f16_to_f32(d16), dmin_round = orc_f16_to_f32(dmin16);
        for (int j = 0; j < 8; j++) {
            uint8_t sc, mn;
            get_scale_min_k4(j, ys, &sc, &mn);
            float d_sub = d_round * (float)sc;
            if (d_sub == 0.0f) continue;
            float dm_sub = dmin_round * (float)mn;
            for (int ii = 0; ii < 32; ii++) {
                int li = nearest_int((x[32 * j + ii] + dm_sub) / d_sub);
                el[32 * j + ii] = (uint8_t)clampi(li, 0, 15);
            }
        }
        uint8_t *out = output + i * ORC_Q4K_BYTES;
        out[0] = (uint8_t)(d16 & 0xff);
        out[1] = (uint8_t)(d16 >> 8);
        out[2] = (uint8_t)(dmin16 & 0xff);
        out[3] = (uint8_t)(dmin16 >> 8);
        memcpy(out + 4, ys, 12);
        uint8_t *qs = out + 16;
        for (int grp = 0; grp < 4; grp++)
            for (int j = 0; j < 32; j++)
                qs[32 * grp + j] =
                    (uint8_t)((el[64 * grp + j] & 0x0F) | ((el[64 * grp + j + 32] & 0x0F) << 4));
    }
}

/* Harness-only Q6_K quantiser: per 16-element group an absmax scale, the super-block scale
 * d = max|group scale| / 127, 6-bit codes round((x / (d*sc))) clamped to [-32, 31]. */
void orc_quantize_row_q6k(const float *input, size_t n, uint8_t *output) {
    size_t nb = n / 256;
    for (size_t i = 0; i < nb; i++) {
        const float *x = input + i * 256;
        uint8_t *out = output + i * ORC_Q6K_BYTES;
        float gscale[16];
        float max_abs_scale = 0.0f;
        for (int g = 0; g < 16; g++) {
            float amax = 0.0f, vmax = 0.0f;
            for (int l = 0; l < 16; l++) {
                float ax = fabsf(x[16 * g + l]);
                if (ax > amax) {
                    amax = ax;
                    vmax = x[16 * g + l];
                }
            }
            gscale[g] = amax > 0.0f ? vmax / -32.0f : 0.0f;
            if (fabsf(gscale[g]) > max_abs_scale) max_abs_scale = fabsf(gscale[g]);
        }
        memset(out, 0, ORC_Q6K_BYTES);
        if (max_abs_scale == 0.0f) continue;
        float iscale = 127.0f / max_abs_scale;
        uint16_t d16 = orc_f32_to_f16(1.0f / iscale);
        float d = orc_f16_to_f32(d16);
        int8_t *sc = (int8_t *)(out + 192);
        uint8_t L[256];
        for (int g = 0; g < 16; g++) {
            int s = clampi(nearest_int(iscale * gscale[g]), -128, 127);
            sc[g] = (int8_t)s;
            float dl = d * (float)s;
            for (int l = 0; l < 16; l++) {
                int q = dl != 0.0f ? nearest_int(x[16 * g + l] / dl) : 0;
                L[16 * g + l] = (uint8_t)(clampi(q, -32, 31) + 32);
            }
        }
        out[208] = (uint8_t)(d16 & 0xff);
        out[209] = (uint8_t)(d16 >> 8);
        uint8_t *ql = out, *qh = out + 128;
        for (int h = 0; h < 2; h++) {
            for (int l = 0; l < 32; l++) {
                uint8_t q1 = L[128 * h + l], q2 = L[128 * h + l + 32];
                uint8_t q3 = L[128 * h + l + 64], q4 = L[128 * h + l + 96];
                ql[64 * h + l] = (uint8_t)((q1 & 0xF) | ((q3 & 0xF) << 4));
                ql[64 * h + l + 32] = (uint8_t)((q2 & 0xF) | ((q4 & 0xF) << 4));
                qh[32 * h + l] =
                    (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
            }
        }
    }
}

/* Harness-only Q8_0 quantiser (GGML convention: d = amax/127, q = round(x/d)). */
/* Q2_K quantiser: harness utility (the reference ships none): per 16-element sub-block a min/max fit
 * on 0..3, 4-bit scales and mins against the block's largest; validated through the reference's
 * dequantiser (round trip). */
void orc_quantize_row_q2k(const float *input, size_t n, uint8_t *output) {
    for (size_t b = 0; b < n / 256; b++) {
        const float *x = input + b * 256;
        uint8_t *blk = output + b * ORC_Q2K_BYTES;
        float sc[16], mn[16], max_sc = 0.f, max_mn = 0.f;
        for (int j = 0; j < 16; j++) {
            float lo = 0.f, hi = x[16 * j];
            for (int l = 0; l < 16; l++) {
                if (x[16 * j + l] < lo) lo = x[16 * j + l];
                if (x[16 * j + l] > hi) hi = x[16 * j + l];
            }
            sc[j] = (hi - lo) / 3.f;
            mn[j] = -lo;
            if (sc[j] > max_sc) max_sc = sc[j];
            if (mn[j] > max_mn) max_mn = mn[j];
        }
        uint16_t dh = orc_f32_to_f16(max_sc / 15.f), mh = orc_f32_to_f16(max_mn / 15.f);
        float d = orc_f16_to_f32(dh), dm = orc_f16_to_f32(mh);
        memset(blk, 0, ORC_Q2K_BYTES);
        blk[80] = (uint8_t)(dh & 0xff);
        blk[81] = (uint8_t)(dh >> 8);
        blk[82] = (uint8_t)(mh & 0xff);
        blk[83] = (uint8_t)(mh >> 8);
        for (int j = 0; j < 16; j++) {
            int ls = clampi(d > 0.f ? nearest_int(sc[j] / d) : 0, 0, 15);
            int lm = clampi(dm > 0.f ? nearest_int(mn[j] / dm) : 0, 0, 15);
            blk[j] = (uint8_t)(ls | (lm << 4));
            float dd = d * (float)ls, mm = dm * (float)lm;
            int half = j / 8, group = j % 8;
            int q_base = half * 32 + (group % 2) * 16, shift = (group / 2) * 2;
            for (int l = 0; l < 16; l++) {
                int q = dd > 0.f ? clampi(nearest_int((x[16 * j + l] + mm) / dd), 0, 3) : 0;
                blk[16 + q_base + l] |= (uint8_t)(q << shift);
            }
        }
    }
}

/* Q3_K quantiser: harness utility (the reference ships none): per 16-element sub-block a symmetric
 * fit on -4..3, six-bit scales (bias 32) against the block's largest; validated through the reference's
 * dequantiser (round trip). */
void orc_quantize_row_q3k(const float *input, size_t n, uint8_t *output) {
    for (size_t b = 0; b < n / 256; b++) {
        const float *x = input + b * 256;
        uint8_t *blk = output + b * ORC_Q3K_BYTES;
        float sc[16], max_sc = 0.f;
        for (int j = 0; j < 16; j++) {
            float amax = 0.f;
            for (int l = 0; l < 16; l++) {
                float a = fabsf(x[16 * j + l]);
                if (a > amax) amax = a;
            }
            sc[j] = amax / 4.f;
            if (sc[j] > max_sc) max_sc = sc[j];
        }
        uint16_t dh = orc_f32_to_f16(max_sc / 31.f);
        float d = orc_f16_to_f32(dh);
        memset(blk, 0, ORC_Q3K_BYTES);
        blk[108] = (uint8_t)(dh & 0xff);
        blk[109] = (uint8_t)(dh >> 8);
        int ls[16];
        for (int j = 0; j < 16; j++) ls[j] = clampi(d > 0.f ? nearest_int(sc[j] / d) : 0, 0, 31) + 32;   /* stored biased, 32..63 */
        /* 6-bit packing: low nibbles of scales 0..7 in bytes 0..7 (low), of 8..15 in their high nibbles;
         * the two top bits of scale j in byte 8 + j % 4 at bit pair j / 4 */
        uint8_t *sb = blk + 96;
        for (int j = 0; j < 16; j++) {
            int lo = ls[j] & 0xF, hi = ls[j] >> 4;
            if (j < 8) sb[j] |= (uint8_t)lo;
            else sb[j - 8] |= (uint8_t)(lo << 4);
            sb[8 + j % 4] |= (uint8_t)(hi << (2 * (j / 4)));
        }
        uint8_t *hm = blk, *q = blk + 32;
        /* element order of the dequantiser: half, plane k, part (16 elements) */
        int y_idx = 0, is = 0;
        for (int half = 0; half < 2; half++)
            for (int k = 0; k < 4; k++)
                for (int part = 0; part < 2; part++) {
                    float dl = d * (float)(ls[is++] - 32);
                    for (int l = 0; l < 16; l++) {
                        int v = dl != 0.f ? clampi(nearest_int(x[y_idx] / dl), -4, 3) : 0;
                        y_idx++;
                        int qv = v & 3;                       /* two low bits of v + 4 */
                        if (v >= 0) hm[l + 16 * part] |= (uint8_t)(1u << (4 * half + k));
                        q[32 * half + l + 16 * part] |= (uint8_t)(qv << (2 * k));
                    }
                }
    }
}

/* Q5_K quantiser: harness utility (the reference ships none).  Per 32-element sub-block a
 * min/max fit on 0..31, super-scales fitted to 6 bits, validated through the reference's
 * dequantiser (round trip). */
void orc_quantize_row_q5k(const float *input, size_t n, uint8_t *output) {
    for (size_t b = 0; b < n / 256; b++) {
        const float *x = input + b * 256;
        uint8_t *blk = output + b * ORC_Q5K_BYTES;
        float sc[8], mn[8], max_sc = 0.f, max_mn = 0.f;
        for (int j = 0; j < 8; j++) {
            float lo = 0.f, hi = x[32 * j];
            for (int l = 0; l < 32; l++) {
                if (x[32 * j + l] < lo) lo = x[32 * j + l];
                if (x[32 * j + l] > hi) hi = x[32 * j + l];
            }
            sc[j] = (hi - lo) / 31.f;
            mn[j] = -lo;
            if (sc[j] > max_sc) max_sc = sc[j];
            if (mn[j] > max_mn) max_mn = mn[j];
        }
        uint16_t dh = orc_f32_to_f16(max_sc / 63.f), mh = orc_f32_to_f16(max_mn / 63.f);
        float d = orc_f16_to_f32(dh), dm = orc_f16_to_f32(mh);
        uint8_t ls[8], lm[8];
        for (int j = 0; j < 8; j++) {
            ls[j] = (uint8_t)clampi(d > 0.f ? nearest_int(sc[j] / d) : 0, 0, 63);
            lm[j] = (uint8_t)clampi(dm > 0.f ? nearest_int(mn[j] / dm) : 0, 0, 63);
        }
        memset(blk, 0, ORC_Q5K_BYTES);
        blk[0] = (uint8_t)(dh & 0xff);
        blk[1] = (uint8_t)(dh >> 8);
        blk[2] = (uint8_t)(mh & 0xff);
        blk[3] = (uint8_t)(mh >> 8);
        uint8_t *ys = blk + 4;
        for (int j = 0; j < 8; j++) {
            if (j < 4) {
                ys[j] = ls[j];
                ys[j + 4] = lm[j];
            } else {
                ys[j + 4] = (uint8_t)((ls[j] & 0xF) | ((lm[j] & 0xF) << 4));
                ys[j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
                ys[j] |= (uint8_t)((lm[j] >> 4) << 6);
            }
        }
        uint8_t *qh = blk + 16, *ql = blk + 48;
        for (int j = 0; j < 8; j++) {
            float dd = d * (float)ls[j], mm = dm * (float)lm[j];
            for (int l = 0; l < 32; l++) {
                int q = dd > 0.f ? clampi(nearest_int((x[32 * j + l] + mm) / dd), 0, 31) : 0;
                int grp = j / 2;
                if (j & 1) ql[32 * grp + l] |= (uint8_t)((q & 0xF) << 4);
                else ql[32 * grp + l] |= (uint8_t)(q & 0xF);
                if (q & 16) qh[l] |= (uint8_t)(1u << j);
            }
        }
    }
}

void orc_quantize_row_q8_0(const float *input, size_t n, uint8_t *output) {
    size_t nb = n / 32;
    for (size_t i = 0; i < nb; i++) {
        const float *x = input + i * 32;
        uint8_t *out = output + i * ORC_Q8_0_BYTES;
        float amax = 0.0f;
        for (int l = 0; l < 32; l++)
            if (fabsf(x[l]) > amax) amax = fabsf(x[l]);
        float d = amax / 127.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        uint16_t d16 = orc_f32_to_f16(d);
        out[0] = (uint8_t)(d16 & 0xff);
        out[1] = (uint8_t)(d16 >> 8);
        for (int l = 0; l < 32; l++) out[2 + l] = (uint8_t)(int8_t)clampi((int)nearbyintf(x[l] * id), -127, 127);
    }
}

typedef struct {
    int type;
    const float *x;
    size_t cols;
    uint8_t *out;
} quant_ctx;
static void quant_rows(size_t b, size_t e, void *p) {
    quant_ctx *c = (quant_ctx *)p;
    size_t rb = orc_row_bytes(c->type, c->cols);
    for (size_t r = b; r < e; r++) {
        const float *x = c->x + r * c->cols;
        uint8_t *o = c->out + r * rb;
        if (c->type == ORC_TYPE_Q4_K) orc_quantize_row_q4k(x, c->cols, o);
        else if (c->type == ORC_TYPE_Q2_K) orc_quantize_row_q2k(x, c->cols, o);
        else if (c->type == ORC_TYPE_Q3_K) orc_quantize_row_q3k(x, c->cols, o);
        else if (c->type == ORC_TYPE_Q5_K) orc_quantize_row_q5k(x, c->cols, o);
        else if (c->type == ORC_TYPE_Q6_K) orc_quantize_row_q6k(x, c->cols, o);
        else orc_quantize_row_q8_0(x, c->cols, o);
    }
}
int orc_quantize_matrix(int type, const float *x, size_t rows, size_t cols, uint8_t *out,
                        int threads) {
    if (orc_row_bytes(type, cols) == 0) return -1;
    quant_ctx c = {type, x, cols, out};
    if (rows <= 64) quant_rows(0, rows, &c);
    else orc_parallel_for(rows, threads, quant_rows, &c);
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * Harness utility, not a restatement of anything in the reference: seeded N(0, sigma) weights
 * quantised block by block with a plain min/max fit (Q4_K), an absmax fit (Q6_K, Q8_0).  It
 * exists so that tests can build full-width random-init matrices (128 256 x 4096 and the like)
 * in a second instead of minutes; the blocks are ordinary GGUF blocks that the dequantisers
 * and dots above read like any other.
 * ---------------------------------------------------------------------------------------- */
static inline uint64_t synth_mix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
static inline void synth_gauss_pair(uint64_t seed, uint64_t idx, float sigma, float *a, float *b) {
    uint64_t r = synth_mix64(seed ^ (idx * 0xd1342543de82ef95ull));
    float u1 = ((float)(uint32_t)(r >> 40) + 1.0f) * (1.0f / 16777217.0f);
    float u2 = (float)(uint32_t)(r & 0xffffff) * (1.0f / 16777216.0f);
    float rad = sigma * sqrtf(-2.0f * logf(u1));
    *a = rad * cosf(6.2831853f * u2);
    *b = rad * sinf(6.2831853f * u2);
}
static void synth_block(int type, uint64_t seed, uint64_t block_index, float sigma, uint8_t *out) {
    float x[256];
    for (int i = 0; i < 256; i += 2) synth_gauss_pair(seed, block_index * 128 + (uint64_t)(i / 2), sigma, &x[i], &x[i + 1]);
    if (type == ORC_TYPE_Q4_K) {
        float sc[8], mn[8], max_sc = 0.0f, max_mn = 0.0f;
        for (int j = 0; j < 8; j++) {
            float lo = 0.0f, hi = x[32 * j];
            for (int l = 0; l < 32; l++) {
                if (x[32 * j + l] < lo) lo = x[32 * j + l];
                if (x[32 * j + l] > hi) hi = x[32 * j + l];
            }
            sc[j] = (hi - lo) / 15.0f;
            mn[j] = -lo;
            if (sc[j] > max_sc) max_sc = sc[j];
            if (mn[j] > max_mn) max_mn = mn[j];
        }
        uint16_t dh = orc_f32_to_f16(max_sc / 63.0f), mh = orc_f32_to_f16(max_mn / 63.0f);
        float d = orc_f16_to_f32(dh), dm = orc_f16_to_f32(mh);
        uint8_t ls[8], lm[8], ys[12] = {0};
        for (int j = 0; j < 8; j++) {
            ls[j] = (uint8_t)clampi(d > 0.0f ? nearest_int(sc[j] / d) : 0, 0, 63);
            lm[j] = (uint8_t)clampi(dm > 0.0f ? nearest_int(mn[j] / dm) : 0, 0, 63);
        }
        for (int j = 0; j < 8; j++) {
            if (j < 4) {
                ys[j] |= ls[j];
                ys[j + 4] |= lm[j];
            } else {
                ys[j + 4] = (uint8_t)((ls[j] & 0xF) | ((lm[j] & 0xF) << 4));
                ys[j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
                ys[j] |= (uint8_t)((lm[j] >> 4) << 6);
            }
        }
        out[0] = (uint8_t)(dh & 0xff);
        out[1] = (uint8_t)(dh >> 8);
        out[2] = (uint8_t)(mh & 0xff);
        out[3] = (uint8_t)(mh >> 8);
        memcpy(out + 4, ys, 12);
        for (int g = 0; g < 4; g++)
            for (int l = 0; l < 32; l++) {
                int q[2];
                for (int h = 0; h < 2; h++) {
                    int j = 2 * g + h;
                    float ds = d * ls[j], ms = dm * lm[j];
                    q[h] = ds > 0.0f ? clampi(nearest_int((x[64 * g + 32 * h + l] + ms) / ds), 0, 15) : 0;
                }
                out[16 + 32 * g + l] = (uint8_t)(q[0] | (q[1] << 4));
            }
    } else if (type == ORC_TYPE_Q2_K) {
        orc_quantize_row_q2k(x, 256, out);
    } else if (type == ORC_TYPE_Q3_K) {
        orc_quantize_row_q3k(x, 256, out);
    } else if (type == ORC_TYPE_Q5_K) {
        orc_quantize_row_q5k(x, 256, out);
    } else if (type == ORC_TYPE_Q6_K) {
        orc_quantize_row_q6k(x, 256, out);
    } else {
        orc_quantize_row_q8_0(x, 256, out);
    }
}
typedef struct {
    int type;
    uint64_t seed;
    float sigma;
    uint8_t *out;
} synth_ctx;
static void synth_blocks(size_t b, size_t e, void *p) {
    synth_ctx *c = (synth_ctx *)p;
    size_t bb = orc_row_bytes(c->type, 256);
    for (size_t i = b; i < e; i++) synth_block(c->type, c->seed, i, c->sigma, c->out + i * bb);
}
int orc_synth_matrix(int type, size_t rows, size_t cols, uint64_t seed, float sigma, uint8_t *out, int threads) {
    if (orc_row_bytes(type, cols) == 0 || cols % 256 != 0) return -1;
    synth_ctx c = {type, seed, sigma, out};
    orc_parallel_for(rows * (cols / 256), threads, synth_blocks, &c);
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * Integer row dots.  Two statements of each: `_lanes` is portable C that reproduces the
 * AVX2 lane structure (8 f32 accumulators per row, one FMA per block, the same horizontal
 * sum order) and is bit-identical to the intrinsic version, which follows
 * crates/rnb-cpu/src/gemm/avx2_dot.rs:621-696 (Q4_K) and :801-885 (Q6_K).
 * ---------------------------------------------------------------------------------------- */
static int g_force_scalar = 0;
void orc_force_scalar(int on) { g_force_scalar = on; }
int orc_have_avx2(void) {
    return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
}

/* crates/rnb-cpu/src/gemm/avx2_dot.rs:147-164 */
static inline void unpack_q4k_scales(const uint8_t *scales12, uint32_t utmp[4]) {
    const uint32_t k1 = 0x3f3f3f3fu, k2 = 0x0f0f0f0fu, k3 = 0x03030303u;
    utmp[0] = rd_u32(scales12);
    utmp[1] = rd_u32(scales12 + 4);
    utmp[2] = rd_u32(scales12 + 8);
    utmp[3] = ((utmp[2] >> 4) & k2) | (((utmp[1] >> 6) & k3) << 4);
    uint32_t uaux = utmp[1] & k1;
    utmp[1] = (utmp[2] & k2) | (((utmp[0] >> 6) & k3) << 4);
    utmp[2] = uaux;
    utmp[0] &= k1;
}

/* hsum_float_8 order (avx2_dot.rs:25-31): (l+l4 pairs) → (+2) → (+1) */
static inline float hsum8(const float a[8]) {
    float r0 = a[4] + a[0], r1 = a[5] + a[1], r2 = a[6] + a[2], r3 = a[7] + a[3];
    float s0 = r0 + r2, s1 = r1 + r3;
    return s0 + s1;
}

float orc_dot_q4k_q8k_lanes(const uint8_t *row, const orc_q8k_block *y, size_t nb) {
    float acc[8] = {0}, acc_m[4] = {0};
    for (size_t i = 0; i < nb; i++) {
        const uint8_t *block = row + i * ORC_Q4K_BYTES;
        float d = y[i].d * orc_f16_to_f32(rd_u16(block));
        float dmin = -y[i].d * orc_f16_to_f32(rd_u16(block + 2));
        uint32_t utmp[4];
        unpack_q4k_scales(block + 4, utmp);
        uint8_t sc[8], mn[8];
        memcpy(sc, &utmp[0], 8);
        memcpy(mn, &utmp[2], 8);
        for (int k = 0; k < 4; k++) {
            int32_t b0 = (int16_t)(y[i].bsums[4 * k] + y[i].bsums[4 * k + 1]);
            int32_t b1 = (int16_t)(y[i].bsums[4 * k + 2] + y[i].bsums[4 * k + 3]);
            int32_t prod = (int32_t)mn[2 * k] * b0 + (int32_t)mn[2 * k + 1] * b1;
            acc_m[k] = fmaf(dmin, (float)prod, acc_m[k]);
        }
        const uint8_t *q4 = block + 16;
        const int8_t *q8 = y[i].qs;
        int32_t sumi[8] = {0};
        for (int j = 0; j < 4; j++) {
            for (int l = 0; l < 8; l++) {
                int32_t lo = 0, hi = 0;
                for (int b = 0; b < 4; b++) {
                    uint8_t q = q4[32 * j + 4 * l + b];
                    lo += (int32_t)(q & 0xF) * q8[64 * j + 4 * l + b];
                    hi += (int32_t)(q >> 4) * q8[64 * j + 32 + 4 * l + b];
                }
                sumi[l] += (int32_t)sc[2 * j] * lo + (int32_t)sc[2 * j + 1] * hi;
            }
        }
        for (int l = 0; l < 8; l++) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    float m0 = acc_m[0] + acc_m[2], m1 = acc_m[1] + acc_m[3];
    return hsum8(acc) + (m0 + m1);
}

/* Q2_K x Q8_K: crates/rnb-cpu/src/gemm/avx2_dot.rs:169-245.  Eight f32 accumulator lanes; per block first
 * the mins term (lane l: mins[2l] * bsums[2l] + mins[2l+1] * bsums[2l+1], one FMA with dmin), then the
 * quants (lane l = bytes 4l..4l+3 of each 32-byte chunk; chunk k of half h is the 2-bit plane k, its
 * scale is sub-block 8h + 2k for lanes 0..3 and 8h + 2k + 1 for lanes 4..7), one FMA with d. */
float orc_dot_q2k_q8k(const uint8_t *row, const orc_q8k_block *y, size_t nb) {
    float acc[8] = {0};
    for (size_t i = 0; i < nb; i++) {
        const uint8_t *block = row + i * ORC_Q2K_BYTES;
        const uint8_t *q2 = block + 16;
        float d = y[i].d * orc_f16_to_f32(rd_u16(block + 80));
        float dmin = -y[i].d * orc_f16_to_f32(rd_u16(block + 82));
        for (int l = 0; l < 8; l++) {
            int32_t prod = (int32_t)(block[2 * l] >> 4) * (int32_t)y[i].bsums[2 * l] + (int32_t)(block[2 * l + 1] >> 4) * (int32_t)y[i].bsums[2 * l + 1];
            acc[l] = fmaf(dmin, (float)prod, acc[l]);
        }
        int32_t sumi[8] = {0};
        for (int h = 0; h < 2; h++)
            for (int k = 0; k < 4; k++)
                for (int l = 0; l < 8; l++) {
                    int32_t p = 0;
                    for (int b = 0; b < 4; b++) p += (int32_t)((q2[32 * h + 4 * l + b] >> (2 * k)) & 3) * (int32_t)y[i].qs[128 * h + 32 * k + 4 * l + b];
                    sumi[l] += (int32_t)(block[8 * h + 2 * k + (l >= 4)] & 0x0F) * p;
                }
        for (int l = 0; l < 8; l++) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    return hsum8(acc);
}

/* Q3_K x Q8_K: crates/rnb-cpu/src/gemm/avx2_dot.rs:247-378.  Eight f32 accumulator lanes, one FMA per
 * block; lane l = bytes 4l..4l+3 of each 32-byte chunk; chunk k of half h is the 2-bit plane k minus 4
 * where hmask bit 4h + k is clear, and takes scale 8h + 2k (lanes 0..3) or 8h + 2k + 1 (lanes 4..7). */
float orc_dot_q3k_q8k(const uint8_t *row, const orc_q8k_block *y, size_t nb) {
    float acc[8] = {0};
    for (size_t i = 0; i < nb; i++) {
        const uint8_t *block = row + i * ORC_Q3K_BYTES;
        const uint8_t *hm = block, *q3 = block + 32;
        float d = y[i].d * orc_f16_to_f32(rd_u16(block + 108));
        int8_t scales[16];
        q3k_scales(block + 96, scales);
        int32_t sumi[8] = {0};
        for (int h = 0; h < 2; h++)
            for (int k = 0; k < 4; k++)
                for (int l = 0; l < 8; l++) {
                    int32_t p = 0;
                    for (int b = 0; b < 4; b++) {
                        int e = 4 * l + b;
                        int v = ((q3[32 * h + e] >> (2 * k)) & 3) - (((hm[e] >> (4 * h + k)) & 1) ? 0 : 4);
                        p += v * (int32_t)y[i].qs[128 * h + 32 * k + e];
                    }
                    sumi[l] += ((int32_t)scales[8 * h + 2 * k + (l >= 4)] - 32) * p;
                }
        for (int l = 0; l < 8; l++) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    return hsum8(acc);
}

/* Q5_K x Q8_K: crates/rnb-cpu/src/gemm/avx2_dot.rs:698-789.  Eight f32 accumulator lanes as for
 * Q4_K (lane l = bytes 4l..4l+3 of every 32-byte group, one FMA per block); the fifth bit comes from
 * the qh plane (bit j of qh[i] belongs to element i of sub-block j); the mins term is ONE scalar:
 * summs += dmin * (sum_j mins_j * bsum32_j), a multiply and an add per block, added to the folded
 * lanes at the end. */
float orc_dot_q5k_q8k(const uint8_t *row, const orc_q8k_block *y, size_t nb) {
    float acc[8] = {0}, summs = 0.0f;
    for (size_t i = 0; i < nb; i++) {
        const uint8_t *block = row + i * ORC_Q5K_BYTES;
        float d = y[i].d * orc_f16_to_f32(rd_u16(block));
        float dmin = -y[i].d * orc_f16_to_f32(rd_u16(block + 2));
        uint32_t utmp[4];
        unpack_q4k_scales(block + 4, utmp);
        uint8_t sc[8], mn[8];
        memcpy(sc, &utmp[0], 8);
        memcpy(mn, &utmp[2], 8);
        int32_t msum = 0;
        for (int j = 0; j < 8; j++) msum += (int32_t)mn[j] * (int32_t)(int16_t)(y[i].bsums[2 * j] + y[i].bsums[2 * j + 1]);
        volatile float mprod = dmin * (float)msum;   /* a rounded product, then a rounded sum: no contraction */
        summs = summs + mprod;
        const uint8_t *qh = block + 16, *q5 = block + 48;
        const int8_t *q8 = y[i].qs;
        int32_t sumi[8] = {0};
        for (int j = 0; j < 4; j++) {
            for (int l = 0; l < 8; l++) {
                int32_t lo = 0, hi = 0;
                for (int b = 0; b < 4; b++) {
                    int e = 4 * l + b;
                    uint8_t q = q5[32 * j + e];
                    int v0 = (q & 0xF) + (((qh[e] >> (2 * j)) & 1) << 4);
                    int v1 = (q >> 4) + (((qh[e] >> (2 * j + 1)) & 1) << 4);
                    lo += v0 * q8[64 * j + e];
                    hi += v1 * q8[64 * j + 32 + e];
                }
                sumi[l] += (int32_t)sc[2 * j] * lo + (int32_t)sc[2 * j + 1] * hi;
            }
        }
        for (int l = 0; l < 8; l++) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    return hsum8(acc) + summs;
}

float orc_dot_q6k_q8k_lanes(const uint8_t *row, const orc_q8k_block *y, size_t nb) {
    float acc[8] = {0};
    for (size_t i = 0; i < nb; i++) {
        const uint8_t *block = row + i * ORC_Q6K_BYTES;
        const uint8_t *ql = block, *qh = block + 128;
        const int8_t *sc = (const int8_t *)(block + 192);
        float d = y[i].d * orc_f16_to_f32(rd_u16(block + 208));
        int32_t sumi[8];
        /* q8sclsub lane l = (bsums[2l]*sc[2l] + bsums[2l+1]*sc[2l+1]) << 5 */
        for (int l = 0; l < 8; l++)
            sumi[l] = -(((int32_t)y[i].bsums[2 * l] * sc[2 * l] +
                         (int32_t)y[i].bsums[2 * l + 1] * sc[2 * l + 1]) *
                        32);
        const int8_t *q8 = y[i].qs;
        for (int n = 0; n < 2; n++) {
            for (int part = 0; part < 4; part++) {
                /* part p covers elements 128n + 32p .. +32; its two 16-groups use scales
                 * sc[8n + 2p] and sc[8n + 2p + 1] (lanes 0-3 / 4-7). */
                for (int l = 0; l < 8; l++) {
                    int32_t s = 0;
                    for (int b = 0; b < 4; b++) {
                        int e = 4 * l + b; /* 0..31 within the part */
                        uint8_t lo4 = (part & 1) ? ql[64 * n + 32 + e] : ql[64 * n + e];
                        int nib = (part & 2) ? (lo4 >> 4) : (lo4 & 0xF);
                        int hi2 = (qh[32 * n + e] >> (2 * part)) & 3;
                        s += (int32_t)(nib | (hi2 << 4)) * q8[128 * n + 32 * part + e];
                    }
                    sumi[l] += (int32_t)sc[8 * n + 2 * part + (l >> 2)] * s;
                }
            }
        }
        for (int l = 0; l < 8; l++) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    return hsum8(acc);
}

__attribute__((target("avx2,fma"))) static inline float hsum_float_8(__m256 x) {
    __m128 res = _mm256_extractf128_ps(x, 1);
    res = _mm_add_ps(res, _mm256_castps256_ps128(x));
    res = _mm_add_ps(res, _mm_movehl_ps(res, res));
    res = _mm_add_ss(res, _mm_movehdup_ps(res));
    return _mm_cvtss_f32(res);
}

__attribute__((target("avx2,fma"))) static float dot_q4k_q8k_avx2(const uint8_t *row,
                                                                   const orc_q8k_block *y,
                                                                   size_t nb) {
    const __m256i m4 = _mm256_set1_epi8(0xF);
    __m256 acc = _mm256_setzero_ps();
    __m128 acc_m = _mm_setzero_ps();
    for (size_t i = 0; i < nb; i++) {
        const uint8_t *block = row + i * ORC_Q4K_BYTES;
        float d = y[i].d * orc_f16_to_f32(rd_u16(block));
        float dmin = -y[i].d * orc_f16_to_f32(rd_u16(block + 2));
        uint32_t utmp[4];
        unpack_q4k_scales(block + 4, utmp);
        const __m256i mins_and_scales = _mm256_cvtepu8_epi16(
            _mm_set_epi32((int)utmp[3], (int)utmp[2], (int)utmp[1], (int)utmp[0]));
        const __m256i q8sums = _mm256_loadu_si256((const __m256i *)y[i].bsums);
        const __m128i q8s = _mm_hadd_epi16(_mm256_extracti128_si256(q8sums, 0),
                                           _mm256_extracti128_si256(q8sums, 1));
        const __m128i prod = _mm_madd_epi16(_mm256_extracti128_si256(mins_and_scales, 1), q8s);
        acc_m = _mm_fmadd_ps(_mm_set1_ps(dmin), _mm_cvtepi32_ps(prod), acc_m);
        const __m128i sc128 = _mm256_extracti128_si256(mins_and_scales, 0);
        const __m256i scales = _mm256_set_m128i(sc128, sc128);
        __m256i sumi = _mm256_setzero_si256();
        const uint8_t *q4 = block + 16;
        const int8_t *q8 = y[i].qs;
        for (int j = 0; j < 4; j++) {
            const __m256i scale_l = _mm256_shuffle_epi8(
                scales, _mm256_set1_epi16((short)(((4 * j + 1) << 8) | (4 * j))));
            const __m256i scale_h = _mm256_shuffle_epi8(
                scales, _mm256_set1_epi16((short)(((4 * j + 3) << 8) | (4 * j + 2))));
            const __m256i q4bits = _mm256_loadu_si256((const __m256i *)q4);
            q4 += 32;
            const __m256i q4l = _mm256_and_si256(q4bits, m4);
            const __m256i q4h = _mm256_and_si256(_mm256_srli_epi16(q4bits, 4), m4);
            const __m256i q8l = _mm256_loadu_si256((const __m256i *)q8);
            q8 += 32;
            __m256i p16l = _mm256_madd_epi16(scale_l, _mm256_maddubs_epi16(q4l, q8l));
            const __m256i q8h = _mm256_loadu_si256((const __m256i *)q8);
            q8 += 32;
            __m256i p16h = _mm256_madd_epi16(scale_h, _mm256_maddubs_epi16(q4h, q8h));
            sumi = _mm256_add_epi32(sumi, _mm256_add_epi32(p16l, p16h));
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    __m128 acc_m_hi = _mm_add_ps(acc_m, _mm_movehl_ps(acc_m, acc_m));
    __m128 acc_m_final = _mm_add_ss(acc_m_hi, _mm_movehdup_ps(acc_m_hi));
    return hsum_float_8(acc) + _mm_cvtss_f32(acc_m_final);
}

__attribute__((target("avx2,fma"))) static float dot_q6k_q8k_avx2(const uint8_t *row,
                                                                   const orc_q8k_block *y,
                                                                   size_t nb) {
    const __m256i m3 = _mm256_set1_epi8(3), m15 = _mm256_set1_epi8(15);
    const __m256i m12 = _mm256_set1_epi8(12), m48 = _mm256_set1_epi8(48);
    const __m256i mtop2 = _mm256_set1_epi8(-64);
    __m256 acc = _mm256_setzero_ps();
    for (size_t i = 0; i < nb; i++) {
        const uint8_t *block = row + i * ORC_Q6K_BYTES;
        const uint8_t *q4 = block, *qh = block + 128;
        float d = y[i].d * orc_f16_to_f32(rd_u16(block + 208));
        const __m256i q8sums = _mm256_loadu_si256((const __m256i *)y[i].bsums);
        const __m128i scales = _mm_loadu_si128((const __m128i *)(block + 192));
        const __m256i q8sclsub =
            _mm256_slli_epi32(_mm256_madd_epi16(q8sums, _mm256_cvtepi8_epi16(scales)), 5);
        __m256i sumi = _mm256_setzero_si256();
        const int8_t *q8 = y[i].qs;
        int is = 0;
        for (int j = 0; j < 2; j++) {
            const __m256i q4bits1 = _mm256_loadu_si256((const __m256i *)q4);
            q4 += 32;
            const __m256i q4bits2 = _mm256_loadu_si256((const __m256i *)q4);
            q4 += 32;
            const __m256i q4bitsh = _mm256_loadu_si256((const __m256i *)qh);
            qh += 32;
            const __m256i q4h_0 = _mm256_slli_epi16(_mm256_and_si256(q4bitsh, m3), 4);
            const __m256i q4h_1 = _mm256_slli_epi16(_mm256_and_si256(q4bitsh, m12), 2);
            const __m256i q4h_2 = _mm256_and_si256(q4bitsh, m48);
            const __m256i q4h_3 = _mm256_srli_epi16(_mm256_and_si256(q4bitsh, mtop2), 2);
            const __m256i q4_0 = _mm256_or_si256(_mm256_and_si256(q4bits1, m15), q4h_0);
            const __m256i q4_1 = _mm256_or_si256(_mm256_and_si256(q4bits2, m15), q4h_1);
            const __m256i q4_2 =
                _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(q4bits1, 4), m15), q4h_2);
            const __m256i q4_3 =
                _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(q4bits2, 4), m15), q4h_3);
            __m256i p[4];
            const __m256i qq[4] = {q4_0, q4_1, q4_2, q4_3};
            for (int t = 0; t < 4; t++) {
                const __m256i q8v = _mm256_loadu_si256((const __m256i *)q8);
                q8 += 32;
                /* scale shuffle: lanes 0-3 ← scales[2*(is+t)], lanes 4-7 ← scales[2*(is+t)+1],
                 * widened to i16 (the SCALE_SHUFFLE_Q6 table of avx2_dot.rs) */
                const int s0 = ((const int8_t *)(block + 192))[2 * (is + t)];
                const int s1 = ((const int8_t *)(block + 192))[2 * (is + t) + 1];
                const __m256i sc16 = _mm256_set_m128i(_mm_set1_epi16((short)s1),
                                                      _mm_set1_epi16((short)s0));
                p[t] = _mm256_madd_epi16(sc16, _mm256_maddubs_epi16(qq[t], q8v));
            }
            is += 4;
            sumi = _mm256_add_epi32(sumi, _mm256_add_epi32(p[0], p[1]));
            sumi = _mm256_add_epi32(sumi, _mm256_add_epi32(p[2], p[3]));
        }
        sumi = _mm256_sub_epi32(sumi, q8sclsub);
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    return hsum_float_8(acc);
}

float orc_dot_q4k_q8k(const uint8_t *row, const orc_q8k_block *y, size_t nb) {
    if (!g_force_scalar && orc_have_avx2()) return dot_q4k_q8k_avx2(row, y, nb);
    return orc_dot_q4k_q8k_lanes(row, y, nb);
}
float orc_dot_q6k_q8k(const uint8_t *row, const orc_q8k_block *y, size_t nb) {
    if (!g_force_scalar && orc_have_avx2()) return dot_q6k_q8k_avx2(row, y, nb);
    return orc_dot_q6k_q8k_lanes(row, y, nb);
}

/* crates/rnb-cpu/src/gemm/quant_gemv.rs:127-141 — f32 activations, sequential sums */
float orc_dot_q8_0_row(const uint8_t *row, const float *x, size_t blocks_per_row) {
    float acc = 0.0f;
    for (size_t bi = 0; bi < blocks_per_row; bi++) {
        const uint8_t *b = row + bi * ORC_Q8_0_BYTES;
        float d = orc_f16_to_f32(rd_u16(b));
        const float *xb = x + bi * 32;
        float block_sum = 0.0f;
        for (int i = 0; i < 32; i++) block_sum += (float)(int8_t)b[2 + i] * xb[i];
        acc += d * block_sum;
    }
    return acc;
}

/* crates/rnb-cpu/src/gemm/quant_gemv.rs:228-314 (dot_quantized_row, non-aarch64 branch):
 * dequantise a block, sum tmp[i]*x[i] sequentially, add per block. */
float orc_dot_dequant_row(int type, const uint8_t *row, const float *x, size_t cols) {
    float acc = 0.0f;
    float tmp[256];
    if (type == ORC_TYPE_Q8_0) { /* dot_basic_blocks_scalar :178-224: one running sum */
        for (size_t b = 0; b < cols / 32; b++) {
            orc_dequantize_q8_0_block(row + b * ORC_Q8_0_BYTES, tmp);
            for (int i = 0; i < 32; i++) acc += tmp[i] * x[b * 32 + i];
        }
        return acc;
    }
    size_t bb = type == ORC_TYPE_Q4_K ? ORC_Q4K_BYTES : ORC_Q6K_BYTES;
    for (size_t b = 0; b < cols / 256; b++) {
        if (type == ORC_TYPE_Q4_K) orc_dequantize_q4k_block(row + b * bb, tmp);
        else orc_dequantize_q6k_block(row + b * bb, tmp);
        float block_acc = 0.0f;
        for (int i = 0; i < 256; i++) block_acc += tmp[i] * x[b * 256 + i];
        acc += block_acc;
    }
    return acc;
}

/* ------------------------------------------------------------------------------------------
 * GEMV drivers.  K-quants: crates/rnb-cpu/src/gemm/quant_gemv.rs:1103-1183
 * (gemv_quantized_avx2: Q8_K per token, row chunks, seq-major out[s*rows+row]).
 * Q8_0: :360-401 (gemv_q8_0, f32 activations).
 * ---------------------------------------------------------------------------------------- */
typedef struct {
    int type;
    const uint8_t *w;
    const float *x;
    const orc_q8k_block *xq;
    float *out;
    size_t rows, cols, seq_len, row_bytes, nb;
} gemv_ctx;

static void gemv_rows(size_t b, size_t e, void *p) {
    gemv_ctx *c = (gemv_ctx *)p;
    for (size_t r = b; r < e; r++) {
        const uint8_t *row = c->w + r * c->row_bytes;
        for (size_t s = 0; s < c->seq_len; s++) {
            float v;
            if (c->type == ORC_TYPE_Q4_K) v = orc_dot_q4k_q8k(row, c->xq + s * c->nb, c->nb);
            else if (c->type == ORC_TYPE_Q2_K) v = orc_dot_q2k_q8k(row, c->xq + s * c->nb, c->nb);
            else if (c->type == ORC_TYPE_Q3_K) v = orc_dot_q3k_q8k(row, c->xq + s * c->nb, c->nb);
            else if (c->type == ORC_TYPE_Q5_K) v = orc_dot_q5k_q8k(row, c->xq + s * c->nb, c->nb);
            else if (c->type == ORC_TYPE_Q6_K) v = orc_dot_q6k_q8k(row, c->xq + s * c->nb, c->nb);
            else v = orc_dot_q8_0_row(row, c->x + s * c->cols, c->cols / 32);
            c->out[s * c->rows + r] = v;
        }
    }
}

int orc_gemv(int type, const uint8_t *w, const float *x, float *out, size_t rows, size_t cols,
             size_t seq_len, int threads) {
    gemv_ctx c;
    memset(&c, 0, sizeof(c));
    c.type = type;
    c.w = w;
    c.x = x;
    c.out = out;
    c.rows = rows;
    c.cols = cols;
    c.seq_len = seq_len;
    c.row_bytes = orc_row_bytes(type, cols);
    if (c.row_bytes == 0) return -1;
    orc_q8k_block *xq = NULL;
    if (type != ORC_TYPE_Q8_0) {
        if (cols % 256) return -1;
        c.nb = cols / 256;
        xq = (orc_q8k_block *)malloc(sizeof(orc_q8k_block) * c.nb * seq_len);
        for (size_t s = 0; s < seq_len; s++) orc_quantize_q8k(x + s * cols, cols, xq + s * c.nb);
        c.xq = xq;
    } else if (cols % 32) {
        return -1;
    }
    orc_parallel_for(rows, threads, gemv_rows, &c);
    free(xq);
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * Decode attention, fp32.
 * 4-pass: crates/rnb-cpu/src/kernels/attention/decode_flash.rs:91-212
 * online: :245-297 (process_head).  f32·f16 dot: x86_helpers.rs:11-54 (two 8-lane
 * accumulators, mul then add, no FMA); scaled add: :58-80.
 * ---------------------------------------------------------------------------------------- */
static float dot_f32_f16_scalar(const float *a, const uint16_t *b, size_t len) {
    float acc0[8] = {0}, acc1[8] = {0};
    size_t i = 0;
    for (; i + 16 <= len; i += 16) {
        for (int l = 0; l < 8; l++) acc0[l] = acc0[l] + a[i + l] * orc_f16_to_f32(b[i + l]);
        for (int l = 0; l < 8; l++)
            acc1[l] = acc1[l] + a[i + 8 + l] * orc_f16_to_f32(b[i + 8 + l]);
    }
    for (; i + 8 <= len; i += 8)
        for (int l = 0; l < 8; l++) acc0[l] = acc0[l] + a[i + l] * orc_f16_to_f32(b[i + l]);
    float acc[8];
    for (int l = 0; l < 8; l++) acc[l] = acc0[l] + acc1[l];
    /* lo+hi, then movehdup add, then movehl add */
    float s0 = acc[0] + acc[4], s1 = acc[1] + acc[5], s2 = acc[2] + acc[6], s3 = acc[3] + acc[7];
    float t0 = s0 + s1, t2 = s2 + s3;
    float total = t0 + t2;
    for (; i < len; i++) total += a[i] * orc_f16_to_f32(b[i]);
    return total;
}
static void scaled_add_f16_scalar(float *out, const uint16_t *v, float scale, size_t len) {
    for (size_t i = 0; i < len; i++) out[i] = out[i] + orc_f16_to_f32(v[i]) * scale;
}
/* The same two routines with F16C/AVX2, as the reference's x86 helpers are written
 * (x86_helpers.rs:11-80): identical lane order, mul then add, so identical bits. */
__attribute__((target("avx2,f16c"))) static float dot_f32_f16_avx2(const float *a,
                                                                   const uint16_t *b,
                                                                   size_t len) {
    __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
    size_t i = 0;
    for (; i + 16 <= len; i += 16) {
        acc0 = _mm256_add_ps(acc0, _mm256_mul_ps(_mm256_loadu_ps(a + i),
                                                 _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(b + i)))));
        acc1 = _mm256_add_ps(acc1, _mm256_mul_ps(_mm256_loadu_ps(a + i + 8),
                                                 _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(b + i + 8)))));
    }
    for (; i + 8 <= len; i += 8)
        acc0 = _mm256_add_ps(acc0, _mm256_mul_ps(_mm256_loadu_ps(a + i),
                                                 _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(b + i)))));
    __m256 acc = _mm256_add_ps(acc0, acc1);
    __m128 sum128 = _mm_add_ps(_mm256_castps256_ps128(acc), _mm256_extractf128_ps(acc, 1));
    __m128 shuf = _mm_movehdup_ps(sum128);
    __m128 sums = _mm_add_ps(sum128, shuf);
    shuf = _mm_movehl_ps(shuf, sums);
    float total = _mm_cvtss_f32(_mm_add_ss(sums, shuf));
    for (; i < len; i++) total += a[i] * orc_f16_to_f32(b[i]);
    return total;
}
__attribute__((target("avx2,f16c"))) static void scaled_add_f16_avx2(float *out, const uint16_t *v,
                                                                     float scale, size_t len) {
    const __m256 s = _mm256_set1_ps(scale);
    size_t i = 0;
    for (; i + 8 <= len; i += 8) {
        __m256 vf = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(v + i)));
        _mm256_storeu_ps(out + i, _mm256_add_ps(_mm256_loadu_ps(out + i), _mm256_mul_ps(vf, s)));
    }
    for (; i < len; i++) out[i] = out[i] + orc_f16_to_f32(v[i]) * scale;
}
static int have_f16c(void) {
    return !g_force_scalar && __builtin_cpu_supports("avx2") && __builtin_cpu_supports("f16c");
}
static float dot_f32_f16(const float *a, const uint16_t *b, size_t len) {
    return have_f16c() ? dot_f32_f16_avx2(a, b, len) : dot_f32_f16_scalar(a, b, len);
}
static void scaled_add_f16(float *out, const uint16_t *v, float scale, size_t len) {
    if (have_f16c()) scaled_add_f16_avx2(out, v, scale, len);
    else scaled_add_f16_scalar(out, v, scale, len);
}

typedef struct {
    const float *q;
    const uint16_t *k, *v;
    float *out;
    size_t num_heads, num_kv_heads, head_dim, kv_len;
    float scale;
    size_t window;   /* sliding window (0 = none): position j is masked when j + window <= kv_len - 1 */
} attn_ctx;
static void attn_heads(size_t hb, size_t he, void *p) {
    attn_ctx *c = (attn_ctx *)p;
    size_t group = c->num_heads / c->num_kv_heads, kv_dim = c->num_kv_heads * c->head_dim;
    size_t head_dim = c->head_dim, kv_len = c->kv_len;
    float *scores = (float *)malloc(sizeof(float) * (kv_len ? kv_len : 1));
    for (size_t h = hb; h < he; h++) {
        size_t kv_h = h / group;
        const float *qh = c->q + h * head_dim;
        for (size_t j = 0; j < kv_len; j++) {
            /* decode_flash.rs:139-146: a masked position scores -inf (its weight is exp(-inf) = 0) */
            if (c->window && j + c->window <= kv_len - 1) {
                scores[j] = -INFINITY;
                continue;
            }
            scores[j] = dot_f32_f16(qh, c->k + j * kv_dim + kv_h * head_dim, head_dim) * c->scale;
        }
        float max_score = -INFINITY;
        for (size_t j = 0; j < kv_len; j++)
            if (scores[j] > max_score) max_score = scores[j];
        float sum = 0.0f;
        for (size_t j = 0; j < kv_len; j++) {
            scores[j] = expf(scores[j] - max_score);
            sum += scores[j];
        }
        float inv_sum = sum > 0.0f ? 1.0f / sum : 0.0f;
        float *o = c->out + h * head_dim;
        for (size_t d = 0; d < head_dim; d++) o[d] = 0.0f;
        for (size_t j = 0; j < kv_len; j++)
            scaled_add_f16(o, c->v + j * kv_dim + kv_h * head_dim, scores[j] * inv_sum, head_dim);
    }
    free(scores);
}
void orc_attention_decode(const float *q, const uint16_t *k, const uint16_t *v, float *out,
                          size_t num_heads, size_t num_kv_heads, size_t head_dim, size_t kv_len,
                          float scale) {
    attn_ctx c = {q, k, v, out, num_heads, num_kv_heads, head_dim, kv_len, scale, 0};
    attn_heads(0, num_heads, &c);
}
/* attention_decode_into_with_scale_window_and_softcap with sliding_window = Some(window), softcap = None
 * (crates/rnb-cpu/src/kernels/attention/decode_flash.rs:91-212): every position is walked, the masked ones
 * with weight zero. */
void orc_attention_decode_window(const float *q, const uint16_t *k, const uint16_t *v, float *out,
                                 size_t num_heads, size_t num_kv_heads, size_t head_dim, size_t kv_len,
                                 float scale, size_t window) {
    attn_ctx c = {q, k, v, out, num_heads, num_kv_heads, head_dim, kv_len, scale, window};
    attn_heads(0, num_heads, &c);
}
/* Heads are independent; the reference runs them in parallel on its thread pool. */
void orc_attention_decode_mt(const float *q, const uint16_t *k, const uint16_t *v, float *out,
                             size_t num_heads, size_t num_kv_heads, size_t head_dim, size_t kv_len,
                             float scale, int threads) {
    attn_ctx c = {q, k, v, out, num_heads, num_kv_heads, head_dim, kv_len, scale, 0};
    if (threads <= 1) {
        attn_heads(0, num_heads, &c);
        return;
    }
    /* orc_parallel_for keeps n <= 64 on one thread; split heads by hand */
    size_t nt = (size_t)threads < num_heads ? (size_t)threads : num_heads;
    size_t chunk = (num_heads + nt - 1) / nt;
    pthread_t tid[256];
    orc_task task[256];
    int n = 0;
    for (size_t b = 0; b < num_heads && n < 256; b += chunk, n++) {
        task[n].fn = attn_heads;
        task[n].ctx = &c;
        task[n].begin = b;
        task[n].end = b + chunk < num_heads ? b + chunk : num_heads;
    }
    for (int i = 1; i < n; i++) pthread_create(&tid[i], NULL, orc_task_main, &task[i]);
    orc_task_main(&task[0]);
    for (int i = 1; i < n; i++) pthread_join(tid[i], NULL);
}

void orc_attention_decode_online(const float *q, const uint16_t *k, const uint16_t *v, float *out,
                                 size_t num_heads, size_t num_kv_heads, size_t head_dim,
                                 size_t kv_len, float scale) {
    size_t group = num_heads / num_kv_heads, kv_dim = num_kv_heads * head_dim;
    for (size_t h = 0; h < num_heads; h++) {
        size_t kv_h = h / group;
        const float *qh = q + h * head_dim;
        float *o = out + h * head_dim;
        float m = -INFINITY, s = 0.0f;
        for (size_t d = 0; d < head_dim; d++) o[d] = 0.0f;
        for (size_t j = 0; j < kv_len; j++) {
            size_t off = j * kv_dim + kv_h * head_dim;
            float x = dot_f32_f16(qh, k + off, head_dim) * scale;
            if (x > m) {
                if (m > -INFINITY) {
                    float alpha = expf(m - x);
                    for (size_t d = 0; d < head_dim; d++) o[d] *= alpha;
                    s *= alpha;
                }
                scaled_add_f16(o, v + off, 1.0f, head_dim);
                s += 1.0f;
                m = x;
            } else {
                float p = expf(x - m);
                scaled_add_f16(o, v + off, p, head_dim);
                s += p;
            }
        }
        if (s > 0.0f) {
            float inv = 1.0f / s;
            for (size_t d = 0; d < head_dim; d++) o[d] *= inv;
        }
    }
}

/* Causal prefill attention, fp32: query i sees keys 0..(kv_len-seq_len+i)
 * (crates/rnb-cpu/src/kernels/attention/batch_f32.rs:76-176).  The reference tiles this
 * with an online softmax; this is the mathematically equal two-pass form. */
typedef struct {
    const float *q, *kf, *vf;
    const uint16_t *kh, *vh;
    float *out;
    size_t seq_len, kv_len, num_heads, num_kv_heads, head_dim;
    float scale;
} prefill_ctx;
static void prefill_rows(size_t b, size_t e, void *p) {
    prefill_ctx *c = (prefill_ctx *)p;
    size_t group = c->num_heads / c->num_kv_heads, kv_dim = c->num_kv_heads * c->head_dim;
    float *scores = (float *)malloc(sizeof(float) * c->kv_len);
    for (size_t i = b; i < e; i++) {
        size_t visible = c->kv_len - c->seq_len + i + 1;
        for (size_t h = 0; h < c->num_heads; h++) {
            size_t kv_h = h / group;
            const float *qh = c->q + (i * c->num_heads + h) * c->head_dim;
            float mx = -INFINITY;
            for (size_t j = 0; j < visible; j++) {
                size_t off = j * kv_dim + kv_h * c->head_dim;
                float dot = 0.0f;
                if (c->kf)
                    for (size_t d = 0; d < c->head_dim; d++) dot += qh[d] * c->kf[off + d];
                else
                    dot = dot_f32_f16(qh, c->kh + off, c->head_dim);
                scores[j] = dot * c->scale;
                if (scores[j] > mx) mx = scores[j];
            }
            float sum = 0.0f;
            for (size_t j = 0; j < visible; j++) {
                scores[j] = expf(scores[j] - mx);
                sum += scores[j];
            }
            float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
            float *o = c->out + (i * c->num_heads + h) * c->head_dim;
            for (size_t d = 0; d < c->head_dim; d++) o[d] = 0.0f;
            for (size_t j = 0; j < visible; j++) {
                size_t off = j * kv_dim + kv_h * c->head_dim;
                float w = scores[j] * inv;
                if (c->vf)
                    for (size_t d = 0; d < c->head_dim; d++) o[d] += w * c->vf[off + d];
                else
                    scaled_add_f16(o, c->vh + off, w, c->head_dim);
            }
        }
    }
    free(scores);
}
void orc_attention_prefill(const float *q, const float *k, const float *v, float *out,
                           size_t seq_len, size_t kv_len, size_t num_heads, size_t num_kv_heads,
                           size_t head_dim, float scale) {
    prefill_ctx c = {q, k, v, NULL, NULL, out, seq_len, kv_len, num_heads, num_kv_heads, head_dim,
                     scale};
    orc_parallel_for(seq_len, 8, prefill_rows, &c);
}
void orc_attention_prefill_f16kv(const float *q, const uint16_t *k, const uint16_t *v, float *out,
                                 size_t seq_len, size_t kv_len, size_t num_heads,
                                 size_t num_kv_heads, size_t head_dim, float scale) {
    prefill_ctx c = {q, NULL, NULL, k, v, out, seq_len, kv_len, num_heads, num_kv_heads, head_dim,
                     scale};
    orc_parallel_for(seq_len, 8, prefill_rows, &c);
}

/* ------------------------------------------------------------------------------------------
 * MoE routing: top-k by logit (descending; ties → lower expert id), weights = softmax over
 * the k selected logits in rank order.
 * crates/rnb-llm/src/engine/models/shared_expert_moe/routing.rs:18-62
 * The exponential is f32::exp, i.e. libm's expf, as in the reference.
 * ---------------------------------------------------------------------------------------- */
size_t orc_moe_route_topk(const float *logits, size_t n_expert, size_t top_k, uint32_t *ids,
                          float *weights) {
    size_t sel = top_k < n_expert ? top_k : n_expert;
    if (sel > 32) sel = 32;
    if (sel == 0) return 0;
    float best_vals[32];
    size_t best_ids[32];
    for (int i = 0; i < 32; i++) {
        best_vals[i] = -INFINITY;
        best_ids[i] = SIZE_MAX;
    }
    for (size_t e = 0; e < n_expert; e++) {
        float value = logits[e];
        for (size_t rank = 0; rank < sel; rank++) {
            if (value > best_vals[rank] || (value == best_vals[rank] && e < best_ids[rank])) {
                for (size_t sh = sel - 1; sh > rank; sh--) {
                    best_vals[sh] = best_vals[sh - 1];
                    best_ids[sh] = best_ids[sh - 1];
                }
                best_vals[rank] = value;
                best_ids[rank] = e;
                break;
            }
        }
    }
    float mx = best_vals[0], sum = 0.0f;
    for (size_t r = 0; r < sel; r++) {
        float w = expf(best_vals[r] - mx);   /* f32::exp, routing.rs:50 */
        ids[r] = (uint32_t)best_ids[r];
        weights[r] = w;
        sum += w;
    }
    if (sum != 0.0f)
        for (size_t r = 0; r < sel; r++) weights[r] /= sum;
    return sel;
}

/* Router logits: the reference computes them on the host with gemv_f32 → dot_f32_row
 * (crates/rnb-llm/src/engine/models/shared_expert_moe/moe_view.rs:146-157,
 *  crates/rnb-cpu/src/gemm/f32_gemv.rs:215-237,266-275): two 8-lane FMA accumulators walking
 * the row 16 elements at a time, acc0+acc1, then (l+l4) → (+2) → (+1), then a scalar tail.
 * Restated lane by lane with fmaf, which is bit-identical to the vector FMA. */
static float dot_f32_row(const float *a, const float *b, size_t n) {
    float acc[16] = {0};
    size_t i = 0;
    for (; i + 16 <= n; i += 16)
        for (int l = 0; l < 16; l++) acc[l] = fmaf(a[i + l], b[i + l], acc[l]);
    float s[8];
    for (int l = 0; l < 8; l++) s[l] = acc[l] + acc[l + 8];
    float r0 = s[0] + s[4], r1 = s[1] + s[5], r2 = s[2] + s[6], r3 = s[3] + s[7];
    float t0 = r0 + r2, t1 = r1 + r3;
    float out = t0 + t1;
    for (; i < n; i++) out += a[i] * b[i];
    return out;
}
void orc_gemv_f32(const float *w, const float *x, float *out, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; r++) out[r] = dot_f32_row(w + r * cols, x, cols);
}

/* Expert FFN: per selected expert gate/up GEMV → SiLU·up → down GEMV → × route weight;
 * experts summed in selection order starting from zero.
 * crates/rnb-llm/src/engine/models/shared_expert_moe/moe_view/fanout.rs:260-327,
 * moe_view.rs:416-423 */
int orc_moe_experts(const uint8_t *const *gate, const uint8_t *const *up,
                    const uint8_t *const *down, const float *route_weights, size_t n_selected,
                    int down_type, size_t n_ff, size_t n_embd, const float *x, float *out,
                    int threads) {
    float *g = (float *)malloc(sizeof(float) * n_ff * 2);
    float *u = g + n_ff;
    float *eo = (float *)malloc(sizeof(float) * n_embd);
    for (size_t i = 0; i < n_embd; i++) out[i] = 0.0f;
    int rc = 0;
    for (size_t e = 0; e < n_selected && rc == 0; e++) {
        rc |= orc_gemv(ORC_TYPE_Q4_K, gate[e], x, g, n_ff, n_embd, 1, threads);
        rc |= orc_gemv(ORC_TYPE_Q4_K, up[e], x, u, n_ff, n_embd, 1, threads);
        orc_silu_mul_inplace(g, u, n_ff);
        rc |= orc_gemv(down_type, down[e], g, eo, n_embd, n_ff, 1, threads);
        for (size_t i = 0; i < n_embd; i++) eo[i] *= route_weights[e];
        for (size_t i = 0; i < n_embd; i++) out[i] += eo[i];
    }
    free(g);
    free(eo);
    return rc;
}

/* ------------------------------------------------------------------------------------------
 * Glue.
 * RMSNorm: crates/rnb-cpu/src/kernels/norm.rs:177-196 (f64 mean square; (x/rms)*w)
 * RoPE:    crates/rnb-cpu/src/kernels/rope.rs:267-293 (adjacent pairs, angle chain)
 * SiLU·up: crates/rnb-cpu/src/kernels/activation.rs:74-89
 * argmax:  crates/rnb-llm/src/sampler/greedy.rs:4-11 (max_by → last of equal maxima)
 * ---------------------------------------------------------------------------------------- */
void orc_rms_norm(const float *x, const float *w, float eps, float *out, size_t hidden,
                  size_t seq_len) {
    for (size_t s = 0; s < seq_len; s++) {
        const float *xs = x + s * hidden;
        double ss = 0.0;
        for (size_t i = 0; i < hidden; i++) ss += (double)xs[i] * (double)xs[i];
        double ms = ss / (double)hidden;
        float rms = (float)sqrt(ms + (double)eps);
        float *o = out + s * hidden;
        for (size_t i = 0; i < hidden; i++) o[i] = (xs[i] / rms) * w[i];
    }
}

void orc_rope_table(size_t pos, size_t head_dim, float theta, float *cos_out, float *sin_out) {
    float theta_scale = powf(theta, -2.0f / (float)head_dim);
    float angle = (float)pos;
    for (size_t i = 0; i < head_dim / 2; i++) {
        cos_out[i] = cosf(angle);
        sin_out[i] = sinf(angle);
        angle *= theta_scale;
    }
}

void orc_rope_inplace(float *data, size_t n, size_t pos_start, size_t head_dim, size_t dim,
                      float theta) {
    if (n == 0 || head_dim == 0) return;
    size_t seq_len = n / dim;
    float cs[512], sn[512];
    for (size_t t = 0; t < seq_len; t++) {
        orc_rope_table(pos_start + t, head_dim, theta, cs, sn);
        for (size_t c = 0; c < dim; c += head_dim) {
            float *chunk = data + t * dim + c;
            for (size_t i = 0; i < head_dim; i += 2) {
                float x0 = chunk[i], x1 = chunk[i + 1];
                chunk[i] = x0 * cs[i / 2] - x1 * sn[i / 2];
                chunk[i + 1] = x0 * sn[i / 2] + x1 * cs[i / 2];
            }
        }
    }
}

/* Half-split ("NeoX") pairing (i, i + head_dim/2) with the same angle chain; used for the
 * synthetic MoE configuration, which has no end-to-end model in the reference. */
void orc_rope_neox_inplace(float *data, size_t n, size_t pos_start, size_t head_dim, size_t dim,
                           float theta) {
    if (n == 0 || head_dim == 0) return;
    size_t seq_len = n / dim, half = head_dim / 2;
    float cs[512], sn[512];
    for (size_t t = 0; t < seq_len; t++) {
        orc_rope_table(pos_start + t, head_dim, theta, cs, sn);
        for (size_t c = 0; c < dim; c += head_dim) {
            float *chunk = data + t * dim + c;
            for (size_t i = 0; i < half; i++) {
                float x0 = chunk[i], x1 = chunk[i + half];
                chunk[i] = x0 * cs[i] - x1 * sn[i];
                chunk[i + half] = x0 * sn[i] + x1 * cs[i];
            }
        }
    }
}

void orc_silu_mul_inplace(float *gate, const float *up, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float g = gate[i];
        gate[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

uint32_t orc_argmax_last(const float *x, size_t n) {
    size_t best = 0;
    for (size_t i = 1; i < n; i++)
        if (x[i] >= x[best]) best = i;
    return (uint32_t)best;
}

/* ------------------------------------------------------------------------------------------
 * Token-level decode of a Llama-style stack (dense or softmax-top-k MoE FFN), built from
 * the routines above in the order the reference's engine runs them:
 * crates/rnb-llm/src/engine/decode.rs:199-564 (norm → q/k/v GEMV → RoPE → f16 KV append →
 * decode attention → o_proj → residual), crates/rnb-llm/src/engine/decode_ffn.rs:294-366
 * (norm → gate/up → SiLU·up → down → residual), crates/rnb-llm/src/engine/logits.rs
 * (final norm → LM head).
 * ---------------------------------------------------------------------------------------- */
struct orc_model {
    orc_model_cfg cfg;
    orc_layer *layers;
    orc_qweight token_embd, output;
    const float *out_norm;
    size_t max_ctx;
    int threads;
    uint16_t **k_cache, **v_cache;
    float *x, *h, *q, *k, *v, *attn, *proj, *g, *u, *logits, *router_logits;
    uint32_t *expert_ids; /* [n_layer][n_expert_used] */
};

orc_model *orc_model_create(const orc_model_cfg *cfg, const orc_layer *layers,
                            orc_qweight token_embd, const float *out_norm, orc_qweight output,
                            size_t max_ctx, int threads) {
    orc_model *m = (orc_model *)calloc(1, sizeof(orc_model));
    m->cfg = *cfg;
    m->layers = (orc_layer *)malloc(sizeof(orc_layer) * (size_t)cfg->n_layer);
    memcpy(m->layers, layers, sizeof(orc_layer) * (size_t)cfg->n_layer);
    m->token_embd = token_embd;
    m->output = output;
    m->out_norm = out_norm;
    m->max_ctx = max_ctx;
    m->threads = threads;
    size_t kv_dim = (size_t)cfg->n_kv_head * (size_t)cfg->head_dim;
    size_t q_dim = (size_t)cfg->n_head * (size_t)cfg->head_dim;
    m->k_cache = (uint16_t **)malloc(sizeof(void *) * (size_t)cfg->n_layer);
    m->v_cache = (uint16_t **)malloc(sizeof(void *) * (size_t)cfg->n_layer);
    for (int l = 0; l < cfg->n_layer; l++) {
        m->k_cache[l] = (uint16_t *)calloc(max_ctx * kv_dim, 2);
        m->v_cache[l] = (uint16_t *)calloc(max_ctx * kv_dim, 2);
    }
    size_t ff = (size_t)(cfg->n_expert ? cfg->n_ff_expert : cfg->n_ff);
    m->x = (float *)calloc((size_t)cfg->hidden, 4);
    m->h = (float *)calloc((size_t)cfg->hidden, 4);
    m->q = (float *)calloc(q_dim, 4);
    m->k = (float *)calloc(kv_dim, 4);
    m->v = (float *)calloc(kv_dim, 4);
    m->attn = (float *)calloc(q_dim, 4);
    m->proj = (float *)calloc((size_t)cfg->hidden, 4);
    m->g = (float *)calloc(ff, 4);
    m->u = (float *)calloc(ff, 4);
    m->logits = (float *)calloc((size_t)cfg->vocab, 4);
    m->router_logits = (float *)calloc((size_t)(cfg->n_expert ? cfg->n_expert : 1), 4);
    m->expert_ids = (uint32_t *)calloc((size_t)cfg->n_layer * 32, 4);
    return m;
}

void orc_model_free(orc_model *m) {
    if (!m) return;
    for (int l = 0; l < m->cfg.n_layer; l++) {
        free(m->k_cache[l]);
        free(m->v_cache[l]);
    }
    free(m->k_cache);
    free(m->v_cache);
    free(m->layers);
    free(m->x);
    free(m->h);
    free(m->q);
    free(m->k);
    free(m->v);
    free(m->attn);
    free(m->proj);
    free(m->g);
    free(m->u);
    free(m->logits);
    free(m->router_logits);
    free(m->expert_ids);
    free(m);
}

void orc_model_reset(orc_model *m) {
    size_t kv_dim = (size_t)m->cfg.n_kv_head * (size_t)m->cfg.head_dim;
    for (int l = 0; l < m->cfg.n_layer; l++) {
        memset(m->k_cache[l], 0, m->max_ctx * kv_dim * 2);
        memset(m->v_cache[l], 0, m->max_ctx * kv_dim * 2);
    }
}

const float *orc_model_decode(orc_model *m, uint32_t token, size_t pos) {
    const orc_model_cfg *c = &m->cfg;
    size_t H = (size_t)c->hidden, hd = (size_t)c->head_dim;
    size_t q_dim = (size_t)c->n_head * hd, kv_dim = (size_t)c->n_kv_head * hd;
    int T = m->threads;
    if (pos >= m->max_ctx) return NULL;
    orc_dequantize_row(m->token_embd.type,
                       m->token_embd.data + (size_t)token * orc_row_bytes(m->token_embd.type, H), H,
                       m->x);
    float scale = 1.0f / sqrtf((float)hd);
    for (int l = 0; l < c->n_layer; l++) {
        const orc_layer *L = &m->layers[l];
        orc_rms_norm(m->x, L->attn_norm, c->rms_eps, m->h, H, 1);
        orc_gemv(L->wq.type, L->wq.data, m->h, m->q, q_dim, H, 1, T);
        orc_gemv(L->wk.type, L->wk.data, m->h, m->k, kv_dim, H, 1, T);
        orc_gemv(L->wv.type, L->wv.data, m->h, m->v, kv_dim, H, 1, T);
        if (c->rope_neox) {
            orc_rope_neox_inplace(m->q, q_dim, pos, hd, q_dim, c->rope_theta);
            orc_rope_neox_inplace(m->k, kv_dim, pos, hd, kv_dim, c->rope_theta);
        } else {
            orc_rope_inplace(m->q, q_dim, pos, hd, q_dim, c->rope_theta);
            orc_rope_inplace(m->k, kv_dim, pos, hd, kv_dim, c->rope_theta);
        }
        orc_f32_to_f16_row(m->k, m->k_cache[l] + pos * kv_dim, kv_dim);
        orc_f32_to_f16_row(m->v, m->v_cache[l] + pos * kv_dim, kv_dim);
        orc_attention_decode(m->q, m->k_cache[l], m->v_cache[l], m->attn, (size_t)c->n_head,
                             (size_t)c->n_kv_head, hd, pos + 1, scale);
        orc_gemv(L->wo.type, L->wo.data, m->attn, m->proj, H, q_dim, 1, T);
        for (size_t i = 0; i < H; i++) m->x[i] += m->proj[i];
        orc_rms_norm(m->x, L->ffn_norm, c->rms_eps, m->h, H, 1);
        if (c->n_expert > 0) {
            size_t ne = (size_t)c->n_expert, k = (size_t)c->n_expert_used;
            size_t ffe = (size_t)c->n_ff_expert;
            orc_gemv_f32(L->router, m->h, m->router_logits, ne, H);
            uint32_t *ids = m->expert_ids + (size_t)l * 32;
            float w[32];
            size_t sel = orc_moe_route_topk(m->router_logits, ne, k, ids, w);
            const uint8_t *gp[32], *up[32], *dp[32];
            size_t gb = ffe * orc_row_bytes(L->gate_exps.type, H);
            size_t db = H * orc_row_bytes(L->down_exps.type, ffe);
            for (size_t e = 0; e < sel; e++) {
                gp[e] = L->gate_exps.data + (size_t)ids[e] * gb;
                up[e] = L->up_exps.data + (size_t)ids[e] * gb;
                dp[e] = L->down_exps.data + (size_t)ids[e] * db;
            }
            orc_moe_experts(gp, up, dp, w, sel, L->down_exps.type, ffe, H, m->h, m->proj, T);
        } else {
            size_t ff = (size_t)c->n_ff;
            orc_gemv(L->gate.type, L->gate.data, m->h, m->g, ff, H, 1, T);
            orc_gemv(L->up.type, L->up.data, m->h, m->u, ff, H, 1, T);
            orc_silu_mul_inplace(m->g, m->u, ff);
            orc_gemv(L->down.type, L->down.data, m->g, m->proj, H, ff, 1, T);
        }
        for (size_t i = 0; i < H; i++) m->x[i] += m->proj[i];
    }
    orc_rms_norm(m->x, m->out_norm, c->rms_eps, m->h, H, 1);
    orc_gemv(m->output.type, m->output.data, m->h, m->logits, (size_t)c->vocab, H, 1, T);
    return m->logits;
}

const uint16_t *orc_model_k_cache(const orc_model *m, int layer) { return m->k_cache[layer]; }
const uint16_t *orc_model_v_cache(const orc_model *m, int layer) { return m->v_cache[layer]; }
const float *orc_model_hidden(const orc_model *m) { return m->x; }
const uint32_t *orc_model_last_expert_ids(const orc_model *m, int layer) {
    return m->expert_ids + (size_t)layer * 32;
}
