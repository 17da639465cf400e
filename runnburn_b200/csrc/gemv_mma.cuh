// Batch-1 Q4_K / Q6_K x Q8_K matvec, integer lane sums on the int8 MMA pipe.
//
// The eight f32 accumulator lanes of rnb-cpu's AVX2 dots (crates/rnb-cpu/src/gemm/avx2_dot.rs:
// 621-696 Q4_K, :801-885 Q6_K) are sums over groups of four consecutive elements of every
// 32-element sub-block.  For 16 weight rows at once that is a 16 x 32 (rows x elements) times
// 32 x 8 (elements x lanes) integer product whose right operand holds the Q8_K activation on a
// block diagonal: column l is non-zero only in elements 4l..4l+3.  One
// mma.sync.m16n8k32.u8.s8 therefore yields the exact int32 lane sums of a sub-block for 16 rows,
// the activation is fetched once per 16 rows instead of once per row, and the per-thread work
// that remains is the nibble masks, one integer multiply by the sub-block scale per lane sum and
// the ordered f32 FMA chain - about a third of the instructions of the dp4a forms, same bits.
//
// Shape of a CTA: a tile of 16 rows, eight MMA warps, a producer warp and a replay warp.  K is cut into
// stages of eight super-blocks of every row (bulk-async copies onto an mbarrier, a ring of
// stages); MMA warp w takes block w of the stage for all 16 rows and leaves, per (block, row), the
// lane sums, the mins products and the block scales as f32 in a double-buffered record area.
// One lane of the producer warp issues the copies as the MMA warps release stages; the replay warp
// replays the records in block order - one FMA per block and accumulator, the only part that has to
// be sequential - then folds the lanes and runs the epilogue.  CTAs are persistent: they walk tiles blockIdx.x, blockIdx.x + gridDim.x, ... with
// the copy ring running across tile boundaries.
//
// Fragment layouts (PTX ISA, mma.m16n8k32 with 8-bit operands; g = lane / 4, t = lane % 4):
//   A: a0 = (row g, k 4t..4t+3), a1 = (row g+8, same k), a2 = (row g, k 16+4t..), a3 = (row g+8, ..)
//   B: b0 = (k 4t..4t+3, column g), b1 = (k 16+4t.., column g)
//   C: c0, c1 = (row g, columns 2t, 2t+1), c2, c3 = (row g+8, columns 2t, 2t+1)
// k slot 4t carries accumulator lane t and k slot 16+4t lane 4+t, so column l is fed by exactly
// one thread: (g = l, t = l % 4), through b0 when l < 4 and b1 otherwise; every other thread holds
// zeros in its B registers.
#pragma once
#include "gemv.cuh"
#include "gemv_stream.cuh"
#include "gemv_pair.cuh"
#include "q8k.cuh"

namespace rnb {

constexpr int GM_ROWS = 16;
constexpr int GM_CHUNK = 8;                              // super-blocks per stage = MMA warps
constexpr int GM_MMA_WARPS = 8;
constexpr int GM_THREADS = 32 * (GM_MMA_WARPS + 2);   // + producer warp + replay warp
constexpr int GM_MAX_STAGES = 6;
constexpr uint32_t GM_REC_BYTES = 64;                    // per (block, row): a[8] | m[4] | d | dmin | pad
constexpr uint32_t GM_PBUF_BYTES = GM_CHUNK * GM_ROWS * GM_REC_BYTES;
constexpr uint32_t GM_ZERO_BYTES = 320;                  // zeros read by threads that feed no column
constexpr uint32_t GM_ACT_BLOCK_BYTES = 256 + 32 + 4;               // qs | bsum16 | d per super-block of a stage
constexpr uint32_t GM_POLL_LIMIT = 1u << 21;
#ifndef GM_MIN_CTAS
#define GM_MIN_CTAS 2
#endif

// Tiled-copy descriptors (CUtensorMap, opaque here) of the launch's weight matrices: with them a
// stage's 16 rows arrive by ONE copy instruction instead of 16, which is what the single issuing
// lane can sustain at the HBM rate.  Matrix i is described as [rows][row_bytes / 8] 8-byte words with a
// box of 16 rows x (row stride / 8) words; rows or words past the end read as zeros.
struct alignas(64) GmTensorMap {
    unsigned long long opaque[16];
};
struct GmTmaps {
    GmTensorMap m[GS_PACK];
};
__device__ __forceinline__ void gm_tma_2d(uint32_t dst, const void *tmap, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

struct GmParams {
    int cols;
    int chunk;            // super-blocks per stage: GM_CHUNK or 2 * GM_CHUNK (each MMA warp then takes two blocks per stage)
    int n_stages;
    int dynamic_table;
    int n_tiles;
    int use_tmap;         // weights arrive through the tiled-copy descriptors (by-value kernel only)
    uint32_t row_stride;  // bytes of a Q4_K weight row per stage; row_stride / 16 is odd (ldmatrix reads 8 rows conflict-free)
    uint32_t row_stride6; // the same for Q6_K rows (equal to row_stride unless descriptors are in use)
    uint32_t act_off;
    uint32_t slot_bytes;
};

__host__ __device__ inline uint32_t gm_smem_bytes(int stages, uint32_t slot_bytes) {
    return (uint32_t)stages * slot_bytes + 2u * GM_PBUF_BYTES + GM_ZERO_BYTES;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// D = A (16 x 32, u8) * B (32 x 8, s8), int32
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
// prmt.b32 in its default mode: selector nibble bits 0-2 pick one of the eight source bytes, bit 3
// replaces the byte by eight copies of its sign bit (the __byte_perm intrinsic documents three
// selector bits only).
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// A 4-byte word of a Q6_K block.  Blocks are 210 bytes: inside a 16-byte aligned stage row the odd
// blocks start two bytes past a word boundary.
template <bool ODD>
__device__ __forceinline__ uint32_t lds_word(uint32_t addr) {
    if (!ODD) return lds32(addr);
    const uint32_t w0 = lds32(addr - 2), w1 = lds32(addr + 2);
    return prmt_b32(w0, w1, 0x5432u);
}
__device__ __forceinline__ void sts_f2(uint32_t addr, float a, float b) {
    asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void sts_f1(uint32_t addr, float a) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_f1(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
#ifdef GM_PROFILE
// Development aid (compiled only with -DGM_PROFILE): SM-clock cycles summed over warps.
// 0 MMA wait for a stage, 1 MMA wait for a record buffer, 2 MMA compute, 3 control wait for records,
// 4 control copy issue, 5 control replay + epilogue, 6 MMA items, 7 control items
static __device__ unsigned long long g_gm_prof[8];
#define GM_PROF_DECL long long prof_t0 = clock64(), prof_a = 0, prof_b = 0, prof_c = 0, prof_n = 0
#define GM_PROF_LAP(acc) do { const long long prof_t1 = clock64(); acc += prof_t1 - prof_t0; prof_t0 = prof_t1; } while (0)
#else
#define GM_PROF_DECL
#define GM_PROF_LAP(acc)
#endif
// Bounded wait that also gives up as soon as another warp of the CTA has flagged a failure.  The
// first probe is inline (the common case: the data is already there); the polling loop is kept out
// of line so that it does not weigh on the callers' code.
static __device__ __noinline__ bool gm_wait_slow(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < GM_POLL_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 16) {
            if (*abort_flag) return false;
            __nanosleep(i > 4096 ? 256 : 40);
        }
    }
    return false;
}
__device__ __forceinline__ bool gm_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    return gm_wait_slow(bar, parity, abort_flag);
}
// 16-byte units 0,1 and 2,3 of a record trade places in rows whose bit 1 is set, so that the
// replay's 16-byte loads of four consecutive rows fall into distinct banks.
__device__ __forceinline__ uint32_t gm_rec_unit(int row, int unit) { return (uint32_t)(unit ^ (row & 2)) * 16u; }

// ---- one Q4_K block of 16 rows (MMA warp) -------------------------------------------------------
// rows_base: stage slot (row r at + r * row_stride), blk_off: byte offset of the block inside a row.
__device__ __forceinline__ void gm_q4k_block(uint32_t rows_base, uint32_t row_stride, uint32_t blk_off, uint32_t act_qs, uint32_t act_bs, float yd,
                                             uint32_t zeros, uint32_t rec, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t rowA = rows_base + (uint32_t)g * row_stride + blk_off, rowB = rowA + 8u * row_stride;
    const uint4 hA = lds128(rowA), hB = lds128(rowB);
    const uint32_t lm = rows_base + (uint32_t)((lane & 7) + ((lane >> 3) & 1) * 8) * row_stride + blk_off + 16u + (uint32_t)(lane >> 4) * 16u;
    const bool feeds = t == (g & 3);
    const uint32_t p0 = (feeds && g < 4) ? act_qs + 4u * g : zeros + 4u * g;
    const uint32_t p1 = (feeds && g >= 4) ? act_qs + 4u * g : zeros + 4u * g;
    const uint32_t scA03 = hA.y & 0x3f3f3f3fu, scA47 = (hA.w & 0x0f0f0f0fu) | ((hA.y >> 2) & 0x30303030u);
    const uint32_t scB03 = hB.y & 0x3f3f3f3fu, scB47 = (hB.w & 0x0f0f0f0fu) | ((hB.y >> 2) & 0x30303030u);
    int loA0 = 0, loA1 = 0, loB0 = 0, loB1 = 0, hiA0 = 0, hiA1 = 0, hiB0 = 0, hiB1 = 0;
#pragma unroll
    for (int gp = 0; gp < 4; gp++) {
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(lm + 32u * gp, r0, r1, r2, r3);
        const uint32_t b0l = lds32(p0 + 64u * gp), b1l = lds32(p1 + 64u * gp);
        const uint32_t b0h = lds32(p0 + 64u * gp + 32u), b1h = lds32(p1 + 64u * gp + 32u);
        const uint32_t swA = gp < 2 ? scA03 : scA47, swB = gp < 2 ? scB03 : scB47;
        // one byte of the scale word each (prmt: selected byte in byte 0, zeros above)
        const int slA = (int)__byte_perm(swA, 0u, 0x4440u + 2u * (gp & 1)), shA = (int)__byte_perm(swA, 0u, 0x4441u + 2u * (gp & 1));
        const int slB = (int)__byte_perm(swB, 0u, 0x4440u + 2u * (gp & 1)), shB = (int)__byte_perm(swB, 0u, 0x4441u + 2u * (gp & 1));
        int c[4];
        mma_u8s8(c, r0 & 0x0f0f0f0fu, r1 & 0x0f0f0f0fu, r2 & 0x0f0f0f0fu, r3 & 0x0f0f0f0fu, b0l, b1l);
        loA0 += slA * c[0];
        loA1 += slA * c[1];
        loB0 += slB * c[2];
        loB1 += slB * c[3];
        // high nibbles stay in place (x16); the sums are exact multiples of 16
        mma_u8s8(c, r0 & 0xf0f0f0f0u, r1 & 0xf0f0f0f0u, r2 & 0xf0f0f0f0u, r3 & 0xf0f0f0f0u, b0h, b1h);
        hiA0 += shA * c[0];
        hiA1 += shA * c[1];
        hiB0 += shB * c[2];
        hiB1 += shB * c[3];
    }
    // mins accumulator lane t: mn[2t] * bsum32[2t] + mn[2t+1] * bsum32[2t+1], bsum32[j] = bsum16[2j] + bsum16[2j+1] (i16)
    const uint2 bs = lds64(act_bs + 8u * t);
    const int b32a = (short)((short)(bs.x & 0xffff) + (short)(bs.x >> 16)), b32b = (short)((short)(bs.y & 0xffff) + (short)(bs.y >> 16));
    const uint32_t mnA = t < 2 ? (hA.z & 0x3f3f3f3fu) : (((hA.w >> 4) & 0x0f0f0f0fu) | ((hA.z >> 2) & 0x30303030u));
    const uint32_t mnB = t < 2 ? (hB.z & 0x3f3f3f3fu) : (((hB.w >> 4) & 0x0f0f0f0fu) | ((hB.z >> 2) & 0x30303030u));
    const uint32_t selm = 0x4440u + 2u * (uint32_t)(t & 1);
    const int mpA = (int)__byte_perm(mnA, 0u, selm) * b32a + (int)__byte_perm(mnA, 0u, selm + 1u) * b32b;
    const int mpB = (int)__byte_perm(mnB, 0u, selm) * b32a + (int)__byte_perm(mnB, 0u, selm + 1u) * b32b;
    const uint32_t recA = rec + (uint32_t)g * GM_REC_BYTES, recB = recA + 8u * GM_REC_BYTES;   // rows g and g+8 share bit 1
    const uint32_t ua = gm_rec_unit(g, t >> 1) + (uint32_t)(t & 1) * 8u, um = gm_rec_unit(g, 2) + 4u * t, ud = gm_rec_unit(g, 3);
    sts_f2(recA + ua, (float)(loA0 + (hiA0 >> 4)), (float)(loA1 + (hiA1 >> 4)));
    sts_f2(recB + ua, (float)(loB0 + (hiB0 >> 4)), (float)(loB1 + (hiB1 >> 4)));
    sts_f1(recA + um, (float)mpA);
    sts_f1(recB + um, (float)mpB);
    if (t == 0) {
        sts_f2(recA + ud, __fmul_rn(yd, f16_bits_to_f32(hA.x & 0xffffu)), __fmul_rn(-yd, f16_bits_to_f32(hA.x >> 16)));
        sts_f2(recB + ud, __fmul_rn(yd, f16_bits_to_f32(hB.x & 0xffffu)), __fmul_rn(-yd, f16_bits_to_f32(hB.x >> 16)));
    }
}

// ---- one Q6_K block of 16 rows (MMA warp) -------------------------------------------------------
// Part P = 4n + p covers elements 32P..32P+31: low nibbles of ql[64n + 32(p&1) ..] for p < 2, high
// nibbles for p >= 2, bits 2p..2p+1 of qh[32n ..]; lanes 0-3 use scale 2P, lanes 4-7 scale 2P+1.
template <bool ODD>
__device__ __forceinline__ void gm_q6k_block(uint32_t rows_base, uint32_t row_stride, uint32_t blk_off, uint32_t act_qs, uint32_t act_bs, float yd,
                                             uint32_t zeros, uint32_t rec, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t rowA = rows_base + (uint32_t)g * row_stride + blk_off, rowB = rowA + 8u * row_stride;
    const bool feeds = t == (g & 3);
    const uint32_t p0 = (feeds && g < 4) ? act_qs + 4u * g : zeros + 4u * g;
    const uint32_t p1 = (feeds && g >= 4) ? act_qs + 4u * g : zeros + 4u * g;
    // sign-extending byte selectors for the scale of this thread's lane half (bytes hh and 2 + hh of a scale word)
    const uint32_t hh = (uint32_t)(t >> 1);
    const uint32_t sel0 = hh | ((hh | 8u) << 4) | ((hh | 8u) << 8) | ((hh | 8u) << 12);
    const uint32_t sel1 = sel0 + 0x2222u;
    int sA0 = 0, sA1 = 0, sB0 = 0, sB1 = 0;
#pragma unroll
    for (int n = 0; n < 2; n++) {
        uint32_t qlA[2][2], qlB[2][2], qhA[2], qhB[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
#pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                qlA[h2][i] = lds_word<ODD>(rowA + 64u * n + 32u * h2 + 16u * i + 4u * t);
                qlB[h2][i] = lds_word<ODD>(rowB + 64u * n + 32u * h2 + 16u * i + 4u * t);
            }
            qhA[i] = lds_word<ODD>(rowA + 128u + 32u * n + 16u * i + 4u * t);
            qhB[i] = lds_word<ODD>(rowB + 128u + 32u * n + 16u * i + 4u * t);
        }
        uint32_t scwA[2], scwB[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            scwA[k] = lds_word<ODD>(rowA + 192u + 8u * n + 4u * k);
            scwB[k] = lds_word<ODD>(rowB + 192u + 8u * n + 4u * k);
        }
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const int P = 4 * n + p;
            uint32_t a[4];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const uint32_t lA = qlA[p & 1][i], lB = qlB[p & 1][i];
                const uint32_t nA = (p & 2) ? (lA >> 4) : lA, nB = (p & 2) ? (lB >> 4) : lB;
                const uint32_t xA = p == 0 ? (qhA[i] << 4) : p == 1 ? (qhA[i] << 2) : p == 2 ? qhA[i] : (qhA[i] >> 2);
                const uint32_t xB = p == 0 ? (qhB[i] << 4) : p == 1 ? (qhB[i] << 2) : p == 2 ? qhB[i] : (qhB[i] >> 2);
                a[2 * i] = (nA & 0x0f0f0f0fu) | (xA & 0x30303030u);
                a[2 * i + 1] = (nB & 0x0f0f0f0fu) | (xB & 0x30303030u);
            }
            const uint32_t b0 = lds32(p0 + 32u * P), b1 = lds32(p1 + 32u * P);
            int c[4];
            mma_u8s8(c, a[0], a[1], a[2], a[3], b0, b1);
            const int scA = (int)prmt_b32(scwA[p >> 1], 0u, (p & 1) ? sel1 : sel0);
            const int scB = (int)prmt_b32(scwB[p >> 1], 0u, (p & 1) ? sel1 : sel0);
            sA0 += scA * c[0];
            sA1 += scA * c[1];
            sB0 += scB * c[2];
            sB1 += scB * c[3];
        }
    }
    // lanes 2t and 2t+1 lose 32 * (bsum16[2l] * sc[2l] + bsum16[2l+1] * sc[2l+1]): scales 4t..4t+3 are one word
    const uint2 bs = lds64(act_bs + 8u * t);
    const int scTA = (int)lds_word<ODD>(rowA + 192u + 4u * t), scTB = (int)lds_word<ODD>(rowB + 192u + 4u * t);
    sA0 -= 32 * __dp2a_lo((int)bs.x, scTA, 0);
    sA1 -= 32 * __dp2a_hi((int)bs.y, scTA, 0);
    sB0 -= 32 * __dp2a_lo((int)bs.x, scTB, 0);
    sB1 -= 32 * __dp2a_hi((int)bs.y, scTB, 0);
    const uint32_t recA = rec + (uint32_t)g * GM_REC_BYTES, recB = recA + 8u * GM_REC_BYTES;
    const uint32_t ua = gm_rec_unit(g, t >> 1) + (uint32_t)(t & 1) * 8u, ud = gm_rec_unit(g, 3);
    sts_f2(recA + ua, (float)sA0, (float)sA1);
    sts_f2(recB + ua, (float)sB0, (float)sB1);
    if (t == 0) {
        sts_f1(recA + ud, __fmul_rn(yd, f16_bits_to_f32(lds16(rowA + 208u))));
        sts_f1(recB + ud, __fmul_rn(yd, f16_bits_to_f32(lds16(rowB + 208u))));
    }
}

// Tail of a gate + up launch (one warp): the CTA that completes a 256-row block of both vectors
// computes SiLU(gate) * up for the block and quantises it to Q8_K; counters[block] is zero before
// the launch and re-armed by the block's last arrival.
static __device__ __noinline__ void gm_silu_tail(const GpTail &tail, int blk, int arrivals, int lane) {
    __threadfence();   // this tile's results are visible device-wide before the tile is counted
    __syncwarp();
    int last = 0;
    if (lane == 0) last = atomicAdd(&tail.counters[blk], 1) == arrivals - 1;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
    const size_t off = (size_t)blk * 256 + lane * 8;
    const float4 g0 = __ldcg(reinterpret_cast<const float4 *>(tail.gate + off)), g1 = __ldcg(reinterpret_cast<const float4 *>(tail.gate + off + 4));
    const float4 u0 = __ldcg(reinterpret_cast<const float4 *>(tail.up + off)), u1 = __ldcg(reinterpret_cast<const float4 *>(tail.up + off + 4));
    const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const float e = expf_libm(-gv[k]);   // libm's expf (as silu_mul_q8k_kernel)
        v[k] = __fmul_rn(__fdiv_rn(gv[k], __fadd_rn(1.0f, e)), uv[k]);
    }
    Q8kDevView dv = q8k_dev_view(tail.xq_out, tail.n);
    q8k_quantize_block_warp(v, lane, dv.qs + blk * 256, dv.d + blk, dv.bsum16 + blk * 16, nullptr);
    if (lane == 0) tail.counters[blk] = 0;
}

// Walks the (tile, part, chunk) items of one CTA in order.
struct GmCursor {
    int tile, part, chunk;
    int jsel, row0, nrows, type, n_parts;
};
__device__ __forceinline__ bool gm_locate(const GemvJob *__restrict__ jobs, int n_jobs, GmCursor &c) {
    int t0 = 0;
    for (int i = 0; i < n_jobs; i++) {
        const int rows = jobs[i].rows, nt = (rows + GM_ROWS - 1) / GM_ROWS;
        if (c.tile < t0 + nt) {
            c.jsel = i;
            c.row0 = (c.tile - t0) * GM_ROWS;
            c.nrows = min(GM_ROWS, rows - c.row0);
            c.type = jobs[i].type;
            c.n_parts = jobs[i].n_parts;
            return true;
        }
        t0 += nt;
    }
    return false;
}
// advances to the next item; returns false when the CTA's tiles are exhausted
__device__ __forceinline__ bool gm_next(const GemvJob *__restrict__ jobs, int n_jobs, int n_chunks, int n_tiles, int tile_step, GmCursor &c) {
    if (++c.chunk < n_chunks) return true;
    c.chunk = 0;
    if (++c.part < c.n_parts) return true;
    c.part = 0;
    c.tile += tile_step;
    if (c.tile >= n_tiles) return false;
    return gm_locate(jobs, n_jobs, c);
}

// PEER: the instantiation whose epilogue also stores the rows into the peers' buffers (sharded decode);
// the single-GPU instantiation carries none of that code.
template <bool PEER>
__device__ __forceinline__ void gemv_mma_body(const GemvJob *__restrict__ jobs, int n_jobs, const GmParams &P, int *__restrict__ dev_error,
                                              const GpTail &tail, const GmTmaps *__restrict__ tmaps) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[GM_MAX_STAGES], empty[GM_MAX_STAGES], pfull[2], pempty[2];
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int S = P.n_stages, cols = P.cols, nb = cols >> 8, CB = P.chunk, n_chunks = (nb + CB - 1) / CB, halves = CB / GM_CHUNK;
    if (blockDim.x != GM_THREADS || S < 1 || S > GM_MAX_STAGES || nb < 1 || (P.row_stride & 15u) || !((P.row_stride >> 4) & 1u) ||
        (P.row_stride6 & 15u) || !((P.row_stride6 >> 4) & 1u) || (P.use_tmap && !tmaps) ||
        P.act_off < (uint32_t)GM_ROWS * max(P.row_stride, P.row_stride6) || (P.act_off & 15u) || P.act_off + (uint32_t)CB * GM_ACT_BLOCK_BYTES > P.slot_bytes || (P.slot_bytes & 127u) ||
        n_jobs < 1 || (CB != GM_CHUNK && CB != 2 * GM_CHUNK)) {
        if (tid == 0) atomicExch(dev_error, DEV_ERR_BAD_JOB);
        return;
    }
    if (P.dynamic_table) pdl_wait();   // the table itself is written by the previous kernel
    pdl_launch_dependents();
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t pbuf = smem_base + (uint32_t)S * P.slot_bytes, zeros = pbuf + 2u * GM_PBUF_BYTES;
    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GM_MMA_WARPS);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&pfull[b], GM_MMA_WARPS);
            mbar_init(&pempty[b], 1);
        }
        s_abort = 0;
        mbar_fence_init();
    }
    for (uint32_t i = tid; i < GM_ZERO_BYTES / 4; i += GM_THREADS) reinterpret_cast<uint32_t *>(smem + (size_t)S * P.slot_bytes + 2u * GM_PBUF_BYTES)[i] = 0u;
    __syncthreads();
    GmCursor cur;
    cur.tile = blockIdx.x;
    cur.part = 0;
    cur.chunk = 0;
    if (cur.tile >= P.n_tiles || !gm_locate(jobs, n_jobs, cur)) return;
    const int tile_step = gridDim.x;

    if (warp < GM_MMA_WARPS) {
        // ------------------------------ MMA warps ------------------------------
        int slot = 0;
        uint32_t it = 0;
        bool more = true, failed = false;
        GM_PROF_DECL;
        while (more) {
            const int nblk = min(CB, nb - cur.chunk * CB);
            const uint32_t slot_base = smem_base + (uint32_t)slot * P.slot_bytes;
            // the stage has landed
            if (!gm_wait(&full[slot], (it / (uint32_t)S) & 1u, &s_abort)) {
                failed = true;
                break;
            }
            GM_PROF_LAP(prof_a);
            for (int h = 0; h < halves; h++) {
                const uint32_t ri = it * (uint32_t)halves + (uint32_t)h, b = ri & 1u;   // record item and its buffer
                const int j = h * GM_CHUNK + warp;                                       // this warp's block of the stage
                // the record buffer is free once the replay of two record items ago is done
                if (ri >= 2 && !gm_wait(&pempty[b], ((ri >> 1) - 1u) & 1u, &s_abort)) {
                    failed = true;
                    break;
                }
                GM_PROF_LAP(prof_b);
                if (j < nblk) {
                    const uint32_t act_qs = slot_base + P.act_off + (uint32_t)j * 256u;
                    const uint32_t act_bs = slot_base + P.act_off + (uint32_t)CB * 256u + (uint32_t)j * 32u;
                    const float yd = lds_f1(slot_base + P.act_off + (uint32_t)CB * 288u + (uint32_t)j * 4u);
                    const uint32_t rec = pbuf + b * GM_PBUF_BYTES + (uint32_t)warp * GM_ROWS * GM_REC_BYTES;
                    if (cur.type == TYPE_Q4_K) gm_q4k_block(slot_base, P.row_stride, (uint32_t)j * Q4K_BYTES, act_qs, act_bs, yd, zeros, rec, lane);
                    else if (j & 1) gm_q6k_block<true>(slot_base, P.row_stride6, (uint32_t)j * Q6K_BYTES, act_qs, act_bs, yd, zeros, rec, lane);
                    else gm_q6k_block<false>(slot_base, P.row_stride6, (uint32_t)j * Q6K_BYTES, act_qs, act_bs, yd, zeros, rec, lane);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&pfull[b]);   // this warp's record of the half (if any) is in place
                GM_PROF_LAP(prof_c);
            }
            if (failed) break;
            if (lane == 0) mbar_arrive(&empty[slot]);   // this warp has consumed the stage's bytes: the producer may refill the slot
            ++it;
            if (++slot == S) slot = 0;
            more = gm_next(jobs, n_jobs, n_chunks, P.n_tiles, tile_step, cur);
            GM_PROF_LAP(prof_c);
#ifdef GM_PROFILE
            prof_n++;
#endif
        }
#ifdef GM_PROFILE
        if (lane == 0) {
            atomicAdd(&g_gm_prof[0], (unsigned long long)prof_a);
            atomicAdd(&g_gm_prof[1], (unsigned long long)prof_b);
            atomicAdd(&g_gm_prof[2], (unsigned long long)prof_c);
            atomicAdd(&g_gm_prof[6], (unsigned long long)prof_n);
        }
#endif
        if (failed && lane == 0) {
            s_abort = 1;
            atomicExch(dev_error, DEV_ERR_MBAR_TIMEOUT);
        }
        return;
    }

    if (warp == GM_MMA_WARPS) {
        // ------------------------------ producer warp: one lane issues every copy ------------------------------
        if (lane != 0) return;
        // copies of item (tile, part, chunk) into a slot: one bulk copy per weight row, three for the activation slices
        auto issue = [&](const GmCursor &c, int slot, bool weights, bool act) {
            const GemvJob &job = jobs[c.jsel];
            const uint32_t blk = c.type == TYPE_Q4_K ? Q4K_BYTES : Q6K_BYTES;
            const int nblk = min(CB, nb - c.chunk * CB);
            const uint32_t wbytes = (uint32_t)nblk * blk, dbytes = ((uint32_t)nblk * 4u + 15u) & ~15u;
            uint64_t *bar = &full[slot];
            uint8_t *dst = smem + (size_t)slot * P.slot_bytes;
            const uint32_t rs = c.type == TYPE_Q4_K ? P.row_stride : P.row_stride6;
            if (weights && P.use_tmap) {
                // one tiled copy: the box is always 16 rows x the whole row stride (zeros past the matrix), and so is its byte count
                mbar_arrive_expect_tx(bar, (uint32_t)GM_ROWS * rs + (uint32_t)nblk * 288u + dbytes);
                gm_tma_2d(smem_u32(dst), &tmaps->m[c.jsel], (int)(((uint32_t)(c.chunk * CB) * blk) >> 3), c.row0, bar);
            } else if (weights) {
                mbar_arrive_expect_tx(bar, wbytes * (uint32_t)c.nrows + (uint32_t)nblk * 288u + dbytes);
                const size_t rb = (size_t)nb * blk;
                const uint8_t *src = job.parts[c.part].w + (size_t)c.row0 * rb + (uint32_t)(c.chunk * CB) * blk;
                uint8_t *d = dst;
                for (int r = 0; r < c.nrows; r++, src += rb, d += rs) bulk_g2s(d, src, wbytes, bar);
            }
            if (act) {
                const uint8_t *x = job.parts[c.part].x;
                const uint32_t b0 = (uint32_t)(c.chunk * CB);
                bulk_g2s(dst + P.act_off, x + b0 * 256u, (uint32_t)nblk * 256u, bar);
                bulk_g2s(dst + P.act_off + (uint32_t)CB * 256u, x + cols + b0 * 32u, (uint32_t)nblk * 32u, bar);
                bulk_g2s(dst + P.act_off + (uint32_t)CB * 288u, x + cols + 32 * nb + b0 * 4u, dbytes, bar);
            }
        };
        GmCursor pc = cur;
        bool p_more = true, failed = false;
        uint32_t issued = 0;
        {
            GmCursor c2 = cur;
            bool m2 = true;
            for (int i = 0; i < S && m2; i++) {
                issue(c2, i, true, false);
                m2 = gm_next(jobs, n_jobs, n_chunks, P.n_tiles, tile_step, c2);
            }
            pdl_wait();   // weights do not depend on the previous kernel; the activation does
            for (int i = 0; i < S && p_more; i++) {
                issue(pc, i, false, true);
                ++issued;
                p_more = gm_next(jobs, n_jobs, n_chunks, P.n_tiles, tile_step, pc);
            }
        }
        int slot = 0;
        while (p_more) {
            // item `issued` goes into the slot that item `issued - S` has occupied
            if (!gm_wait(&empty[slot], ((issued / (uint32_t)S) - 1u) & 1u, &s_abort)) {
                failed = true;
                break;
            }
            issue(pc, slot, true, true);
            ++issued;
            if (++slot == S) slot = 0;
            p_more = gm_next(jobs, n_jobs, n_chunks, P.n_tiles, tile_step, pc);
        }
        if (failed) {
            s_abort = 1;
            atomicExch(dev_error, DEV_ERR_MBAR_TIMEOUT);
        }
        // Every copy this lane started must land before the CTA's shared memory goes away: the consumers
        // wait for each of them in the normal course; after a failure wait here (bounded) for the last S.
        if (failed || s_abort) {
            const uint32_t first = issued > (uint32_t)S ? issued - (uint32_t)S : 0u;
            for (uint32_t n = first; n < issued; n++) {
                bool landed = false;
                for (uint32_t k = 0; k < (1u << 18) && !landed; k++) landed = mbar_try_wait(&full[n % (uint32_t)S], (n / (uint32_t)S) & 1u);
            }
        }
        return;
    }

    // ------------------------------ replay warp ------------------------------
    pdl_wait();
    // thread (row r = lane / 2, half hq = lane % 2) carries accumulator lanes 4hq..4hq+3 and mins lanes 2hq, 2hq+1
    const int r = lane >> 1, hq = lane & 1;
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, accm[2] = {0.f, 0.f}, acc_total = 0.f;
    const uint32_t ra = (uint32_t)r * GM_REC_BYTES + gm_rec_unit(r, hq), rd = (uint32_t)r * GM_REC_BYTES + gm_rec_unit(r, 3);
    const uint32_t rm = (uint32_t)r * GM_REC_BYTES + gm_rec_unit(r, 2) + 8u * (uint32_t)hq;
    uint32_t it = 0;
    bool more = true, failed = false;
    GM_PROF_DECL;
    float res_pref = 0.f;
    while (more) {
        const int nblk_stage = min(CB, nb - cur.chunk * CB);
        const bool q4 = cur.type == TYPE_Q4_K;
        if (cur.chunk == 0 && cur.part == 0) {
            // the residual of this tile's rows is fetched now and used when the tile is done
            const GemvJob &tj = jobs[cur.jsel];
            res_pref = (r < cur.nrows && hq == 0 && tj.residual) ? tj.residual[(size_t)cur.row0 + r] : 0.f;
        }
        for (int h = 0; h < halves; h++) {
            const uint32_t ri = it * (uint32_t)halves + (uint32_t)h, b = ri & 1u;
            const int nblk = max(0, min(GM_CHUNK, nblk_stage - h * GM_CHUNK));
            if (!gm_wait(&pfull[b], (ri >> 1) & 1u, &s_abort)) {
                failed = true;
                break;
            }
            GM_PROF_LAP(prof_a);
            const uint32_t recs = pbuf + b * GM_PBUF_BYTES;
            if (nblk == GM_CHUNK) {
                // all records first, then the ordered chains: the loads overlap instead of alternating with the FMAs
                float4 sv[GM_CHUNK];
                float2 mv[GM_CHUNK], dv[GM_CHUNK];
#pragma unroll
                for (int j = 0; j < GM_CHUNK; j++) {
                    const uint32_t rj = recs + (uint32_t)j * GM_ROWS * GM_REC_BYTES;
                    sv[j] = lds_f4(rj + ra);
                    dv[j] = lds_f2(rj + rd);
                    if (q4) mv[j] = lds_f2(rj + rm);
                }
#pragma unroll
                for (int j = 0; j < GM_CHUNK; j++) {
                    acc[0] = __fmaf_rn(dv[j].x, sv[j].x, acc[0]);
                    acc[1] = __fmaf_rn(dv[j].x, sv[j].y, acc[1]);
                    acc[2] = __fmaf_rn(dv[j].x, sv[j].z, acc[2]);
                    acc[3] = __fmaf_rn(dv[j].x, sv[j].w, acc[3]);
                    if (q4) {
                        accm[0] = __fmaf_rn(dv[j].y, mv[j].x, accm[0]);
                        accm[1] = __fmaf_rn(dv[j].y, mv[j].y, accm[1]);
                    }
                }
            } else {
                for (int j = 0; j < nblk; j++) {
                    const uint32_t rj = recs + (uint32_t)j * GM_ROWS * GM_REC_BYTES;
                    const float4 s = lds_f4(rj + ra);
                    const float2 d = lds_f2(rj + rd);
                    acc[0] = __fmaf_rn(d.x, s.x, acc[0]);
                    acc[1] = __fmaf_rn(d.x, s.y, acc[1]);
                    acc[2] = __fmaf_rn(d.x, s.z, acc[2]);
                    acc[3] = __fmaf_rn(d.x, s.w, acc[3]);
                    if (q4) {
                        const float2 m = lds_f2(rj + rm);
                        accm[0] = __fmaf_rn(d.y, m.x, accm[0]);
                        accm[1] = __fmaf_rn(d.y, m.y, accm[1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&pempty[b]);
            GM_PROF_LAP(prof_b);
        }
        if (failed) break;
        if (cur.chunk == n_chunks - 1) {
            // fold: (l + l4) -> (+2) -> (+1); mins (a0 + a2) + (a1 + a3)
            const float v0 = __fadd_rn(acc[0], __shfl_xor_sync(0xffffffffu, acc[0], 1));
            const float v1 = __fadd_rn(acc[1], __shfl_xor_sync(0xffffffffu, acc[1], 1));
            const float v2 = __fadd_rn(acc[2], __shfl_xor_sync(0xffffffffu, acc[2], 1));
            const float v3 = __fadd_rn(acc[3], __shfl_xor_sync(0xffffffffu, acc[3], 1));
            float dot = __fadd_rn(__fadd_rn(v0, v2), __fadd_rn(v1, v3));
            // mins: (m0 + m2) + (m1 + m3); the pair of threads of a row holds (m0, m1) and (m2, m3)
            const float m02 = __fadd_rn(accm[0], __shfl_xor_sync(0xffffffffu, accm[0], 1));
            const float m13 = __fadd_rn(accm[1], __shfl_xor_sync(0xffffffffu, accm[1], 1));
            if (q4) dot = __fadd_rn(dot, __fadd_rn(m02, m13));
            const GemvJob &job = jobs[cur.jsel];
            if (job.parts[cur.part].scale) dot = __fmul_rn(dot, __ldg(job.parts[cur.part].scale));
            acc_total = cur.n_parts == 1 ? dot : __fadd_rn(acc_total, dot);
#pragma unroll
            for (int k = 0; k < 4; k++) acc[k] = 0.f;
            accm[0] = accm[1] = 0.f;
            if (cur.part == cur.n_parts - 1) {
                const bool live = r < cur.nrows && hq == 0;
                const size_t o = (size_t)cur.row0 + r;
                float val = acc_total;
                if (live && job.residual) val = __fadd_rn(res_pref, acc_total);
                acc_total = 0.f;
                const int epi = job.epi;
                if (epi == GEMV_EPI_NONE) {
                    if (live) {
                        job.y[o] = val;
                        if (PEER && tail.kind == 2) peer_store(tail.peer, o, val);
                    }
                } else {
                    // q/k/v: adjacent-pair RoPE and/or the f16 KV append on the rows just produced; rows 2i and
                    // 2i+1 sit two lanes apart
                    const float other = __shfl_xor_sync(0xffffffffu, val, 2);
                    if (live) {
                        const int pos = *job.epi_pos;
                        float outv = val;
                        if (epi == GEMV_EPI_ROPE_F32 || epi == GEMV_EPI_ROPE_F16_CACHE) {
                            const int jj = (int)(o & (size_t)127), i = jj >> 1;
                            const float *cs = job.epi_rope + (size_t)pos * 128;
                            const float cc = cs[i], sn = cs[64 + i];
                            const float x0 = (jj & 1) ? other : val, x1 = (jj & 1) ? val : other;
                            outv = (jj & 1) ? __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cc)) : __fsub_rn(__fmul_rn(x0, cc), __fmul_rn(x1, sn));
                        }
                        if (epi == GEMV_EPI_ROPE_F32) job.y[o] = outv;
                        else job.epi_cache[(size_t)pos * job.epi_kv_dim + o] = __half_as_ushort(__float2half_rn(outv));
                    }
                }
                if (tail.kind == 1) gm_silu_tail(tail, cur.row0 >> 8, n_jobs * (256 / GM_ROWS), lane);
            }
        }
        ++it;
        more = gm_next(jobs, n_jobs, n_chunks, P.n_tiles, tile_step, cur);
        GM_PROF_LAP(prof_c);
#ifdef GM_PROFILE
        prof_n++;
#endif
    }
#ifdef GM_PROFILE
    if (lane == 0) {
        atomicAdd(&g_gm_prof[3], (unsigned long long)prof_a);
        atomicAdd(&g_gm_prof[4], (unsigned long long)prof_b);
        atomicAdd(&g_gm_prof[5], (unsigned long long)prof_c);
        atomicAdd(&g_gm_prof[7], (unsigned long long)prof_n);
    }
#endif
    if (failed && lane == 0) {
        s_abort = 1;
        atomicExch(dev_error, DEV_ERR_MBAR_TIMEOUT);
    }
    if (PEER && tail.kind == 2 && !failed) {
        // every CTA of the grid arrives once, with or without tiles; the last raises the peers' flags
        __threadfence_system();
        __syncwarp();
        if (lane == 0) peer_arrive(tail.peer);
    }
}

RNB_GLOBAL void __launch_bounds__(GM_THREADS, GM_MIN_CTAS)
gemv_mma_kernel(const GemvJob *__restrict__ jobs, int n_jobs, const GmParams P, int *__restrict__ dev_error) {
    GpTail none;
    none.kind = 0;
    none.peer.peers = nullptr;
    gemv_mma_body<false>(jobs, n_jobs, P, dev_error, none, nullptr);
}
RNB_GLOBAL void __launch_bounds__(GM_THREADS, GM_MIN_CTAS)
gemv_mma_kernel_1(const __grid_constant__ GemvJobPack jobs, int n_jobs, const GmParams P, int *__restrict__ dev_error,
                  const __grid_constant__ GpTail tail, const __grid_constant__ GmTmaps tmaps) {
    gemv_mma_body<false>(jobs.j, n_jobs, P, dev_error, tail, &tmaps);
}
RNB_GLOBAL void __launch_bounds__(GM_THREADS, GM_MIN_CTAS)
gemv_mma_kernel_1_peer(const __grid_constant__ GemvJobPack jobs, int n_jobs, const GmParams P, int *__restrict__ dev_error,
                       const __grid_constant__ GpTail tail, const __grid_constant__ GmTmaps tmaps) {
    gemv_mma_body<true>(jobs.j, n_jobs, P, dev_error, tail, &tmaps);
}

}  // namespace rnb
