// Q5_K x Q8_K (and, below, Q2_K x Q8_K) matvec, bit-exact with rnb-cpu's AVX2 dots
// (crates/rnb-cpu/src/gemm/avx2_dot.rs:698-789): eight f32 accumulator lanes per row (lane l sums
// bytes 4l..4l+3 of every 32-byte group), one FMA per block in block order, the fold 4-2-1 at
// the end, and the mins term kept as ONE scalar that takes a rounded product and a rounded sum
// per block.  Block layout (176 bytes): d f16 | dmin f16 | scales[12] | qh[32] | qs[128]
// (crates/rnb-cpu/src/quantize/blocks.rs:90-98); bit j of qh[i] is the fifth bit of element i of
// sub-block j.
//
// One warp per row: its four 8-lane groups take four consecutive blocks at a time; integer lane
// sums are exact in any order, the f32 chain is then replayed in block order with the four
// blocks' values fetched by shuffle (every group carries the same accumulators).  Weights are
// read straight from global memory with 4-byte loads: this kernel serves the formats beside the
// Q4_K_M set and is built for parity first; it does not stage through shared memory.
#pragma once
#include "common.cuh"

namespace rnb {

constexpr int TYPE_Q5_K = 13;
constexpr int Q5K_BYTES = 176;
constexpr int G5_WARPS = 4;

// xq: Q8K-dev layout of the activation (qs[cols] | bsum16[cols/16] | d[cols/256]); seq tokens, xq_stride bytes apart
RNB_GLOBAL void __launch_bounds__(G5_WARPS * 32)
gemv_q5k_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, size_t xq_stride, float *__restrict__ y, int rows, int cols, int seq) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * G5_WARPS + warp;
    if (row >= rows) return;
    const int nb = cols >> 8, l = lane & 7, g = lane >> 3;
    const uint8_t *wrow = w + (size_t)row * nb * Q5K_BYTES;
    for (int s = 0; s < seq; s++) {
        const uint8_t *x = xq + (size_t)s * xq_stride;
        const int8_t *qs = reinterpret_cast<const int8_t *>(x);
        const int16_t *bsum16 = reinterpret_cast<const int16_t *>(x + cols);
        const float *xd = reinterpret_cast<const float *>(x + cols + 32 * nb);
        float acc = 0.f, summs = 0.f;
        for (int b0 = 0; b0 < nb; b0 += 4) {
            const int b = b0 + g;
            int sumi = 0;
            float dd = 0.f, mprod = 0.f;
            if (b < nb) {
                const uint8_t *blk = wrow + (size_t)b * Q5K_BYTES;
                const uint32_t hdr = *reinterpret_cast<const uint32_t *>(blk);
                const float yd = xd[b];
                dd = __fmul_rn(yd, __half2float(__ushort_as_half((unsigned short)(hdr & 0xffffu))));
                const float dmin = __fmul_rn(-yd, __half2float(__ushort_as_half((unsigned short)(hdr >> 16))));
                // 6-bit scales and mins of the eight sub-blocks (the reference's unpack of the 12 packed bytes)
                uint32_t u0 = *reinterpret_cast<const uint32_t *>(blk + 4), u1 = *reinterpret_cast<const uint32_t *>(blk + 8),
                         u2 = *reinterpret_cast<const uint32_t *>(blk + 12);
                const uint32_t u3 = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
                const uint32_t ua = u1 & 0x3f3f3f3fu;
                u1 = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
                u2 = ua;
                u0 &= 0x3f3f3f3fu;
                // scales: bytes of (u0, u1); mins: bytes of (u2, u3)
                int msum = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int mn = (int)(((j < 4 ? u2 : u3) >> (8 * (j & 3))) & 0xffu);
                    const int bs = (int)(short)(bsum16[b * 16 + 2 * j] + bsum16[b * 16 + 2 * j + 1]);   // 16-bit wrap as the AVX2 hadd
                    msum += mn * bs;
                }
                mprod = __fmul_rn(dmin, (float)msum);
                const uint32_t qh = *reinterpret_cast<const uint32_t *>(blk + 16 + 4 * l);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t ql = *reinterpret_cast<const uint32_t *>(blk + 48 + 32 * j + 4 * l);
                    const int v0 = (int)((ql & 0x0f0f0f0fu) | (((qh >> (2 * j)) & 0x01010101u) << 4));
                    const int v1 = (int)(((ql >> 4) & 0x0f0f0f0fu) | (((qh >> (2 * j + 1)) & 0x01010101u) << 4));
                    const int a0 = *reinterpret_cast<const int *>(qs + b * 256 + 64 * j + 4 * l);
                    const int a1 = *reinterpret_cast<const int *>(qs + b * 256 + 64 * j + 32 + 4 * l);
                    const int sc0 = (int)(((j < 2 ? u0 : u1) >> (8 * ((2 * j) & 3))) & 0xffu);
                    const int sc1 = (int)(((j < 2 ? u0 : u1) >> (8 * ((2 * j + 1) & 3))) & 0xffu);
                    sumi += sc0 * __dp4a(v0, a0, 0) + sc1 * __dp4a(v1, a1, 0);   // weights 0..31: positive as signed bytes
                }
            }
            // the four blocks' FMAs in block order; every group ends up with the same eight lanes
#pragma unroll
            for (int gg = 0; gg < 4; gg++) {
                const int si = __shfl_sync(0xffffffffu, sumi, l + 8 * gg);
                const float di = __shfl_sync(0xffffffffu, dd, l + 8 * gg);
                const float mi = __shfl_sync(0xffffffffu, mprod, l + 8 * gg);
                if (b0 + gg < nb) {
                    acc = __fmaf_rn(di, (float)si, acc);
                    summs = __fadd_rn(summs, mi);
                }
            }
        }
        // fold: (l + l4) -> (+2) -> (+1), then the scalar mins term
        float r = __fadd_rn(__shfl_sync(0xffffffffu, acc, (l + 4) & 7), acc);   // lanes 0..3: a[l+4] + a[l]
        r = __fadd_rn(r, __shfl_sync(0xffffffffu, r, (l + 2) & 7));            // lanes 0, 1: (r0 + r2), (r1 + r3)
        r = __fadd_rn(r, __shfl_sync(0xffffffffu, r, (l + 1) & 7));            // lane 0: s0 + s1
        if (lane == 0) y[(size_t)s * rows + row] = __fadd_rn(r, summs);
    }
}

// Q2_K x Q8_K, bit-exact with crates/rnb-cpu/src/gemm/avx2_dot.rs:169-245.  Block (84 bytes): scales[16]
// (low nibble scale, high nibble min) | qs[64] | d f16 | dmin f16 (crates/rnb-cpu/src/quantize/blocks.rs:63-69).
// Eight accumulator lanes; per block first the mins term (lane l: min[2l] * bsum[2l] + min[2l+1] * bsum[2l+1],
// one FMA with dmin), then the quants (lane l = bytes 4l..4l+3 of each 32-byte chunk; chunk k of half h is the
// 2-bit plane k and takes sub-block scale 8h + 2k for lanes 0..3, 8h + 2k + 1 for lanes 4..7), one FMA with d.
// Same warp-per-row scheme as the Q5_K kernel above.
constexpr int TYPE_Q2_K = 10;
constexpr int Q2K_BYTES = 84;
RNB_GLOBAL void __launch_bounds__(G5_WARPS * 32)
gemv_q2k_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, size_t xq_stride, float *__restrict__ y, int rows, int cols, int seq) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * G5_WARPS + warp;
    if (row >= rows) return;
    const int nb = cols >> 8, l = lane & 7, g = lane >> 3;
    const uint8_t *wrow = w + (size_t)row * nb * Q2K_BYTES;
    for (int s = 0; s < seq; s++) {
        const uint8_t *x = xq + (size_t)s * xq_stride;
        const int8_t *qs = reinterpret_cast<const int8_t *>(x);
        const int16_t *bsum16 = reinterpret_cast<const int16_t *>(x + cols);
        const float *xd = reinterpret_cast<const float *>(x + cols + 32 * nb);
        float acc = 0.f;
        for (int b0 = 0; b0 < nb; b0 += 4) {
            const int b = b0 + g;
            int sumi = 0, prod = 0;
            float dd = 0.f, dmin = 0.f;
            if (b < nb) {
                const uint8_t *blk = wrow + (size_t)b * Q2K_BYTES;
                const uint32_t tail = *reinterpret_cast<const uint32_t *>(blk + 80);
                const float yd = xd[b];
                dd = __fmul_rn(yd, __half2float(__ushort_as_half((unsigned short)(tail & 0xffffu))));
                dmin = __fmul_rn(-yd, __half2float(__ushort_as_half((unsigned short)(tail >> 16))));
                const uint32_t sc_lo = *reinterpret_cast<const uint32_t *>(blk + ((2 * l) & ~3));   // holds scales bytes 2l, 2l + 1
                const int m0 = (int)((sc_lo >> (8 * ((2 * l) & 3) + 4)) & 0xfu), m1 = (int)((sc_lo >> (8 * ((2 * l + 1) & 3) + 4)) & 0xfu);
                prod = m0 * (int)bsum16[b * 16 + 2 * l] + m1 * (int)bsum16[b * 16 + 2 * l + 1];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t q2 = *reinterpret_cast<const uint32_t *>(blk + 16 + 32 * h + 4 * l);
                    const uint32_t scw = *reinterpret_cast<const uint32_t *>(blk + 8 * h), scw2 = *reinterpret_cast<const uint32_t *>(blk + 8 * h + 4);
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int v = (int)((q2 >> (2 * k)) & 0x03030303u);
                        const int a = *reinterpret_cast<const int *>(qs + b * 256 + 128 * h + 32 * k + 4 * l);
                        const int si = 2 * k + (l >= 4);                                        // sub-block within the half
                        const int sc = (int)(((si < 4 ? scw : scw2) >> (8 * (si & 3))) & 0xfu);
                        sumi += sc * __dp4a(v, a, 0);
                    }
                }
            }
#pragma unroll
            for (int gg = 0; gg < 4; gg++) {
                const int pi = __shfl_sync(0xffffffffu, prod, l + 8 * gg), si = __shfl_sync(0xffffffffu, sumi, l + 8 * gg);
                const float di = __shfl_sync(0xffffffffu, dd, l + 8 * gg), mi = __shfl_sync(0xffffffffu, dmin, l + 8 * gg);
                if (b0 + gg < nb) {
                    acc = __fmaf_rn(mi, (float)pi, acc);
                    acc = __fmaf_rn(di, (float)si, acc);
                }
            }
        }
        float r = __fadd_rn(__shfl_sync(0xffffffffu, acc, (l + 4) & 7), acc);
        r = __fadd_rn(r, __shfl_sync(0xffffffffu, r, (l + 2) & 7));
        r = __fadd_rn(r, __shfl_sync(0xffffffffu, r, (l + 1) & 7));
        if (lane == 0) y[(size_t)s * rows + row] = r;
    }
}

// Q3_K x Q8_K, bit-exact with crates/rnb-cpu/src/gemm/avx2_dot.rs:247-378.  Block (110 bytes, so only 2-byte
// aligned): hmask[32] | qs[64] | scales[12] | d f16 (crates/rnb-cpu/src/quantize/blocks.rs:72-78).  Sixteen
// six-bit scales with bias 32; an element is its two low bits minus 4 where its hmask bit (4h + k for plane k of
// half h) is clear.  Eight lanes, one FMA per block; lane / scale assignment as for Q2_K.
constexpr int TYPE_Q3_K = 11;
constexpr int Q3K_BYTES = 110;
__device__ __forceinline__ uint32_t ld32_a2(const uint8_t *p) {   // 4 bytes from a 2-byte aligned address
    const unsigned short *h = reinterpret_cast<const unsigned short *>(p);
    return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}
RNB_GLOBAL void __launch_bounds__(G5_WARPS * 32)
gemv_q3k_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, size_t xq_stride, float *__restrict__ y, int rows, int cols, int seq) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * G5_WARPS + warp;
    if (row >= rows) return;
    const int nb = cols >> 8, l = lane & 7, g = lane >> 3;
    const uint8_t *wrow = w + (size_t)row * nb * Q3K_BYTES;
    for (int s = 0; s < seq; s++) {
        const uint8_t *x = xq + (size_t)s * xq_stride;
        const int8_t *qs = reinterpret_cast<const int8_t *>(x);
        const float *xd = reinterpret_cast<const float *>(x + cols + 32 * nb);
        float acc = 0.f;
        for (int b0 = 0; b0 < nb; b0 += 4) {
            const int b = b0 + g;
            int sumi = 0;
            float dd = 0.f;
            if (b < nb) {
                const uint8_t *blk = wrow + (size_t)b * Q3K_BYTES;
                dd = __fmul_rn(xd[b], __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blk + 108))));
                // the 16 scales as bytes of aux[0..3] (the reference's unpack of the 12 packed bytes), still biased by 32
                const uint32_t a0 = ld32_a2(blk + 96), a1 = ld32_a2(blk + 100), a2 = ld32_a2(blk + 104);
                uint32_t aux[4];
                aux[0] = (a0 & 0x0f0f0f0fu) | (((a2 >> 0) & 0x03030303u) << 4);
                aux[1] = (a1 & 0x0f0f0f0fu) | (((a2 >> 2) & 0x03030303u) << 4);
                aux[2] = ((a0 >> 4) & 0x0f0f0f0fu) | (((a2 >> 4) & 0x03030303u) << 4);
                aux[3] = ((a1 >> 4) & 0x0f0f0f0fu) | (((a2 >> 6) & 0x03030303u) << 4);
                const uint32_t nhm = ~ld32_a2(blk + 4 * l);   // set where 4 is subtracted
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t q3 = ld32_a2(blk + 32 + 32 * h + 4 * l);
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int lo = (int)((q3 >> (2 * k)) & 0x03030303u);
                        const int hi = (int)(((nhm >> (4 * h + k)) & 0x01010101u) << 2);
                        const int a = *reinterpret_cast<const int *>(qs + b * 256 + 128 * h + 32 * k + 4 * l);
                        const int si = 8 * h + 2 * k + (l >= 4);
                        const int sc = (int)((aux[si >> 2] >> (8 * (si & 3))) & 0xffu) - 32;
                        sumi += sc * (__dp4a(lo, a, 0) - __dp4a(hi, a, 0));
                    }
                }
            }
#pragma unroll
            for (int gg = 0; gg < 4; gg++) {
                const int si = __shfl_sync(0xffffffffu, sumi, l + 8 * gg);
                const float di = __shfl_sync(0xffffffffu, dd, l + 8 * gg);
                if (b0 + gg < nb) acc = __fmaf_rn(di, (float)si, acc);
            }
        }
        float r = __fadd_rn(__shfl_sync(0xffffffffu, acc, (l + 4) & 7), acc);
        r = __fadd_rn(r, __shfl_sync(0xffffffffu, r, (l + 2) & 7));
        r = __fadd_rn(r, __shfl_sync(0xffffffffu, r, (l + 1) & 7));
        if (lane == 0) y[(size_t)s * rows + row] = r;
    }
}

}  // namespace rnb
