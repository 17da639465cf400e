// Dequant-fused batch-1 matvec over GGUF block formats: Q4_K x Q8_K, Q6_K x Q8_K, Q8_0 x f32.
//
// This is an HBM stream, not a contraction: each CTA pulls one tile of whole weight rows
// (a contiguous byte range, because rows of blocks are stored back to back) into shared
// memory with a single bulk-async copy per matrix, signalled on an mbarrier, then unpacks
// nibbles/scales in registers and accumulates with dp4a.  Several CTAs are resident per SM,
// so copies of later tiles overlap the arithmetic of earlier ones.  The Q8_K activation is
// small (<= 30 KB) and is read through L1 with 16-byte loads.
//
// Numerics follow rnb-cpu's integer dots (crates/rnb-cpu/src/gemm/avx2_dot.rs:621-696 Q4_K,
// :801-885 Q6_K): exact int32 sums inside a block, fp32 accumulation across blocks.  Q8_0
// uses f32 activations like rnb-cpu's x86 path (crates/rnb-cpu/src/gemm/quant_gemv.rs:127-141).
#pragma once
#include "common.cuh"

namespace rnb {

constexpr int GEMV_THREADS = 128;
constexpr int GEMV_MAX_PARTS = 8;

// y[row] = residual[row] + sum_p scale_p * dot(W_p[row, :], x_p)
// One "part" per (matrix, activation) pair; ordinary matvecs have one part, the MoE down
// projection has one part per routed expert (summed in selection order).
struct GemvPart {
    const uint8_t *w;    // rows x row_bytes, device
    const uint8_t *x;    // Q8K-dev layout (K-quants) or float[cols] (Q8_0)
    const float *scale;  // optional device scalar (route weight); null = 1
};
struct GemvJob {
    float *y;
    const float *residual;  // optional
    int rows;
    int type;
    int n_parts;
    int tile0;  // index of this job's first tile within the launch
    int rows_per_tile;
    int seq;          // tokens sharing the weight tile (1 for decode); outputs are seq-major
    size_t x_stride;  // bytes between consecutive tokens' activations
    GemvPart parts[GEMV_MAX_PARTS];
    // Optional epilogue of the batch-1 streaming kernel (decode q/k/v): rotate adjacent row pairs
    // with the cos/sin row of the current position and/or write the row as f16 into a KV cache.
    int epi;                  // GEMV_EPI_*
    int epi_kv_dim;           // elements per cache position
    const float *epi_rope;    // [pos][cos 64 | sin 64]
    const int *epi_pos;       // device scalar: position of this token
    uint16_t *epi_cache;      // K or V cache of the layer
    // Expert-gathered form (two-threads-per-row kernel): `rows` are virtual rows, dyn_rows per selected expert;
    // virtual row v reads row ids[v / dyn_rows] * dyn_rows + v % dyn_rows of the stacked expert tensor parts[0].w
    // against the activation parts[0].x + (v / dyn_rows) * dyn_x_stride.  The ids are written by an earlier
    // kernel of the same stream.  null = plain rows.
    const uint32_t *dyn_ids;
    int dyn_rows;
    uint32_t dyn_x_stride;
};
constexpr int GEMV_EPI_NONE = 0, GEMV_EPI_ROPE_F32 = 1, GEMV_EPI_ROPE_F16_CACHE = 2, GEMV_EPI_F16_CACHE = 3;

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// 8 bytes from shared memory at any 2-byte-aligned address (Q6_K/Q8_0 blocks are 210/34 bytes).
__device__ __forceinline__ uint2 lds8_unaligned(uint32_t addr) {
    const uint32_t base = addr & ~3u, sh = (addr & 3u) * 8u;
    const uint32_t w0 = lds32(base), w1 = lds32(base + 4), w2 = lds32(base + 8);
    return make_uint2(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh));
}

// All three formats reproduce rnb-cpu's x86 results BIT FOR BIT.  The AVX2 dots keep eight f32
// accumulator lanes per row (lane l sums bytes 4l..4l+3 of every 32-byte group), add one FMA
// per block in block order, and fold the lanes 4, 2, 1 apart at the end
// (crates/rnb-cpu/src/gemm/avx2_dot.rs:25-31,621-696,801-885).  Here a warp owns a row and its
// four 8-lane groups take four consecutive blocks at a time; integer lane sums are exact in
// any order, so they are reduce-scattered inside a group until thread t of the group holds
// the sum of ONE accumulator lane, and then every thread replays the four blocks' FMAs in
// block order with the lane sums fetched by shuffle.

// ---- Q4_K ------------------------------------------------------------------------------------
// Thread t of a group owns qs bytes 16t..16t+15: 64-element group g = t/2, half h = t%2; its
// four words are accumulator lanes 4h..4h+3 of sub-blocks 2g (low nibbles) and 2g+1 (high).
// After the reduce-scatter it holds lane 4h+g.  Threads also carry the mins term: accumulator
// lane k = t%4 of acc_m is mn[2k]*bsum32[2k] + mn[2k+1]*bsum32[2k+1].
struct Q4kTerms {
    int lane_sum;   // sumi lane (4h+g) of this block
    int min_prod;   // acc_m integer for lane t%4
    float d, dmin;  // y.d*d and -y.d*dmin
};
__device__ __forceinline__ Q4kTerms q4k_block_terms(const uint8_t *blk, int t, const int8_t *xq,
                                                    float yd, const int16_t *bsum16, bool valid) {
    Q4kTerms r;
    r.lane_sum = 0;
    r.min_prod = 0;
    r.d = 0.f;
    r.dmin = 0.f;
    int v0 = 0, v1 = 0, v2 = 0, v3 = 0;
    const int g = t >> 1, h = t & 1;
    if (valid) {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
        const uint4 q = *reinterpret_cast<const uint4 *>(blk + 16 + 16 * t);
        const uint4 alo = ldg_nc_u4(xq + 64 * g + 16 * h);
        const uint4 ahi = ldg_nc_u4(xq + 64 * g + 32 + 16 * h);
        // 6-bit scale/min unpack (get_scale_min_k4) for all 8 sub-blocks at once
        const uint32_t sc03 = hdr.y & 0x3f3f3f3fu;
        const uint32_t mn03 = hdr.z & 0x3f3f3f3fu;
        const uint32_t sc47 = (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
        const uint32_t mn47 = ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
        const uint32_t scw = g < 2 ? sc03 : sc47;
        const int sc_lo = (scw >> (16 * (g & 1))) & 0xff;
        const int sc_hi = (scw >> (16 * (g & 1) + 8)) & 0xff;
        v0 = sc_lo * __dp4a((int)(q.x & 0x0f0f0f0fu), (int)alo.x, 0) + sc_hi * __dp4a((int)((q.x >> 4) & 0x0f0f0f0fu), (int)ahi.x, 0);
        v1 = sc_lo * __dp4a((int)(q.y & 0x0f0f0f0fu), (int)alo.y, 0) + sc_hi * __dp4a((int)((q.y >> 4) & 0x0f0f0f0fu), (int)ahi.y, 0);
        v2 = sc_lo * __dp4a((int)(q.z & 0x0f0f0f0fu), (int)alo.z, 0) + sc_hi * __dp4a((int)((q.z >> 4) & 0x0f0f0f0fu), (int)ahi.z, 0);
        v3 = sc_lo * __dp4a((int)(q.w & 0x0f0f0f0fu), (int)alo.w, 0) + sc_hi * __dp4a((int)((q.w >> 4) & 0x0f0f0f0fu), (int)ahi.w, 0);
        // mins: lane k = t%4 pairs sub-blocks 2k, 2k+1; bsum32[j] = bsum16[2j] + bsum16[2j+1] (i16)
        const int k = t & 3;
        const uint32_t mnw = k < 2 ? mn03 : mn47;
        const int mn_a = (mnw >> (16 * (k & 1))) & 0xff, mn_b = (mnw >> (16 * (k & 1) + 8)) & 0xff;
        const uint2 bs = ldg_nc_u2(bsum16 + 4 * k);  // four consecutive i16, 8-byte aligned
        const int b32a = (short)((short)(bs.x & 0xffff) + (short)(bs.x >> 16));
        const int b32b = (short)((short)(bs.y & 0xffff) + (short)(bs.y >> 16));
        r.min_prod = mn_a * b32a + mn_b * b32b;
        r.d = __fmul_rn(yd, f16_bits_to_f32(hdr.x & 0xffffu));
        r.dmin = __fmul_rn(-yd, f16_bits_to_f32(hdr.x >> 16));
    }
    // reduce over g (bits 1,2 of t), scattering the four words: thread (g,h) ends with word g
    const int g0 = g & 1, g1 = g >> 1;
    const int a0 = (g0 ? v1 : v0) + __shfl_xor_sync(0xffffffffu, g0 ? v0 : v1, 2);
    const int a1 = (g0 ? v3 : v2) + __shfl_xor_sync(0xffffffffu, g0 ? v2 : v3, 2);
    r.lane_sum = (g1 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, g1 ? a0 : a1, 4);
    return r;
}

// ---- Q6_K ------------------------------------------------------------------------------------
// Thread t = (n = t/4, m = t%4) owns l = 8m..8m+7 of half n in each of the four 32-element
// parts, i.e. accumulator lanes 2m and 2m+1; after exchanging with the other half it holds
// lane 2m+n, from which the reference subtracts 32*(bsums[2l]*sc[2l] + bsums[2l+1]*sc[2l+1]).
__device__ __forceinline__ void q6k_block_terms(uint32_t blk, int t, const int8_t *xq, float yd,
                                                const int16_t *bsum16, bool valid, int &lane_sum,
                                                float &d) {
    const int n = t >> 2, m = t & 3;
    int u0 = 0, u1 = 0, corr = 0;
    d = 0.f;
    const int l = 2 * m + n;
    if (valid) {
        const uint2 qla = lds8_unaligned(blk + 64 * n + 8 * m);
        const uint2 qlb = lds8_unaligned(blk + 64 * n + 32 + 8 * m);
        const uint2 qh = lds8_unaligned(blk + 128 + 32 * n + 8 * m);
        const int8_t *xa = xq + 128 * n + 8 * m;
        const uint2 a0 = ldg_nc_u2(xa), a1 = ldg_nc_u2(xa + 32), a2 = ldg_nc_u2(xa + 64), a3 = ldg_nc_u2(xa + 96);
        const uint32_t sc = blk + 192 + 8 * n + (m >> 1);
        int s0, s1, s2, s3, sa, sb, dh;
        asm volatile("ld.shared.s8 %0, [%1];" : "=r"(s0) : "r"(sc));
        asm volatile("ld.shared.s8 %0, [%1];" : "=r"(s1) : "r"(sc + 2));
        asm volatile("ld.shared.s8 %0, [%1];" : "=r"(s2) : "r"(sc + 4));
        asm volatile("ld.shared.s8 %0, [%1];" : "=r"(s3) : "r"(sc + 6));
        asm volatile("ld.shared.s8 %0, [%1];" : "=r"(sa) : "r"(blk + 192 + 2 * l));
        asm volatile("ld.shared.s8 %0, [%1];" : "=r"(sb) : "r"(blk + 192 + 2 * l + 1));
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dh) : "r"(blk + 208));
#pragma unroll
        for (int w = 0; w < 2; w++) {
            const uint32_t la = w ? qla.y : qla.x, lb = w ? qlb.y : qlb.x, hh = w ? qh.y : qh.x;
            const uint32_t q0 = (la & 0x0f0f0f0fu) | ((hh << 4) & 0x30303030u);
            const uint32_t q1 = (lb & 0x0f0f0f0fu) | ((hh << 2) & 0x30303030u);
            const uint32_t q2 = ((la >> 4) & 0x0f0f0f0fu) | (hh & 0x30303030u);
            const uint32_t q3 = ((lb >> 4) & 0x0f0f0f0fu) | ((hh >> 2) & 0x30303030u);
            const int acc = s0 * __dp4a((int)q0, (int)(w ? a0.y : a0.x), 0) + s1 * __dp4a((int)q1, (int)(w ? a1.y : a1.x), 0) +
                            s2 * __dp4a((int)q2, (int)(w ? a2.y : a2.x), 0) + s3 * __dp4a((int)q3, (int)(w ? a3.y : a3.x), 0);
            if (w) u1 = acc;
            else u0 = acc;
        }
        const uint32_t bs = __ldg(reinterpret_cast<const uint32_t *>(bsum16 + 2 * l));
        corr = 32 * ((int)(short)(bs & 0xffff) * sa + (int)(short)(bs >> 16) * sb);
        d = __fmul_rn(yd, f16_bits_to_f32((uint32_t)dh));
    }
    lane_sum = (n ? u1 : u0) + __shfl_xor_sync(0xffffffffu, n ? u0 : u1, 4) - corr;
}

// ---- Q8_0: one lane per 32-element block, f32 activations -------------------------------------
// rnb-cpu (crates/rnb-cpu/src/gemm/quant_gemv.rs:127-141): block_sum += q*x in element order,
// acc += d*block_sum in block order, multiplies and adds unfused.
__device__ __forceinline__ void q8_0_block_terms(uint32_t blk, const float *x, bool valid,
                                                 float &block_sum, float &d) {
    block_sum = 0.f;
    d = 0.f;
    if (!valid) return;
    // 34 bytes at a 2-byte-aligned address: d (f16) then 32 int8
    const uint32_t base = blk & ~3u, sh = (blk & 3u) * 8u;
    uint32_t w[10];
#pragma unroll
    for (int i = 0; i < 10; i++) w[i] = lds32(base + 4 * i);
    uint32_t b[9];
#pragma unroll
    for (int i = 0; i < 9; i++) b[i] = __funnelshift_r(w[i], w[i + 1], sh);
    d = f16_bits_to_f32(b[0] & 0xffffu);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        // quants 4i..4i+3 live in bytes 2+4i .. 5+4i: upper half of b[i], lower half of b[i+1]
        const uint32_t qw = __funnelshift_r(b[i], b[i + 1], 16);
        const float4 xv = *reinterpret_cast<const float4 *>(x + 4 * i);
        sum = __fadd_rn(sum, __fmul_rn((float)(int8_t)(qw & 0xff), xv.x));
        sum = __fadd_rn(sum, __fmul_rn((float)(int8_t)((qw >> 8) & 0xff), xv.y));
        sum = __fadd_rn(sum, __fmul_rn((float)(int8_t)((qw >> 16) & 0xff), xv.z));
        sum = __fadd_rn(sum, __fmul_rn((float)(int8_t)(qw >> 24), xv.w));
    }
    block_sum = sum;
}

// Shared memory: [part 0 tile][part 1 tile]...; each part region is part_stride bytes
// (tile bytes rounded up to 16, plus 16 bytes of slack for the unaligned readers).
// `dynamic_table`: the job table itself is written by the previous kernel (routed experts), so
// it may only be read after the dependency wait.
__device__ __forceinline__ void gemv_tile_body(const GemvJob *__restrict__ jobs, int n_jobs,
                                               int cols, uint32_t part_stride,
                                               int *__restrict__ dev_error, int dynamic_table) {
    if (dynamic_table) pdl_wait();
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ int s_mode;  // 1 = bulk copy in flight, 0 = cooperative copy needed

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = blockIdx.x;
    int j = 0;
    for (int i = 1; i < n_jobs; i++)
        if (tile >= jobs[i].tile0) j = i;
    const GemvJob *job = jobs + j;
    const int type = job->type, n_parts = job->n_parts, R = job->rows_per_tile;
    const int row0 = (tile - job->tile0) * R;
    const int nrows = min(R, job->rows - row0);
    const size_t rb = row_bytes_of(type, (size_t)cols);
    const uint32_t bytes = (uint32_t)(nrows * rb);
    if (nrows <= 0 || n_parts < 1 || n_parts > GEMV_MAX_PARTS || rb == 0 ||
        ((bytes + 15u) & ~15u) + 16u > part_stride) {
        if (tid == 0) atomicExch(dev_error, DEV_ERR_BAD_JOB);
        return;
    }

    pdl_launch_dependents();
    if (tid == 0) {
        bool aligned = (bytes & 15u) == 0;
        for (int p = 0; p < n_parts; p++)
            aligned = aligned && (((uintptr_t)(job->parts[p].w + (size_t)row0 * rb) & 15u) == 0);
        s_mode = aligned ? 1 : 0;
        mbar_init(&bar, 1);
        mbar_fence_init();
        if (aligned) {
            // weights never depend on the previous kernel: start streaming before pdl_wait
            mbar_arrive_expect_tx(&bar, bytes * (uint32_t)n_parts);
            for (int p = 0; p < n_parts; p++)
                bulk_g2s(smem + (size_t)p * part_stride, job->parts[p].w + (size_t)row0 * rb,
                         bytes, &bar);
        }
    }
    __syncthreads();
    if (s_mode == 0) {  // misaligned source or ragged tail: plain loads
        for (int p = 0; p < n_parts; p++) {
            const uint8_t *src = job->parts[p].w + (size_t)row0 * rb;
            uint8_t *dst = smem + (size_t)p * part_stride;
            for (uint32_t i = tid; i < bytes; i += GEMV_THREADS) dst[i] = src[i];
        }
        __syncthreads();
    }
    pdl_wait();  // activations / residual come from the previous kernel
    if (s_mode == 1 && !mbar_wait_bounded(&bar, 0)) {
        if (tid == 0) atomicExch(dev_error, DEV_ERR_MBAR_TIMEOUT);
        return;
    }

    const int t = lane & 7, bsub = lane >> 3;
    const int seq = job->seq < 1 ? 1 : job->seq;
    for (int rs = warp; rs < nrows * seq; rs += GEMV_THREADS / 32) {
        const int r = rs / seq, s = rs - r * seq;
        float acc = 0.0f;
        for (int p = 0; p < n_parts; p++) {
            const uint8_t *rowp = smem + (size_t)p * part_stride + (size_t)r * rb;
            const uint8_t *xbase = job->parts[p].x + (size_t)s * job->x_stride;
            float dot;
            if (type == TYPE_Q4_K) {
                const int nb = cols >> 8;
                const int8_t *qs = reinterpret_cast<const int8_t *>(xbase);
                const int16_t *bs = reinterpret_cast<const int16_t *>(xbase + cols);
                const float *xd = reinterpret_cast<const float *>(xbase + cols + 32 * nb);
                float lane_acc = 0.f, min_acc = 0.f;  // AVX lane 4h+g of acc, lane t%4 of acc_m
                for (int b0 = 0; b0 < nb; b0 += 4) {
                    const int b = b0 + bsub;
                    const bool valid = b < nb;
                    const int bc = valid ? b : b0;
                    const Q4kTerms tm = q4k_block_terms(rowp + bc * Q4K_BYTES, t, qs + bc * 256, __ldg(xd + bc), bs + bc * 16, valid);
                    const int nvalid = min(4, nb - b0);
#pragma unroll
                    for (int bb = 0; bb < 4; bb++) {
                        const int ls = __shfl_sync(0xffffffffu, tm.lane_sum, bb * 8 + t);
                        const float dd = __shfl_sync(0xffffffffu, tm.d, bb * 8 + t);
                        const int mp = __shfl_sync(0xffffffffu, tm.min_prod, bb * 8 + (t & 3));
                        const float dm = __shfl_sync(0xffffffffu, tm.dmin, bb * 8 + t);
                        if (bb < nvalid) {
                            lane_acc = __fmaf_rn(dd, (float)ls, lane_acc);
                            min_acc = __fmaf_rn(dm, (float)mp, min_acc);
                        }
                    }
                }
                // hsum_float_8: (l + l4) -> (+2) -> (+1); thread (g,h) holds lane 4h+g
                float hs = lane_acc;
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 1));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 4));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 2));
                float ms = min_acc;  // (a0+a2), (a1+a3), then their sum
                ms = __fadd_rn(ms, __shfl_xor_sync(0xffffffffu, ms, 2));
                ms = __fadd_rn(ms, __shfl_xor_sync(0xffffffffu, ms, 1));
                dot = __fadd_rn(hs, ms);
            } else if (type == TYPE_Q6_K) {
                const int nb = cols >> 8;
                const int8_t *qs = reinterpret_cast<const int8_t *>(xbase);
                const int16_t *bs = reinterpret_cast<const int16_t *>(xbase + cols);
                const float *xd = reinterpret_cast<const float *>(xbase + cols + 32 * nb);
                const uint32_t rows32 = smem_u32(rowp);
                float lane_acc = 0.f;  // AVX lane 2m+n
                for (int b0 = 0; b0 < nb; b0 += 4) {
                    const int b = b0 + bsub;
                    const bool valid = b < nb;
                    const int bc = valid ? b : b0;
                    int lsum;
                    float dmine;
                    q6k_block_terms(rows32 + bc * Q6K_BYTES, t, qs + bc * 256, __ldg(xd + bc), bs + bc * 16, valid, lsum, dmine);
                    const int nvalid = min(4, nb - b0);
#pragma unroll
                    for (int bb = 0; bb < 4; bb++) {
                        const int ls = __shfl_sync(0xffffffffu, lsum, bb * 8 + t);
                        const float dd = __shfl_sync(0xffffffffu, dmine, bb * 8 + t);
                        if (bb < nvalid) lane_acc = __fmaf_rn(dd, (float)ls, lane_acc);
                    }
                }
                // thread (n,m) holds lane 2m+n: +4 is m^2 (t^2), +2 is m^1 (t^1), +1 is n^1 (t^4)
                float hs = lane_acc;
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 2));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 1));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 4));
                dot = hs;
            } else {  // TYPE_Q8_0
                const int nb32 = cols >> 5;
                const float *xf = reinterpret_cast<const float *>(xbase);
                const uint32_t rows32 = smem_u32(rowp);
                float a = 0.f;
                for (int b0 = 0; b0 < nb32; b0 += 32) {
                    const int b = b0 + lane;
                    const bool valid = b < nb32;
                    const int bc = valid ? b : b0;
                    float bsum, dd;
                    q8_0_block_terms(rows32 + bc * Q8_0_BYTES, xf + bc * 32, valid, bsum, dd);
                    const int nvalid = min(32, nb32 - b0);
                    for (int bb = 0; bb < nvalid; bb++)  // nvalid is warp-uniform
                        a = __fadd_rn(a, __fmul_rn(__shfl_sync(0xffffffffu, dd, bb), __shfl_sync(0xffffffffu, bsum, bb)));
                }
                dot = a;
            }
            // expert_out *= route weight; out += expert_out (moe_view/fanout.rs:301-303, moe_view.rs:416-423)
            if (job->parts[p].scale) dot = __fmul_rn(dot, __ldg(job->parts[p].scale));
            acc = n_parts == 1 ? dot : __fadd_rn(acc, dot);
        }
        if (lane == 0) {
            const size_t o = (size_t)s * job->rows + row0 + r;
            job->y[o] = job->residual ? __fadd_rn(job->residual[o], acc) : acc;
        }
    }
}

// Job table in global memory (multi-matrix launches: q/k/v, gate/up, routed experts).
RNB_GLOBAL void __launch_bounds__(GEMV_THREADS)
gemv_tile_kernel(const GemvJob *__restrict__ jobs, int n_jobs, int cols, uint32_t part_stride,
                 int *__restrict__ dev_error, int dynamic_table) {
    gemv_tile_body(jobs, n_jobs, cols, part_stride, dev_error, dynamic_table);
}
// Single job passed by value in kernel-parameter space (no table upload).
RNB_GLOBAL void __launch_bounds__(GEMV_THREADS)
gemv_tile_kernel_1(const __grid_constant__ GemvJob job, int cols, uint32_t part_stride,
                   int *__restrict__ dev_error) {
    gemv_tile_body(&job, 1, cols, part_stride, dev_error, 0);
}

// LM-head epilogue: greedy argmax with the reference CPU sampler's tie rule (the LAST of equal
// maxima, crates/rnb-llm/src/sampler/greedy.rs:4-11).  Single CTA.
RNB_GLOBAL void __launch_bounds__(1024)
argmax_last_kernel(const float *__restrict__ x, int n, uint32_t *__restrict__ idx_out,
                   float *__restrict__ val_out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sv[32];
    __shared__ int si[32];
    float best = -INFINITY;
    int bi = -1;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = x[i];
        if (bi < 0 || v >= best) {  // ascending i per thread: >= keeps the last
            best = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) {
            best = ov;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 0; w < (int)(blockDim.x >> 5); w++)
            if (si[w] >= 0 && (bi < 0 || sv[w] > best || (sv[w] == best && si[w] > bi))) {
                best = sv[w];
                bi = si[w];
            }
        *idx_out = (uint32_t)bi;
        if (val_out) *val_out = best;
    }
}

// Two-stage form for long vectors (the 128k-entry logits): stage 1 leaves one (value, index)
// candidate per CTA of 1024 threads x 4 elements, stage 2 is argmax_last_pairs_kernel.
RNB_GLOBAL void __launch_bounds__(1024)
argmax_last_partial_kernel(const float *__restrict__ x, int n, float *__restrict__ vals, uint32_t *__restrict__ idxs) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sv[32];
    __shared__ int si[32];
    float best = -INFINITY;
    int bi = -1;
    const int i0 = blockIdx.x * 4096;
    for (int i = i0 + threadIdx.x; i < n && i < i0 + 4096; i += 1024) {
        const float v = x[i];
        if (bi < 0 || v >= best) {
            best = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) {
            best = ov;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 0; w < 32; w++)
            if (si[w] >= 0 && (bi < 0 || sv[w] > best || (sv[w] == best && si[w] > bi))) {
                best = sv[w];
                bi = si[w];
            }
        vals[blockIdx.x] = best;
        idxs[blockIdx.x] = (uint32_t)bi;
    }
}
// one warp: last index of the maximum among n (value, index) candidates
RNB_GLOBAL void __launch_bounds__(32)
argmax_last_pairs_kernel(const float *__restrict__ vals, const uint32_t *__restrict__ idxs, int n, uint32_t *__restrict__ idx_out,
                         float *__restrict__ val_out) {
    pdl_launch_dependents();
    pdl_wait();
    float best = -INFINITY;
    long long bi = -1;
    for (int i = threadIdx.x; i < n; i += 32) {
        const float v = vals[i];
        const long long id = idxs[i];
        if (bi < 0 || v > best || (v == best && id > bi)) {
            best = v;
            bi = id;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) {
            best = ov;
            bi = oi;
        }
    }
    if (threadIdx.x == 0) {
        *idx_out = (uint32_t)bi;
        if (val_out) *val_out = best;
    }
}

}  // namespace rnb
