// Batch-1 matvec, streaming form: the kernel the decode path uses for Q4_K and Q6_K.
//
// Bit-exactness with rnb-cpu's AVX2 dots needs, per row, one f32 FMA per block IN BLOCK ORDER
// on each of eight accumulator lanes (see gemv.cuh).  Only that last step is sequential; the
// integer lane sums in front of it are exact in any order.  So every pipeline stage runs in two
// phases:
//   phase 1  all 128 threads: 8 threads per (row, block) item unpack nibbles/scales, dp4a
//            against the Q8_K activation, and leave the block's 8 integer lane sums (+4 for
//            the Q4_K mins term) and its two f32 scales in shared memory;
//   phase 2  one thread per (row, accumulator lane) replays the FMAs over the stage's blocks
//            in order, carrying its accumulator across stages.
// A CTA owns R rows (2, 4 or 8).  Rows are cut along K into chunks of up to 8 super-blocks;
// one chunk of every row plus the matching slice of the activation is a pipeline stage,
// fetched by the bulk-async copy engine onto the stage's mbarrier while earlier stages are
// consumed.  Several CTAs per SM keep a few hundred KB of weights in flight.
#pragma once
#include "gemv.cuh"

namespace rnb {

constexpr int GS_MAX_STAGES = 8;
constexpr int GS_THREADS = 128;
constexpr int GS_MAX_ROWS = 8;
constexpr int GS_MAX_CHUNK = 8;

struct GsParams {
    int cols;
    int rows_per_cta;     // 2, 4 or 8
    int chunk_blocks;     // super-blocks (256 elements) per stage, <= GS_MAX_CHUNK
    int n_stages;         // 1..GS_MAX_STAGES
    uint32_t row_stride;  // bytes of shared memory per weight row per stage (16-byte multiple)
    uint32_t act_off;     // offset of the activation slice inside a stage
    uint32_t slot_bytes;  // bytes per stage
    int dynamic_table;
};

// unsigned bytes x signed bytes
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// 8 bytes at any 2-byte aligned shared-memory address (Q6_K blocks are 210 bytes long)
__device__ __forceinline__ uint2 smem_load8_unaligned(const uint8_t *p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t *w = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
    const uint32_t sh = (uint32_t)(a & 3) * 8u;
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
    return make_uint2(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh));
}

// Q4_K item: thread t of the group owns qs bytes 16t..16t+15 (64-element group g = t/2, half
// h = t%2 -> accumulator lanes 4h..4h+3 of sub-blocks 2g / 2g+1); after the reduce-scatter it
// holds lane 4h+g.  Lane k = t%4 of the mins accumulator is mn[2k]*bsum32[2k] + mn[2k+1]*bsum32[2k+1].
__device__ __forceinline__ void gs_q4k_item(const uint8_t *blk, const uint8_t *act, const int16_t *bs16, float yd,
                                            int t, bool valid, int *s_int, int *s_min, float *s_d, float *s_dm) {
    int v0 = 0, v1 = 0, v2 = 0, v3 = 0, min_prod = 0;
    float d = 0.f, dmin = 0.f;
    const int g = t >> 1, h = t & 1;
    if (valid) {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
        const uint4 q = *reinterpret_cast<const uint4 *>(blk + 16 + 16 * t);
        const uint4 alo = *reinterpret_cast<const uint4 *>(act + 64 * g + 16 * h);
        const uint4 ahi = *reinterpret_cast<const uint4 *>(act + 64 * g + 32 + 16 * h);
        const uint32_t sc03 = hdr.y & 0x3f3f3f3fu;
        const uint32_t mn03 = hdr.z & 0x3f3f3f3fu;
        const uint32_t sc47 = (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
        const uint32_t mn47 = ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
        const uint32_t scw = g < 2 ? sc03 : sc47;
        // high nibbles stay in place (x16): scale the low side by 16 too and shift once at the end
        const int sc_lo16 = (int)((scw >> (16 * (g & 1))) & 0xff) << 4;
        const int sc_hi = (int)((scw >> (16 * (g & 1) + 8)) & 0xff);
        v0 = sc_lo16 * __dp4a((int)(q.x & 0x0f0f0f0fu), (int)alo.x, 0) + sc_hi * dp4a_us(q.x & 0xf0f0f0f0u, ahi.x, 0);
        v1 = sc_lo16 * __dp4a((int)(q.y & 0x0f0f0f0fu), (int)alo.y, 0) + sc_hi * dp4a_us(q.y & 0xf0f0f0f0u, ahi.y, 0);
        v2 = sc_lo16 * __dp4a((int)(q.z & 0x0f0f0f0fu), (int)alo.z, 0) + sc_hi * dp4a_us(q.z & 0xf0f0f0f0u, ahi.z, 0);
        v3 = sc_lo16 * __dp4a((int)(q.w & 0x0f0f0f0fu), (int)alo.w, 0) + sc_hi * dp4a_us(q.w & 0xf0f0f0f0u, ahi.w, 0);
        const int k = t & 3;
        const uint32_t mnw = k < 2 ? mn03 : mn47;
        const int mn_a = (mnw >> (16 * (k & 1))) & 0xff, mn_b = (mnw >> (16 * (k & 1) + 8)) & 0xff;
        const uint2 bs = *reinterpret_cast<const uint2 *>(bs16 + 4 * k);
        const int b32a = (short)((short)(bs.x & 0xffff) + (short)(bs.x >> 16));
        const int b32b = (short)((short)(bs.y & 0xffff) + (short)(bs.y >> 16));
        min_prod = mn_a * b32a + mn_b * b32b;
        d = __fmul_rn(yd, f16_bits_to_f32(hdr.x & 0xffffu));
        dmin = __fmul_rn(-yd, f16_bits_to_f32(hdr.x >> 16));
    }
    const int g0 = g & 1, g1 = g >> 1;
    const int a0 = (g0 ? v1 : v0) + __shfl_xor_sync(0xffffffffu, g0 ? v0 : v1, 2);
    const int a1 = (g0 ? v3 : v2) + __shfl_xor_sync(0xffffffffu, g0 ? v2 : v3, 2);
    const int lane_sum = ((g1 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, g1 ? a0 : a1, 4)) >> 4;  // exact: a multiple of 16
    if (valid) {
        s_int[4 * h + g] = lane_sum;
        if (t < 4) s_min[t] = min_prod;
        if (t == 0) {
            *s_d = d;
            *s_dm = dmin;
        }
    }
}

// Q6_K item: thread t = (n = t/4, m = t%4) owns l = 8m..8m+7 of half n in each 32-element
// part, i.e. accumulator lanes 2m and 2m+1; after the exchange with the other half it holds
// lane 2m+n, from which the reference subtracts 32*(bsums[2l]*sc[2l] + bsums[2l+1]*sc[2l+1]).
__device__ __forceinline__ void gs_q6k_item(const uint8_t *blk, const uint8_t *act, const int16_t *bs16, float yd,
                                            int t, bool valid, int *s_int, float *s_d) {
    const int n = t >> 2, m = t & 3, l = 2 * m + n;
    int u0 = 0, u1 = 0, corr = 0;
    float d = 0.f;
    if (valid) {
        const uint2 qla = smem_load8_unaligned(blk + 64 * n + 8 * m);
        const uint2 qlb = smem_load8_unaligned(blk + 64 * n + 32 + 8 * m);
        const uint2 qh = smem_load8_unaligned(blk + 128 + 32 * n + 8 * m);
        const uint8_t *xa = act + 128 * n + 8 * m;
        const uint2 a0 = *reinterpret_cast<const uint2 *>(xa), a1 = *reinterpret_cast<const uint2 *>(xa + 32),
                    a2 = *reinterpret_cast<const uint2 *>(xa + 64), a3 = *reinterpret_cast<const uint2 *>(xa + 96);
        const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192);
        const int s0 = sc[8 * n + (m >> 1)], s1 = sc[8 * n + (m >> 1) + 2], s2 = sc[8 * n + (m >> 1) + 4],
                  s3 = sc[8 * n + (m >> 1) + 6];
        const int sa = sc[2 * l], sb = sc[2 * l + 1];
        const uint32_t dh = *reinterpret_cast<const uint16_t *>(blk + 208);
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
        const uint32_t bs = *reinterpret_cast<const uint32_t *>(bs16 + 2 * l);
        corr = 32 * ((int)(short)(bs & 0xffff) * sa + (int)(short)(bs >> 16) * sb);
        d = __fmul_rn(yd, f16_bits_to_f32(dh));
    }
    const int lane_sum = (n ? u1 : u0) + __shfl_xor_sync(0xffffffffu, n ? u0 : u1, 4) - corr;
    if (valid) {
        s_int[l] = lane_sum;
        if (t == 0) *s_d = d;
    }
}

__device__ __forceinline__ void gemv_stream_body(const GemvJob *__restrict__ jobs, int n_jobs,
                                                 const GsParams P, int *__restrict__ dev_error) {
    if (P.dynamic_table) pdl_wait();
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[GS_MAX_STAGES];
    // phase-1 results, double-buffered by stage parity: [buf][row][block][lane]
    __shared__ int s_int[2][GS_MAX_ROWS][GS_MAX_CHUNK][8];
    __shared__ int s_min[2][GS_MAX_ROWS][GS_MAX_CHUNK][4];
    __shared__ float s_d[2][GS_MAX_ROWS][GS_MAX_CHUNK], s_dm[2][GS_MAX_ROWS][GS_MAX_CHUNK];
    __shared__ float s_ms[GS_MAX_ROWS];

    const int tid = threadIdx.x;
    const int R = P.rows_per_cta;
    const int tile = blockIdx.x;
    int jsel = 0;
    for (int i = 1; i < n_jobs; i++)
        if (tile >= jobs[i].tile0) jsel = i;
    const GemvJob *job = jobs + jsel;
    const int type = job->type, n_parts = job->n_parts;
    const int row0 = (tile - job->tile0) * R;
    const int nrows = min(R, job->rows - row0);
    const int cols = P.cols, nb = cols >> 8, CB = P.chunk_blocks, S = P.n_stages;
    const uint32_t blk_bytes = type == TYPE_Q4_K ? Q4K_BYTES : Q6K_BYTES;
    const size_t rb = (size_t)nb * blk_bytes;
    const int n_chunks = (nb + CB - 1) / CB;
    const int n_items = n_parts * n_chunks;
    if (nrows <= 0 || n_parts < 1 || n_parts > GEMV_MAX_PARTS || nb < 1 || S < 1 || S > GS_MAX_STAGES || CB < 1 ||
        CB > GS_MAX_CHUNK || R < 1 || R > GS_MAX_ROWS || (type != TYPE_Q4_K && type != TYPE_Q6_K) ||
        (uint32_t)CB * blk_bytes + 16u > P.row_stride || (P.row_stride & 15u) || (P.act_off & 15u) ||
        (uint32_t)R * P.row_stride > P.act_off || P.act_off + (uint32_t)CB * 288u > P.slot_bytes ||
        job->rows_per_tile != R || blockDim.x != GS_THREADS) {
        if (tid == 0) atomicExch(dev_error, DEV_ERR_BAD_JOB);
        return;
    }

    pdl_launch_dependents();
    // bulk copies need 16-byte aligned sources and sizes: whole-row alignment decides
    bool tma = (rb & 15u) == 0;
    for (int p = 0; p < n_parts; p++)
        tma = tma && (((uintptr_t)job->parts[p].w & 15u) == 0) && (((uintptr_t)job->parts[p].x & 15u) == 0);
    if (type == TYPE_Q6_K) tma = tma && (CB % 8 == 0);

    // stage = R weight-row chunks + the activation's qs and bsum16 slices for the same blocks
    auto issue_weights = [&](int item) {  // thread 0 only
        const int p = item / n_chunks, c = item - p * n_chunks;
        const int nblk = min(CB, nb - c * CB);
        const uint32_t bytes = (uint32_t)nblk * blk_bytes;
        uint64_t *bar = &full[item % S];
        uint8_t *dst = smem + (size_t)(item % S) * P.slot_bytes;
        const uint8_t *src = job->parts[p].w + (size_t)row0 * rb + (size_t)c * CB * blk_bytes;
        mbar_arrive_expect_tx(bar, bytes * (uint32_t)nrows + (uint32_t)nblk * 288u);
        for (int r = 0; r < nrows; r++) bulk_g2s(dst + (size_t)r * P.row_stride, src + (size_t)r * rb, bytes, bar);
    };
    auto issue_act = [&](int item) {  // thread 0 only, after the dependency wait
        const int p = item / n_chunks, c = item - p * n_chunks;
        const int nblk = min(CB, nb - c * CB);
        uint64_t *bar = &full[item % S];
        uint8_t *dst = smem + (size_t)(item % S) * P.slot_bytes + P.act_off;
        const uint8_t *x = job->parts[p].x;
        bulk_g2s(dst, x + (size_t)c * CB * 256, (uint32_t)nblk * 256u, bar);
        bulk_g2s(dst + CB * 256, x + cols + (size_t)c * CB * 32, (uint32_t)nblk * 32u, bar);
    };

    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(&full[s], 1);
        mbar_fence_init();
        if (tma)  // weights never depend on the previous kernel: start streaming before pdl_wait
            for (int i = 0; i < S && i < n_items; i++) issue_weights(i);
    }
    __syncthreads();
    pdl_wait();  // activations, residual and route weights come from earlier kernels
    if (tma && tid == 0)
        for (int i = 0; i < S && i < n_items; i++) issue_act(i);

    const int t = tid & 7, grp = tid >> 3;  // 16 groups of 8 threads
    // phase-2 roles: threads 0..8R-1 own (row, accumulator lane); threads 64..64+4R-1 own (row, mins lane)
    const bool lane_owner = tid < 8 * R;
    const bool min_owner = type == TYPE_Q4_K && tid >= 64 && tid < 64 + 4 * R;
    const int o_row = lane_owner ? (tid >> 3) : ((tid - 64) >> 2);
    const int o_lane = lane_owner ? (tid & 7) : ((tid - 64) & 3);
    float chain = 0.f, acc_total = 0.f;

    for (int item = 0; item < n_items; item++) {
        const int p = item / n_chunks, c = item - p * n_chunks;
        const int nblk = min(CB, nb - c * CB);
        const int buf = item & 1;
        uint8_t *slot = smem + (size_t)(item % S) * P.slot_bytes;
        if (tma) {
            if (!mbar_wait_bounded(&full[item % S], (uint32_t)((item / S) & 1))) {
                // Give the copies still in flight a bounded chance to land before the shared
                // memory is released, flag the error and leave (every thread takes this path).
                for (int k = item + 1; k < n_items && k < item + S; k++) mbar_wait_bounded(&full[k % S], (uint32_t)((k / S) & 1));
                if (tid == 0) atomicExch(dev_error, DEV_ERR_MBAR_TIMEOUT);
                return;
            }
        } else {  // misaligned rows: stage the same bytes with plain loads
            const uint32_t bytes = (uint32_t)nblk * blk_bytes;
            const uint8_t *src = job->parts[p].w + (size_t)row0 * rb + (size_t)c * CB * blk_bytes;
            for (int q = 0; q < nrows; q++)
                for (uint32_t i = tid; i < bytes; i += GS_THREADS) slot[(size_t)q * P.row_stride + i] = src[(size_t)q * rb + i];
            const uint8_t *x = job->parts[p].x;
            for (uint32_t i = tid; i < (uint32_t)nblk * 256u; i += GS_THREADS) slot[P.act_off + i] = x[(size_t)c * CB * 256 + i];
            for (uint32_t i = tid; i < (uint32_t)nblk * 32u; i += GS_THREADS) slot[P.act_off + CB * 256 + i] = x[cols + (size_t)c * CB * 32 + i];
            __syncthreads();
        }
        // ---- phase 1: integer lane sums of every (row, block) of the stage ----
        const float *xd = reinterpret_cast<const float *>(job->parts[p].x + cols + 32 * nb) + c * CB;
        const uint8_t *act = slot + P.act_off;
        const int16_t *bs16 = reinterpret_cast<const int16_t *>(slot + P.act_off + CB * 256);
        const int n_work = R * nblk;
#pragma unroll 2
        for (int w0 = 0; w0 < n_work; w0 += GS_THREADS / 8) {
            const int wi = w0 + grp;
            const int r = wi / nblk, j = wi - r * nblk;
            const bool valid = wi < n_work && r < nrows;
            const int rc = valid ? r : 0, jc = valid ? j : 0;
            const uint8_t *blk = slot + (size_t)rc * P.row_stride + (size_t)jc * blk_bytes;
            const float yd = valid ? __ldg(xd + jc) : 0.f;
            if (type == TYPE_Q4_K)
                gs_q4k_item(blk, act + jc * 256, bs16 + jc * 16, yd, t, valid, s_int[buf][rc][jc], s_min[buf][rc][jc], &s_d[buf][rc][jc], &s_dm[buf][rc][jc]);
            else
                gs_q6k_item(blk, act + jc * 256, bs16 + jc * 16, yd, t, valid, s_int[buf][rc][jc], &s_d[buf][rc][jc]);
        }
        __syncthreads();  // stage consumed, phase-1 results visible
        if (tma && tid == 0 && item + S < n_items) {
            issue_weights(item + S);
            issue_act(item + S);
        }
        // ---- phase 2: the sequential part, one FMA per block in block order ----
        if (lane_owner && o_row < nrows) {
#pragma unroll 4
            for (int j = 0; j < nblk; j++) chain = __fmaf_rn(s_d[buf][o_row][j], (float)s_int[buf][o_row][j][o_lane], chain);
        } else if (min_owner && o_row < nrows) {
#pragma unroll 4
            for (int j = 0; j < nblk; j++) chain = __fmaf_rn(s_dm[buf][o_row][j], (float)s_min[buf][o_row][j][o_lane], chain);
        }
        if (c == n_chunks - 1) {  // rows finished for this part: fold the accumulator lanes
            // hsum_float_8: (l + l4) -> (+2) -> (+1); mins: (a0 + a2) + (a1 + a3).  Both orders are
            // xor 4, 2, 1 over the owner's lane index (the mins lanes simply have no bit 2).
            float f = chain;
            if (tid < 64 + 32) {  // whole warps of owners take the shuffles
                const float o4 = __shfl_xor_sync(0xffffffffu, f, 4);
                if (lane_owner) f = __fadd_rn(f, o4);
                f = __fadd_rn(f, __shfl_xor_sync(0xffffffffu, f, 2));
                f = __fadd_rn(f, __shfl_xor_sync(0xffffffffu, f, 1));
            }
            if (min_owner && o_lane == 0) s_ms[o_row] = f;
            __syncthreads();
            if (lane_owner && o_lane == 0 && o_row < nrows) {
                float dot = type == TYPE_Q4_K ? __fadd_rn(f, s_ms[o_row]) : f;
                // expert_out *= route weight; out += expert_out, experts in selection order
                if (job->parts[p].scale) dot = __fmul_rn(dot, __ldg(job->parts[p].scale));
                acc_total = n_parts == 1 ? dot : __fadd_rn(acc_total, dot);
            }
            chain = 0.f;
            __syncthreads();  // s_ms is reused by the next part
        }
    }
    if (lane_owner && o_lane == 0 && o_row < nrows) {
        const size_t o = (size_t)row0 + o_row;
        job->y[o] = job->residual ? __fadd_rn(job->residual[o], acc_total) : acc_total;
    }
}

RNB_GLOBAL void __launch_bounds__(GS_THREADS)
gemv_stream_kernel(const GemvJob *__restrict__ jobs, int n_jobs, const GsParams P, int *__restrict__ dev_error) {
    gemv_stream_body(jobs, n_jobs, P, dev_error);
}
RNB_GLOBAL void __launch_bounds__(GS_THREADS)
gemv_stream_kernel_1(const __grid_constant__ GemvJob job, const GsParams P, int *__restrict__ dev_error) {
    gemv_stream_body(&job, 1, P, dev_error);
}

}  // namespace rnb
