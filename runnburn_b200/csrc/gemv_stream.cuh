// Batch-1 matvec, streaming form: the kernel the decode path uses for Q4_K and Q6_K.
//
// Bit-exactness with rnb-cpu's AVX2 dots needs, per row, one f32 FMA per block IN BLOCK ORDER
// on each of eight accumulator lanes (see gemv.cuh for the lane algebra).  Eight threads own
// one weight row for its whole length: per block they unpack nibbles and scales, dp4a against
// the Q8_K activation, reduce-scatter the integer partial sums (exact in any order) until
// each thread holds ONE accumulator lane, and issue that lane's FMA - so the ordered chain
// lives in registers and needs no hand-off.  A warp is four rows, a CTA is 1, 2 or 4 warps.
// Rows are cut along K into chunks of up to 8 super-blocks; one chunk of every row of the CTA
// plus the matching slice of the activation is a pipeline stage, fetched by the bulk-async
// copy engine onto the stage's mbarrier while the previous stage is consumed.  Many small
// CTAs per SM keep a few hundred KB of weights in flight.
#pragma once
#include "gemv.cuh"

namespace rnb {

constexpr int GS_MAX_STAGES = 8;
constexpr int GS_MAX_CHUNK = 8;                          // blocks per stage; also the slot pitch

struct GsParams {
    int cols;
    int rows_per_cta;     // 4, 8 or 16 (blockDim.x = 8 * rows)
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

// 8 bytes of a Q6_K block in shared memory.  Blocks are 210 bytes long, so inside a 16-byte
// aligned row even blocks start 4-byte aligned (MIS = 0: two word loads) and odd blocks 2 bytes
// past a word boundary (MIS = 2: three word loads and two funnel shifts).
template <int MIS>
__device__ __forceinline__ uint2 smem_load8(const uint8_t *p) {
    const uint32_t *w = reinterpret_cast<const uint32_t *>(p - MIS);
    if (MIS == 0) return make_uint2(w[0], w[1]);
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
    return make_uint2(__funnelshift_r(w0, w1, 16), __funnelshift_r(w1, w2, 16));
}

// ---- Q6_K: thread t = (n = t/4, m = t%4) owns l = 8m..8m+7 of half n in each
// 32-element part, i.e. accumulator lanes 2m and 2m+1; after the exchange with the other half it
// holds lane 2m+n, from which the reference subtracts 32*(bsums[2l]*sc[2l] + bsums[2l+1]*sc[2l+1]).
template <int MIS>
__device__ __forceinline__ int gs_q6k_lanes(const uint8_t *blk, const uint8_t *act, const int16_t *bs16, float yd, int t,
                                            bool valid, float2 *dd) {
    const int n = t >> 2, m = t & 3, l = 2 * m + n;
    int u0 = 0, u1 = 0, corr = 0;
    if (valid) {
        const uint2 qla = smem_load8<MIS>(blk + 64 * n + 8 * m);
        const uint2 qlb = smem_load8<MIS>(blk + 64 * n + 32 + 8 * m);
        const uint2 qh = smem_load8<MIS>(blk + 128 + 32 * n + 8 * m);
        const uint8_t *xa = act + 128 * n + 8 * m;
        const uint2 a0 = *reinterpret_cast<const uint2 *>(xa), a1 = *reinterpret_cast<const uint2 *>(xa + 32),
                    a2 = *reinterpret_cast<const uint2 *>(xa + 64), a3 = *reinterpret_cast<const uint2 *>(xa + 96);
        const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192);
        const int s0 = sc[8 * n + (m >> 1)], s1 = sc[8 * n + (m >> 1) + 2], s2 = sc[8 * n + (m >> 1) + 4],
                  s3 = sc[8 * n + (m >> 1) + 6];
        const int sa = sc[2 * l], sb = sc[2 * l + 1];
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
        if (t == 0) {
            const uint32_t dh = *reinterpret_cast<const uint16_t *>(blk + 208);
            *dd = make_float2(__fmul_rn(yd, f16_bits_to_f32(dh)), 0.f);
        }
    }
    return (n ? u1 : u0) + __shfl_xor_sync(0xffffffffu, n ? u0 : u1, 4) - corr;
}

struct Q4kStep {
    int lane_sum, min_prod;
    float d, dmin;
};
// Thread t of the group owns qs bytes 16t..16t+15 (64-element group g = t/2, half h = t%2 ->
// accumulator lanes 4h..4h+3 of sub-blocks 2g / 2g+1); after the reduce-scatter it holds lane
// 4h+g.  High nibbles stay in place (x16) and the low scale is pre-multiplied by 16, so one
// exact shift at the end replaces four.  Lane k = t%4 of the mins accumulator is
// mn[2k]*bsum32[2k] + mn[2k+1]*bsum32[2k+1].
__device__ __forceinline__ Q4kStep gr_q4k_step(const uint8_t *blk, const uint8_t *act, const int16_t *bs16, float yd, int t) {
    const int g = t >> 1, h = t & 1, k = t & 3;
    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
    const uint4 q = *reinterpret_cast<const uint4 *>(blk + 16 + 16 * t);
    const uint4 alo = *reinterpret_cast<const uint4 *>(act + 64 * g + 16 * h);
    const uint4 ahi = *reinterpret_cast<const uint4 *>(act + 64 * g + 32 + 16 * h);
    const uint2 bs = *reinterpret_cast<const uint2 *>(bs16 + 4 * k);
    const uint32_t sc03 = hdr.y & 0x3f3f3f3fu, mn03 = hdr.z & 0x3f3f3f3fu;
    const uint32_t sc47 = (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
    const uint32_t mn47 = ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
    const uint32_t scw = g < 2 ? sc03 : sc47, mnw = k < 2 ? mn03 : mn47;
    const int sc_lo16 = (int)((scw >> (16 * (g & 1))) & 0xff) << 4, sc_hi = (int)((scw >> (16 * (g & 1) + 8)) & 0xff);
    const int mn_a = (mnw >> (16 * (k & 1))) & 0xff, mn_b = (mnw >> (16 * (k & 1) + 8)) & 0xff;
    const int v0 = sc_lo16 * __dp4a((int)(q.x & 0x0f0f0f0fu), (int)alo.x, 0) + sc_hi * dp4a_us(q.x & 0xf0f0f0f0u, ahi.x, 0);
    const int v1 = sc_lo16 * __dp4a((int)(q.y & 0x0f0f0f0fu), (int)alo.y, 0) + sc_hi * dp4a_us(q.y & 0xf0f0f0f0u, ahi.y, 0);
    const int v2 = sc_lo16 * __dp4a((int)(q.z & 0x0f0f0f0fu), (int)alo.z, 0) + sc_hi * dp4a_us(q.z & 0xf0f0f0f0u, ahi.z, 0);
    const int v3 = sc_lo16 * __dp4a((int)(q.w & 0x0f0f0f0fu), (int)alo.w, 0) + sc_hi * dp4a_us(q.w & 0xf0f0f0f0u, ahi.w, 0);
    const int b32a = (short)((short)(bs.x & 0xffff) + (short)(bs.x >> 16));
    const int b32b = (short)((short)(bs.y & 0xffff) + (short)(bs.y >> 16));
    Q4kStep r;
    r.min_prod = mn_a * b32a + mn_b * b32b;
    r.d = __fmul_rn(yd, f16_bits_to_f32(hdr.x & 0xffffu));
    r.dmin = __fmul_rn(-yd, f16_bits_to_f32(hdr.x >> 16));
    const int g0 = g & 1, g1 = g >> 1;
    const int a0 = (g0 ? v1 : v0) + __shfl_xor_sync(0xffffffffu, g0 ? v0 : v1, 2);
    const int a1 = (g0 ? v3 : v2) + __shfl_xor_sync(0xffffffffu, g0 ? v2 : v3, 2);
    r.lane_sum = ((g1 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, g1 ? a0 : a1, 4)) >> 4;
    return r;
}

template <int TYPE>
__device__ __forceinline__ void gr_run(const GemvJob *__restrict__ job, const GsParams &P, const int row0, const int nrows,
                                       uint8_t *smem, uint64_t *full, int *__restrict__ dev_error) {
    constexpr uint32_t BLK = TYPE == TYPE_Q4_K ? Q4K_BYTES : Q6K_BYTES;
    const int tid = threadIdx.x, lane = tid & 31;
    const int R = P.rows_per_cta, cols = P.cols, nb = cols >> 8, CB = P.chunk_blocks, S = P.n_stages, n_parts = job->n_parts;
    const uint32_t row_stride = P.row_stride, act_off = P.act_off, slot_bytes = P.slot_bytes;
    const uint32_t rb = (uint32_t)nb * BLK;
    const int n_chunks = (nb + CB - 1) / CB;
    const int n_items = n_parts * n_chunks;
    bool tma = (rb & 15u) == 0;
    for (int p = 0; p < n_parts; p++)
        tma = tma && (((uintptr_t)job->parts[p].w & 15u) == 0) && (((uintptr_t)job->parts[p].x & 15u) == 0);
    if (TYPE == TYPE_Q6_K) tma = tma && (CB % 8 == 0);
    auto issue = [&](int p, int c, int slot_idx, bool weights, bool act) {  // thread 0 only
        const int nblk = min(CB, nb - c * CB);
        const uint32_t bytes = (uint32_t)nblk * BLK;
        uint64_t *bar = &full[slot_idx];
        uint8_t *dst = smem + (uint32_t)slot_idx * slot_bytes;
        if (weights) {
            const uint8_t *src = job->parts[p].w + (size_t)row0 * rb + (uint32_t)(c * CB) * BLK;
            mbar_arrive_expect_tx(bar, bytes * (uint32_t)nrows + (uint32_t)nblk * 288u);
            for (int r = 0; r < nrows; r++) bulk_g2s(dst + (uint32_t)r * row_stride, src + (size_t)r * rb, bytes, bar);
        }
        if (act) {
            const uint8_t *x = job->parts[p].x;
            bulk_g2s(dst + act_off, x + (uint32_t)(c * CB) * 256u, (uint32_t)nblk * 256u, bar);
            bulk_g2s(dst + act_off + CB * 256, x + cols + (uint32_t)(c * CB) * 32u, (uint32_t)nblk * 32u, bar);
        }
    };
    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(&full[s], 1);
        mbar_fence_init();
        if (tma) {
            int p = 0, c = 0;
            for (int i = 0; i < S && i < n_items; i++) {
                issue(p, c, i, true, false);
                if (++c == n_chunks) c = 0, ++p;
            }
        }
    }
    __syncthreads();
    pdl_wait();
    if (tma && tid == 0) {
        int p = 0, c = 0;
        for (int i = 0; i < S && i < n_items; i++) {
            issue(p, c, i, false, true);
            if (++c == n_chunks) c = 0, ++p;
        }
    }
    const int t = lane & 7;
    const int r = tid >> 3;  // this group's row within the CTA
    const bool live = r < nrows;
    const uint32_t row_off = (uint32_t)(live ? r : 0) * row_stride;
    float lane_acc = 0.f, min_acc = 0.f, acc_total = 0.f;
    int p = 0, c = 0, slot_idx = 0, parity = 0, pn = 0, cn = 0;
    for (int i = 0; i < S; i++)
        if (++cn == n_chunks) cn = 0, ++pn;
    for (int item = 0; item < n_items; item++) {
        const int nblk = min(CB, nb - c * CB);
        uint8_t *slot = smem + (uint32_t)slot_idx * slot_bytes;
        if (tma) {
            if (!mbar_wait_bounded(&full[slot_idx], (uint32_t)parity)) {
                for (int k = item + 1; k < n_items && k < item + S; k++) mbar_wait_bounded(&full[k % S], (uint32_t)((k / S) & 1));
                if (tid == 0) atomicExch(dev_error, DEV_ERR_MBAR_TIMEOUT);
                return;
            }
        } else {
            const uint32_t bytes = (uint32_t)nblk * BLK;
            const uint8_t *src = job->parts[p].w + (size_t)row0 * rb + (uint32_t)(c * CB) * BLK;
            for (int q = 0; q < nrows; q++)
                for (uint32_t k = tid; k < bytes; k += blockDim.x) slot[(uint32_t)q * row_stride + k] = src[(size_t)q * rb + k];
            const uint8_t *x = job->parts[p].x;
            for (uint32_t k = tid; k < (uint32_t)nblk * 256u; k += blockDim.x) slot[act_off + k] = x[(uint32_t)(c * CB) * 256u + k];
            for (uint32_t k = tid; k < (uint32_t)nblk * 32u; k += blockDim.x) slot[act_off + CB * 256 + k] = x[cols + (uint32_t)(c * CB) * 32u + k];
            __syncthreads();
        }
        const float *xd = reinterpret_cast<const float *>(job->parts[p].x + cols + 32 * nb) + c * CB;
        const uint8_t *rowp = slot + row_off;
        const uint8_t *act = slot + act_off;
        const int16_t *bs16 = reinterpret_cast<const int16_t *>(slot + act_off + CB * 256);
        // every thread of a warp runs the same trip count; dead groups (rows past the end) read
        // row 0 and simply do not store
        if (TYPE == TYPE_Q4_K) {
            if (nblk == GS_MAX_CHUNK) {
#pragma unroll
                for (int j = 0; j < GS_MAX_CHUNK; j++) {
                    const Q4kStep st = gr_q4k_step(rowp + j * Q4K_BYTES, act + j * 256, bs16 + j * 16, __ldg(xd + j), t);
                    lane_acc = __fmaf_rn(st.d, (float)st.lane_sum, lane_acc);
                    min_acc = __fmaf_rn(st.dmin, (float)st.min_prod, min_acc);
                }
            } else {
                for (int j = 0; j < nblk; j++) {
                    const Q4kStep st = gr_q4k_step(rowp + j * Q4K_BYTES, act + j * 256, bs16 + j * 16, __ldg(xd + j), t);
                    lane_acc = __fmaf_rn(st.d, (float)st.lane_sum, lane_acc);
                    min_acc = __fmaf_rn(st.dmin, (float)st.min_prod, min_acc);
                }
            }
        } else {
            float2 dd;
            // even blocks sit 4-byte aligned in the row, odd blocks 2 bytes off: two code shapes
#pragma unroll 2
            for (int j = 0; j + 1 < nblk; j += 2) {
                const uint8_t *b0 = rowp + j * Q6K_BYTES, *b1 = b0 + Q6K_BYTES;
                const uint32_t dh0 = *reinterpret_cast<const uint16_t *>(b0 + 208), dh1 = *reinterpret_cast<const uint16_t *>(b1 + 208);
                const int ls0 = gs_q6k_lanes<0>(b0, act + j * 256, bs16 + j * 16, 0.f, t, true, &dd);
                const int ls1 = gs_q6k_lanes<2>(b1, act + (j + 1) * 256, bs16 + (j + 1) * 16, 0.f, t, true, &dd);
                lane_acc = __fmaf_rn(__fmul_rn(__ldg(xd + j), f16_bits_to_f32(dh0)), (float)ls0, lane_acc);
                lane_acc = __fmaf_rn(__fmul_rn(__ldg(xd + j + 1), f16_bits_to_f32(dh1)), (float)ls1, lane_acc);
            }
            if (nblk & 1) {
                const int j = nblk - 1;
                const uint8_t *b0 = rowp + j * Q6K_BYTES;
                const uint32_t dh0 = *reinterpret_cast<const uint16_t *>(b0 + 208);
                const int ls0 = gs_q6k_lanes<0>(b0, act + j * 256, bs16 + j * 16, 0.f, t, true, &dd);
                lane_acc = __fmaf_rn(__fmul_rn(__ldg(xd + j), f16_bits_to_f32(dh0)), (float)ls0, lane_acc);
            }
        }
        __syncthreads();  // slot consumed by every group
        if (tma && tid == 0 && item + S < n_items) issue(pn, cn, slot_idx, true, true);
        if (c == n_chunks - 1) {
            float dot;
            if (TYPE == TYPE_Q4_K) {
                float hs = lane_acc;  // thread (g,h) holds lane 4h+g: (l + l4) -> (+2) -> (+1)
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 1));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 4));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 2));
                float ms = min_acc;  // lane t%4: (a0 + a2) + (a1 + a3)
                ms = __fadd_rn(ms, __shfl_xor_sync(0xffffffffu, ms, 2));
                ms = __fadd_rn(ms, __shfl_xor_sync(0xffffffffu, ms, 1));
                dot = __fadd_rn(hs, ms);
            } else {
                float hs = lane_acc;  // thread (n,m) holds lane 2m+n: +4 is t^2, +2 is t^1, +1 is t^4
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 2));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 1));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 4));
                dot = hs;
            }
            if (job->parts[p].scale) dot = __fmul_rn(dot, __ldg(job->parts[p].scale));
            acc_total = n_parts == 1 ? dot : __fadd_rn(acc_total, dot);
            lane_acc = 0.f;
            min_acc = 0.f;
        }
        if (++c == n_chunks) c = 0, ++p;
        if (++cn == n_chunks) cn = 0, ++pn;
        if (++slot_idx == S) slot_idx = 0, parity ^= 1;
    }
    const size_t o = (size_t)row0 + r;
    float val = acc_total;
    if (live && t == 0 && job->residual) val = __fadd_rn(job->residual[o], acc_total);
    const int epi = job->epi;
    if (epi == GEMV_EPI_NONE) {
        if (live && t == 0) job->y[o] = val;
        return;
    }
    // q/k/v epilogue: what rope_kv_append_kernel does, on the rows this CTA has just produced.
    // Rows 2i and 2i+1 of a head are a rotation pair (adjacent-pair RoPE); they sit in
    // neighbouring 8-lane groups of one warp (rows per CTA is a multiple of 4, row0 is even).
    const float other = __shfl_xor_sync(0xffffffffu, val, 8);
    if (!(live && t == 0)) return;
    const int pos = *job->epi_pos;
    float outv = val;
    if (epi == GEMV_EPI_ROPE_F32 || epi == GEMV_EPI_ROPE_F16_CACHE) {
        const int j = (int)(o & (size_t)127), i = j >> 1;
        const float *cs = job->epi_rope + (size_t)pos * 128;
        const float c = cs[i], sn = cs[64 + i];
        const float x0 = (j & 1) ? other : val, x1 = (j & 1) ? val : other;
        outv = (j & 1) ? __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c)) : __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
    }
    if (epi == GEMV_EPI_ROPE_F32) job->y[o] = outv;
    else job->epi_cache[(size_t)pos * job->epi_kv_dim + o] = __half_as_ushort(__float2half_rn(outv));
}

__device__ __forceinline__ void gemv_stream_body(const GemvJob *__restrict__ jobs, int n_jobs, const GsParams &P,
                                                   int *__restrict__ dev_error) {
    if (P.dynamic_table) pdl_wait();
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[GS_MAX_STAGES];
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
    const int nb = P.cols >> 8, CB = P.chunk_blocks, S = P.n_stages;
    const uint32_t blk_bytes = type == TYPE_Q4_K ? Q4K_BYTES : Q6K_BYTES;
    if (nrows <= 0 || n_parts < 1 || n_parts > GEMV_MAX_PARTS || nb < 1 || S < 1 || S > GS_MAX_STAGES || CB < 1 ||
        CB > GS_MAX_CHUNK || (int)blockDim.x != R * 8 || (R & 3) || R > 16 || (type != TYPE_Q4_K && type != TYPE_Q6_K) ||
        (uint32_t)CB * blk_bytes + 16u > P.row_stride || (P.row_stride & 15u) || (P.act_off & 15u) ||
        (uint32_t)R * P.row_stride > P.act_off || P.act_off + (uint32_t)CB * 288u > P.slot_bytes || job->rows_per_tile != R) {
        if (tid == 0) atomicExch(dev_error, DEV_ERR_BAD_JOB);
        return;
    }
    pdl_launch_dependents();
    if (type == TYPE_Q4_K) gr_run<TYPE_Q4_K>(job, P, row0, nrows, smem, full, dev_error);
    else gr_run<TYPE_Q6_K>(job, P, row0, nrows, smem, full, dev_error);
}
RNB_GLOBAL void __launch_bounds__(128)
gemv_stream_kernel(const GemvJob *__restrict__ jobs, int n_jobs, const GsParams P, int *__restrict__ dev_error) {
    gemv_stream_body(jobs, n_jobs, P, dev_error);
}
// Static job tables travel as a kernel parameter (constant bank): no dependent global loads
// before the first copy can be issued.  Tables written on the device (MoE) use the kernel above.
constexpr int GS_PACK = 3;
struct GemvJobPack {
    GemvJob j[GS_PACK];
};
RNB_GLOBAL void __launch_bounds__(128)
gemv_stream_kernel_1(const __grid_constant__ GemvJobPack jobs, int n_jobs, const GsParams P, int *__restrict__ dev_error) {
    gemv_stream_body(jobs.j, n_jobs, P, dev_error);
}

}  // namespace rnb
