// Batch-1 matvec, streaming form: the kernel the decode path uses.
//
// Eight threads own one weight row and walk its blocks in order, so the f32 accumulation is
// rnb-cpu's AVX2 order without any exchange between rows (see gemv.cuh for the lane algebra).
// A CTA of NW warps owns 4*NW rows.  Rows are cut along K into chunks of CB super-blocks; a
// chunk of every row of the CTA is one pipeline stage, fetched by the bulk-async copy engine
// (one copy per row, completion counted on the stage's mbarrier) while earlier stages are
// being consumed.  Several small CTAs per SM keep hundreds of KB of weights in flight.
#pragma once
#include "gemv.cuh"

namespace rnb {

constexpr int GS_MAX_STAGES = 8;

struct GsParams {
    int cols;
    int chunk_blocks;     // super-blocks (256 elements) per stage
    int n_stages;         // 1..GS_MAX_STAGES
    uint32_t row_stride;  // bytes of shared memory per row per stage (>= chunk bytes + 16)
    int dynamic_table;
};

__device__ __forceinline__ void gemv_stream_body(const GemvJob *__restrict__ jobs, int n_jobs,
                                                 const GsParams P, int *__restrict__ dev_error) {
    if (P.dynamic_table) pdl_wait();
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[GS_MAX_STAGES];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rows_per_cta = (int)(blockDim.x >> 5) * 4;
    const int tile = blockIdx.x;
    int jsel = 0;
    for (int i = 1; i < n_jobs; i++)
        if (tile >= jobs[i].tile0) jsel = i;
    const GemvJob *job = jobs + jsel;
    const int type = job->type, n_parts = job->n_parts;
    const int row0 = (tile - job->tile0) * rows_per_cta;
    const int nrows = min(rows_per_cta, job->rows - row0);
    const int cols = P.cols, nb = cols >> 8, CB = P.chunk_blocks, S = P.n_stages;
    const uint32_t blk_bytes = type == TYPE_Q4_K ? Q4K_BYTES : type == TYPE_Q6_K ? Q6K_BYTES : 8 * Q8_0_BYTES;
    const size_t rb = (size_t)nb * blk_bytes;
    const int n_chunks = (nb + CB - 1) / CB;
    const int n_items = n_parts * n_chunks;
    if (nrows <= 0 || n_parts < 1 || n_parts > GEMV_MAX_PARTS || nb < 1 || S < 1 || S > GS_MAX_STAGES ||
        (uint32_t)CB * blk_bytes + 16u > P.row_stride || (P.row_stride & 15u) != 0 || job->rows_per_tile != rows_per_cta) {
        if (tid == 0) atomicExch(dev_error, DEV_ERR_BAD_JOB);
        return;
    }
    const uint32_t slot_bytes = (uint32_t)rows_per_cta * P.row_stride;

    pdl_launch_dependents();
    // bulk copies need 16-byte aligned sources and sizes: whole-row alignment decides
    bool tma = (rb & 15u) == 0;
    for (int p = 0; p < n_parts; p++) tma = tma && (((uintptr_t)job->parts[p].w & 15u) == 0);
    if (type == TYPE_Q6_K) tma = tma && (CB % 8 == 0);

    auto issue = [&](int item) {  // thread 0 only
        const int p = item / n_chunks, c = item - p * n_chunks;
        const int nblk = min(CB, nb - c * CB);
        const uint32_t bytes = (uint32_t)nblk * blk_bytes;
        uint64_t *bar = &full[item % S];
        uint8_t *dst = smem + (size_t)(item % S) * slot_bytes;
        const uint8_t *src = job->parts[p].w + (size_t)row0 * rb + (size_t)c * CB * blk_bytes;
        mbar_arrive_expect_tx(bar, bytes * (uint32_t)nrows);
        for (int r = 0; r < nrows; r++) bulk_g2s(dst + (size_t)r * P.row_stride, src + (size_t)r * rb, bytes, bar);
    };

    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(&full[s], 1);
        mbar_fence_init();
        if (tma)  // weights never depend on the previous kernel: start streaming before pdl_wait
            for (int i = 0; i < S && i < n_items; i++) issue(i);
    }
    __syncthreads();
    pdl_wait();  // activations, residual and route weights come from earlier kernels

    const int t = lane & 7;
    const int r = warp * 4 + (lane >> 3);  // this group's row within the CTA
    const bool live = r < nrows;
    const int rr = live ? r : 0;
    float acc_total = 0.f;
    float lane_acc = 0.f, min_acc = 0.f;

    for (int item = 0; item < n_items; item++) {
        const int p = item / n_chunks, c = item - p * n_chunks;
        const int nblk = min(CB, nb - c * CB);
        uint8_t *slot = smem + (size_t)(item % S) * slot_bytes;
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
                for (uint32_t i = tid; i < bytes; i += blockDim.x) slot[(size_t)q * P.row_stride + i] = src[(size_t)q * rb + i];
            __syncthreads();
        }
        const uint8_t *rowp = slot + (size_t)rr * P.row_stride;
        const uint8_t *xbase = job->parts[p].x;
        const int b0 = c * CB;
        if (type == TYPE_Q4_K) {
            const int8_t *qs = reinterpret_cast<const int8_t *>(xbase);
            const int16_t *bs = reinterpret_cast<const int16_t *>(xbase + cols);
            const float *xd = reinterpret_cast<const float *>(xbase + cols + 32 * nb);
#pragma unroll 2
            for (int j = 0; j < nblk; j++) {
                const int b = b0 + j;
                const Q4kTerms tm = q4k_block_terms(rowp + j * Q4K_BYTES, t, qs + b * 256, __ldg(xd + b), bs + b * 16, live);
                lane_acc = __fmaf_rn(tm.d, (float)tm.lane_sum, lane_acc);
                min_acc = __fmaf_rn(tm.dmin, (float)tm.min_prod, min_acc);
            }
        } else if (type == TYPE_Q6_K) {
            const int8_t *qs = reinterpret_cast<const int8_t *>(xbase);
            const int16_t *bs = reinterpret_cast<const int16_t *>(xbase + cols);
            const float *xd = reinterpret_cast<const float *>(xbase + cols + 32 * nb);
            const uint32_t row32 = smem_u32(rowp);
#pragma unroll 2
            for (int j = 0; j < nblk; j++) {
                const int b = b0 + j;
                int ls;
                float dd;
                q6k_block_terms(row32 + j * Q6K_BYTES, t, qs + b * 256, __ldg(xd + b), bs + b * 16, live, ls, dd);
                lane_acc = __fmaf_rn(dd, (float)ls, lane_acc);
            }
        } else {  // Q8_0: a 256-element unit is 8 blocks, thread t takes block t of the unit
            const float *xf = reinterpret_cast<const float *>(xbase);
            const uint32_t row32 = smem_u32(rowp);
            for (int j = 0; j < nblk; j++) {
                float bsum, dd;
                q8_0_block_terms(row32 + (j * 8 + t) * Q8_0_BYTES, xf + ((b0 + j) * 8 + t) * 32, live, bsum, dd);
#pragma unroll
                for (int jj = 0; jj < 8; jj++) {  // block order, every thread of the group alike
                    const float sb = __shfl_sync(0xffffffffu, bsum, (lane & ~7) + jj);
                    const float sd = __shfl_sync(0xffffffffu, dd, (lane & ~7) + jj);
                    lane_acc = __fadd_rn(lane_acc, __fmul_rn(sd, sb));
                }
            }
        }
        if (c == n_chunks - 1) {  // row finished for this part: fold the accumulator lanes
            float dot;
            if (type == TYPE_Q4_K) {
                float hs = lane_acc;  // thread (g,h) holds lane 4h+g: (l + l4) -> (+2) -> (+1)
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 1));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 4));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 2));
                float ms = min_acc;  // lane t%4: (a0 + a2) + (a1 + a3)
                ms = __fadd_rn(ms, __shfl_xor_sync(0xffffffffu, ms, 2));
                ms = __fadd_rn(ms, __shfl_xor_sync(0xffffffffu, ms, 1));
                dot = __fadd_rn(hs, ms);
            } else if (type == TYPE_Q6_K) {
                float hs = lane_acc;  // thread (n,m) holds lane 2m+n: +4 is t^2, +2 is t^1, +1 is t^4
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 2));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 1));
                hs = __fadd_rn(hs, __shfl_xor_sync(0xffffffffu, hs, 4));
                dot = hs;
            } else {
                dot = lane_acc;
            }
            // expert_out *= route weight; out += expert_out, experts in selection order
            if (job->parts[p].scale) dot = __fmul_rn(dot, __ldg(job->parts[p].scale));
            acc_total = n_parts == 1 ? dot : __fadd_rn(acc_total, dot);
            lane_acc = 0.f;
            min_acc = 0.f;
        }
        __syncthreads();  // every thread is done with this slot: refill it with the item S ahead
        if (tma && tid == 0 && item + S < n_items) issue(item + S);
    }
    if (live && t == 0) {
        const size_t o = (size_t)row0 + r;
        job->y[o] = job->residual ? __fadd_rn(job->residual[o], acc_total) : acc_total;
    }
}

__global__ void __launch_bounds__(128)
gemv_stream_kernel(const GemvJob *__restrict__ jobs, int n_jobs, const GsParams P, int *__restrict__ dev_error) {
    gemv_stream_body(jobs, n_jobs, P, dev_error);
}
__global__ void __launch_bounds__(128)
gemv_stream_kernel_1(const __grid_constant__ GemvJob job, const GsParams P, int *__restrict__ dev_error) {
    gemv_stream_body(&job, 1, P, dev_error);
}

}  // namespace rnb
