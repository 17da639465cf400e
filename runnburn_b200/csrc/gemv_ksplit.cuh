// Batch-1 Q6_K matvec for long rows and few of them (ffn_down: 4096 x 14336): K-split form.
//
// With 4096 rows the eight-threads-per-row kernel has only ~7 warps per SM, each walking a
// 56-block row serially: latency-bound at a quarter of the HBM rate.  Only the per-lane FMA
// chain of a row has to run in block order (see gemv.cuh); the integer lane sums of different
// blocks are independent.  Here a CTA owns 4 rows and 4 warps; a pipeline stage is one chunk
// of 8 super-blocks of every row (bulk-async copies onto an mbarrier, a ring of stages); warp w
// unpacks and dots blocks 2w and 2w+1 of the stage for all four rows (eight threads per row,
// integer partial sums reduce-scattered to one accumulator lane each) and leaves the lane
// sums, as f32, with the block scales in shared memory; after one CTA barrier warp 0 replays
// the stage's eight blocks in order, one FMA per block and lane, while the other warps start
// the next stage.  Four times the warps per row, same bytes, same bits.
#pragma once
#include "gemv.cuh"
#include "gemv_stream.cuh"

namespace rnb {

constexpr int GK_ROWS = 4;
constexpr int GK_CHUNK = 8;      // super-blocks per stage: 8 x 210 bytes is the shortest 16-byte multiple
constexpr int GK_MAX_STAGES = 6;
constexpr int GK_THREADS = 128;
constexpr uint32_t GK_ROW_STRIDE = GK_CHUNK * Q6K_BYTES + 16;                  // 1696: 16-byte multiple
constexpr uint32_t GK_ACT_OFF = GK_ROWS * GK_ROW_STRIDE;                       // qs | bsum16 | d
constexpr uint32_t GK_SLOT = ((GK_ACT_OFF + GK_CHUNK * 292 + 127) / 128) * 128;
constexpr uint32_t GK_RES_FLOATS = GK_CHUNK * GK_ROWS * 9;                     // per stage: 8 lane sums + d per (block, row)
__host__ __device__ constexpr uint32_t gk_smem(int stages) { return (uint32_t)stages * GK_SLOT + 2u * GK_RES_FLOATS * 4u; }

// grid = ceil(rows / 4); 128 threads; dynamic shared memory gk_smem(S).  cols % 2048 == 0, operands 16-byte aligned.
RNB_GLOBAL void __launch_bounds__(GK_THREADS)
gemv_ksplit_q6k_kernel(const __grid_constant__ GemvJob job, int cols, int S, int *__restrict__ dev_error) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[GK_MAX_STAGES];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = cols >> 8, n_chunks = nb / GK_CHUNK;
    const int row0 = blockIdx.x * GK_ROWS, nrows = min(GK_ROWS, job.rows - row0);
    if (nrows <= 0 || job.type != TYPE_Q6_K || job.n_parts != 1 || nb < GK_CHUNK || (nb % GK_CHUNK) != 0 || blockDim.x != GK_THREADS || S < 1 || S > GK_MAX_STAGES) {
        if (tid == 0) atomicExch(dev_error, DEV_ERR_BAD_JOB);
        return;
    }
    pdl_launch_dependents();
    float *res = reinterpret_cast<float *>(smem + (uint32_t)S * GK_SLOT);
    const uint32_t rb = (uint32_t)nb * Q6K_BYTES;
    const uint8_t *w = job.parts[0].w + (size_t)row0 * rb, *x = job.parts[0].x;
    auto issue = [&](int c, int s, bool weights, bool act) {   // thread 0
        uint64_t *bar = &full[s];
        uint8_t *dst = smem + (uint32_t)s * GK_SLOT;
        if (weights) {
            mbar_arrive_expect_tx(bar, (uint32_t)nrows * GK_CHUNK * Q6K_BYTES + GK_CHUNK * 292u);
            for (int r = 0; r < nrows; r++) bulk_g2s(dst + (uint32_t)r * GK_ROW_STRIDE, w + (size_t)r * rb + (uint32_t)(c * GK_CHUNK) * Q6K_BYTES, GK_CHUNK * Q6K_BYTES, bar);
        }
        if (act) {
            bulk_g2s(dst + GK_ACT_OFF, x + (uint32_t)(c * GK_CHUNK) * 256u, GK_CHUNK * 256u, bar);
            bulk_g2s(dst + GK_ACT_OFF + GK_CHUNK * 256, x + cols + (uint32_t)(c * GK_CHUNK) * 32u, GK_CHUNK * 32u, bar);
            bulk_g2s(dst + GK_ACT_OFF + GK_CHUNK * 288, x + cols + 32 * nb + (uint32_t)(c * GK_CHUNK) * 4u, GK_CHUNK * 4u, bar);
        }
    };
    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(&full[s], 1);
        mbar_fence_init();
        for (int i = 0; i < S && i < n_chunks; i++) issue(i, i, true, false);
    }
    __syncthreads();
    pdl_wait();   // the weights do not depend on the previous kernel; the activation does
    if (tid == 0)
        for (int i = 0; i < S && i < n_chunks; i++) issue(i, i, false, true);
    const int r = lane >> 3, t = lane & 7;                 // phase 1: row of the CTA, thread of the row
    const uint32_t row_off = (uint32_t)(r < nrows ? r : 0) * GK_ROW_STRIDE;   // dead rows read row 0 and are never stored
    float acc = 0.f;                                       // phase 2 (warp 0): row = lane / 8, accumulator lane = lane % 8
    int s = 0;
    uint32_t parity = 0;
    for (int c = 0; c < n_chunks; c++) {
        bool ok = true;
        if (warp == 0) ok = mbar_wait_bounded(&full[s], parity);   // one warp polls; the rest park at the barrier
        if (!__syncthreads_and(ok)) {
            if (tid == 0) {
                for (int k = c + 1; k < n_chunks && k < c + S; k++) mbar_wait_bounded(&full[k % S], (uint32_t)((k / S) & 1));   // drain what is in flight
                atomicExch(dev_error, DEV_ERR_MBAR_TIMEOUT);
            }
            return;
        }
        if (warp != 0) mbar_try_wait(&full[s], parity);   // completed: acquires the copied bytes
        const uint8_t *slot = smem + (uint32_t)s * GK_SLOT;
        const uint8_t *act = slot + GK_ACT_OFF;
        const int16_t *bs16 = reinterpret_cast<const int16_t *>(slot + GK_ACT_OFF + GK_CHUNK * 256);
        const float *xd = reinterpret_cast<const float *>(slot + GK_ACT_OFF + GK_CHUNK * 288);
        float *rs = res + (uint32_t)(c & 1) * GK_RES_FLOATS;
        {
            // ---- phase 1: blocks 2*warp (4-byte aligned in the row) and 2*warp + 1 (2 bytes off) ----
            const int j0 = 2 * warp, j1 = j0 + 1;
            const uint8_t *b0 = slot + row_off + j0 * Q6K_BYTES, *b1 = b0 + Q6K_BYTES;
            float2 dd;
            const int ls0 = gs_q6k_lanes<0>(b0, act + j0 * 256, bs16 + j0 * 16, 0.f, t, true, &dd);
            const int ls1 = gs_q6k_lanes<2>(b1, act + j1 * 256, bs16 + j1 * 16, 0.f, t, true, &dd);
            const int l = 2 * (t & 3) + (t >> 2);   // thread (n = t/4, m = t%4) holds accumulator lane 2m + n
            rs[(j0 * GK_ROWS + r) * 9 + l] = (float)ls0;
            rs[(j1 * GK_ROWS + r) * 9 + l] = (float)ls1;
            if (t == 0) {
                rs[(j0 * GK_ROWS + r) * 9 + 8] = __fmul_rn(xd[j0], f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(b0 + 208)));
                rs[(j1 * GK_ROWS + r) * 9 + 8] = __fmul_rn(xd[j1], f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(b1 + 208)));
            }
        }
        __syncthreads();   // results of the stage complete, stage consumed
        if (tid == 0 && c + S < n_chunks) issue(c + S, s, true, true);
        if (warp == 0) {
            // ---- phase 2: ordered replay of the stage's eight blocks ----
            const float *rr = rs + (lane >> 3) * 9;
            const int l = lane & 7;
#pragma unroll
            for (int j = 0; j < GK_CHUNK; j++) acc = __fmaf_rn(rr[j * GK_ROWS * 9 + 8], rr[j * GK_ROWS * 9 + l], acc);
        }
        if (++s == S) s = 0, parity ^= 1u;
    }
    if (warp == 0) {
        // lanes: (l + l4) -> (+2) -> (+1)
        float v = acc;
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
        if (job.parts[0].scale) v = __fmul_rn(v, __ldg(job.parts[0].scale));
        const int cr = lane >> 3;
        if ((lane & 7) == 0 && cr < nrows) {
            const size_t o = (size_t)row0 + cr;
            job.y[o] = job.residual ? __fadd_rn(job.residual[o], v) : v;
        }
    }
}

}  // namespace rnb
