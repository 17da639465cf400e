// Batch-1 Q4_K matvec for row-rich matrices: two threads per row, one warp per CTA.
//
// Same arithmetic as gemv_stream.cuh (bit-exact with rnb-cpu's AVX2 order), different split of
// a row: thread h of a pair owns bytes 16h..16h+15 of every 32-byte qs group, which are exactly
// accumulator lanes 4h..4h+3, so the integer lane sums need no exchange between threads and a
// block's scales are decoded twice instead of eight times - about half the instructions per
// block of the eight-thread form.  A warp therefore covers 16 rows; it is the whole CTA and
// owns a private ring of stages (K-chunks of 2 super-blocks of every row + the matching
// slices of the Q8_K activation), so refills need a warp-level sync only and ~20 such warps
// fit on an SM.  Worth it when the matrix has rows to spare (gate/up, expert stacks): with few
// rows the eight-thread kernel has more warps to hide latency with.
#pragma once
#include "gemv.cuh"
#include "gemv_stream.cuh"
#include "q8k.cuh"

namespace rnb {

constexpr int GP_ROWS = 16;
constexpr int GP_MAX_STAGES = 8;
constexpr int GP_MAX_CHUNK = 8;

struct GpParams {
    int cols;
    int chunk;            // super-blocks per stage
    int n_stages;
    uint32_t row_stride;  // 16-byte multiple, = 32 or 96 mod 128: the 16-byte loads of a quarter-warp hit 8 bank groups
    uint32_t act_off;     // activation slice inside a stage: qs | bsum16 | d
    uint32_t slot_bytes;
    int rows_per_tile;    // expert-gathered form only: 4, 8 or 16 rows per one-warp CTA (the other lanes idle).
                          // The dense form is 16.
};

// Optional tail for a gate + up launch: the CTA that completes a 256-row block of both vectors
// (16 gate tiles + 16 up tiles) computes silu(gate) * up for the block and quantises it to Q8_K -
// the work of silu_mul_q8k_kernel, spread over the blocks as they finish, without a launch.
// counters[block] is zero before the launch and re-armed by the block's last CTA.
struct GpTail {
    int kind;            // 0 = none, 1 = SiLU * up + Q8_K, 2 = peer publish (integer-MMA kernel, one plain job),
                         // 3 = ordered sum of the selected experts' rows (expert-gathered down projection)
    int n;               // length of the gate / up vectors (multiple of 256); kind 3: rows per expert
    const float *gate, *up;   // kind 3: gate = the experts' raw rows [k][n], up = the k route weights
    uint8_t *xq_out;     // Q8K-dev layout of the n-vector
    int *counters;       // n / 256 ints; kind 3: n / rows per tile
    PeerOut peer;        // kind 2: where the finished rows also go
    int vec_n;           // kind 1: the n elements are n / vec_n vectors, each quantised on its own (0 = one vector)
    int sum_k;           // kind 3: experts per token
    float *sum_out;      // kind 3: out[row] = residual[row] + sum over experts in order of weight * row
    const float *sum_res;
};

struct Q4kPairAcc {
    float a[4], m[2];
};
// One block for thread h: lane sums of lanes 4h..4h+3 and of mins lanes 2h, 2h+1, then the
// block's FMAs.  High nibbles stay in place (x16), the low scale is pre-multiplied by 16, one
// exact shift per lane replaces the nibble shifts.
__device__ __forceinline__ void gp_q4k_block(const uint8_t *blk, const uint8_t *act, const int16_t *bs16, float yd, int h,
                                             Q4kPairAcc &A) {
    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
    const uint32_t sc03 = hdr.y & 0x3f3f3f3fu, mn03 = hdr.z & 0x3f3f3f3fu;
    const uint32_t sc47 = (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
    const uint32_t mn47 = ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
    int s0 = 0, s1 = 0, s2 = 0, s3 = 0;
#pragma unroll
    for (int g = 0; g < 4; g++) {
        const uint4 q = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * g + 16 * h);
        const uint4 alo = *reinterpret_cast<const uint4 *>(act + 64 * g + 16 * h);
        const uint4 ahi = *reinterpret_cast<const uint4 *>(act + 64 * g + 32 + 16 * h);
        const uint32_t scw = g < 2 ? sc03 : sc47;
        const int sl = (int)((scw >> (16 * (g & 1))) & 0xffu) << 4, sh = (int)((scw >> (16 * (g & 1) + 8)) & 0xffu);
        s0 += sl * __dp4a((int)(q.x & 0x0f0f0f0fu), (int)alo.x, 0) + sh * dp4a_us(q.x & 0xf0f0f0f0u, ahi.x, 0);
        s1 += sl * __dp4a((int)(q.y & 0x0f0f0f0fu), (int)alo.y, 0) + sh * dp4a_us(q.y & 0xf0f0f0f0u, ahi.y, 0);
        s2 += sl * __dp4a((int)(q.z & 0x0f0f0f0fu), (int)alo.z, 0) + sh * dp4a_us(q.z & 0xf0f0f0f0u, ahi.z, 0);
        s3 += sl * __dp4a((int)(q.w & 0x0f0f0f0fu), (int)alo.w, 0) + sh * dp4a_us(q.w & 0xf0f0f0f0u, ahi.w, 0);
    }
    const uint4 bs = *reinterpret_cast<const uint4 *>(bs16 + 8 * h);
    const uint32_t mnw = h ? mn47 : mn03;
    const int b0 = (short)((short)(bs.x & 0xffff) + (short)(bs.x >> 16)), b1 = (short)((short)(bs.y & 0xffff) + (short)(bs.y >> 16));
    const int b2 = (short)((short)(bs.z & 0xffff) + (short)(bs.z >> 16)), b3 = (short)((short)(bs.w & 0xffff) + (short)(bs.w >> 16));
    const int mp0 = (int)(mnw & 0xffu) * b0 + (int)((mnw >> 8) & 0xffu) * b1;
    const int mp1 = (int)((mnw >> 16) & 0xffu) * b2 + (int)(mnw >> 24) * b3;
    const float d = __fmul_rn(yd, f16_bits_to_f32(hdr.x & 0xffffu));
    const float dmin = __fmul_rn(-yd, f16_bits_to_f32(hdr.x >> 16));
    A.a[0] = __fmaf_rn(d, (float)(s0 >> 4), A.a[0]);
    A.a[1] = __fmaf_rn(d, (float)(s1 >> 4), A.a[1]);
    A.a[2] = __fmaf_rn(d, (float)(s2 >> 4), A.a[2]);
    A.a[3] = __fmaf_rn(d, (float)(s3 >> 4), A.a[3]);
    A.m[0] = __fmaf_rn(dmin, (float)mp0, A.m[0]);
    A.m[1] = __fmaf_rn(dmin, (float)mp1, A.m[1]);
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// grid = tiles of 16 rows, 32 threads.  Operands must be 16-byte aligned (the host checks).
// DYN: the expert-gathered instantiation (virtual rows, ids read after the wait on the previous kernel, tails 1 with
// per-expert vectors and 3); the dense instantiation carries none of that code.
template <bool DYN>
__device__ __forceinline__ void gemv_pair_body(const GemvJobPack &jobs, int n_jobs, const GpParams &P, int *__restrict__ dev_error, const GpTail &tail) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[GP_MAX_STAGES];
    const int lane = threadIdx.x, r = lane >> 1, h = lane & 1;
    const int tile = blockIdx.x;
    int jsel = 0;
    for (int i = 1; i < n_jobs; i++)
        if (tile >= jobs.j[i].tile0) jsel = i;
    const GemvJob &job = jobs.j[jsel];
    const int RPT = DYN ? P.rows_per_tile : GP_ROWS;
    const int row0 = (tile - job.tile0) * RPT, nrows = min(RPT, job.rows - row0);
    const int cols = P.cols, nb = cols >> 8, CB = P.chunk, S = P.n_stages;
    if (nrows <= 0 || job.n_parts != 1 || job.type != TYPE_Q4_K || nb < 1 || CB < 1 || CB > GP_MAX_CHUNK || S < 1 || S > GP_MAX_STAGES ||
        blockDim.x != 32 || (P.row_stride & 15u) || (uint32_t)CB * Q4K_BYTES > P.row_stride || (P.act_off & 15u) ||
        RPT < 1 || RPT > GP_ROWS || (uint32_t)RPT * P.row_stride > P.act_off || P.act_off + (uint32_t)CB * 288u + 32u > P.slot_bytes) {
        if (lane == 0) atomicExch(dev_error, DEV_ERR_BAD_JOB);
        return;
    }
    pdl_launch_dependents();
    const uint32_t rb = (uint32_t)nb * Q4K_BYTES;
    const int n_chunks = (nb + CB - 1) / CB;
    const uint8_t *w = job.parts[0].w + (size_t)row0 * rb, *x = job.parts[0].x;   // w: first row of this tile
    // every row's first thread fetches that row's chunk; lane 1 fetches the activation slice
    auto issue_w = [&](int c, int slot_idx) {
        if (h != 0) return;
        uint64_t *bar = &full[slot_idx];
        if (r < nrows) {
            const uint32_t bytes = (uint32_t)min(CB, nb - c * CB) * Q4K_BYTES;
            mbar_arrive_expect_tx(bar, bytes);
            bulk_g2s(smem + (uint32_t)slot_idx * P.slot_bytes + (uint32_t)r * P.row_stride, w + (size_t)r * rb + (uint32_t)(c * CB) * Q4K_BYTES,
                     bytes, bar);
        } else {
            mbar_arrive(bar);
        }
    };
    auto issue_a = [&](int c, int slot_idx) {
        if (lane != 1) return;
        uint64_t *bar = &full[slot_idx];
        const uint32_t nblk = (uint32_t)min(CB, nb - c * CB);
        // the block scales are 4 bytes each: copy the 16-byte groups that contain this chunk's
        const uint32_t d_first = (uint32_t)(c * CB) * 4u, d_lo = d_first & ~15u, d_bytes = ((d_first + nblk * 4u + 15u) & ~15u) - d_lo;
        uint8_t *dst = smem + (uint32_t)slot_idx * P.slot_bytes + P.act_off;
        mbar_arrive_expect_tx(bar, nblk * 288u + d_bytes);
        bulk_g2s(dst, x + (uint32_t)(c * CB) * 256u, nblk * 256u, bar);
        bulk_g2s(dst + CB * 256, x + cols + (uint32_t)(c * CB) * 32u, nblk * 32u, bar);
        bulk_g2s(dst + CB * 288, x + cols + 32 * nb + d_lo, d_bytes, bar);
    };
    if (lane == 0) {
        for (int s = 0; s < S; s++) mbar_init(&full[s], GP_ROWS + 1);
        mbar_fence_init();
    }
    __syncwarp();
    if (DYN) {
        // the ids come from an earlier kernel: nothing can be fetched before the wait
        pdl_wait();
        const int e = row0 / job.dyn_rows;
        const uint32_t id = __ldcg(job.dyn_ids + e);
        w = job.parts[0].w + ((size_t)id * (size_t)job.dyn_rows + (size_t)(row0 - e * job.dyn_rows)) * rb;
        x += (size_t)e * job.dyn_x_stride;
    }
    for (int i = 0; i < S && i < n_chunks; i++) issue_w(i, i);
    if (!DYN) pdl_wait();   // the weights do not depend on the previous kernel; the activation does
    for (int i = 0; i < S && i < n_chunks; i++) issue_a(i, i);
    const uint32_t row_off = (uint32_t)(r < nrows ? r : 0) * P.row_stride + 0u;   // dead rows read row 0 and do not store
    Q4kPairAcc A = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f}};
    int slot_idx = 0;
    uint32_t parity = 0;
    for (int c = 0; c < n_chunks; c++) {
        const int nblk = min(CB, nb - c * CB);
        uint8_t *slot = smem + (uint32_t)slot_idx * P.slot_bytes;
        if (!mbar_wait_bounded(&full[slot_idx], parity)) {
            for (int k = c + 1; k < n_chunks && k < c + S; k++) mbar_wait_bounded(&full[k % S], (uint32_t)((k / S) & 1));
            if (lane == 0) atomicExch(dev_error, DEV_ERR_MBAR_TIMEOUT);
            return;
        }
        const uint8_t *rowp = slot + row_off;
        const uint8_t *act = slot + P.act_off;
        const int16_t *bs16 = reinterpret_cast<const int16_t *>(slot + P.act_off + CB * 256);
        const float *xd = reinterpret_cast<const float *>(slot + P.act_off + CB * 288) + (((uint32_t)(c * CB) * 4u & 15u) >> 2);
#pragma unroll 2
        for (int j = 0; j < nblk; j++) gp_q4k_block(rowp + j * Q4K_BYTES, act + j * 256, bs16 + j * 16, xd[j], h, A);
        __syncwarp();   // stage consumed by every row
        if (c + S < n_chunks) {
            issue_w(c + S, slot_idx);
            issue_a(c + S, slot_idx);
        }
        if (++slot_idx == S) slot_idx = 0, parity ^= 1u;
    }
    // lanes 4h+w: (l + l4) across the pair, then (v0 + v2) + (v1 + v3); mins lanes 2h, 2h+1: (a0 + a2) + (a1 + a3)
    const float v0 = __fadd_rn(A.a[0], __shfl_xor_sync(0xffffffffu, A.a[0], 1));
    const float v1 = __fadd_rn(A.a[1], __shfl_xor_sync(0xffffffffu, A.a[1], 1));
    const float v2 = __fadd_rn(A.a[2], __shfl_xor_sync(0xffffffffu, A.a[2], 1));
    const float v3 = __fadd_rn(A.a[3], __shfl_xor_sync(0xffffffffu, A.a[3], 1));
    const float hs = __fadd_rn(__fadd_rn(v0, v2), __fadd_rn(v1, v3));
    const float x0 = __fadd_rn(A.m[0], __shfl_xor_sync(0xffffffffu, A.m[0], 1));
    const float x1 = __fadd_rn(A.m[1], __shfl_xor_sync(0xffffffffu, A.m[1], 1));
    float dot = __fadd_rn(hs, __fadd_rn(x0, x1));
    if (job.parts[0].scale) dot = __fmul_rn(dot, __ldg(job.parts[0].scale));
    if (r < nrows && h == 0) {
        const size_t o = (size_t)row0 + r;
        job.y[o] = job.residual ? __fadd_rn(job.residual[o], dot) : dot;
    }
    if (tail.kind == 1) {
        const int blk = row0 >> 8;
        __threadfence();   // this tile's 16 results are visible device-wide before the tile is counted
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atomicAdd(&tail.counters[blk], 1) == n_jobs * (256 / RPT) - 1;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) return;
        __threadfence();
        const size_t off = (size_t)blk * 256 + lane * 8;
        const float4 g0 = __ldcg(reinterpret_cast<const float4 *>(tail.gate + off)), g1 = __ldcg(reinterpret_cast<const float4 *>(tail.gate + off + 4));
        const float4 u0 = __ldcg(reinterpret_cast<const float4 *>(tail.up + off)), u1 = __ldcg(reinterpret_cast<const float4 *>(tail.up + off + 4));
        const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float e = expf_libm(-gv[j]);   // as silu_mul_q8k_kernel: libm's expf
            v[j] = __fmul_rn(__fdiv_rn(gv[j], __fadd_rn(1.0f, e)), uv[j]);
        }
        int vb = blk, vn = tail.n;
        uint8_t *xq = tail.xq_out;
        if (DYN && tail.vec_n) {
            // one Q8_K vector per expert
            vn = tail.vec_n;
            const int vec = blk / (vn >> 8);
            vb = blk - vec * (vn >> 8);
            xq += (size_t)vec * q8k_dev_bytes((size_t)vn);
        }
        Q8kDevView dv = q8k_dev_view(xq, vn);
        q8k_quantize_block_warp(v, lane, dv.qs + vb * 256, dv.d + vb, dv.bsum16 + vb * 16, nullptr);
        if (lane == 0) tail.counters[blk] = 0;
    }
    if (DYN && tail.kind == 3) {
        // the tile that completes its 16 rows over all experts folds them in selection order:
        // out = residual + ((0 + w0 * r0) + w1 * r1 + ...), the order of the multi-part matvec
        const int e = row0 / tail.n, lrow0 = row0 - e * tail.n, ctr = lrow0 / RPT;
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atomicAdd(&tail.counters[ctr], 1) == tail.sum_k - 1;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) return;
        __threadfence();
        if (lane < RPT && lrow0 + lane < tail.n) {
            const size_t o = (size_t)lrow0 + lane;
            float acc = 0.f;
            for (int k = 0; k < tail.sum_k; k++) acc = __fadd_rn(acc, __fmul_rn(__ldcg(tail.gate + (size_t)k * tail.n + o), __ldcg(tail.up + k)));
            tail.sum_out[o] = tail.sum_res ? __fadd_rn(__ldcg(tail.sum_res + o), acc) : acc;
        }
        if (lane == 0) tail.counters[ctr] = 0;
    }
}
RNB_GLOBAL void __launch_bounds__(32)
gemv_pair_q4k_kernel(const __grid_constant__ GemvJobPack jobs, int n_jobs, const GpParams P, int *__restrict__ dev_error,
                     const __grid_constant__ GpTail tail) {
    gemv_pair_body<false>(jobs, n_jobs, P, dev_error, tail);
}
RNB_GLOBAL void __launch_bounds__(32)
gemv_pair_q4k_dyn_kernel(const __grid_constant__ GemvJobPack jobs, int n_jobs, const GpParams P, int *__restrict__ dev_error,
                         const __grid_constant__ GpTail tail) {
    gemv_pair_body<true>(jobs, n_jobs, P, dev_error, tail);
}

}  // namespace rnb
