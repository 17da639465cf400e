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
};

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

// ---- Q4_K: 8 lanes per 256-element block; lane t owns 16 bytes of qs ----------------------
// qs bytes 16t..16t+15 belong to 64-element group g = t/2, half h = t%2: low nibbles are
// elements 64g+16h+(0..15) (sub-block 2g), high nibbles 64g+32+16h+(0..15) (sub-block 2g+1).
// Lane t also owns the min correction of sub-block t.
__device__ __forceinline__ float q4k_block_partial(const uint8_t *blk, int t, const int8_t *xq,
                                                   float yd, int bsum32_t) {
    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
    const uint4 q = *reinterpret_cast<const uint4 *>(blk + 16 + 16 * t);
    const int g = t >> 1, h = t & 1;
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
    const int mn = ((t < 4 ? mn03 : mn47) >> (8 * (t & 3))) & 0xff;
    int lo = 0, hi = 0;
    lo = __dp4a((int)(q.x & 0x0f0f0f0fu), (int)alo.x, lo);
    hi = __dp4a((int)((q.x >> 4) & 0x0f0f0f0fu), (int)ahi.x, hi);
    lo = __dp4a((int)(q.y & 0x0f0f0f0fu), (int)alo.y, lo);
    hi = __dp4a((int)((q.y >> 4) & 0x0f0f0f0fu), (int)ahi.y, hi);
    lo = __dp4a((int)(q.z & 0x0f0f0f0fu), (int)alo.z, lo);
    hi = __dp4a((int)((q.z >> 4) & 0x0f0f0f0fu), (int)ahi.z, hi);
    lo = __dp4a((int)(q.w & 0x0f0f0f0fu), (int)alo.w, lo);
    hi = __dp4a((int)((q.w >> 4) & 0x0f0f0f0fu), (int)ahi.w, hi);
    const float d = f16_bits_to_f32(hdr.x & 0xffffu);
    const float dmin = f16_bits_to_f32(hdr.x >> 16);
    return yd * (d * (float)(sc_lo * lo + sc_hi * hi) - dmin * (float)(mn * bsum32_t));
}

// ---- Q6_K: 8 lanes per block; lane t = (n = t/4, m = t%4) owns l = 8m..8m+7 of half n -----
__device__ __forceinline__ float q6k_block_partial(uint32_t blk, int t, const int8_t *xq,
                                                   float yd) {
    const int n = t >> 2, m = t & 3;
    const uint2 qla = lds8_unaligned(blk + 64 * n + 8 * m);
    const uint2 qlb = lds8_unaligned(blk + 64 * n + 32 + 8 * m);
    const uint2 qh = lds8_unaligned(blk + 128 + 32 * n + 8 * m);
    const int8_t *xa = xq + 128 * n + 8 * m;
    const uint2 a0 = ldg_nc_u2(xa), a1 = ldg_nc_u2(xa + 32), a2 = ldg_nc_u2(xa + 64),
                a3 = ldg_nc_u2(xa + 96);
    int i0 = 0, i1 = 0, i2 = 0, i3 = 0;
#pragma unroll
    for (int w = 0; w < 2; w++) {
        const uint32_t la = w ? qla.y : qla.x, lb = w ? qlb.y : qlb.x, hh = w ? qh.y : qh.x;
        const uint32_t v0 = (la & 0x0f0f0f0fu) | ((hh << 4) & 0x30303030u);
        const uint32_t v1 = (lb & 0x0f0f0f0fu) | ((hh << 2) & 0x30303030u);
        const uint32_t v2 = ((la >> 4) & 0x0f0f0f0fu) | (hh & 0x30303030u);
        const uint32_t v3 = ((lb >> 4) & 0x0f0f0f0fu) | ((hh >> 2) & 0x30303030u);
        i0 = __dp4a((int)__vsub4(v0, 0x20202020u), (int)(w ? a0.y : a0.x), i0);
        i1 = __dp4a((int)__vsub4(v1, 0x20202020u), (int)(w ? a1.y : a1.x), i1);
        i2 = __dp4a((int)__vsub4(v2, 0x20202020u), (int)(w ? a2.y : a2.x), i2);
        i3 = __dp4a((int)__vsub4(v3, 0x20202020u), (int)(w ? a3.y : a3.x), i3);
    }
    const uint32_t sc = blk + 192 + 8 * n + (m >> 1);
    int s0, s1, s2, s3, dh;
    asm volatile("ld.shared.s8 %0, [%1];" : "=r"(s0) : "r"(sc));
    asm volatile("ld.shared.s8 %0, [%1];" : "=r"(s1) : "r"(sc + 2));
    asm volatile("ld.shared.s8 %0, [%1];" : "=r"(s2) : "r"(sc + 4));
    asm volatile("ld.shared.s8 %0, [%1];" : "=r"(s3) : "r"(sc + 6));
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dh) : "r"(blk + 208));
    const int isum = s0 * i0 + s1 * i1 + s2 * i2 + s3 * i3;
    return (yd * f16_bits_to_f32((uint32_t)dh)) * (float)isum;
}

// ---- Q8_0: one lane per 32-element block, f32 activations ---------------------------------
__device__ __forceinline__ float q8_0_block_partial(uint32_t blk, const float *x) {
    // 34 bytes at a 2-byte-aligned address: d (f16) then 32 int8
    const uint32_t base = blk & ~3u, sh = (blk & 3u) * 8u;
    uint32_t w[10];
#pragma unroll
    for (int i = 0; i < 10; i++) w[i] = lds32(base + 4 * i);
    uint32_t b[9];
#pragma unroll
    for (int i = 0; i < 9; i++) b[i] = __funnelshift_r(w[i], w[i + 1], sh);
    const float d = f16_bits_to_f32(b[0] & 0xffffu);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        // quants 4i..4i+3 live in bytes 2+4i .. 5+4i: upper half of b[i], lower half of b[i+1]
        const uint32_t qw = __funnelshift_r(b[i], b[i + 1], 16);
        const float4 xv = *reinterpret_cast<const float4 *>(x + 4 * i);
        sum = fmaf((float)(int8_t)(qw & 0xff), xv.x, sum);
        sum = fmaf((float)(int8_t)((qw >> 8) & 0xff), xv.y, sum);
        sum = fmaf((float)(int8_t)((qw >> 16) & 0xff), xv.z, sum);
        sum = fmaf((float)(int8_t)(qw >> 24), xv.w, sum);
    }
    return d * sum;
}

// Shared memory: [part 0 tile][part 1 tile]...; each part region is part_stride bytes
// (tile bytes rounded up to 16, plus 16 bytes of slack for the unaligned readers).
__device__ __forceinline__ void gemv_tile_body(const GemvJob *__restrict__ jobs, int n_jobs,
                                               int cols, uint32_t part_stride,
                                               int *__restrict__ dev_error) {
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
            float part = 0.0f;
            if (type == TYPE_Q4_K) {
                const int nb = cols >> 8;
                const int8_t *qs = reinterpret_cast<const int8_t *>(xbase);
                const float *xd = reinterpret_cast<const float *>(xbase + cols);
                const int16_t *bs = reinterpret_cast<const int16_t *>(xbase + cols + 4 * nb);
#pragma unroll 4
                for (int b = bsub; b < nb; b += 4)
                    part += q4k_block_partial(rowp + b * Q4K_BYTES, t, qs + b * 256, __ldg(xd + b),
                                              (int)__ldg(bs + b * 8 + t));
            } else if (type == TYPE_Q6_K) {
                const int nb = cols >> 8;
                const int8_t *qs = reinterpret_cast<const int8_t *>(xbase);
                const float *xd = reinterpret_cast<const float *>(xbase + cols);
                const uint32_t rows32 = smem_u32(rowp);
#pragma unroll 2
                for (int b = bsub; b < nb; b += 4)
                    part += q6k_block_partial(rows32 + b * Q6K_BYTES, t, qs + b * 256, __ldg(xd + b));
            } else {  // TYPE_Q8_0
                const int nb32 = cols >> 5;
                const float *xf = reinterpret_cast<const float *>(xbase);
                const uint32_t rows32 = smem_u32(rowp);
                for (int b = lane; b < nb32; b += 32)
                    part += q8_0_block_partial(rows32 + b * Q8_0_BYTES, xf + b * 32);
            }
            part = warp_sum(part);
            const float sc = job->parts[p].scale ? __ldg(job->parts[p].scale) : 1.0f;
            acc = fmaf(sc, part, acc);
        }
        if (lane == 0) {
            const size_t o = (size_t)s * job->rows + row0 + r;
            job->y[o] = job->residual ? job->residual[o] + acc : acc;
        }
    }
}

// Job table in global memory (multi-matrix launches: q/k/v, gate/up, routed experts).
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_tile_kernel(const GemvJob *__restrict__ jobs, int n_jobs, int cols, uint32_t part_stride,
                 int *__restrict__ dev_error) {
    gemv_tile_body(jobs, n_jobs, cols, part_stride, dev_error);
}
// Single job passed by value in kernel-parameter space (no table upload).
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_tile_kernel_1(const __grid_constant__ GemvJob job, int cols, uint32_t part_stride,
                   int *__restrict__ dev_error) {
    gemv_tile_body(&job, 1, cols, part_stride, dev_error);
}

// LM-head epilogue: greedy argmax with the reference CPU sampler's tie rule (the LAST of equal
// maxima, crates/rnb-llm/src/sampler/greedy.rs:4-11).  Single CTA.
__global__ void __launch_bounds__(1024)
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

}  // namespace rnb
