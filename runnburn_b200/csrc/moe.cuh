// MoE routing on device: router logits, softmax top-k, and the expert-gathered matvec job
// tables, so that a decode step needs no host round trip between routing and the experts.
#pragma once
#include "common.cuh"
#include "gemv.cuh"

namespace rnb {

// Router logits: f32 [n_expert][hidden] x f32 h.  16 threads per expert reproduce the exact
// accumulation order of the reference's host routine (dot_f32_avx2_fma,
// crates/rnb-cpu/src/gemm/f32_gemv.rs:215-237,266-275): thread j owns accumulator lane j of
// the two 8-lane FMA registers, then lanes are folded 8, 4, 2, 1 apart.  Bit-identical
// logits are what makes the selected expert ids identical.  hidden % 16 == 0.
// The loads of a batch of steps are issued together (the chain of FMAs is latency-bound on its
// loads otherwise).  Any number of experts per CTA (blockDim / 16).
__device__ __forceinline__ void router_logits_body(const float *__restrict__ w, const float *__restrict__ h, int n_expert,
                                                   int hidden, float *logits) {
    pdl_launch_dependents();
    // WB steps of router weights per batch (elements j, j + 16, ...) are in registers before they are needed: the
    // first batch is fetched before the wait on the previous kernel (a 2048-wide row is one batch, so nothing of the
    // row is left to fetch after the wait); the hidden state follows in sub-batches of HB steps.
    constexpr int WB = 128, HB = 64;
    const int j = threadIdx.x & 15;
    const int e = blockIdx.x * (blockDim.x >> 4) + (threadIdx.x >> 4);
    const bool live = e < n_expert;
    const float *wr = w + (size_t)(live ? e : 0) * hidden;
    float wv[WB];
    const int full = hidden / (16 * WB) * (16 * WB);
    if (full > 0) {
#pragma unroll
        for (int u = 0; u < WB; u++) wv[u] = __ldg(wr + u * 16 + j);
    }
    pdl_wait();
    float acc = 0.0f;
    for (int base = 0; base < full; base += 16 * WB) {
#pragma unroll
        for (int sub = 0; sub < WB / HB; sub++) {
            float hv[HB];
#pragma unroll
            for (int u = 0; u < HB; u++) hv[u] = h[base + (sub * HB + u) * 16 + j];
#pragma unroll
            for (int u = 0; u < HB; u++) acc = __fmaf_rn(wv[sub * HB + u], hv[u], acc);
        }
        if (base + 16 * WB < full) {
#pragma unroll
            for (int u = 0; u < WB; u++) wv[u] = __ldg(wr + base + 16 * WB + u * 16 + j);
        }
    }
    for (int i = full + j; i < hidden; i += 16) acc = __fmaf_rn(wr[i], h[i], acc);
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
    if (live && j == 0) logits[e] = acc;
}
RNB_GLOBAL void __launch_bounds__(128)
router_logits_kernel(const float *__restrict__ w, const float *__restrict__ h, int n_expert,
                     int hidden, float *__restrict__ logits) {
    router_logits_body(w, h, n_expert, hidden, logits);
}

// Top-k by logit (descending, ties -> lower expert id), weights = softmax over the selected
// logits in rank order: crates/rnb-llm/src/engine/models/shared_expert_moe/routing.rs:18-62;
// same contract as the reference's rnb_moe_route_topk_f32
// (crates/rnb-backend/cuda/cuda/kernels/quant_batch_and_ops.cuh:4782-4912).
// One warp per token; n_expert <= 1024, top_k <= 32.  exp is libm's expf (expf_libm), as the CPU's routing.
// Returns the id this lane selected (lane r holds rank r; other lanes return 0).
__device__ __forceinline__ uint32_t moe_route_topk_warp(const float *logits, int token, int n_expert, int top_k,
                                                        uint32_t *__restrict__ ids_out, float *__restrict__ weights_out) {
    const int lane = threadIdx.x;
    const float *lg = logits + (size_t)token * n_expert;
    uint32_t *ids = ids_out + (size_t)token * top_k;
    float *wts = weights_out + (size_t)token * top_k;
    const int sel = min(min(top_k, n_expert), 32);
    uint32_t taken = 0;  // bit s <-> expert lane + 32*s
    float my_val = 0.0f;
    uint32_t my_id = 0;
    // up to 256 experts: the lane's logits are read once and kept in registers (every round of the selection would
    // otherwise wait on the L2 again)
    constexpr int RC = 8;
    const bool cached = n_expert <= 32 * RC;
    float cv[RC];
    if (cached) {
#pragma unroll
        for (int s = 0; s < RC; s++) cv[s] = lane + 32 * s < n_expert ? __ldcg(lg + lane + 32 * s) : 0.0f;
    }
    for (int r = 0; r < sel; r++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        if (cached) {
#pragma unroll
            for (int s = 0; s < RC; s++) {
                const int e = lane + 32 * s;
                if (e < n_expert && !(taken & (1u << s)) && (bi == 0x7fffffff || cv[s] > best)) {
                    best = cv[s];
                    bi = e;
                }
            }
        } else {
            for (int s = 0, e = lane; e < n_expert; s++, e += 32) {
                if (taken & (1u << s)) continue;
                const float v = __ldcg(lg + e);   // may have been written by other CTAs of the same launch
                if (bi == 0x7fffffff || v > best) {  // ascending e: strict > keeps the lowest id
                    best = v;
                    bi = e;
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) {
                best = ov;
                bi = oi;
            }
        }
        if ((bi & 31) == lane && bi != 0x7fffffff) taken |= 1u << (bi >> 5);
        if (lane == r) {
            my_val = best;
            my_id = (uint32_t)bi;
            ids[r] = my_id;
        }
    }
    const float mx = __shfl_sync(0xffffffffu, my_val, 0);
    float w = lane < sel ? expf_libm(__fsub_rn(my_val, mx)) : 0.0f;   // libm's expf, as the CPU's .exp()
    float sum = 0.0f;
    for (int r = 0; r < sel; r++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, w, r));
    if (lane < sel) wts[lane] = sum != 0.0f ? __fdiv_rn(w, sum) : w;
    return my_id;
}
RNB_GLOBAL void __launch_bounds__(32)
moe_route_topk_kernel(const float *__restrict__ logits, int n_expert, int top_k,
                      uint32_t *__restrict__ ids_out, float *__restrict__ weights_out) {
    pdl_launch_dependents();
    pdl_wait();
    moe_route_topk_warp(logits, (int)blockIdx.x, n_expert, top_k, ids_out, weights_out);
}

// Fills the per-layer job tables of the expert-gathered matvecs from the routed ids:
//   gate_up job e (0..k-1) / (k..2k-1): rows n_ff, weights at base + id*stride, activation hq
//   down job: one job with k parts (weight slice, that expert's activation, route weight)
struct MoeLayerPtrs {
    const uint8_t *gate_base, *up_base, *down_base;
    size_t gate_stride, down_stride;
};
__device__ __forceinline__ void moe_fill_jobs_warp(size_t id, const float *__restrict__ weights, int top_k,
                                                   const MoeLayerPtrs &lp, GemvJob *__restrict__ gate_up_jobs, GemvJob *__restrict__ down_job) {
    const int e = threadIdx.x;
    if (e >= top_k) return;
    gate_up_jobs[e].parts[0].w = lp.gate_base + id * lp.gate_stride;
    gate_up_jobs[top_k + e].parts[0].w = lp.up_base + id * lp.gate_stride;
    down_job->parts[e].w = lp.down_base + id * lp.down_stride;
    down_job->parts[e].scale = weights + e;
}
// Router logits, routing and job tables in one launch (one token): CTAs of one warp compute two
// experts' logits each; the CTA that finishes last (a counter that it re-arms) selects the experts
// and points the expert-gathered matvecs at them.
RNB_GLOBAL void __launch_bounds__(32)
router_route_fill_kernel(const float *__restrict__ w, const float *__restrict__ h, int n_expert, int hidden, float *logits,
                         int top_k, uint32_t *__restrict__ ids_out, float *__restrict__ weights_out, MoeLayerPtrs lp,
                         GemvJob *__restrict__ gate_up_jobs, GemvJob *__restrict__ down_job, int *__restrict__ counter) {
    router_logits_body(w, h, n_expert, hidden, logits);
    __threadfence();   // this CTA's logits are visible device-wide before the CTA is counted
    __syncwarp();
    int last = 0;
    if (threadIdx.x == 0) last = atomicAdd(counter, 1) == (int)gridDim.x - 1;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
    const uint32_t id = moe_route_topk_warp(logits, 0, n_expert, top_k, ids_out, weights_out);   // one token: its row of ids / weights
    moe_fill_jobs_warp(id, weights_out, top_k, lp, gate_up_jobs, down_job);
    if (threadIdx.x == 0) *counter = 0;
}

}  // namespace rnb
