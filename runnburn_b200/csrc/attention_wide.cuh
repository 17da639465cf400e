// Decode attention for head_dim 256 and 512 (attention_decode_hd256 / attention_decode_hd512,
// crates/rnb-backend/cuda/src/runtime/api/attention_api.rs:1906-1941,1980-2015; CPU routine
// crates/rnb-cpu/src/kernels/attention/decode_flash.rs:91-212 with head_dim as a parameter).
// Split-KV on CUDA cores in fp32: parity with the CPU routine within the tolerance of the long-context
// hd128 path (the summation order differs by design), not tuned - the tuned kernels are the hd128 ones.
#pragma once
#include "common.cuh"

namespace rnb {

constexpr int AW_THREADS = 128;   // 4 warps per CTA, each walks every fourth position of the chunk
constexpr int AW_MAX_CHUNKS = 256;

// partials: [head][chunk][HD + 2] = unnormalised output, running max, running sum
template <int HD_>
RNB_GLOBAL void __launch_bounds__(AW_THREADS)
attention_wide_partials_kernel(const float *__restrict__ q, const uint16_t *__restrict__ k, const uint16_t *__restrict__ v, int kv_len,
                               int num_heads, int num_kv_heads, float scale, float *__restrict__ partials) {
    constexpr int PER = HD_ / 32;   // dims per lane: 8 (hd256) or 16 (hd512), contiguous
    static_assert(PER % 8 == 0, "a lane reads whole 16-byte groups of f16");
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_acc[AW_THREADS / 32][HD_];
    __shared__ float s_m[AW_THREADS / 32], s_l[AW_THREADS / 32];
    const int head = blockIdx.x, chunk = blockIdx.y, n_chunks = gridDim.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kv_h = head / (num_heads / num_kv_heads);
    const size_t kv_dim = (size_t)num_kv_heads * HD_;
    const int chunk_len = (kv_len + n_chunks - 1) / n_chunks;
    const int p0 = min(kv_len, chunk * chunk_len), p1 = min(kv_len, p0 + chunk_len);
    float qv[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) qv[i] = q[(size_t)head * HD_ + lane * PER + i] * scale;
    float m = -INFINITY, l = 0.f, acc[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) acc[i] = 0.f;
    for (int j = p0 + warp; j < p1; j += AW_THREADS / 32) {
        const uint16_t *kr = k + (size_t)j * kv_dim + (size_t)kv_h * HD_ + lane * PER;
        const uint16_t *vr = v + (size_t)j * kv_dim + (size_t)kv_h * HD_ + lane * PER;
        float kf[PER], vf[PER];
#pragma unroll
        for (int g8 = 0; g8 < PER / 8; g8++) {
            const uint4 kb = *reinterpret_cast<const uint4 *>(kr + 8 * g8), vb = *reinterpret_cast<const uint4 *>(vr + 8 * g8);
            const uint32_t kw[4] = {kb.x, kb.y, kb.z, kb.w}, vw[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                kf[8 * g8 + 2 * i] = f16_bits_to_f32(kw[i] & 0xffffu);
                kf[8 * g8 + 2 * i + 1] = f16_bits_to_f32(kw[i] >> 16);
                vf[8 * g8 + 2 * i] = f16_bits_to_f32(vw[i] & 0xffffu);
                vf[8 * g8 + 2 * i + 1] = f16_bits_to_f32(vw[i] >> 16);
            }
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < PER; i++) s = fmaf(qv[i], kf[i], s);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float m_new = fmaxf(m, s);
        const float corr = m == -INFINITY ? 0.f : expf(m - m_new), p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < PER; i++) acc[i] = fmaf(p, vf[i], acc[i] * corr);
        m = m_new;
    }
#pragma unroll
    for (int i = 0; i < PER; i++) s_acc[warp][lane * PER + i] = acc[i];
    if (lane == 0) {
        s_m[warp] = m;
        s_l[warp] = l;
    }
    __syncthreads();
    // fold the four warps' states in warp order
    float M = -INFINITY;
    for (int w = 0; w < AW_THREADS / 32; w++) M = fmaxf(M, s_m[w]);
    float *dst = partials + ((size_t)head * n_chunks + chunk) * (HD_ + 2);
    for (int d = threadIdx.x; d < HD_; d += AW_THREADS) {
        float o = 0.f;
        for (int w = 0; w < AW_THREADS / 32; w++)
            if (s_m[w] != -INFINITY) o += s_acc[w][d] * expf(s_m[w] - M);
        dst[d] = o;
    }
    if (threadIdx.x == 0) {
        float L = 0.f;
        for (int w = 0; w < AW_THREADS / 32; w++)
            if (s_m[w] != -INFINITY) L += s_l[w] * expf(s_m[w] - M);
        dst[HD_] = M;
        dst[HD_ + 1] = L;
    }
}

template <int HD_>
RNB_GLOBAL void __launch_bounds__(HD_ / 2)
attention_wide_merge_kernel(const float *__restrict__ partials, int n_chunks, float *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x;
    const float *src = partials + (size_t)head * n_chunks * (HD_ + 2);
    float M = -INFINITY;
    for (int c = 0; c < n_chunks; c++) M = fmaxf(M, src[(size_t)c * (HD_ + 2) + HD_]);
    float L = 0.f;
    for (int c = 0; c < n_chunks; c++) {
        const float mc = src[(size_t)c * (HD_ + 2) + HD_];
        if (mc != -INFINITY) L += src[(size_t)c * (HD_ + 2) + HD_ + 1] * expf(mc - M);
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int d = threadIdx.x; d < HD_; d += HD_ / 2) {
        float o = 0.f;
        for (int c = 0; c < n_chunks; c++) {
            const float mc = src[(size_t)c * (HD_ + 2) + HD_];
            if (mc != -INFINITY) o += src[(size_t)c * (HD_ + 2) + d] * expf(mc - M);
        }
        out[(size_t)head * HD_ + d] = o * inv;
    }
}

inline int attention_wide_chunks(size_t kv_len, size_t num_heads, int sm_count) {
    long want = (2L * sm_count + (long)num_heads - 1) / (long)num_heads;
    const long max_c = (long)((kv_len + 31) / 32);
    if (want > max_c) want = max_c;
    if (want > AW_MAX_CHUNKS) want = AW_MAX_CHUNKS;
    return want < 1 ? 1 : (int)want;
}
inline size_t attention_wide_scratch_bytes(size_t num_heads, int n_chunks, size_t head_dim) {
    return num_heads * (size_t)n_chunks * (head_dim + 2) * sizeof(float);
}

}  // namespace rnb
