// GGML Q8_K activation quantisation on device, bit-exact with rnb-cpu's
// quantize_q8k_block_ggml (crates/rnb-cpu/src/gemm/activation_q8.rs:149-173), plus the two
// producers that feed it on the decode path (RMSNorm, SiLU·up).
#pragma once
#include "common.cuh"

namespace rnb {

// One warp quantises one 256-element block; lane holds elements 8*lane .. 8*lane+7.
// Writes the device layout (qs / d / bsum16) and, when `ref_block` is given, the reference's
// 292-byte Q8KBlock as well.
__device__ __forceinline__ void q8k_quantize_block_warp(const float (&v)[8], int lane,
                                                        int8_t *qs_out, float *d_out,
                                                        int16_t *bsum16_out, uint8_t *ref_block) {
    // first element with the strictly largest |x|
    float amax = 0.0f, mval = 0.0f;
    int idx = 256;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float ax = fabsf(v[j]);
        if (ax > amax) {
            amax = ax;
            mval = v[j];
            idx = lane * 8 + j;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float oa = __shfl_xor_sync(0xffffffffu, amax, o);
        float ov = __shfl_xor_sync(0xffffffffu, mval, o);
        int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oa > amax || (oa == amax && oi < idx)) {
            amax = oa;
            mval = ov;
            idx = oi;
        }
    }
    int q[8];
    float d = 0.0f;
    if (amax == 0.0f) {
#pragma unroll
        for (int j = 0; j < 8; j++) q[j] = 0;
    } else {
        const float iscale = __fdiv_rn(-127.0f, mval);
        d = __fdiv_rn(1.0f, iscale);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            int r = __float2int_rn(__fmul_rn(iscale, v[j]));  // ties to even
            q[j] = r > 127 ? 127 : r;                        // upper clamp only
        }
    }
    int s = 0;
#pragma unroll
    for (int j = 0; j < 8; j++) s += q[j];
    const int s16 = s + __shfl_xor_sync(0xffffffffu, s, 1);      // 16-element sum
    const uint32_t w0 = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) |
                        ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    const uint32_t w1 = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) |
                        ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    if (qs_out) {
        *reinterpret_cast<uint2 *>(qs_out + lane * 8) = make_uint2(w0, w1);
        if (lane == 0) *d_out = d;
        if ((lane & 1) == 0) bsum16_out[lane >> 1] = (int16_t)s16;
    }
    if (ref_block) {
        uint32_t *words = reinterpret_cast<uint32_t *>(ref_block);  // 292 = 4*73: 4-byte aligned
        if (lane == 0) words[0] = __float_as_uint(d);
        words[1 + lane * 2] = w0;
        words[2 + lane * 2] = w1;
        if ((lane & 1) == 0)
            reinterpret_cast<int16_t *>(ref_block + 260)[lane >> 1] = (int16_t)s16;
    }
}

struct Q8kDevView {
    int8_t *qs;
    float *d;
    int16_t *bsum16;
};
__device__ __forceinline__ Q8kDevView q8k_dev_view(uint8_t *base, int cols) {
    Q8kDevView v;
    const int nb = cols / 256;
    v.qs = reinterpret_cast<int8_t *>(base);
    v.bsum16 = reinterpret_cast<int16_t *>(base + cols);
    v.d = reinterpret_cast<float *>(base + cols + 32 * nb);
    return v;
}

// x: [seq][cols] f32.  dev_out: [seq] device-layout vectors (stride q8k_dev_bytes(cols)), may
// be null.  ref_out: [seq][cols/256] reference 292-byte blocks, may be null.
RNB_GLOBAL void __launch_bounds__(128)
quantize_q8k_kernel(const float *__restrict__ x, int cols, int seq, uint8_t *dev_out,
                    uint8_t *ref_out) {
    pdl_launch_dependents();
    pdl_wait();
    const int nb = cols / 256;
    const int lane = threadIdx.x & 31;
    const int gb = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (gb >= nb * seq) return;
    const int s = gb / nb, b = gb % nb;
    const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)s * cols + b * 256 + lane * 8);
    const float4 a = src[0], c = src[1];
    const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
    Q8kDevView dv{nullptr, nullptr, nullptr};
    if (dev_out) dv = q8k_dev_view(dev_out + (size_t)s * q8k_dev_bytes(cols), cols);
    q8k_quantize_block_warp(v, lane, dev_out ? dv.qs + b * 256 : nullptr, dv.d + b,
                            dv.bsum16 + b * 16,
                            ref_out ? ref_out + ((size_t)s * nb + b) * Q8K_BYTES : nullptr);
}

// RMSNorm with an f64 mean square and (x / rms) * w, as rnb-cpu's rms_norm_into_f64
// (crates/rnb-cpu/src/kernels/norm.rs:177-196), fused with the Q8_K quantisation of the
// result.  One CTA per token.  `h_out` (f32 normalised vector) is optional.
template <int THREADS>
RNB_GLOBAL void __launch_bounds__(THREADS)
rmsnorm_q8k_kernel(const float *__restrict__ x, const float *__restrict__ w, float eps, int hidden,
                   float *__restrict__ h_out, uint8_t *__restrict__ xq_out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ double red[THREADS / 32];
    __shared__ float s_rms;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *xs = x + (size_t)blockIdx.x * hidden;
    double ss = 0.0;
    for (int i = tid; i < hidden; i += THREADS) {
        const double v = (double)xs[i];
        ss += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int i = 0; i < THREADS / 32; i++) t += red[i];
        s_rms = (float)sqrt(t / (double)hidden + (double)eps);
    }
    __syncthreads();
    const float rms = s_rms;
    const int nb = hidden / 256;
    Q8kDevView dv{nullptr, nullptr, nullptr};
    if (xq_out) dv = q8k_dev_view(xq_out + (size_t)blockIdx.x * q8k_dev_bytes(hidden), hidden);
    for (int b = warp; b < nb; b += THREADS / 32) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int i = b * 256 + lane * 8 + j;
            v[j] = __fmul_rn(__fdiv_rn(xs[i], rms), w[i]);
        }
        if (h_out) {
            float *ho = h_out + (size_t)blockIdx.x * hidden + b * 256 + lane * 8;
            *reinterpret_cast<float4 *>(ho) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4 *>(ho + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
        if (xq_out) q8k_quantize_block_warp(v, lane, dv.qs + b * 256, dv.d + b, dv.bsum16 + b * 16, nullptr);
    }
}

// The same for one token, spread over hidden / 256 CTAs: every CTA sums the squares of the whole
// vector (same order in every CTA, so all agree on the rms to the bit) and then normalises and
// quantises its own 256-element block.  One CTA doing all blocks in turn spends most of its time
// in dependent latency; this form is a single round of loads, one reduction and one block.
RNB_GLOBAL void __launch_bounds__(128)
rmsnorm_q8k_blocks_kernel(const float *__restrict__ x, const float *__restrict__ w, float eps, int hidden,
                          float *__restrict__ h_out, uint8_t *__restrict__ xq_out, const PeerWait pw = PeerWait{}) {
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, b = blockIdx.x;
    // the norm weights do not depend on the previous kernel
    const float4 w0 = __ldg(reinterpret_cast<const float4 *>(w + b * 256 + lane * 8)), w1 = __ldg(reinterpret_cast<const float4 *>(w + b * 256 + lane * 8 + 4));
    pdl_wait();
    peer_wait(pw);   // sharded decode: the other ranks' slices of x arrive by peer stores
    __shared__ double red[4];
    double ss = 0.0;
    for (int i = tid * 4; i < hidden; i += 128 * 4) {
        const float4 v = *reinterpret_cast<const float4 *>(x + i);
        ss += (double)v.x * (double)v.x;
        ss += (double)v.y * (double)v.y;
        ss += (double)v.z * (double)v.z;
        ss += (double)v.w * (double)v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp != 0) return;
    const double total = ((red[0] + red[1]) + red[2]) + red[3];
    const float rms = (float)sqrt(total / (double)hidden + (double)eps);
    const float4 a = *reinterpret_cast<const float4 *>(x + b * 256 + lane * 8), c = *reinterpret_cast<const float4 *>(x + b * 256 + lane * 8 + 4);
    const float xv[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w}, wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = __fmul_rn(__fdiv_rn(xv[j], rms), wv[j]);
    if (h_out) {
        float *ho = h_out + b * 256 + lane * 8;
        *reinterpret_cast<float4 *>(ho) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(ho + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (xq_out) {
        Q8kDevView dv = q8k_dev_view(xq_out, hidden);
        q8k_quantize_block_warp(v, lane, dv.qs + b * 256, dv.d + b, dv.bsum16 + b * 16, nullptr);
    }
}

// act = silu(gate) * up with g / (1 + exp(-g)) (crates/rnb-cpu/src/kernels/activation.rs:74-89),
// fused with Q8_K quantisation.  exp is libm's expf evaluated as the C library does (expf_libm),
// so the value fed to the quantiser has the CPU's bits.
RNB_GLOBAL void __launch_bounds__(128)
silu_mul_q8k_kernel(const float *__restrict__ gate, const float *__restrict__ up, int n, int seq,
                    float *__restrict__ act_out, uint8_t *__restrict__ xq_out) {
    pdl_launch_dependents();
    pdl_wait();
    const int nb = n / 256;
    const int lane = threadIdx.x & 31;
    const int gb = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (gb >= nb * seq) return;
    const int s = gb / nb, b = gb % nb;
    const size_t off = (size_t)s * n + b * 256 + lane * 8;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float g = gate[off + j];
        const float e = expf_libm(-g);   // libm's expf, as the CPU's (-g).exp()
        v[j] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, e)), up[off + j]);
    }
    if (act_out) {
        *reinterpret_cast<float4 *>(act_out + off) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(act_out + off + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (xq_out) {
        Q8kDevView dv = q8k_dev_view(xq_out + (size_t)s * q8k_dev_bytes(n), n);
        q8k_quantize_block_warp(v, lane, dv.qs + b * 256, dv.d + b, dv.bsum16 + b * 16, nullptr);
    }
}

}  // namespace rnb
