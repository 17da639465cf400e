// KV-cache append (RoPE + f32->f16) and split-KV flash-decode attention with GQA, head_dim 128.
//
// Layouts follow the reference everywhere: q/out f32 [head][128]; K/V f16 [pos][kv_head][128]
// (crates/rnb-cpu/src/kernels/attention/decode_flash.rs:13-15,
//  crates/rnb-backend/cuda/cuda/kernels/gdn_attention.cuh:1733-1734).
// Decode attention is a pure KV stream: each K/V row is read from HBM once per KV group and
// shared by the `group` query heads that map to it; all arithmetic is fp32.
#pragma once
#include "common.cuh"
#include "q8k.cuh"

namespace rnb {

constexpr int HD = 128;

// RoPE on q and k with a host-built cos/sin table row (the reference's fused path also builds
// its tables on the host: crates/rnb-backend/cuda/src/runtime/state/rope_cache.rs:33-54; the
// values here come from the CPU angle chain of crates/rnb-cpu/src/kernels/rope.rs:267-293),
// then K/V rows are rounded to f16 (round-to-nearest-even, as half::f16::from_f32 in
// crates/rnb-llm/src/kv_cache.rs:126-141) and written at row `pos` of the layer's cache.
// grid = num_heads + 2*num_kv_heads CTAs of 64 threads; thread i owns rotation pair i.
// rope_table: [max_pos][2][64] (cos then sin) indexed by position when table_by_pos != 0,
// else a single row.  Position = *pos_dev (optional device scalar) + pos_offset.
RNB_GLOBAL void __launch_bounds__(64)
rope_kv_append_kernel(float *__restrict__ q, const float *__restrict__ k,
                      const float *__restrict__ v, const float *__restrict__ rope_table,
                      const int *__restrict__ pos_dev, int pos_offset, int table_by_pos,
                      int num_heads, int num_kv_heads, int neox, uint16_t *__restrict__ k_cache,
                      uint16_t *__restrict__ v_cache, uint16_t *__restrict__ k_row_out,
                      uint16_t *__restrict__ v_row_out) {
    pdl_launch_dependents();
    pdl_wait();
    const int pos = (pos_dev ? *pos_dev : 0) + pos_offset;
    const int i = threadIdx.x;
    const float *cs = rope_table + (size_t)(table_by_pos ? pos : 0) * 128;
    const float c = cs[i], s = cs[64 + i];
    const int i0 = neox ? i : 2 * i, i1 = neox ? i + 64 : 2 * i + 1;
    int h = blockIdx.x;
    if (h < num_heads) {
        float *qh = q + (size_t)h * HD;
        const float x0 = qh[i0], x1 = qh[i1];
        qh[i0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        qh[i1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
        return;
    }
    h -= num_heads;
    const size_t kv_dim = (size_t)num_kv_heads * HD;
    if (h < num_kv_heads) {
        const float *kh = k + (size_t)h * HD;
        const float x0 = kh[i0], x1 = kh[i1];
        const uint16_t r0 = __half_as_ushort(__float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s))));
        const uint16_t r1 = __half_as_ushort(__float2half_rn(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c))));
        if (k_cache) {
            uint16_t *dst = k_cache + (size_t)pos * kv_dim + (size_t)h * HD;
            dst[i0] = r0;
            dst[i1] = r1;
        }
        if (k_row_out) {
            k_row_out[(size_t)h * HD + i0] = r0;
            k_row_out[(size_t)h * HD + i1] = r1;
        }
        return;
    }
    h -= num_kv_heads;
    const float *vh = v + (size_t)h * HD;
    const uint16_t r0 = __half_as_ushort(__float2half_rn(vh[i])),
                   r1 = __half_as_ushort(__float2half_rn(vh[i + 64]));
    if (v_cache) {
        uint16_t *dst = v_cache + (size_t)pos * kv_dim + (size_t)h * HD;
        dst[i] = r0;
        dst[i + 64] = r1;
    }
    if (v_row_out) {
        v_row_out[(size_t)h * HD + i] = r0;
        v_row_out[(size_t)h * HD + i + 64] = r1;
    }
}

// Plain f32 -> f16 row append (no RoPE) for callers that rotate elsewhere.
RNB_GLOBAL void kv_append_f16_kernel(const float *__restrict__ src, uint16_t *__restrict__ dst,
                                     size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __half_as_ushort(__float2half_rn(src[i]));
}

// ---- split-KV flash decode ------------------------------------------------------------------
// grid = (num_kv_heads, n_chunks); 128 threads.  Chunk c covers positions
// [c*chunk_len, min(kv_len, (c+1)*chunk_len)) with chunk_len = ceil(kv_len / n_chunks) rounded
// up to 8.  Warp w walks positions c0+w, c0+w+4, ...; lane l owns dims 4l..4l+3 of the row.
// Per (head, chunk) the kernel writes an un-normalised accumulator, the running max and the
// running sum into `partials` ([num_heads][n_chunks][HD + 2] floats); flash_decode_reduce
// merges chunks with the usual log-sum-exp rule.
constexpr int FD_THREADS = 128;
constexpr int FD_PART_STRIDE = HD + 2;

// four consecutive K/V elements as f32, from an f16 cache (decode) or f32 tensors (prefill API)
__device__ __forceinline__ float4 kv_load4(const uint16_t *p) {
    const uint2 b = ldg_nc_u2(p);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&b.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&b.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ float4 kv_load4(const float *p) {
    const uint4 b = ldg_nc_u4(p);
    return make_float4(__uint_as_float(b.x), __uint_as_float(b.y), __uint_as_float(b.z),
                       __uint_as_float(b.w));
}

// G = query heads handled per pass (<= group size).  When `direct_out` is given the merged,
// normalised result is written there ([head][128]) instead of a partial record.
template <int G, typename KVT>
__device__ __forceinline__ void fd_process(const float *__restrict__ q, const KVT *__restrict__ k,
                                           const KVT *__restrict__ v, int kv_h, int head0,
                                           int heads_here, size_t kv_dim, int p_begin, int p_end,
                                           float scale, int n_chunks, int chunk,
                                           float *__restrict__ partials, float *s_acc, float *s_ml,
                                           float *__restrict__ direct_out = nullptr) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float qr[G][4], acc[G][4], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
        const float4 qv = g < heads_here
                              ? *reinterpret_cast<const float4 *>(q + (size_t)(head0 + g) * HD + 4 * lane)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
        qr[g][0] = qv.x * scale;
        qr[g][1] = qv.y * scale;
        qr[g][2] = qv.z * scale;
        qr[g][3] = qv.w * scale;
        acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
        m[g] = -INFINITY;
        l[g] = 0.f;
    }
    const size_t head_off = (size_t)kv_h * HD + 4 * lane;
#pragma unroll 2
    for (int p = p_begin + warp; p < p_end; p += FD_THREADS / 32) {
        const float4 kk = kv_load4(k + (size_t)p * kv_dim + head_off);
        const float4 vv = kv_load4(v + (size_t)p * kv_dim + head_off);
        float sc[G];
#pragma unroll
        for (int g = 0; g < G; g++)
            sc[g] = qr[g][0] * kk.x + qr[g][1] * kk.y + qr[g][2] * kk.z + qr[g][3] * kk.w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int g = 0; g < G; g++) sc[g] += __shfl_xor_sync(0xffffffffu, sc[g], o);
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float mn = fmaxf(m[g], sc[g]);
            const float corr = expf(m[g] - mn);  // m = -inf on the first position -> 0
            const float pw = expf(sc[g] - mn);
            acc[g][0] = acc[g][0] * corr + pw * vv.x;
            acc[g][1] = acc[g][1] * corr + pw * vv.y;
            acc[g][2] = acc[g][2] * corr + pw * vv.z;
            acc[g][3] = acc[g][3] * corr + pw * vv.w;
            l[g] = l[g] * corr + pw;
            m[g] = mn;
        }
    }
    // merge the 4 warps' states through shared memory
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; g++) {
        float *a = s_acc + ((size_t)(warp * G + g)) * HD + 4 * lane;
        a[0] = acc[g][0];
        a[1] = acc[g][1];
        a[2] = acc[g][2];
        a[3] = acc[g][3];
        if (lane == 0) {
            s_ml[(warp * G + g) * 2] = m[g];
            s_ml[(warp * G + g) * 2 + 1] = l[g];
        }
    }
    __syncthreads();
    for (int g = 0; g < heads_here; g++) {
        const int d = threadIdx.x;  // 128 threads <-> 128 dims
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < FD_THREADS / 32; w++) M = fmaxf(M, s_ml[(w * G + g) * 2]);
        float a = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < FD_THREADS / 32; w++) {
            const float mw = s_ml[(w * G + g) * 2];
            const float f = mw == -INFINITY ? 0.f : expf(mw - M);
            a += s_acc[((size_t)(w * G + g)) * HD + d] * f;
            L += s_ml[(w * G + g) * 2 + 1] * f;
        }
        if (direct_out) {
            direct_out[(size_t)(head0 + g) * HD + d] = L > 0.f ? a / L : 0.f;
            continue;
        }
        float *out = partials + ((size_t)(head0 + g) * n_chunks + chunk) * FD_PART_STRIDE;
        out[d] = a;
        if (d == 0) {
            out[HD] = M;
            out[HD + 1] = L;
        }
    }
}

RNB_GLOBAL void __launch_bounds__(FD_THREADS)
flash_decode_partials_kernel(const float *__restrict__ q, const uint16_t *__restrict__ k,
                             const uint16_t *__restrict__ v, const int *__restrict__ kv_len_dev,
                             int kv_len_host, int num_heads, int num_kv_heads, float scale,
                             float *__restrict__ partials) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_acc[(FD_THREADS / 32) * 4 * HD];
    __shared__ float s_ml[(FD_THREADS / 32) * 4 * 2];
    const int kv_len = kv_len_dev ? *kv_len_dev + kv_len_host : kv_len_host;
    const int n_chunks = gridDim.y, chunk = blockIdx.y, kv_h = blockIdx.x;
    int chunk_len = (kv_len + n_chunks - 1) / n_chunks;
    chunk_len = (chunk_len + 7) & ~7;
    const int p_begin = min(kv_len, chunk * chunk_len), p_end = min(kv_len, p_begin + chunk_len);
    const int group = num_heads / num_kv_heads;
    const size_t kv_dim = (size_t)num_kv_heads * HD;
    for (int g0 = 0; g0 < group; g0 += 4) {
        const int here = min(4, group - g0);
        fd_process<4, uint16_t>(q, k, v, kv_h, kv_h * group + g0, here, kv_dim, p_begin, p_end,
                                scale, n_chunks, chunk, partials, s_acc, s_ml);
        __syncthreads();
    }
}

// grid = num_heads, 128 threads (one per output dim).
RNB_GLOBAL void __launch_bounds__(HD)
flash_decode_reduce_kernel(const float *__restrict__ partials, int n_chunks,
                           float *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, d = threadIdx.x;
    const float *base = partials + (size_t)h * n_chunks * FD_PART_STRIDE;
    float M = -INFINITY;
#pragma unroll 8
    for (int c = 0; c < n_chunks; c++) M = fmaxf(M, base[(size_t)c * FD_PART_STRIDE + HD]);
    float a = 0.f, L = 0.f;
#pragma unroll 8
    for (int c = 0; c < n_chunks; c++) {
        const float *pc = base + (size_t)c * FD_PART_STRIDE;
        const float mc = pc[HD];
        const float f = mc == -INFINITY ? 0.f : expf(mc - M);
        a += pc[d] * f;
        L += pc[HD + 1] * f;
    }
    out[(size_t)h * HD + d] = L > 0.f ? a / L : 0.f;
}

// Chunk merge fused with the Q8_K quantisation of the attention output (the o_proj input):
// grid = num_heads / 2, 256 threads; two heads are exactly one 256-element Q8_K block.
// The 128 threads of a head first agree on the global max and the per-chunk rescale factors
// (kept in shared memory), then each sums its output dimension over the chunks.
constexpr int FD_MAX_CHUNKS = 1024;
RNB_GLOBAL void __launch_bounds__(2 * HD)
flash_decode_reduce_q8k_kernel(const float *__restrict__ partials, int n_chunks, int num_heads,
                               float *__restrict__ out, uint8_t *__restrict__ xq_out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(16) float s_out[2 * HD];
    __shared__ float s_f[2][FD_MAX_CHUNKS];
    __shared__ float s_red[2][4];
    const int hs = threadIdx.x >> 7, d = threadIdx.x & (HD - 1), wq = d >> 5, lane = d & 31;
    const int h = blockIdx.x * 2 + hs;
    const float *base = partials + (size_t)h * n_chunks * FD_PART_STRIDE;
    float m = -INFINITY;
    for (int c = d; c < n_chunks; c += HD) m = fmaxf(m, base[(size_t)c * FD_PART_STRIDE + HD]);
    m = warp_max(m);
    if (lane == 0) s_red[hs][wq] = m;
    __syncthreads();
    const float M = fmaxf(fmaxf(s_red[hs][0], s_red[hs][1]), fmaxf(s_red[hs][2], s_red[hs][3]));
    __syncthreads();
    float l = 0.f;
    for (int c = d; c < n_chunks; c += HD) {
        const float mc = base[(size_t)c * FD_PART_STRIDE + HD];
        const float f = mc == -INFINITY ? 0.f : expf(mc - M);
        s_f[hs][c] = f;
        l += base[(size_t)c * FD_PART_STRIDE + HD + 1] * f;
    }
    l = warp_sum(l);
    if (lane == 0) s_red[hs][wq] = l;
    __syncthreads();
    const float L = (s_red[hs][0] + s_red[hs][1]) + (s_red[hs][2] + s_red[hs][3]);
    float a = 0.f;
#pragma unroll 8
    for (int c = 0; c < n_chunks; c++) a += base[(size_t)c * FD_PART_STRIDE + d] * s_f[hs][c];
    const float o = L > 0.f ? a / L : 0.f;
    if (out) out[(size_t)h * HD + d] = o;
    s_out[threadIdx.x] = o;
    __syncthreads();
    if (threadIdx.x < 32) {
        const float4 v0 = *reinterpret_cast<const float4 *>(s_out + lane * 8), v1 = *reinterpret_cast<const float4 *>(s_out + lane * 8 + 4);
        const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        Q8kDevView dv = q8k_dev_view(xq_out, num_heads * HD);
        const int b = blockIdx.x;
        q8k_quantize_block_warp(v, lane, dv.qs + b * 256, dv.d + b, dv.bsum16 + b * 16, nullptr);
    }
}

}  // namespace rnb
