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
    // gridDim.y > 1: a batch of consecutive tokens (prefill), token t = blockIdx.y at position base + t,
    // its q/k/v rows t * (heads or kv heads) * 128 further on
    q += (size_t)blockIdx.y * num_heads * HD;
    k += (size_t)blockIdx.y * num_kv_heads * HD;
    v += (size_t)blockIdx.y * num_kv_heads * HD;
    const int pos = (pos_dev ? *pos_dev : 0) + pos_offset + (int)blockIdx.y;
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

// The same work for a batch of consecutive tokens (prefill): one CTA of 256 threads per token,
// thread (g = tid / 64, i = tid % 64) owns rotation pair i of heads g, g + 4, ... - the cos/sin of
// the pair is read once.  Same arithmetic and rounding as rope_kv_append_kernel.
RNB_GLOBAL void __launch_bounds__(256)
rope_kv_append_tokens_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v, const float *__restrict__ rope_table,
                             int pos0, int num_heads, int num_kv_heads, int neox, uint16_t *__restrict__ k_cache, uint16_t *__restrict__ v_cache) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, pos = pos0 + t, i = threadIdx.x & 63, g = threadIdx.x >> 6;
    const float *cs = rope_table + (size_t)pos * 128;
    const float c = cs[i], s = cs[64 + i];
    const int i0 = neox ? i : 2 * i, i1 = neox ? i + 64 : 2 * i + 1;
    const size_t kv_dim = (size_t)num_kv_heads * HD;
    float *qt = q + (size_t)t * num_heads * HD;
    for (int h = g; h < num_heads; h += 4) {
        float *qh = qt + (size_t)h * HD;
        const float x0 = qh[i0], x1 = qh[i1];
        qh[i0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        qh[i1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
    const float *kt = k + (size_t)t * kv_dim, *vt = v + (size_t)t * kv_dim;
    uint16_t *kd = k_cache + (size_t)pos * kv_dim, *vd = v_cache + (size_t)pos * kv_dim;
    for (int h = g; h < num_kv_heads; h += 4) {
        const float *kh = kt + (size_t)h * HD;
        const float x0 = kh[i0], x1 = kh[i1];
        kd[(size_t)h * HD + i0] = __half_as_ushort(__float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s))));
        kd[(size_t)h * HD + i1] = __half_as_ushort(__float2half_rn(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c))));
    }
    for (size_t e = threadIdx.x; e < kv_dim; e += 256) vd[e] = __half_as_ushort(__float2half_rn(vt[e]));
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
constexpr int FD_MAX_CHUNKS = 1024;   // merge kernels keep one rescale factor per chunk in shared memory

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

// ---- split-KV flash decode on the tensor cores (f16 caches) ---------------------------------
// Same grid, chunking and partial-record format as flash_decode_partials_kernel, but the K/V
// rows of a chunk are staged in shared memory by 256-byte bulk copies (one per row, completing
// on an mbarrier per 16-position block) and both products run as m16n8k16 MMAs with fp32
// accumulators, with the (up to 8) query heads of a KV group as the N dimension:
//   S^T[pos][head] = K[pos][dim] . Q^T[dim][head]     A = K rows as stored, B = query
//   O^T[dim][head] += V^T[dim][pos] . P^T[pos][head]  A = V rows read transposed, B = P
// K and V are exact f16 values; the pre-scaled f32 query and the f32 probabilities are each
// split into two f16 terms (hi + lo), so the products keep ~22 mantissa bits.
// Warp w owns positions [16w, 16w+16) of each 64-position staging pass and keeps its own
// running (max, sum, O); the four warps are merged through shared memory at the end.
constexpr int FDM_THREADS = 128;
constexpr int FDM_SUPER = 64;             // positions staged per pass
constexpr int FDM_ROW = 2 * HD + 16;      // padded row: ldmatrix without bank conflicts
constexpr int FDM_KV_BYTES = 2 * FDM_SUPER * FDM_ROW;
constexpr int FDM_ACC_STRIDE = HD + 4;    // merge scratch row (floats), padded against conflicts

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ void mma_f16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (x, y) -> f16x2 "hi" and the f16x2 remainder "lo"
__device__ __forceinline__ void split_f16x2(float x, float y, uint32_t &hi, uint32_t &lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}

// PREFILL = false: decode, grid (kv heads, chunks), one query, partial records out.
// PREFILL = true: causal prefill, grid (kv heads, query blocks); the 8 MMA columns are
// (8 / group) consecutive queries x the group's heads, query i sees positions
// 0 .. kv_len - seq_len + i, and the normalised result is written straight to `out`
// ([seq][head][128]); no chunking, the CTA walks all visible positions.
// Optional tail of the decode kernel: the CTA that completes a KV head's last chunk (arrival counter,
// re-armed by that CTA) merges the chunks of the group's query heads and writes the attention
// output as f32 and / or as Q8_K blocks (two heads = one 256-element block), which saves the merge
// launch.  counters: one int per KV head, zero before the launch.
struct FdMerge {
    int *counters;       // null: no counter-based merge
    float *out;          // [heads][128] f32, optional
    uint8_t *xq_out;     // Q8K-dev layout of the heads x 128 vector, optional (needs an even head group)
    int cluster;         // > 0: the launch is one thread-block cluster of this many chunks per KV head; the
                         // cluster's CTA b merges heads 2b, 2b + 1 of the group after a cluster barrier
};
template <bool PREFILL>
__device__ __forceinline__ void fdm_body(const float *__restrict__ q, const uint16_t *__restrict__ k, const uint16_t *__restrict__ v,
                                         const int *__restrict__ kv_len_dev, int kv_len_host, int seq_len, int num_heads, int num_kv_heads,
                                         float scale, float *__restrict__ partials, float *__restrict__ out, int *__restrict__ err_flag,
                                         const FdMerge merge = FdMerge{nullptr, nullptr, nullptr, 0}) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(128) uint8_t s_kv[FDM_KV_BYTES];   // K rows then V rows; merge scratch later
    __shared__ __align__(8) uint64_t s_bar[FDM_SUPER / 16];
    __shared__ float s_ml[(FDM_THREADS / 32) * 8 * 2];
    static_assert((FDM_THREADS / 32) * 8 * FDM_ACC_STRIDE * 4 <= FDM_KV_BYTES, "merge scratch must fit the staging area");
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int kv_len = kv_len_dev ? *kv_len_dev + kv_len_host : kv_len_host;
    const int n_chunks = gridDim.y, chunk = blockIdx.y, kv_h = blockIdx.x;
    const int group = num_heads / num_kv_heads;
    const int qpc = PREFILL ? (group >= 8 ? 1 : 8 / group) : 1;   // queries per CTA
    const int i0 = PREFILL ? (int)blockIdx.y * qpc : 0;
    int p_begin, p_end;
    if (PREFILL) {
        p_begin = 0;
        p_end = max(0, min(kv_len, kv_len - seq_len + min(i0 + qpc, seq_len)));   // what the CTA's last query sees
    } else {
        int chunk_len = (kv_len + n_chunks - 1) / n_chunks;
        chunk_len = (chunk_len + 15) & ~15;
        p_begin = min(kv_len, chunk * chunk_len);
        p_end = min(kv_len, p_begin + chunk_len);
    }
    const size_t kv_dim = (size_t)num_kv_heads * HD;
    uint8_t *s_k = s_kv, *s_v = s_kv + FDM_SUPER * FDM_ROW;
    if (tid < FDM_SUPER / 16) mbar_init(&s_bar[tid], 32);   // 16 K-row + 16 V-row issuers per block
    mbar_fence_init();
    uint32_t phase = 0;
    const int my_row = tid & (FDM_SUPER - 1), my_is_v = tid >> 6;
    const int mi = lane >> 3, mr = lane & 7;   // ldmatrix: this lane addresses row mr of matrix mi

    for (int g0 = 0; g0 < group; g0 += 8) {
        const int heads_here = min(8, group - g0), head0 = kv_h * group + g0;
        const int cols = PREFILL ? heads_here * qpc : heads_here;   // live MMA columns: (query, head) pairs
        // column c -> (query c / heads_here, head c % heads_here); this thread's B-fragment column is g
        const int my_qi = g / heads_here, my_hh = g % heads_here;
        const bool col_live = g < cols && (!PREFILL || i0 + my_qi < seq_len);
        // query B fragments: column g, dims ks*16 + {2t, 2t+1} and + 8
        uint32_t qh[8][2], ql[8][2];
        const float *qrow = q + ((size_t)(PREFILL ? i0 + my_qi : 0) * num_heads + head0 + my_hh) * HD;
#pragma unroll
        for (int ks = 0; ks < 8; ks++)
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                float2 qv = make_float2(0.f, 0.f);
                if (col_live) qv = *reinterpret_cast<const float2 *>(qrow + ks * 16 + hf * 8 + 2 * t);
                split_f16x2(qv.x * scale, qv.y * scale, qh[ks][hf], ql[ks][hf]);
            }
        // causal limit of the two columns this thread owns in the score tile (2t, 2t+1)
        int lim[2] = {kv_len, kv_len};
        if (PREFILL) {
#pragma unroll
            for (int e = 0; e < 2; e++) lim[e] = kv_len - seq_len + i0 + (2 * t + e) / heads_here + 1;
        }
        float o[8][4];   // O^T tile mt: (dim 16mt+g | +8, head 2t | 2t+1)
#pragma unroll
        for (int n = 0; n < 8; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // heads 2t, 2t+1 (l: this thread's share)

        for (int sp = p_begin; sp < p_end; sp += FDM_SUPER) {
            const int n_here = min(FDM_SUPER, p_end - sp);
            __syncthreads();   // everyone is done with the previous pass's rows (and barrier init)
            {
                uint64_t *bar = &s_bar[my_row >> 4];
                if (my_row < n_here) {
                    const uint16_t *src = (my_is_v ? v : k) + (size_t)(sp + my_row) * kv_dim + (size_t)kv_h * HD;
                    mbar_arrive_expect_tx(bar, 2 * HD);
                    bulk_g2s((my_is_v ? s_v : s_k) + my_row * FDM_ROW, src, 2 * HD, bar);
                } else {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
                }
            }
            const int rows = min(16, n_here - 16 * warp);
            if (rows > 0) {
                // rows past the end of a ragged block hold stale bytes: zero them so that a
                // masked probability (0) never meets a NaN/Inf pattern
                if (rows < 16) {
                    const int n_seg = (16 - rows) * 16;   // 16-byte segments per array
                    for (int i = lane; i < 2 * n_seg; i += 32) {
                        const int which = i / n_seg, j = i % n_seg;
                        uint8_t *row = (which ? s_v : s_k) + (16 * warp + rows + j / 16) * FDM_ROW;
                        *reinterpret_cast<uint4 *>(row + (j % 16) * 16) = make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                }
                if (!mbar_wait_bounded(&s_bar[warp], phase)) {
                    if (lane == 0 && err_flag) atomicExch(err_flag, DEV_ERR_MBAR_TIMEOUT);
                } else {
                    // ---- S^T = K Q^T for this warp's 16 positions ----
                    float sc[4] = {0.f, 0.f, 0.f, 0.f};   // (pos g, head 2t) (g, 2t+1) (g+8, 2t) (g+8, 2t+1)
                    const uint32_t k_base = smem_u32(s_k) + (16 * warp + (mi & 1) * 8 + mr) * FDM_ROW + (mi >> 1) * 16;
#pragma unroll
                    for (int ks = 0; ks < 8; ks++) {
                        uint32_t a[4];
                        ldmatrix_x4(a, k_base + ks * 32);
                        mma_f16_16816(sc, a, qh[ks][0], qh[ks][1]);
                        mma_f16_16816(sc, a, ql[ks][0], ql[ks][1]);
                    }
                    if (g >= rows) sc[0] = sc[1] = -INFINITY;
                    if (g + 8 >= rows) sc[2] = sc[3] = -INFINITY;
                    if (PREFILL) {
                        const int pa = sp + 16 * warp + g;   // absolute position of rows g and g + 8
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            if (pa >= lim[e]) sc[e] = -INFINITY;
                            if (pa + 8 >= lim[e]) sc[2 + e] = -INFINITY;
                        }
                    }
                    // ---- online softmax per head (column): max over the 16 positions ----
                    float corr[2], pr[4];
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        float mx = fmaxf(sc[e], sc[2 + e]);
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                        const float m_new = fmaxf(m_run[e], mx);   // stays -inf while everything is masked
                        corr[e] = m_run[e] == -INFINITY ? 0.f : expf(m_run[e] - m_new);
                        pr[e] = sc[e] == -INFINITY ? 0.f : expf(sc[e] - m_new);
                        pr[2 + e] = sc[2 + e] == -INFINITY ? 0.f : expf(sc[2 + e] - m_new);
                        l_run[e] = l_run[e] * corr[e] + (pr[e] + pr[2 + e]);
                        m_run[e] = m_new;
                    }
#pragma unroll
                    for (int n = 0; n < 8; n++) {
                        o[n][0] *= corr[0];
                        o[n][1] *= corr[1];
                        o[n][2] *= corr[0];
                        o[n][3] *= corr[1];
                    }
                    // P^T as B fragments: transpose the two 8x8 (pos x head) tiles across the warp
                    uint32_t p_lo_h, p_lo_l, p_hi_h, p_hi_l;
                    split_f16x2(pr[0], pr[1], p_lo_h, p_lo_l);   // positions 0..7
                    split_f16x2(pr[2], pr[3], p_hi_h, p_hi_l);   // positions 8..15
                    const uint32_t b0h = movmatrix_trans(p_lo_h), b0l = movmatrix_trans(p_lo_l);
                    const uint32_t b1h = movmatrix_trans(p_hi_h), b1l = movmatrix_trans(p_hi_l);
                    // ---- O^T += V^T P^T: A tiles are V[pos][dim] read transposed ----
                    const uint32_t v_base = smem_u32(s_v) + (16 * warp + (mi >> 1) * 8 + mr) * FDM_ROW + (mi & 1) * 16;
#pragma unroll
                    for (int mt = 0; mt < 8; mt++) {
                        uint32_t a[4];
                        ldmatrix_x4_trans(a, v_base + mt * 32);
                        mma_f16_16816(o[mt], a, b0h, b1h);
                        mma_f16_16816(o[mt], a, b0l, b1l);
                    }
                }
            }
            phase ^= 1;
        }
        // ---- merge the four warps (staging area reused as [warp][8 heads][128] f32) ----
#pragma unroll
        for (int e = 0; e < 2; e++) {
            l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 4);
            l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 8);
            l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 16);
        }
        __syncthreads();
        float *s_acc = reinterpret_cast<float *>(s_kv);
#pragma unroll
        for (int mt = 0; mt < 8; mt++) {
            float *r0 = s_acc + (size_t)(warp * 8 + 2 * t) * FDM_ACC_STRIDE + mt * 16 + g;
            r0[0] = o[mt][0];
            r0[FDM_ACC_STRIDE] = o[mt][1];
            r0[8] = o[mt][2];
            r0[FDM_ACC_STRIDE + 8] = o[mt][3];
        }
        if (g == 0) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                s_ml[(warp * 8 + 2 * t + e) * 2] = m_run[e];
                s_ml[(warp * 8 + 2 * t + e) * 2 + 1] = l_run[e];
            }
        }
        __syncthreads();
        for (int hh = 0; hh < cols; hh++) {
            const int d = tid;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < FDM_THREADS / 32; w++) M = fmaxf(M, s_ml[(w * 8 + hh) * 2]);
            float a = 0.f, L = 0.f;
#pragma unroll
            for (int w = 0; w < FDM_THREADS / 32; w++) {
                const float mw = s_ml[(w * 8 + hh) * 2];
                const float f = mw == -INFINITY ? 0.f : expf(mw - M);
                a += s_acc[(size_t)(w * 8 + hh) * FDM_ACC_STRIDE + d] * f;
                L += s_ml[(w * 8 + hh) * 2 + 1] * f;
            }
            if (PREFILL) {
                const int qi = hh / heads_here;
                if (i0 + qi < seq_len) out[((size_t)(i0 + qi) * num_heads + head0 + hh % heads_here) * HD + d] = L > 0.f ? a / L : 0.f;
            } else {
                float *rec = partials + ((size_t)(head0 + hh) * n_chunks + chunk) * FD_PART_STRIDE;
                rec[d] = a;
                if (d == 0) {
                    rec[HD] = M;
                    rec[HD + 1] = L;
                }
            }
        }
        // the next head pass overwrites s_kv through the async proxy after these generic reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (!PREFILL && merge.cluster > 0) {
        // ---- all chunks of this KV head are one cluster: barrier, then CTA b merges the group's heads 2b, 2b + 1 ----
        __threadfence();
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        const int hA = 2 * chunk;                       // first head of this CTA's pair within the group
        if (hA >= group) return;
        float *s_o = reinterpret_cast<float *>(s_kv);   // [2][128] merged rows
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 2; e++) {
            float o_val = 0.f;
            const int head = kv_h * group + hA + e;
            if (hA + e < group) {
                const float *base = partials + (size_t)head * n_chunks * FD_PART_STRIDE;
                float M = -INFINITY;
                for (int c = 0; c < n_chunks; c++) M = fmaxf(M, __ldcg(base + (size_t)c * FD_PART_STRIDE + HD));
                float a = 0.f, L = 0.f;
#pragma unroll 4
                for (int c = 0; c < n_chunks; c++) {
                    const float mc = __ldcg(base + (size_t)c * FD_PART_STRIDE + HD);
                    const float f = mc == -INFINITY ? 0.f : expf(mc - M);
                    L += __ldcg(base + (size_t)c * FD_PART_STRIDE + HD + 1) * f;
                    a += __ldcg(base + (size_t)c * FD_PART_STRIDE + tid) * f;
                }
                o_val = L > 0.f ? a / L : 0.f;
                if (merge.out) merge.out[(size_t)head * HD + tid] = o_val;
            }
            s_o[e * HD + tid] = o_val;
        }
        __syncthreads();
        if (merge.xq_out && warp == 0) {
            const float4 v0 = *(reinterpret_cast<const float4 *>(s_o) + 2 * lane), v1 = *(reinterpret_cast<const float4 *>(s_o) + 2 * lane + 1);
            const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            Q8kDevView dv = q8k_dev_view(merge.xq_out, num_heads * HD);
            const int blk = (kv_h * group) / 2 + chunk;
            q8k_quantize_block_warp(vv, lane, dv.qs + blk * 256, dv.d + blk, dv.bsum16 + blk * 16, nullptr);
        }
        return;
    }
    if (PREFILL || !merge.counters) return;
    // ---- last CTA of this KV head: merge its chunks --------------------------------------------
    __shared__ int s_last;
    __threadfence();   // this CTA's records are visible device-wide before it is counted
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&merge.counters[kv_h], 1) == n_chunks - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float *s_f = reinterpret_cast<float *>(s_kv);                                   // [warp][n_chunks] rescale factors
    float *s_o = reinterpret_cast<float *>(s_kv) + (FDM_THREADS / 32) * FD_MAX_CHUNKS;   // [head of the group][128] merged rows
    static_assert(((FDM_THREADS / 32) * FD_MAX_CHUNKS + 16 * HD) * 4 <= FDM_KV_BYTES, "merge tail scratch must fit the staging area");
    float *my_f = s_f + warp * FD_MAX_CHUNKS;
    for (int g0 = 0; g0 < group; g0 += 16) {
        const int n_here = min(16, group - g0);
        // warp w merges heads w, w + 4, ... of this slice: lane = output dims 4 lane .. 4 lane + 3
        for (int hh = warp; hh < n_here; hh += FDM_THREADS / 32) {
            const int head = kv_h * group + g0 + hh;
            const float *base = partials + (size_t)head * n_chunks * FD_PART_STRIDE;
            float m = -INFINITY;
            for (int c = lane; c < n_chunks; c += 32) m = fmaxf(m, __ldcg(base + (size_t)c * FD_PART_STRIDE + HD));
            const float M = warp_max(m);
            float l = 0.f;
            for (int c = lane; c < n_chunks; c += 32) {
                const float mc = __ldcg(base + (size_t)c * FD_PART_STRIDE + HD);
                const float f = mc == -INFINITY ? 0.f : expf(mc - M);
                my_f[c] = f;
                l += __ldcg(base + (size_t)c * FD_PART_STRIDE + HD + 1) * f;
            }
            const float L = warp_sum(l);
            __syncwarp();
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
            for (int c = 0; c < n_chunks; c++) {
                // records are 130 floats apart: 8-byte alignment is all that holds for every chunk
                const float2 *rp = reinterpret_cast<const float2 *>(base + (size_t)c * FD_PART_STRIDE) + 2 * lane;
                const float2 r0 = __ldcg(rp), r1 = __ldcg(rp + 1);
                const float f = my_f[c];
                a.x += r0.x * f;
                a.y += r0.y * f;
                a.z += r1.x * f;
                a.w += r1.y * f;
            }
            const float4 o4 = L > 0.f ? make_float4(a.x / L, a.y / L, a.z / L, a.w / L) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (merge.out) *(reinterpret_cast<float4 *>(merge.out + (size_t)head * HD) + lane) = o4;
            *(reinterpret_cast<float4 *>(s_o + hh * HD) + lane) = o4;
            __syncwarp();
        }
        __syncthreads();
        if (merge.xq_out) {
            // heads 2b, 2b + 1 of the slice are one Q8_K block; the slice starts at an even head
            for (int bq = warp; 2 * bq + 1 < n_here; bq += FDM_THREADS / 32) {
                const float4 v0 = *(reinterpret_cast<const float4 *>(s_o + 2 * bq * HD) + 2 * lane), v1 = *(reinterpret_cast<const float4 *>(s_o + 2 * bq * HD) + 2 * lane + 1);
                const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                Q8kDevView dv = q8k_dev_view(merge.xq_out, num_heads * HD);
                const int blk = (kv_h * group + g0) / 2 + bq;
                q8k_quantize_block_warp(vv, lane, dv.qs + blk * 256, dv.d + blk, dv.bsum16 + blk * 16, nullptr);
            }
        }
        __syncthreads();
    }
    if (tid == 0) merge.counters[kv_h] = 0;
}

RNB_GLOBAL void __launch_bounds__(FDM_THREADS, 4)
flash_decode_mma_kernel(const float *__restrict__ q, const uint16_t *__restrict__ k,
                        const uint16_t *__restrict__ v, const int *__restrict__ kv_len_dev,
                        int kv_len_host, int num_heads, int num_kv_heads, float scale,
                        float *__restrict__ partials, int *__restrict__ err_flag, const FdMerge merge) {
    fdm_body<false>(q, k, v, kv_len_dev, kv_len_host, 1, num_heads, num_kv_heads, scale, partials, nullptr, err_flag, merge);
}
// Causal prefill attention on the same machinery: grid (kv heads, ceil(seq / queries per CTA)).
RNB_GLOBAL void __launch_bounds__(FDM_THREADS, 4)
prefill_attention_mma_kernel(const float *__restrict__ q, const uint16_t *__restrict__ k, const uint16_t *__restrict__ v, int seq_len,
                             int kv_len, int num_heads, int num_kv_heads, float scale, float *__restrict__ out, int *__restrict__ err_flag) {
    fdm_body<true>(q, k, v, nullptr, kv_len, seq_len, num_heads, num_kv_heads, scale, nullptr, out, err_flag);
}

// Chunk merge: grid = num_heads, 512 threads.  The threads first agree on the global max and
// the per-chunk rescale factors (shared memory), then thread (group g = tid / 128, dim d) sums
// dimension d over the chunks c = g, g + 4, ...; the four groups are added at the end.  A head
// sharded onto one GPU of eight has hundreds of chunks: a serial walk would take tens of us.
RNB_GLOBAL void __launch_bounds__(4 * HD)
flash_decode_reduce_kernel(const float *__restrict__ partials, int n_chunks,
                           float *__restrict__ out, const PeerOut po = PeerOut{}) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_f[FD_MAX_CHUNKS];
    __shared__ float s_red[16];
    __shared__ float s_part[4][HD];
    const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *base = partials + (size_t)h * n_chunks * FD_PART_STRIDE;
    float m = -INFINITY;
    for (int c = tid; c < n_chunks; c += 4 * HD) m = fmaxf(m, base[(size_t)c * FD_PART_STRIDE + HD]);
    m = warp_max(m);
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < 16; i++) M = fmaxf(M, s_red[i]);
    __syncthreads();
    float l = 0.f;
    for (int c = tid; c < n_chunks; c += 4 * HD) {
        const float mc = base[(size_t)c * FD_PART_STRIDE + HD];
        const float f = mc == -INFINITY ? 0.f : expf(mc - M);
        s_f[c] = f;
        l += base[(size_t)c * FD_PART_STRIDE + HD + 1] * f;
    }
    l = warp_sum(l);
    if (lane == 0) s_red[warp] = l;
    __syncthreads();
    float L = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i++) L += s_red[i];
    const int g = tid >> 7, d = tid & (HD - 1);
    float a = 0.f;
#pragma unroll 8
    for (int c = g; c < n_chunks; c += 4) a += base[(size_t)c * FD_PART_STRIDE + d] * s_f[c];
    s_part[g][d] = a;
    __syncthreads();
    if (g == 0) {
        const float t = (s_part[0][d] + s_part[1][d]) + (s_part[2][d] + s_part[3][d]);
        const float o = L > 0.f ? t / L : 0.f;
        out[(size_t)h * HD + d] = o;
        if (po.peers) {
            // sharded decode: the head's row also goes straight into every peer's gathered buffer
            peer_store(po, (size_t)h * HD + d, o);
            __threadfence_system();
        }
    }
    if (po.peers) {
        __syncthreads();
        if (tid == 0) peer_arrive(po);
    }
}

// Chunk merge fused with the Q8_K quantisation of the attention output (the o_proj input):
// grid = num_heads / 2, 256 threads; two heads are exactly one 256-element Q8_K block.
// The 128 threads of a head first agree on the global max and the per-chunk rescale factors
// (kept in shared memory), then each sums its output dimension over the chunks.
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

// Chunk merge fused with the Q8_K quantisation of the attention output (the o_proj input):
// grid = num_heads / 2, 1024 threads; two heads are exactly one 256-element Q8_K block.
// Thread (head hs, chunk group g, dim d): the 512 threads of a head first agree on the global max
// and the per-chunk rescale factors (shared memory), then group g sums dimension d over the chunks
// g, g + 4, ... and the four groups are added in a fixed order.
constexpr int FDR_GROUPS = 4;
RNB_GLOBAL void __launch_bounds__(2 * FDR_GROUPS * HD)
flash_decode_reduce_q8k_wide_kernel(const float *__restrict__ partials, int n_chunks, int num_heads,
                               float *__restrict__ out, uint8_t *__restrict__ xq_out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(16) float s_out[2 * HD];
    __shared__ float s_f[2][FD_MAX_CHUNKS];
    __shared__ float s_red[2][FDR_GROUPS * 4];
    __shared__ float s_part[2][FDR_GROUPS][HD];
    const int tid = threadIdx.x, hs = tid / (FDR_GROUPS * HD), th = tid % (FDR_GROUPS * HD), g = th >> 7, d = th & (HD - 1), wq = th >> 5, lane = tid & 31;
    const int h = blockIdx.x * 2 + hs;
    const float *base = partials + (size_t)h * n_chunks * FD_PART_STRIDE;
    float m = -INFINITY;
    for (int c = th; c < n_chunks; c += FDR_GROUPS * HD) m = fmaxf(m, base[(size_t)c * FD_PART_STRIDE + HD]);
    m = warp_max(m);
    if (lane == 0) s_red[hs][wq] = m;
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < FDR_GROUPS * 4; i++) M = fmaxf(M, s_red[hs][i]);
    __syncthreads();
    float l = 0.f;
    for (int c = th; c < n_chunks; c += FDR_GROUPS * HD) {
        const float mc = base[(size_t)c * FD_PART_STRIDE + HD];
        const float f = mc == -INFINITY ? 0.f : expf(mc - M);
        s_f[hs][c] = f;
        l += base[(size_t)c * FD_PART_STRIDE + HD + 1] * f;
    }
    l = warp_sum(l);
    if (lane == 0) s_red[hs][wq] = l;
    __syncthreads();
    float L = 0.f;
#pragma unroll
    for (int i = 0; i < FDR_GROUPS * 4; i++) L += s_red[hs][i];
    float a = 0.f;
#pragma unroll 8
    for (int c = g; c < n_chunks; c += FDR_GROUPS) a += base[(size_t)c * FD_PART_STRIDE + d] * s_f[hs][c];
    s_part[hs][g][d] = a;
    __syncthreads();
    if (g == 0) {
        const float t = (s_part[hs][0][d] + s_part[hs][1][d]) + (s_part[hs][2][d] + s_part[hs][3][d]);
        const float o = L > 0.f ? t / L : 0.f;
        if (out) out[(size_t)h * HD + d] = o;
        s_out[hs * HD + d] = o;
    }
    __syncthreads();
    if (tid < 32) {
        const float4 v0 = *reinterpret_cast<const float4 *>(s_out + lane * 8), v1 = *reinterpret_cast<const float4 *>(s_out + lane * 8 + 4);
        const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        Q8kDevView dv = q8k_dev_view(xq_out, num_heads * HD);
        const int b = blockIdx.x;
        q8k_quantize_block_warp(v, lane, dv.qs + b * 256, dv.d + b, dv.bsum16 + b * 16, nullptr);
    }
}

// ---------------------------------------------------------------------------------------------
// Reference-order decode attention: the same floating-point operations in the same order as
// rnb-cpu's four-pass decode kernel (crates/rnb-cpu/src/kernels/attention/decode_flash.rs:91-212
// with the f32·f16 helpers of x86_helpers.rs:11-80), so the result is bit-identical to the CPU's:
//   score_j = hsum(16 lanes, each 8 sequential mul-then-add steps over dims 16i + lane) * scale
//   m = max_j score_j;  p_j = expf(score_j - m);  sum = ((p_0 + p_1) + p_2) + ...  (f32, in order)
//   w_j = p_j * (1 / sum);  out_d = ((v_0d * w_0) + v_1d * w_1) + ...              (mul, then add)
// The chunked tensor-core kernel above reassociates all three sums; its result differs in the last
// bits, which the Q8_K rounding of the o_proj input can amplify.  This kernel is the one used for
// short contexts, where the in-order sums cost less than a microsecond.
//
// expf is the C library's on the reference's platform: glibc's single-precision routine evaluates
// 2^(k/32) * P(r) in binary64 (a 32-entry table of 2^(i/32) and a cubic in r) and rounds once to
// f32.  The same evaluation here agrees with it on every input up to the binary64 rounding of
// intermediate steps, which is 2^29 times finer than an f32 ulp.
// ---------------------------------------------------------------------------------------------
constexpr int AX_THREADS = 512;       // two heads per CTA
constexpr int AX_MAX_LEN = 4096;      // scores of both heads: 2 * 4 bytes * 4096 positions = 32 KB
constexpr int AX_STAGE_BYTES = 32768; // staged K or V rows: 128 positions of one KV head, or 64 of two
constexpr int AX_STAGE_VECS = AX_STAGE_BYTES / 16 / AX_THREADS;   // 16-byte loads per thread per tile
inline size_t ax_smem_bytes(int max_len) { return (size_t)AX_STAGE_BYTES + (size_t)max_len * 2 * sizeof(float); }

// One tile of K or V rows into registers (16-byte loads, all in flight together), then into the
// staging buffer.  `shared_kv`: both heads of the CTA read the same KV head, the tile is 128
// positions of it; otherwise 64 positions of each head's KV head (slot = head).
struct AxTile {
    uint4 r[AX_STAGE_VECS];
};
__device__ __forceinline__ void ax_fetch(AxTile &t, const uint16_t *__restrict__ base, size_t kv_dim, size_t off0, size_t off1, bool shared_kv,
                                         int pos0, int kv_len, int tid) {
#pragma unroll
    for (int i = 0; i < AX_STAGE_VECS; i++) {
        const int idx = tid + AX_THREADS * i;
        const int slot = shared_kv ? 0 : idx >> 10, p = shared_kv ? idx >> 4 : (idx & 1023) >> 4, seg = idx & 15;
        t.r[i] = make_uint4(0, 0, 0, 0);
        if (pos0 + p < kv_len) t.r[i] = *reinterpret_cast<const uint4 *>(base + (size_t)(pos0 + p) * kv_dim + (slot ? off1 : off0) + seg * 8);
    }
}
__device__ __forceinline__ void ax_store(const AxTile &t, uint16_t *stage, int tid) {
#pragma unroll
    for (int i = 0; i < AX_STAGE_VECS; i++) *reinterpret_cast<uint4 *>(stage + (size_t)(tid + AX_THREADS * i) * 8) = t.r[i];
}

// grid = ceil(num_heads / 2); dynamic shared memory = ax_smem_bytes(max_len).  Writes `out`
// ([num_heads][128] f32) and/or the Q8_K blocks of the output (`xq_out`, needs an even head
// count: two heads are one 256-element block).  K and V must be 16-byte aligned.  A context
// longer than max_len raises the error flag and writes nothing.
RNB_GLOBAL void __launch_bounds__(AX_THREADS)
attention_decode_exact_kernel(const float *__restrict__ q, const uint16_t *__restrict__ k, const uint16_t *__restrict__ v,
                              const int *__restrict__ kv_len_dev, int kv_len_host, int max_len, int num_heads, int num_kv_heads,
                              float scale, float *__restrict__ out, uint8_t *__restrict__ xq_out, int *__restrict__ err_flag) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) uint8_t s_dyn[];
    uint16_t *stage = reinterpret_cast<uint16_t *>(s_dyn);                    // [slot][position][128]
    float *s_score = reinterpret_cast<float *>(s_dyn + AX_STAGE_BYTES);       // [2][max_len]
    __shared__ unsigned long long s_tab[32];
    __shared__ float s_red[2][8];
    __shared__ float s_inv[2];
    __shared__ __align__(16) float s_o[2 * HD];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kv_len = kv_len_dev ? *kv_len_dev + kv_len_host : kv_len_host;
    if (kv_len < 1 || kv_len > max_len) {
        if (tid == 0 && err_flag) atomicExch(err_flag, DEV_ERR_BAD_JOB);
        return;
    }
    if (tid < 32) s_tab[tid] = c_exp2_tab32[tid];
    const int group = num_heads / num_kv_heads;
    const size_t kv_dim = (size_t)num_kv_heads * HD;
    const int h0 = blockIdx.x * 2, h1 = min(h0 + 1, num_heads - 1);           // an odd head count repeats the last head
    const size_t off0 = (size_t)(h0 / group) * HD, off1 = (size_t)(h1 / group) * HD;
    const bool shared_kv = off0 == off1;
    const int tile_pos = shared_kv ? 128 : 64;
    const int n_tiles = (kv_len + tile_pos - 1) / tile_pos;

    // pass 1: scores.  Half-warp (16 lanes) per position, lane l owns dims 16 i + l.
    {
        const int l16 = lane & 15, hw = tid >> 4;                             // 32 half-warps
        // the two halves of a warp can run different trip counts: shuffles name the own half only
        const unsigned hmask = (lane & 16) ? 0xffff0000u : 0x0000ffffu;
        // shared KV head: every half-warp serves both heads of its positions; else 16 half-warps per head
        const int slot = shared_kv ? 0 : hw >> 4, p_first = shared_kv ? hw : hw & 15, p_step = shared_kv ? 32 : 16;
        const int ha = shared_kv ? h0 : (slot ? h1 : h0), hb = shared_kv ? h1 : ha;
        float qa[8], qb[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            qa[i] = q[(size_t)ha * HD + 16 * i + l16];
            qb[i] = q[(size_t)hb * HD + 16 * i + l16];
        }
        AxTile t;
        ax_fetch(t, k, kv_dim, off0, off1, shared_kv, 0, kv_len, tid);
        for (int ti = 0; ti < n_tiles; ti++) {
            const int pos0 = ti * tile_pos, n_here = min(tile_pos, kv_len - pos0);
            __syncthreads();
            ax_store(t, stage, tid);
            __syncthreads();
            if (ti + 1 < n_tiles) ax_fetch(t, k, kv_dim, off0, off1, shared_kv, pos0 + tile_pos, kv_len, tid);
            for (int p = p_first; p < n_here; p += p_step) {
                const uint16_t *row = stage + ((size_t)slot * 64 + p) * HD + l16;
                float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float kf = __half2float(__ushort_as_half(row[16 * i]));
                    acc0 = __fadd_rn(acc0, __fmul_rn(qa[i], kf));
                    acc1 = __fadd_rn(acc1, __fmul_rn(qb[i], kf));
                }
                // lanes l and l + 8 are the reference's two accumulators; then lo + hi, movehdup, movehl
#pragma unroll
                for (int o = 8; o >= 4; o >>= 1) {
                    acc0 = __fadd_rn(acc0, __shfl_xor_sync(hmask, acc0, o));
                    acc1 = __fadd_rn(acc1, __shfl_xor_sync(hmask, acc1, o));
                }
                acc0 = __fadd_rn(acc0, __shfl_xor_sync(hmask, acc0, 1));
                acc1 = __fadd_rn(acc1, __shfl_xor_sync(hmask, acc1, 1));
                acc0 = __fadd_rn(acc0, __shfl_xor_sync(hmask, acc0, 2));
                acc1 = __fadd_rn(acc1, __shfl_xor_sync(hmask, acc1, 2));
                if (l16 == 0) {
                    if (shared_kv) {
                        s_score[pos0 + p] = __fmul_rn(acc0, scale);
                        s_score[max_len + pos0 + p] = __fmul_rn(acc1, scale);
                    } else {
                        s_score[(size_t)slot * max_len + pos0 + p] = __fmul_rn(acc0, scale);
                    }
                }
            }
        }
    }
    __syncthreads();
    const int hs = warp >> 3, th = tid & 255;                                 // head slot, thread within the head
    const int h = h0 + hs;
    const bool live = h < num_heads;
    float *sc = s_score + (size_t)hs * max_len;
    // V rows of the first tile travel while the softmax runs
    AxTile tv;
    ax_fetch(tv, v, kv_dim, off0, off1, shared_kv, 0, kv_len, tid);
    // pass 2: max
    float m = -INFINITY;
    for (int j = th; j < kv_len; j += 256) m = fmaxf(m, sc[j]);
    m = warp_max(m);
    if (lane == 0) s_red[hs][warp & 7] = m;
    __syncthreads();
    float M = s_red[hs][0];
#pragma unroll
    for (int i = 1; i < 8; i++) M = fmaxf(M, s_red[hs][i]);
    // pass 3: exponentials in parallel, their sum in position order by one thread per head
    for (int j = th; j < kv_len; j += 256) sc[j] = expf_libm_smem(__fsub_rn(sc[j], M), s_tab);
    __syncthreads();
    if (th == 0) {
        float sum = 0.0f;
        int j = 0;
        for (; j + 32 <= kv_len; j += 32) {
            float4 p[8];
#pragma unroll
            for (int u = 0; u < 8; u++) p[u] = *reinterpret_cast<const float4 *>(sc + j + 4 * u);
#pragma unroll
            for (int u = 0; u < 8; u++) sum = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(sum, p[u].x), p[u].y), p[u].z), p[u].w);
        }
        for (; j < kv_len; j++) sum = __fadd_rn(sum, sc[j]);
        s_inv[hs] = sum > 0.0f ? __fdiv_rn(1.0f, sum) : 0.0f;
    }
    __syncthreads();
    // pass 4: weights in parallel, then one thread per output dim walks the positions in order
    {
        const float inv = s_inv[hs];
        for (int j = th; j < kv_len; j += 256) sc[j] = __fmul_rn(sc[j], inv);
    }
    float o = 0.0f;
    const int v_slot = shared_kv ? 0 : hs;
    for (int ti = 0; ti < n_tiles; ti++) {
        const int pos0 = ti * tile_pos, n_here = min(tile_pos, kv_len - pos0);
        __syncthreads();                                                      // weights written / previous tile consumed
        ax_store(tv, stage, tid);
        __syncthreads();
        if (ti + 1 < n_tiles) ax_fetch(tv, v, kv_dim, off0, off1, shared_kv, pos0 + tile_pos, kv_len, tid);
        if (th < HD) {
            const uint16_t *col = stage + (size_t)v_slot * 64 * HD + th;
            const float *w = sc + pos0;
            int p = 0;
            for (; p + 8 <= n_here; p += 8) {
                float x[8], wt[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    x[u] = __half2float(__ushort_as_half(col[(size_t)(p + u) * HD]));
                    wt[u] = w[p + u];
                }
#pragma unroll
                for (int u = 0; u < 8; u++) o = __fadd_rn(o, __fmul_rn(x[u], wt[u]));
            }
            for (; p < n_here; p++) o = __fadd_rn(o, __fmul_rn(__half2float(__ushort_as_half(col[(size_t)p * HD])), w[p]));
        }
    }
    if (th < HD) {
        if (live && out) out[(size_t)h * HD + th] = o;
        s_o[hs * HD + th] = live ? o : 0.0f;
    }
    if (!xq_out) return;
    __syncthreads();
    if (tid < 32) {
        const float4 v0 = *reinterpret_cast<const float4 *>(s_o + lane * 8), v1 = *reinterpret_cast<const float4 *>(s_o + lane * 8 + 4);
        const float vals[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        Q8kDevView dv = q8k_dev_view(xq_out, num_heads * HD);
        const int b = blockIdx.x;
        q8k_quantize_block_warp(vals, lane, dv.qs + b * 256, dv.d + b, dv.bsum16 + b * 16, nullptr);
    }
}

}  // namespace rnb
