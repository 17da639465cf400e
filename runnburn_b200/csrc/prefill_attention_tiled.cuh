// Causal prefill attention, query-tiled: one CTA owns 128 (query, head) rows of one KV head -
// 128 / group consecutive query positions x the group's heads - and walks the visible keys in
// tiles of 64, so a K/V tile fetched once serves all 128 rows (the split-KV decode kernel reused
// for prefill served 8).  Arithmetic as in the decode kernel: scores and P*V on mma.sync
// m16n8k16 (f16 operands, fp32 accumulators), q and the probabilities enter as f16 "hi" + f16
// remainder "lo" so that the products keep fp32-level accuracy against the f16 cache;
// softmax(q.K^T * scale).V per head with the online maximum, as rnb-cpu's
// attention_with_scale_window_and_softcap (crates/rnb-cpu/src/kernels/attention/batch_f32.rs:76+);
// query i sees keys 0 .. kv_len - seq_len + i.
//
// 8 warps, warp w owns rows 16w .. 16w+15; row r = (query r / group, head r % group).  K and V
// tiles (64 keys x 128 dims f16, 272-byte padded rows) are double-buffered with cp.async;
// keys past the end of the cache are zero-filled and always masked.
#pragma once
#include "attention.cuh"

namespace rnb {

constexpr int PAT_ROWS = 128;                      // (query, head) rows per CTA
constexpr int PAT_KEYS = 64;                       // keys per tile
constexpr int PAT_THREADS = 256;
constexpr int PAT_PITCH = 2 * HD + 16;             // bytes per padded K/V row
constexpr int PAT_TILE_BYTES = PAT_KEYS * PAT_PITCH;
constexpr size_t PAT_SMEM = 4 * (size_t)PAT_TILE_BYTES;   // 2 stages x (K, V)

// grid = (ceil(seq_len / (128 / group)), num_kv_heads); group = num_heads / num_kv_heads in {1, 2, 4, 8, 16}.
RNB_GLOBAL void __launch_bounds__(PAT_THREADS, 1)
prefill_attention_tiled_kernel(const float *__restrict__ q, const uint16_t *__restrict__ k, const uint16_t *__restrict__ v, int seq_len, int kv_len,
                               int num_heads, int num_kv_heads, float scale, float *__restrict__ out) {
    extern __shared__ __align__(128) uint8_t pat_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = num_heads / num_kv_heads, qpc = PAT_ROWS / group;
    const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;   // long rows first
    const int kv_h = blockIdx.y;
    const int i0 = qb * qpc;
    const int shift = kv_len - seq_len;                    // query i sits at position shift + i
    const int last_q = min(i0 + qpc, seq_len) - 1;
    const int n_keys = min(kv_len, shift + last_q + 1);    // keys visible to the CTA's last query
    const int n_tiles = (n_keys + PAT_KEYS - 1) / PAT_KEYS;
    const uint32_t smem_base = smem_u32(pat_smem);

    // ---- K/V tile t -> stage t & 1: 2 x 64 rows x 16 chunks of 16 bytes, 8 per thread ----
    auto load_tile = [&](int t) {
        const uint32_t st = smem_base + (uint32_t)(t & 1) * 2u * PAT_TILE_BYTES;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int idx = i * PAT_THREADS + tid;          // 0..2047
            const int which = idx >> 10, row = (idx >> 4) & 63, c = idx & 15;
            const int key = t * PAT_KEYS + row;
            const uint16_t *base = which ? v : k;
            const uint16_t *src = base + ((size_t)min(key, kv_len - 1) * num_kv_heads + kv_h) * HD + c * 8;
            const uint32_t nbytes = key < kv_len ? 16u : 0u;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(st + (uint32_t)which * PAT_TILE_BYTES + (uint32_t)row * PAT_PITCH + (uint32_t)c * 16u),
                         "l"(src), "r"(nbytes)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n_tiles > 0) load_tile(0);

    // ---- this thread's two rows: g = lane / 4 -> rows 16w + g and 16w + g + 8 ----
    const int g = lane >> 2, tq = lane & 3;
    int qi[2], hd[2], pos[2];
    bool live[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int r = warp * 16 + g + 8 * h;
        qi[h] = i0 + r / group;
        hd[h] = kv_h * group + r % group;
        live[h] = qi[h] < seq_len;
        pos[h] = live[h] ? shift + qi[h] : kv_len - 1;   // dead rows see everything (finite numbers) and are never stored
    }
    // q A-fragments (hi, lo): k-step ks covers dims 16ks..16ks+15; regs: (row g, dims 2tq..), (row g+8, same), (row g, +8), (row g+8, +8)
    uint32_t qh[8][4], ql[8][4];
#pragma unroll
    for (int ks = 0; ks < 8; ks++)
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int half = 0; half < 2; half++) {
                float2 x = make_float2(0.f, 0.f);
                if (live[h]) x = *reinterpret_cast<const float2 *>(q + ((size_t)qi[h] * num_heads + hd[h]) * HD + ks * 16 + half * 8 + 2 * tq);
                split_f16x2(x.x, x.y, qh[ks][h + 2 * half], ql[ks][h + 2 * half]);
            }
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sl2 = scale * 1.4426950408889634f;   // scores are kept in log2 units: exp(x) = exp2(x * log2 e)
    const int mi = lane >> 3, mr = lane & 7;         // ldmatrix: this lane addresses row mr of matrix mi

    for (int t = 0; t < n_tiles; t++) {
        if (t + 1 < n_tiles) {
            load_tile(t + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const uint32_t k_st = smem_base + (uint32_t)(t & 1) * 2u * PAT_TILE_BYTES, v_st = k_st + PAT_TILE_BYTES;
        // ---- S = q . K^T for 16 rows x 64 keys ----
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            // B fragments of key tile j: matrices (dims 16ks2*2 + 8 mi) for two k-steps per ldmatrix
            const uint32_t row_addr = k_st + (uint32_t)(j * 8 + mr) * PAT_PITCH + (uint32_t)mi * 16u;
#pragma unroll
            for (int kp = 0; kp < 4; kp++) {
                uint32_t b[4];
                ldmatrix_x4(b, row_addr + (uint32_t)kp * 64u);
                mma_f16_16816(s[j], qh[2 * kp], b[0], b[1]);
                mma_f16_16816(s[j], ql[2 * kp], b[0], b[1]);
                mma_f16_16816(s[j], qh[2 * kp + 1], b[2], b[3]);
                mma_f16_16816(s[j], ql[2 * kp + 1], b[2], b[3]);
            }
        }
        // ---- scale, causal mask, online softmax (rows g and g + 8; a row's 64 scores live in a quad) ----
        const int key0 = t * PAT_KEYS + 2 * tq;
        const bool need_mask = t * PAT_KEYS + PAT_KEYS - 1 > min(pos[0], pos[1]);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int h = e >> 1, key = key0 + j * 8 + (e & 1);
                float x = s[j][e] * sl2;
                if (need_mask && key > pos[h]) x = -INFINITY;
                s[j][e] = x;
                mx[h] = fmaxf(mx[h], x);
            }
        float corr[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            m_use[h] = m_new == -INFINITY ? 0.f : m_new;   // a fully masked row so far: keep everything at zero
            corr[h] = exp2f(m_run[h] - m_use[h]);           // exp2(-inf) = 0 on the first tile
            m_run[h] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        uint32_t ph[4][4], pl[4][4];   // P as A fragments of the 4 key k-steps (16 keys each)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
            const float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
            rs[0] += p0 + p1;
            rs[1] += p2 + p3;
            // key tile j = half (j & 1) of k-step j / 2: regs (row g), (row g + 8) then the + 8 keys pair
            split_f16x2(p0, p1, ph[j >> 1][2 * (j & 1)], pl[j >> 1][2 * (j & 1)]);
            split_f16x2(p2, p3, ph[j >> 1][2 * (j & 1) + 1], pl[j >> 1][2 * (j & 1) + 1]);
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
            l_run[h] = l_run[h] * corr[h] + rs[h];
        }
#pragma unroll
        for (int j = 0; j < 16; j++) {
            o[j][0] *= corr[0];
            o[j][1] *= corr[0];
            o[j][2] *= corr[1];
            o[j][3] *= corr[1];
        }
        // ---- O += P . V: k-step kk = keys 16kk..16kk+15, dim tiles jp*2, jp*2+1 per transposed ldmatrix ----
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            const uint32_t row_addr = v_st + (uint32_t)(kk * 16 + (mi & 1) * 8 + mr) * PAT_PITCH + (uint32_t)(mi >> 1) * 16u;
#pragma unroll
            for (int jp = 0; jp < 8; jp++) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, row_addr + (uint32_t)jp * 32u);
                mma_f16_16816(o[2 * jp], ph[kk], b[0], b[1]);
                mma_f16_16816(o[2 * jp], pl[kk], b[0], b[1]);
                mma_f16_16816(o[2 * jp + 1], ph[kk], b[2], b[3]);
                mma_f16_16816(o[2 * jp + 1], pl[kk], b[2], b[3]);
            }
        }
        __syncthreads();   // every warp is done with this stage before the copy of tile t + 2 lands in it
    }
    // ---- normalise and store: row h of this thread, dims 8j + 2tq, + 1 ----
#pragma unroll
    for (int h = 0; h < 2; h++) {
        if (!live[h]) continue;
        const float inv = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;
        float *dst = out + ((size_t)qi[h] * num_heads + hd[h]) * HD + 2 * tq;
#pragma unroll
        for (int j = 0; j < 16; j++) *reinterpret_cast<float2 *>(dst + 8 * j) = make_float2(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
    }
}

}  // namespace rnb
