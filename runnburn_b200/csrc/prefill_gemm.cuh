// Prefill matmul on the 5th-generation tensor cores: Y[t][row] = sum_k W[row][k] * X[t][k] for a
// batch of tokens, W in GGUF Q4_K / Q6_K blocks, dequantised tile-wise to bf16 in shared
// memory and multiplied with tcgen05.mma (bf16 x bf16 -> fp32 accumulators in tensor memory).
// Replaces the reference's dequant -> f16 + cublasGemmEx path (q4k_f16_gemm_batch,
// crates/rnb-backend/cuda/src/runtime/gemv.rs:2335-2421); the dequantisation follows
// crates/rnb-cpu/src/quantize/dequant.rs:353-381 (Q4_K) and :780-807 (Q6_K) in f32 and rounds
// once to bf16.
//
// One CTA owns a 512-token x 128-row output tile: two fp32 accumulators of 128 rows x 256 tokens =
// all 512 columns of the SM's tensor memory; the weight tile is the M operand (TMEM lane = weight
// row), a token half the N operand.  A dequantised weight tile serves 512 tokens - the dequantising
// warps, not the tensor pipe, bounded a 256 x 256 tile.  K advances 64 elements (one Q4_K group, a
// quarter of a super-block) per pipeline stage; a stage holds the token tile (512 x 64 bf16 = 64 KB,
// brought in by two tiled TMA copies; rows past the end of the batch read as zeros) and the weight
// tile (128 x 64 bf16), both K-major in the 128-byte swizzle the MMA descriptors expect:
//   byte offset of (row r, 16-byte chunk c) = (r / 8) * 1024 + (r % 8) * 128 + ((c ^ (r % 8)) * 16).
// Two stages of 80 KB; a stage is refilled as soon as the MMAs that read it have been committed.
// Warp roles: 0-7 dequantise (thread t owns weight row t / 2 and half t % 2 of the 64-element group:
// Q4_K low or high nibbles, Q6_K the first or second 32 elements), thread 0 also issues the token
// copies; warp 8 allocates tensor memory and issues the MMAs (eight per stage: 2 token halves x 4
// K-steps of 16); afterwards warps 0-7 read the accumulators back (tcgen05.ld, one TMEM lane quarter
// per warp) and store f32 rows.  Every wait is bounded; a timeout sets the error flag and all roles
// still meet at the final barrier, where the tensor memory is freed.
#pragma once
#include <cuda_bf16.h>

#include <type_traits>

#include "common.cuh"

namespace rnb {

constexpr int PG_TOK = 512;      // tokens per CTA
constexpr int PG_ROWS = 128;     // weight rows per CTA
constexpr int PG_K = 64;         // elements per stage
constexpr int PG_STAGES = 2;
constexpr int PG_THREADS = 288;
constexpr uint32_t PG_A_BYTES = PG_TOK * 128;    // token tile of a stage
constexpr uint32_t PG_B_BYTES = PG_ROWS * 128;   // weight tile of a stage
constexpr uint32_t PG_STAGE_BYTES = PG_A_BYTES + PG_B_BYTES;
constexpr size_t PG_SMEM = (size_t)PG_STAGES * PG_STAGE_BYTES + 1024;   // + slack to align to 1024
constexpr int PG_BOX_ROWS = 256;                 // tokens per TMA copy

// K-major, 128-byte swizzle, 8-row groups 1024 bytes apart; descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t pg_smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3ffffu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// D = f32, A = B = bf16, both K-major, N = 256 (a token half), M = 128 (the weight rows)
constexpr uint32_t PG_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

__device__ __forceinline__ void pg_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(PG_IDESC), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void pg_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pg_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void pg_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void pg_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void pg_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pg_tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
        "%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
          "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// q in 0..255 -> exact f32 without an int-to-float conversion: 2^23 + q, minus 2^23
__device__ __forceinline__ float pg_byte_to_f32(uint32_t word, int byte) {
    return __uint_as_float(__byte_perm(word, 0x4b000000u, 0x7650 + byte) ) - 8388608.0f;
}
// same, minus 32 (Q6_K's offset): 2^23 + q - (2^23 + 32) is exact
__device__ __forceinline__ float pg_byte_to_f32_m32(uint32_t word, int byte) {
    return __uint_as_float(__byte_perm(word, 0x4b000000u, 0x7650 + byte)) - 8388640.0f;
}
__device__ __forceinline__ uint32_t pg_pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// ---- raw bytes of a weight group (64 elements of one row) --------------------------------------
// The two threads of a row fetch disjoint halves of what both need (the block header once per
// block, the group's 32 qs bytes every stage) and exchange them by shuffle when the bytes are
// used: every byte of a weight tile crosses the L2 -> SM path once.
struct PgRawQ4 {
    uint2 hdr_half;   // bytes 8h .. 8h+7 of {d, dmin, 12 scale bytes}; valid for group 0 of a block
    uint4 qm;         // qs bytes 16h .. 16h+15 of the group
};
__device__ __forceinline__ void pg_load_q4(PgRawQ4 &r, const uint8_t *blk, int g, int h) {
    if (g == 0) r.hdr_half = ldg_nc_u2(blk + 8 * h);
    r.qm = ldg_nc_u4(blk + 16 + 32 * g + 16 * h);
}
__device__ __forceinline__ uint4 pg_pair_exchange(const uint4 &mine) {
    return make_uint4(__shfl_xor_sync(0xffffffffu, mine.x, 1), __shfl_xor_sync(0xffffffffu, mine.y, 1), __shfl_xor_sync(0xffffffffu, mine.z, 1),
                      __shfl_xor_sync(0xffffffffu, mine.w, 1));
}
// Q6_K: group g of a block = elements 64g..64g+63 = for half n = g/2 the pair (q1,q2) if g even,
// (q3,q4) if g odd, l = 0..31 each; y = (d*sc)*(q-32): dequant.rs:780-807.  Blocks are 210 bytes,
// so rows are only 2-byte aligned: bytes are fetched as aligned 16-byte windows and shifted into place (pg_ldg_window).
// f32 -> bf16 rows (activation), padded to a multiple of 8 columns by construction (cols % 256 == 0)
RNB_GLOBAL void __launch_bounds__(256)
f32_to_bf16_kernel(const float *__restrict__ x, uint16_t *__restrict__ y, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= n) return;
    const float4 a = *reinterpret_cast<const float4 *>(x + i), b = *reinterpret_cast<const float4 *>(x + i + 4);
    *reinterpret_cast<uint4 *>(y + i) = make_uint4(pg_pack_bf16(a.x, a.y), pg_pack_bf16(a.z, a.w), pg_pack_bf16(b.x, b.y), pg_pack_bf16(b.z, b.w));
}

// Residual add + RMSNorm of a batch of token rows, written straight as the bf16 token matrix of
// the next matmul: x += t (when t is given; x is updated in place), then (x / rms) * w with the
// f64 mean square of rnb-cpu's rms_norm_into (crates/rnb-cpu/src/kernels/norm.rs:177-196) in the
// reduction order of rmsnorm_q8k_kernel, rounded once to bf16.  One CTA per token; hidden % 8 == 0.
template <int THREADS>
RNB_GLOBAL void __launch_bounds__(THREADS)
add_rmsnorm_bf16_kernel(float *__restrict__ x, const float *__restrict__ t, const float *__restrict__ w, float eps, int hidden,
                        uint16_t *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ double red[THREADS / 32];
    __shared__ float s_rms;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float *xs = x + (size_t)blockIdx.x * hidden;
    double ss = 0.0;
    if (t) {
        const float *ts = t + (size_t)blockIdx.x * hidden;
        for (int i = tid; i < hidden; i += THREADS) {
            const float v = __fadd_rn(xs[i], ts[i]);
            xs[i] = v;
            ss += (double)v * (double)v;
        }
    } else {
        for (int i = tid; i < hidden; i += THREADS) {
            const double v = (double)xs[i];
            ss += v * v;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();   // also orders this CTA's writes of xs before the reads below
    if (tid == 0) {
        double a = 0.0;
        for (int i = 0; i < THREADS / 32; i++) a += red[i];
        s_rms = (float)sqrt(a / (double)hidden + (double)eps);
    }
    __syncthreads();
    const float rms = s_rms;
    uint16_t *os = out + (size_t)blockIdx.x * hidden;
    for (int i = tid * 8; i < hidden; i += THREADS * 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = __fmul_rn(__fdiv_rn(xs[i + j], rms), w[i + j]);
        *reinterpret_cast<uint4 *>(os + i) = make_uint4(pg_pack_bf16(v[0], v[1]), pg_pack_bf16(v[2], v[3]), pg_pack_bf16(v[4], v[5]), pg_pack_bf16(v[6], v[7]));
    }
}

// silu(gate) * up (g / (1 + exp(-g)), crates/rnb-cpu/src/kernels/activation.rs:74-89, libm's expf as in
// silu_mul_q8k_kernel) written straight as the bf16 token matrix of the down
// matmul: the f32 value is rounded to bf16 exactly as f32_to_bf16_kernel would round it.
RNB_GLOBAL void __launch_bounds__(256)
silu_mul_bf16_kernel(const float *__restrict__ gate, const float *__restrict__ up, uint16_t *__restrict__ y, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= n) return;
    const float4 g0 = *reinterpret_cast<const float4 *>(gate + i), g1 = *reinterpret_cast<const float4 *>(gate + i + 4);
    const float4 u0 = *reinterpret_cast<const float4 *>(up + i), u1 = *reinterpret_cast<const float4 *>(up + i + 4);
    const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float e = expf_libm(-gv[j]);
        v[j] = __fmul_rn(__fdiv_rn(gv[j], __fadd_rn(1.0f, e)), uv[j]);
    }
    *reinterpret_cast<uint4 *>(y + i) = make_uint4(pg_pack_bf16(v[0], v[1]), pg_pack_bf16(v[2], v[3]), pg_pack_bf16(v[4], v[5]), pg_pack_bf16(v[6], v[7]));
}

// 128-byte, 64-byte aligned descriptor of the bf16 token matrix [seq][cols] (a CUtensorMap, kept
// opaque here): boxes of 64 columns x 256 tokens, 128-byte swizzle, zero fill past the end.
struct alignas(64) PgTensorMap {
    unsigned long long opaque[16];
};
// tiled 2-D copy global -> shared; x (elements of the inner dimension) * 2 bytes must be a multiple of 16
__device__ __forceinline__ void pg_tma_2d(uint32_t dst, const void *tmap, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

// Up to three matrices that share the token tile go out in one launch (q/k/v, gate/up): the
// x dimension of the grid runs over the 256-row tiles of all of them.
constexpr int PG_MAX_JOBS = 3;
struct PgJob {
    const uint8_t *w;
    float *y;     // [seq][rows]
    int rows, type, tile0, pad;
    // gate + up form (w2 != null): a tile is 64 rows of w (gate) on TMEM lanes 0-63 and the same 64 rows of w2 (up) on
    // lanes 64-127; the epilogue writes silu(gate) * up as bf16 [seq][rows] to yb - the token matrix of the down matmul
    const uint8_t *w2;
    uint16_t *yb;
};
struct PgJobs {
    PgJob j[PG_MAX_JOBS];
    int n;
};

// Half h of a Q4_K group: h = 0 -> low nibbles (chunks 0-3), h = 1 -> high nibbles (chunks 4-7).
// y = (d*sc)*q - (dmin*m) (crates/rnb-cpu/src/quantize/dequant.rs:353-381), evaluated with one fused
// multiply-add per element: the f32 value can differ from the two-rounding form in its last bit,
// which survives the rounding to bf16 only next to a tie.
__device__ __forceinline__ void pg_dequant_q4(const uint4 &hdr, const uint4 &q0, const uint4 &q1, int g, int h, uint8_t *row_base, int rr) {
    const float d = f16_bits_to_f32(hdr.x & 0xffffu), dmin = f16_bits_to_f32(hdr.x >> 16);
    const uint32_t sc03 = hdr.y & 0x3f3f3f3fu, mn03 = hdr.z & 0x3f3f3f3fu;
    const uint32_t sc47 = (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
    const uint32_t mn47 = ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
    const uint32_t scw = g < 2 ? sc03 : sc47, mnw = g < 2 ? mn03 : mn47;
    const int sh = 16 * (g & 1) + 8 * h;
    const float ds = __fmul_rn(d, (float)((scw >> sh) & 0xffu)), nm = -__fmul_rn(dmin, (float)((mnw >> sh) & 0xffu));
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    const int nsh = 4 * h;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        uint32_t o[4];
#pragma unroll
        for (int w = 0; w < 2; w++) {
            const uint32_t n4 = (qw[2 * c + w] >> nsh) & 0x0f0f0f0fu;
            o[2 * w] = pg_pack_bf16(__fmaf_rn(ds, pg_byte_to_f32(n4, 0), nm), __fmaf_rn(ds, pg_byte_to_f32(n4, 1), nm));
            o[2 * w + 1] = pg_pack_bf16(__fmaf_rn(ds, pg_byte_to_f32(n4, 2), nm), __fmaf_rn(ds, pg_byte_to_f32(n4, 3), nm));
        }
        *reinterpret_cast<uint4 *>(row_base + (((c + 4 * h) ^ rr) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}
// Half h of the Q6_K groups of half-block n: h = 0 -> ql[64n .. 64n+31] (q1 / q3), h = 1 -> ql[64n+32 ..] (q2 / q4).
struct PgRawQ6 {
    uint32_t ql[8], qh[4];   // qh: words 4h .. 4h+3 of the half-block's 32 bytes, the pair exchanges them when used
    uint32_t sc[2];
    float d;
};
// NW consecutive words from a 2-byte aligned address out of NV aligned 16-byte loads (4 NV >= NW + 4): the words of the
// loaded window are shifted by whole words with two levels of selects, then funnel-shifted by the odd half-word.  The
// threads of a warp read rows that lie kilobytes apart, so every load instruction costs 32 cache-line accesses
// whatever its width: seven 16-byte loads per half block instead of eighteen 4-byte ones is what lifts the Q6_K
// producer off the load pipe.  An aligned 16-byte load that contains one byte of the tensor cannot leave its page.
template <int NW, int NV>
__device__ __forceinline__ void pg_ldg_window(const uint8_t *p, uint32_t *out, uint32_t *raw = nullptr) {
    static_assert(4 * NV >= NW + 4, "window too small");
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint8_t *base = reinterpret_cast<const uint8_t *>(a & ~(uintptr_t)15);
    const uint32_t off = (uint32_t)(a & 15), k = off >> 2, sh = (off & 3u) * 8u;
    uint32_t v[4 * NV];
#pragma unroll
    for (int j = 0; j < NV; j++) {
        const uint4 t = ldg_nc_u4(base + 16 * j);
        v[4 * j] = t.x, v[4 * j + 1] = t.y, v[4 * j + 2] = t.z, v[4 * j + 3] = t.w;
    }
    if (raw) {
#pragma unroll
        for (int i = 0; i < 4 * NV; i++) raw[i] = v[i];
    }
    uint32_t s1[NW + 2], s2[NW + 1];
#pragma unroll
    for (int i = 0; i < NW + 2; i++) s1[i] = (k & 2u) ? v[i + 2] : v[i];
#pragma unroll
    for (int i = 0; i < NW + 1; i++) s2[i] = (k & 1u) ? s1[i + 1] : s1[i];
#pragma unroll
    for (int i = 0; i < NW; i++) out[i] = __funnelshift_r(s2[i], s2[i + 1], sh);
}
__device__ __forceinline__ void pg_load_q6(PgRawQ6 &r, const uint8_t *blk, int n, int h) {
    pg_ldg_window<8, 3>(blk + 64 * n + 32 * h, r.ql);
    pg_ldg_window<4, 2>(blk + 128 + 32 * n + 16 * h, r.qh);
    // scales (16 bytes at 192) and d (2 bytes at 208): one 18-byte window = two aligned 16-byte loads
    uint32_t sc4[4], raw[8];
    pg_ldg_window<4, 2>(blk + 192, sc4, raw);
    r.sc[0] = n ? sc4[2] : sc4[0];
    r.sc[1] = n ? sc4[3] : sc4[1];
    // d sits 16 bytes after the window's first byte: in the second 16-byte load, at the same offset
    const uint32_t dpos = (uint32_t)(reinterpret_cast<uintptr_t>(blk + 192) & 15u), dk = dpos >> 2;
    const uint32_t dlo = (dk & 2u) ? ((dk & 1u) ? raw[7] : raw[6]) : ((dk & 1u) ? raw[5] : raw[4]);
    r.d = f16_bits_to_f32((dlo >> ((dpos & 2u) * 8u)) & 0xffffu);
}
__device__ __forceinline__ void pg_dequant_q6(const PgRawQ6 &r, int g, int h, uint8_t *row_base, int rr) {
    const bool odd = g & 1;
    uint32_t qh[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t other = __shfl_xor_sync(0xffffffffu, r.qh[i], 1);
        qh[i] = h ? other : r.qh[i];
        qh[4 + i] = h ? r.qh[i] : other;
    }
    const uint32_t scw = (odd ? r.sc[1] : r.sc[0]) >> (16 * h);   // this half's two scale bytes
    const float ds0 = __fmul_rn(r.d, (float)(int)(int8_t)(scw & 0xffu)), ds1 = __fmul_rn(r.d, (float)(int)(int8_t)((scw >> 8) & 0xffu));
    // the two high bits of this half's elements sit at bit 2h (even group) or 4 + 2h (odd group) of qh
    const int hs = (odd ? 4 : 0) + 2 * h;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        uint32_t o[4];
        const float sa = c < 2 ? ds0 : ds1;
#pragma unroll
        for (int w = 0; w < 2; w++) {
            const int i = 2 * c + w;
            const uint32_t lo = (odd ? (r.ql[i] >> 4) : r.ql[i]) & 0x0f0f0f0fu;
            const uint32_t q = lo | (((qh[i] >> hs) << 4) & 0x30303030u);
            o[2 * w] = pg_pack_bf16(__fmul_rn(sa, pg_byte_to_f32_m32(q, 0)), __fmul_rn(sa, pg_byte_to_f32_m32(q, 1)));
            o[2 * w + 1] = pg_pack_bf16(__fmul_rn(sa, pg_byte_to_f32_m32(q, 2)), __fmul_rn(sa, pg_byte_to_f32_m32(q, 3)));
        }
        *reinterpret_cast<uint4 *>(row_base + (((c + 4 * h) ^ rr) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}


// grid = (sum over jobs of ceil(rows / 128), ceil(seq / 512)); 288 threads; dynamic shared memory PG_SMEM.
RNB_GLOBAL void __launch_bounds__(PG_THREADS, 1)
prefill_gemm_kernel(const __grid_constant__ PgJobs jobs, const __grid_constant__ PgTensorMap tmap_x, int seq, int cols,
                         int *__restrict__ err_flag) {
    extern __shared__ __align__(1024) uint8_t pg_smem_raw[];
    __shared__ __align__(8) uint64_t full[PG_STAGES], empty[PG_STAGES], done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int s_failed;
    pdl_launch_dependents();
    pdl_wait();
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(pg_smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int jsel = 0;
    for (int i = 1; i < jobs.n; i++)
        if ((int)blockIdx.x >= jobs.j[i].tile0) jsel = i;
    const PgJob &job = jobs.j[jsel];
    const int rows = job.rows, TYPE = job.type;
    const uint8_t *__restrict__ w = job.w;
    float *__restrict__ y = job.y;
    const uint32_t BLK = TYPE == TYPE_Q4_K ? Q4K_BYTES : Q6K_BYTES;
    const bool pair = job.w2 != nullptr;
    const int n0 = ((int)blockIdx.x - job.tile0) * (pair ? PG_ROWS / 2 : PG_ROWS), m0 = blockIdx.y * PG_TOK;
    const int nb = cols >> 8, KT = cols / PG_K;
    if (tid == 0) {
        for (int s = 0; s < PG_STAGES; s++) {
            mbar_init(&full[s], 9);    // one arrival per producer warp + the thread that issues the token copies
            mbar_init(&empty[s], 1);   // tcgen05.commit
        }
        mbar_init(&done_bar, 1);
        mbar_fence_init();
        s_failed = 0;
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pg_fence_before();
    __syncthreads();
    pg_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    bool ok = true;

    if (warp < 8) {
        const int row = tid >> 1, h = tid & 1, rr = row & 7;
        const size_t rb = (size_t)nb * BLK;
        // rows past the end repeat the last one (never stored)
        const uint8_t *wr = pair ? (row < PG_ROWS / 2 ? w : job.w2) + (size_t)min(n0 + (row & (PG_ROWS / 2 - 1)), rows - 1) * rb
                                 : w + (size_t)min(n0 + row, rows - 1) * rb;
        uint8_t *const brow = smem + PG_A_BYTES + (row >> 3) * 1024 + rr * 128;
        // token tile of stage kt: thread 0 announces the bytes and issues the two copies
        auto issue_tokens = [&](int kt) {
            if (tid != 0) return;
            const int s = kt % PG_STAGES;
            const uint32_t dst = smem_u32(smem + (uint32_t)s * PG_STAGE_BYTES);
            mbar_arrive_expect_tx(&full[s], PG_A_BYTES);
#pragma unroll
            for (int i = 0; i < PG_TOK / PG_BOX_ROWS; i++)
                pg_tma_2d(dst + (uint32_t)i * (PG_BOX_ROWS * 128), &tmap_x, kt * PG_K, m0 + i * PG_BOX_ROWS, &full[s]);
        };
        auto stage_tail = [&](int kt) -> bool {
            pg_proxy_fence();
            __syncwarp();
            if (lane == 0) pg_arrive(&full[kt % PG_STAGES]);
            if (kt + 1 < KT) {
                // the next stage may be written once the MMAs that read it have been committed
                if (!mbar_wait_bounded(&empty[(kt + 1) % PG_STAGES], (uint32_t)((((kt + 1) / PG_STAGES) & 1) ^ 1))) return false;
                issue_tokens(kt + 1);
            }
            return true;
        };
        ok = mbar_wait_bounded(&empty[0], 1u);
        if (ok) issue_tokens(0);
        if (TYPE == TYPE_Q4_K) {
            PgRawQ4 cur, nxt;
            uint4 hdr = make_uint4(0u, 0u, 0u, 0u);
            pg_load_q4(cur, wr, 0, h);
            for (int kt = 0; kt < KT && ok; kt++) {
                const int g = kt & 3;
                if (kt + 1 < KT) pg_load_q4(nxt, wr + (size_t)((kt + 1) >> 2) * BLK, (kt + 1) & 3, h);
                if (g == 0) {   // a new block: put the header halves together
                    const uint32_t ox = __shfl_xor_sync(0xffffffffu, cur.hdr_half.x, 1), oy = __shfl_xor_sync(0xffffffffu, cur.hdr_half.y, 1);
                    hdr = h ? make_uint4(ox, oy, cur.hdr_half.x, cur.hdr_half.y) : make_uint4(cur.hdr_half.x, cur.hdr_half.y, ox, oy);
                }
                const uint4 other = pg_pair_exchange(cur.qm);
                pg_dequant_q4(hdr, h ? other : cur.qm, h ? cur.qm : other, g, h, brow + (uint32_t)(kt % PG_STAGES) * PG_STAGE_BYTES, rr);
                ok = __all_sync(0xffffffffu, stage_tail(kt));   // warp-uniform: the shuffles above need the whole warp
                cur = nxt;
            }
        } else {
            PgRawQ6 cur, nxt;
            pg_load_q6(cur, wr, 0, h);
            for (int kt = 0; kt < KT && ok; kt++) {
                // a half block (128 elements) serves two stages: fetch the next half two stages ahead
                if (!(kt & 1) && kt + 2 < KT) pg_load_q6(nxt, wr + (size_t)((kt + 2) >> 2) * BLK, ((kt + 2) >> 1) & 1, h);
                pg_dequant_q6(cur, kt & 3, h, brow + (uint32_t)(kt % PG_STAGES) * PG_STAGE_BYTES, rr);
                ok = __all_sync(0xffffffffu, stage_tail(kt));   // warp-uniform: the shuffles in the dequantisation need the whole warp
                if (kt & 1) cur = nxt;
            }
        }
    } else {
        // ---- MMA issuer: per stage 2 token halves x 4 K-steps of 16; the weight tile is the M operand (128 rows =
        // 128 TMEM lanes), a token half the N operand (256 columns): fewer shared-memory reads per flop than four
        // 128 x 128 products ----
        for (int kt = 0; kt < KT && ok; kt++) {
            const int s = kt % PG_STAGES;
            ok = mbar_wait_bounded(&full[s], (uint32_t)((kt / PG_STAGES) & 1));
            if (!ok) break;
            pg_fence_after();
            if (lane == 0) {
                const uint32_t x_addr = smem_u32(smem + (uint32_t)s * PG_STAGE_BYTES), w_addr = x_addr + PG_A_BYTES;
#pragma unroll
                for (int nh = 0; nh < 2; nh++)
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        pg_mma(tmem_base + (uint32_t)nh * 256u, pg_smem_desc(w_addr + (uint32_t)k * 32u),
                               pg_smem_desc(x_addr + (uint32_t)nh * 256u * 128u + (uint32_t)k * 32u), (kt > 0 || k > 0) ? 1u : 0u);
                pg_commit(&empty[s]);
            }
            __syncwarp();
        }
        if (ok && lane == 0) pg_commit(&done_bar);
        __syncwarp();
    }
    if (!ok) atomicExch(&s_failed, 1);

    // ---- epilogue: warps 0-7; TMEM lane = weight row (lane quarter = warp % 4), column = token (half = warp / 4).
    // A warp's 32 lanes hold 32 consecutive rows of one token: each store instruction writes 128 contiguous bytes ----
    if (warp < 8) {
        bool fin = ok && mbar_wait_bounded(&done_bar, 0u);
        // token copies that were announced but never consumed must land before the CTA exits
        if (!fin) {
            atomicExch(&s_failed, 1);
            for (int s = 0; s < PG_STAGES; s++) mbar_wait_bounded(&full[s], 0u);
        }
        pg_fence_after();
        if (pair) {
            // gate rows sit on lanes 0-63 (lane quarters 0, 1), the same rows of up on lanes 64-127 (quarters 2, 3): the
            // eight warps put their 32 rows x 32 tokens into shared memory (the operand stages are free by now), then
            // each computes silu(gate) * up for 16 of the 32 tokens of its row.  Every warp takes part in every
            // barrier, whatever its own wait returned.
            float *ex = reinterpret_cast<float *>(smem);
            const int q = warp & 3, nh = warp >> 2, qp = q & 1;
            const int row = n0 + qp * 32 + lane, t_lo = (q >> 1) * 16;
#pragma unroll 1
            for (int cc = 0; cc < 256 / 32; cc++) {
                // two exchange buffers in turn: the barrier of the next pass also covers the reads of this one
                float *buf = ex + (size_t)(cc & 1) * (8 * 32 * 33);
                float *mine = buf + (size_t)warp * (32 * 33);
                const float *gsrc = buf + (size_t)(nh * 4 + qp) * (32 * 33), *usrc = buf + (size_t)(nh * 4 + qp + 2) * (32 * 33);
                uint32_t v[32];
                if (fin) pg_tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(nh * 256 + cc * 32), v);
#pragma unroll
                for (int i = 0; i < 32; i++) mine[lane * 33 + i] = fin ? __uint_as_float(v[i]) : 0.f;
                asm volatile("bar.sync 1, 256;" ::: "memory");
                const int tok0 = m0 + nh * 256 + cc * 32 + t_lo;
                if (fin && row < rows) {
                    uint16_t *dst = job.yb + (size_t)tok0 * rows + row;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const float g = gsrc[lane * 33 + t_lo + i], u = usrc[lane * 33 + t_lo + i];
                        // fast exponential and division: their 2^-21 relative error disappears in the bf16 rounding below
                        const float a = __fdividef(g, 1.0f + __expf(-g)) * u;
                        if (tok0 + i < seq) dst[(size_t)i * rows] = (uint16_t)(pg_pack_bf16(a, 0.f) & 0xffffu);
                    }
                }
            }
        } else if (fin) {
            const int q = warp & 3, nh = warp >> 2;
            const int row = n0 + q * 32 + lane;
#pragma unroll 1
            for (int cc = 0; cc < 256 / 32; cc++) {
                uint32_t v[32];
                pg_tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(nh * 256 + cc * 32), v);
                const int tok0 = m0 + nh * 256 + cc * 32;
                if (row < rows) {
                    float *dst = y + (size_t)tok0 * rows + row;
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (tok0 + i < seq) dst[(size_t)i * rows] = __uint_as_float(v[i]);
                }
            }
        }
    }
    pg_fence_before();
    __syncthreads();
    if (warp == 8) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
        if (lane == 0 && s_failed && err_flag) atomicExch(err_flag, DEV_ERR_GEMM_TIMEOUT);
    }
}

}  // namespace rnb
