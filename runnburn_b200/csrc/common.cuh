// Shared device/host helpers for the sm_100a batch-1 decode/prefill kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

// Kernels live in headers shared by several translation units: internal linkage keeps each
// unit's copy private.
#define RNB_GLOBAL static __global__

namespace rnb {

constexpr int QK_K = 256;
constexpr int Q4K_BYTES = 144;
constexpr int Q6K_BYTES = 210;
constexpr int Q8_0_BYTES = 34;
constexpr int Q8K_BYTES = 292;  // rnb-cpu Q8KBlock: f32 d @0, i8 qs[256] @4, i16 bsums[16] @260

// GGML type ids, as the reference passes them across its operator API (`down_quant: u32`).
constexpr int TYPE_Q8_0 = 8;
constexpr int TYPE_Q4_K = 12;
constexpr int TYPE_Q6_K = 14;

// Device-side error word values (State::dev_error).
constexpr int DEV_ERR_NONE = 0;
constexpr int DEV_ERR_MBAR_TIMEOUT = 1;   // a bounded mbarrier wait gave up
constexpr int DEV_ERR_BAD_JOB = 2;        // job table inconsistent with the launch
constexpr int DEV_ERR_GEMM_TIMEOUT = 3;   // tensor-core matmul: a pipeline wait gave up
constexpr int DEV_ERR_PEER_TIMEOUT = 4;   // multi-GPU exchange: a peer's slice did not arrive in time

__host__ __device__ inline size_t row_bytes_of(int type, size_t cols) {
    switch (type) {
    case TYPE_Q4_K: return cols / 256 * Q4K_BYTES;
    case TYPE_Q6_K: return cols / 256 * Q6K_BYTES;
    case TYPE_Q8_0: return cols / 32 * Q8_0_BYTES;
    case 10: return cols / 256 * 84;    // Q2_K (gemv_q5k.cuh)
    case 11: return cols / 256 * 110;   // Q3_K (gemv_q5k.cuh)
    case 13: return cols / 256 * 176;   // Q5_K (gemv_q5k.cuh)
    default: return 0;
    }
}

// ---------------------------------------------------------------------------------------
// Device-internal activation layout ("Q8K-dev"): the same numbers as rnb-cpu's Q8KBlock
// array, regrouped so that the matvec kernels can use 16-byte loads:
//   int8  qs[K]            @ 0
//   int16 bsum16[K/256*16] @ K                  (sum of each 16-element group, as Q8KBlock.bsums)
//   float d[K/256]         @ K + 32*(K/256)
// ---------------------------------------------------------------------------------------
__host__ __device__ inline size_t q8k_dev_bytes(size_t cols) {
    size_t nb = cols / 256;
    return (cols + nb * 4 + nb * 32 + 15) & ~(size_t)15;
}

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)h));
}

// ---- mbarrier + 1-D bulk async copy (TMA engine, CTA-local destination) ----------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
                 : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gsrc, uint32_t bytes,
                                         uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (seconds at worst), returns false on timeout so
// the caller can flag the error and leave without touching the data.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
    }
    return false;
}

// Programmatic dependent launch: let the next kernel in the stream start its prologue, and
// wait for the previous kernel's memory to be visible.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_nc_u4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_nc_u2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- expf as the C library of the reference's platform evaluates it --------------------------------
// rnb-cpu calls f32::exp (libm's expf) in softmax, SiLU and the MoE routing weights.  glibc's
// single-precision routine computes 2^(k/32) * P(r) in binary64 (a 32-entry table of 2^(i/32) and a
// cubic in r) and rounds once to f32; it is NOT the correctly rounded exponential in about one input
// in a thousand, so a device exp rounded from double differs from it there by one ulp.  The same
// evaluation here agrees with libm on every input up to the binary64 rounding of intermediate steps,
// which is 2^29 times finer than an f32 ulp (checked against the host libm on 262 million inputs).
// (global memory, not the constant bank: the index differs per thread, and two cache lines serve a warp)
static __device__ const unsigned long long c_exp2_tab32[32] = {   // bits(2^(i/32)) - (i << 47)
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull,
};
// LOAD(i) returns table entry i: from global memory (expf_libm) or from a shared-memory copy where a whole CTA
// evaluates at once (expf_libm_smem).
template <class Load>
__device__ __forceinline__ float expf_libm_with(float x, Load load) {
    if (x != x) return x;
    if (x < -0x1.9fe368p6f) return 0.0f;            // below the smallest subnormal
    if (x > 0x1.62e42ep6f) return INFINITY;
    const double z = __dmul_rn(0x1.71547652b82fep+5, (double)x);   // x * 32 / ln 2
    double kd = __dadd_rn(z, 0x1.8p52);                           // round to nearest integer
    const unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
    kd = __dsub_rn(kd, 0x1.8p52);
    const double r = __dsub_rn(z, kd);
    const double s = __longlong_as_double((long long)(load((int)(ki & 31)) + (ki << 47)));
    const double p = __dadd_rn(__dmul_rn(0x1.c6af84b912394p-20, r), 0x1.ebfce50fac4f3p-13);
    const double r2 = __dmul_rn(r, r);
    double y = __dadd_rn(__dmul_rn(0x1.62e42ff0c52d6p-6, r), 1.0);
    y = __dadd_rn(__dmul_rn(p, r2), y);
    return __double2float_rn(__dmul_rn(y, s));
}
__device__ __forceinline__ float expf_libm(float x) {
    return expf_libm_with(x, [](int i) { return __ldg(c_exp2_tab32 + i); });
}
__device__ __forceinline__ float expf_libm_smem(float x, const unsigned long long *tab) {
    return expf_libm_with(x, [tab](int i) { return tab[i]; });
}

// ---- multi-GPU: a producer's epilogue stores its slice of a gathered f32 buffer straight into
// every peer's copy (plain peer stores over NVLink; the buffers sit at the same offset of each
// rank's IPC-mapped arena), and the consumer waits for the other ranks' slices in its prologue.
// Flags: one int per (exchange, source rank) on every GPU, raised to the step's sequence number
// by the producer's last CTA after all of its CTAs' stores are visible system-wide.
struct PeerOut {
    char *const *peers;    // device array [world] of arena bases, own included; null: off
    int world, rank;
    size_t buf_off;        // byte offset of the gathered buffer in an arena
    int count;             // f32 elements per rank slice
    size_t flag_off;       // byte offset of this exchange's flag row (ints indexed by source rank)
    const int *seq_ptr;    // device scalar: sequence number of this step
    int *arrivals;         // local counter of CTAs done, zero between launches
    int n_arrive;          // CTAs that will call peer_arrive
};
struct PeerWait {
    const int *flags;      // this GPU's flag row of the exchange; null: off
    int world, rank;
    const int *seq_ptr;
    int *err;
};
// element `idx` of this rank's slice into every other rank's buffer (the own copy is the caller's)
__device__ __forceinline__ void peer_store(const PeerOut &po, size_t idx, float v) {
    for (int p = 1; p < po.world; p++) {
        const int r = (po.rank + p) % po.world;
        reinterpret_cast<float *>(po.peers[r] + po.buf_off)[(size_t)po.rank * po.count + idx] = v;
    }
}
// Once per CTA, by ONE thread, after every storing thread of the CTA has run
// __threadfence_system() and the CTA (or warp) has synchronised.
__device__ __forceinline__ void peer_arrive(const PeerOut &po) {
    const int before = atomicAdd(po.arrivals, 1);
    if (before != po.n_arrive - 1) return;
    *po.arrivals = 0;
    // one system-scope fence orders the other CTAs' stores (observed through the counter) before all
    // the flags; a release store per peer would each wait for the previous flag's round trip
    __threadfence_system();
    const int seq = *po.seq_ptr;
    for (int p = 1; p < po.world; p++) {
        const int r = (po.rank + p) % po.world;
        int *theirs = reinterpret_cast<int *>(po.peers[r] + po.flag_off) + po.rank;
        asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(seq) : "memory");
    }
}
// All threads of the CTA call it (it synchronises the CTA): thread t < world waits, bounded, for
// rank t's flag.  After a timeout the error word is set and later waits return at once.
static __device__ __noinline__ void peer_wait_slow(const PeerWait &w);
__device__ __forceinline__ void peer_wait(const PeerWait &w) {
    if (w.flags) peer_wait_slow(w);   // out of line: single-GPU launches pay one test
}
static __device__ __noinline__ void peer_wait_slow(const PeerWait &w) {
    const int t = threadIdx.x;
    if (t < w.world && t != w.rank && *reinterpret_cast<volatile int *>(w.err) == 0) {
        const int seq = *w.seq_ptr;
        bool ok = false;
        for (uint32_t i = 0; i < (1u << 21) && !ok; i++) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(w.flags + t) : "memory");
            ok = v >= seq;
            if (!ok && i > 32) __nanosleep(i > 2048 ? 512 : 64);
        }
        if (!ok) atomicExch(w.err, DEV_ERR_PEER_TIMEOUT);
    }
    __syncthreads();
}

#endif  // __CUDACC__

}  // namespace rnb
