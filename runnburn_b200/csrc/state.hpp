// Host-side state of the operator library: one CUDA context per process, its streams, the
// resident weight cache, grow-only scratch buffers and pinned staging — the role CudaState
// plays in the reference (crates/rnb-backend/cuda/src/runtime/types.rs:346+,
// state/init.rs:86-410, state/q4k_cache.rs, state/buffers.rs).
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/rnb_b200.h"
#include "common.cuh"

namespace rnb {

extern thread_local std::string g_last_error;

inline int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}
inline int fail_cuda(cudaError_t e, const char *what) {
    // a sticky error would poison later calls with a stale code: clear the non-sticky ones
    cudaGetLastError();
    return fail(e == cudaErrorMemoryAllocation ? RNB_B200_OUT_OF_MEMORY : RNB_B200_CUDA_ERROR,
                "%s failed: %s (%d)", what, cudaGetErrorString(e), (int)e);
}
#define RNB_CU(call)                                        \
    do {                                                    \
        cudaError_t e_ = (call);                            \
        if (e_ != cudaSuccess) return fail_cuda(e_, #call); \
    } while (0)
#define RNB_TRY(call)                  \
    do {                               \
        int rc_ = (call);              \
        if (rc_ != RNB_B200_OK) return rc_; \
    } while (0)

// DeviceResidencyPlan::from_snapshot — crates/rnb-memory/src/device_residency.rs:40-91:
// dynamic reserve = clamp(total/16 rounded up to 256 MiB, 512 MiB, 2 GiB);
// resident_limit = free - reserve (saturating).
inline uint64_t resident_limit_for(uint64_t total, uint64_t free_bytes) {
    const uint64_t MiB = 1ull << 20;
    uint64_t reserve = total / 16;
    reserve = (reserve + 256 * MiB - 1) / (256 * MiB) * (256 * MiB);
    if (reserve < 512 * MiB) reserve = 512 * MiB;
    if (reserve > 2048 * MiB) reserve = 2048 * MiB;
    return free_bytes > reserve ? free_bytes - reserve : 0;
}

struct DevBuf {
    void *p = nullptr;
    size_t cap = 0;
    int ensure(size_t n) {
        if (n <= cap) return RNB_B200_OK;
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
        size_t want = (n + 255) & ~(size_t)255;
        cudaError_t e = cudaMalloc(&p, want);
        if (e != cudaSuccess) return fail_cuda(e, "cudaMalloc(scratch)");
        cap = want;
        return RNB_B200_OK;
    }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
    }
    template <class T>
    T *as() const {
        return reinterpret_cast<T *>(p);
    }
};
struct PinnedBuf {
    void *p = nullptr;
    size_t cap = 0;
    int ensure(size_t n) {
        if (n <= cap) return RNB_B200_OK;
        if (p) cudaFreeHost(p);
        p = nullptr;
        cap = 0;
        size_t want = (n + 4095) & ~(size_t)4095;
        cudaError_t e = cudaMallocHost(&p, want);
        if (e != cudaSuccess) return fail_cuda(e, "cudaMallocHost(staging)");
        cap = want;
        return RNB_B200_OK;
    }
    void release() {
        if (p) cudaFreeHost(p);
        p = nullptr;
        cap = 0;
    }
    template <class T>
    T *as() const {
        return reinterpret_cast<T *>(p);
    }
};

struct Resident {
    uint8_t *dev = nullptr;
    size_t bytes = 0;
    uint64_t epoch = 0;
    bool pinned = false;  // registered MoE layers are never evicted
};
struct KvMirror {
    const uint16_t *host_k = nullptr, *host_v = nullptr;
    uint16_t *dk = nullptr, *dv = nullptr;
    size_t rows_cap = 0, rows_have = 0, kv_dim = 0;
};

struct State {
    bool is_open = false;
    int device = 0, sm_count = 148;
    cudaStream_t stream = nullptr;
    size_t total = 0, resident_limit = 0, resident_bytes = 0, limit_override = 0;
    std::map<std::pair<const void *, size_t>, Resident> resident;
    uint64_t epoch = 0;
    rnb_b200_cache_snapshot ctr{};
    DevBuf in_f32, xq, xq2, out_f32, mid_a, mid_b, mid_c, jobs, partials, misc, xb;
    std::vector<DevBuf> transient_pool;   // over-budget weights of the current call, one buffer per upload
    size_t transient_used = 0;
    PinnedBuf pin_in, pin_out, pin_jobs;
    int *dev_error = nullptr;
    std::map<size_t, KvMirror> kv_mirrors;
    std::vector<std::pair<void *, size_t>> registered;
    int fail_next_allocs = 0;  // host-side fault injection for tests (fake OOM)

    int open();
    void close();
    int resident_ptr(const uint8_t *host, size_t len, bool pin, const uint8_t **dev_out);
    int transient_upload(const uint8_t *host, size_t len, const uint8_t **dev_out);
    void evict_all(bool include_pinned);
    int h2d(void *dst, const void *src, size_t n, PinnedBuf &stage, size_t stage_off = 0);
    int check_dev_error();
};

State &state();
std::mutex &state_mutex();

}  // namespace rnb
