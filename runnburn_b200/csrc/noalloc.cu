// Decode attention for callers that are not allowed to allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: a plug-in slot inside an
// inference server whose memory pool is sized once at start-up and then frozen, a sandboxed
// worker whose allocator hooks abort on any late allocation, or a real-time loop that may not
// take the driver's allocation locks.  The split-KV attention kernel needs a scratch area for
// its per-chunk partial results; every other entry point takes that area from the caller or
// from the library's grow-only buffers.  This one keeps it in a fixed array that is part of the
// loaded module, so the call path contains no cudaMalloc, cudaFree or allocating library call.
#include "attention.cuh"
#include "launch.hpp"

namespace rnb {

constexpr int NA_MAX_HEADS = 64;
constexpr int NA_MAX_CHUNKS = 32;
constexpr int NA_MAX_DEVICES = 64;

// Partial records of one call: [head][chunk][128 accumulator floats + running max + running sum].
// 64 * 32 * 130 * 4 bytes = 1 064 960 bytes, resident on every device that loads the library
// until the process exits.
static __device__ __align__(256) float g_na_partials[NA_MAX_HEADS * NA_MAX_CHUNKS * FD_PART_STRIDE];

// Status word of this entry point, beside the scratch and just as fixed: a kernel whose bounded
// wait gave up writes a non-zero code here (the rows it skipped are then wrong).  Read and cleared
// by rnb_b200_attention_decode_hd128_noalloc_status.
static __device__ int g_na_status;

// In host code the symbols' names are only handles; kernels need the device addresses, which are
// looked up once per device (with that device current) and cached here.
struct NaDevice {
    float *partials = nullptr;
    int *status = nullptr;
};
static NaDevice g_na_dev[NA_MAX_DEVICES];
static std::mutex g_na_mutex;

static int na_device(NaDevice *out) {
    int dev = -1;
    RNB_CU(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NA_MAX_DEVICES) return fail(RNB_B200_UNSUPPORTED, "no-alloc attention: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> g(g_na_mutex);
    if (!g_na_dev[dev].partials) {
        void *p = nullptr, *st = nullptr;
        RNB_CU(cudaGetSymbolAddress(&p, g_na_partials));
        RNB_CU(cudaGetSymbolAddress(&st, g_na_status));
        g_na_dev[dev].status = static_cast<int *>(st);
        g_na_dev[dev].partials = static_cast<float *>(p);
    }
    *out = g_na_dev[dev];
    return RNB_B200_OK;
}

}  // namespace rnb

using namespace rnb;

extern "C" int rnb_b200_attention_decode_hd128_noalloc(const float *q_dev, const uint16_t *k_dev, const uint16_t *v_dev,
                                                       size_t kv_len, size_t num_heads, size_t num_kv_heads, float scale,
                                                       float *out_dev, void *stream) {
    if (!q_dev || !k_dev || !v_dev || !out_dev) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    if (num_kv_heads == 0 || num_heads == 0 || num_heads % num_kv_heads != 0)
        return fail(RNB_B200_VALIDATION_FAILED, "attention: num_heads(%zu) must be a multiple of num_kv_heads(%zu)", num_heads, num_kv_heads);
    if (num_heads > (size_t)NA_MAX_HEADS)
        return fail(RNB_B200_VALIDATION_FAILED, "no-alloc attention supports at most %d query heads, got %zu", NA_MAX_HEADS, num_heads);
    if (kv_len == 0 || kv_len > (size_t)0x7fffffff) return fail(RNB_B200_VALIDATION_FAILED, "attention kv_len must be in 1..2^31-1, got %zu", kv_len);
    // the kernels read q with 16-byte loads and K/V with 8-byte (16-byte on the tensor-core path) loads:
    // a misaligned pointer would raise a device fault instead of an error code
    if (((uintptr_t)q_dev & 15u) || ((uintptr_t)k_dev & 7u) || ((uintptr_t)v_dev & 7u) || ((uintptr_t)out_dev & 3u))
        return fail(RNB_B200_VALIDATION_FAILED, "attention operands are not aligned: q needs 16 bytes, k and v 8 bytes, out 4 bytes");
    NaDevice nd;
    RNB_TRY(na_device(&nd));
    float *partials = nd.partials;
    int sm = 148, dev = 0;
    RNB_CU(cudaGetDevice(&dev));
    RNB_CU(cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev));
    int n_chunks = flash_decode_default_chunks(kv_len, num_kv_heads, sm);
    if (n_chunks > NA_MAX_CHUNKS) n_chunks = NA_MAX_CHUNKS;
    // Every (head, chunk) record that the merge reads is rewritten by this call's first kernel
    // (empty chunks write max = -inf, sum = 0), so nothing in the array has to start at zero.
    return launch_flash_decode((cudaStream_t)stream, q_dev, k_dev, v_dev, nullptr, (int)kv_len, (int)num_heads, (int)num_kv_heads,
                               scale, partials, n_chunks, out_dev, nd.status);
}

extern "C" int rnb_b200_attention_decode_hd128_noalloc_status(int *status_out, void *stream) {
    if (!status_out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    NaDevice nd;
    RNB_TRY(na_device(&nd));
    int v = 0;
    RNB_CU(cudaMemcpyAsync(&v, nd.status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    RNB_CU(cudaStreamSynchronize((cudaStream_t)stream));
    if (v != 0) RNB_CU(cudaMemsetAsync(nd.status, 0, sizeof(int), (cudaStream_t)stream));
    *status_out = v;
    return RNB_B200_OK;
}
