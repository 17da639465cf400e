// C ABI of the operator library (declarations and reference citations: include/rnb_b200.h).
// Host logic only: validation with the reference's messages, residency, staging, launches.
#include <math.h>

#include <algorithm>

#include "launch.hpp"
#include "prefill.cuh"
#include "attention_wide.cuh"

namespace rnb {

thread_local std::string g_last_error;

State &state() {
    static State s;
    return s;
}
std::mutex &state_mutex() {
    static std::mutex m;
    return m;
}
bool use_pdl() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("RNB_B200_PDL");
        v = (e && *e && strcmp(e, "0") == 0) ? 0 : 1;   // on unless RNB_B200_PDL=0
    }
    return v == 1;
}
const GemvTuning &gemv_tuning() {
    static GemvTuning t = [] {
        GemvTuning v{0, 8, 2};
        auto env_int = [](const char *name, int dflt, int lo, int hi) {
            const char *e = getenv(name);
            if (!e || !*e) return dflt;
            int x = atoi(e);
            return x < lo ? lo : (x > hi ? hi : x);
        };
        v.rows = env_int("RNB_B200_GEMV_ROWS", v.rows, 0, 16);
        v.chunk_blocks = env_int("RNB_B200_GEMV_CHUNK", v.chunk_blocks, 1, GS_MAX_CHUNK);
        v.stages = env_int("RNB_B200_GEMV_STAGES", v.stages, 1, GS_MAX_STAGES);
        return v;
    }();
    return t;
}
int encode_weight_map(GmTensorMap *out, const uint8_t *w, size_t rows, size_t row_bytes, uint32_t box_bytes) {
    static_assert(sizeof(GmTensorMap) == sizeof(CUtensorMap) && alignof(GmTensorMap) >= alignof(CUtensorMap), "descriptor size");
    typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                    const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiled encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        RNB_CU(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !fn) return fail(RNB_B200_UNSUPPORTED, "the driver has no cuTensorMapEncodeTiled");
        encode = reinterpret_cast<EncodeTiled>(fn);
    }
    if (((uintptr_t)w & 15u) || (row_bytes & 15u) || (box_bytes & 15u) || box_bytes / 8 > 256 || rows == 0)
        return fail(RNB_B200_VALIDATION_FAILED, "weight matrix cannot be described for tiled copies (alignment or box width)");
    const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(box_bytes / 8), (cuuint32_t)GM_ROWS};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(reinterpret_cast<CUtensorMap *>(out), CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t *>(w), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(RNB_B200_CUDA_ERROR, "cuTensorMapEncodeTiled(weights) failed with driver code %d", (int)r);
    return RNB_B200_OK;
}
static size_t g_gemv_smem_max = 0;
size_t gemv_smem_max() { return g_gemv_smem_max; }
int gemv_kernel_setup() {
    static bool done = false;
    if (done) return RNB_B200_OK;
    int dev = 0, optin = 0;
    RNB_CU(cudaGetDevice(&dev));
    RNB_CU(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cudaFuncAttributes fa;
    RNB_CU(cudaFuncGetAttributes(&fa, gemv_tile_kernel));
    size_t stat = fa.sharedSizeBytes;
    RNB_CU(cudaFuncGetAttributes(&fa, gemv_tile_kernel_1));
    if (fa.sharedSizeBytes > stat) stat = fa.sharedSizeBytes;
    RNB_CU(cudaFuncGetAttributes(&fa, gemv_stream_kernel));
    if (fa.sharedSizeBytes > stat) stat = fa.sharedSizeBytes;
    RNB_CU(cudaFuncGetAttributes(&fa, gemv_stream_kernel_1));
    if (fa.sharedSizeBytes > stat) stat = fa.sharedSizeBytes;
    const size_t dyn = (size_t)optin - ((stat + 1023) & ~(size_t)1023);
    RNB_CU(cudaFuncSetAttribute(gemv_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    RNB_CU(cudaFuncSetAttribute(gemv_tile_kernel_1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    RNB_CU(cudaFuncSetAttribute(gemv_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    RNB_CU(cudaFuncSetAttribute(gemv_stream_kernel_1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    RNB_CU(cudaFuncSetAttribute(gemv_pair_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    RNB_CU(cudaFuncSetAttribute(gemv_pair_q4k_dyn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    RNB_CU(cudaFuncSetAttribute(gemv_ksplit_q6k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    RNB_CU(cudaFuncSetAttribute(gemv_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    RNB_CU(cudaFuncSetAttribute(gemv_mma_kernel_1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    RNB_CU(cudaFuncSetAttribute(gemv_mma_kernel_1_peer, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    RNB_TRY(attention_exact_setup());
    g_gemv_smem_max = dyn;
    done = true;
    return RNB_B200_OK;
}

// ---------------------------------------------------------------------------------------------
// State
// ---------------------------------------------------------------------------------------------
int State::open() {
    if (is_open) return RNB_B200_OK;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(RNB_B200_CUDA_ERROR, "no usable CUDA device (%s); this library has no CPU fallback",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    }
    const char *env = getenv("RNB_CUDA_DEVICE");
    device = env ? atoi(env) : 0;
    if (device < 0 || device >= n) return fail(RNB_B200_VALIDATION_FAILED, "RNB_CUDA_DEVICE=%d out of range (%d devices)", device, n);
    RNB_CU(cudaSetDevice(device));
    cudaDeviceProp prop;
    RNB_CU(cudaGetDeviceProperties(&prop, device));
    sm_count = prop.multiProcessorCount;
    if (prop.major < 10)
        return fail(RNB_B200_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                    prop.major, prop.minor);
    size_t free_b = 0;
    RNB_CU(cudaMemGetInfo(&free_b, &total));
    resident_limit = limit_override ? limit_override : (size_t)resident_limit_for(total, free_b);
    RNB_CU(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    RNB_CU(cudaMalloc((void **)&dev_error, sizeof(int)));
    RNB_CU(cudaMemsetAsync(dev_error, 0, sizeof(int), stream));
    memset(&ctr, 0, sizeof(ctr));
    is_open = true;
    return RNB_B200_OK;
}

void State::evict_all(bool include_pinned) {
    for (auto it = resident.begin(); it != resident.end();) {
        if (include_pinned || !it->second.pinned) {
            cudaFree(it->second.dev);
            resident_bytes -= it->second.bytes;
            ctr.evictions++;
            it = resident.erase(it);
        } else {
            ++it;
        }
    }
}

void State::close() {
    if (!is_open) return;
    cudaSetDevice(device);
    cudaStreamSynchronize(stream);
    evict_all(true);
    for (auto &kv : kv_mirrors) {
        cudaFree(kv.second.dk);
        cudaFree(kv.second.dv);
    }
    kv_mirrors.clear();
    for (auto &r : registered) cudaHostUnregister(r.first);
    registered.clear();
    DevBuf *bufs[] = {&in_f32, &xq, &xq2, &out_f32, &mid_a, &mid_b, &mid_c, &jobs, &partials, &misc, &xb};
    for (DevBuf *b : bufs) b->release();
    for (DevBuf &b : transient_pool) b.release();
    transient_pool.clear();
    transient_used = 0;
    pin_in.release();
    pin_out.release();
    pin_jobs.release();
    cudaFree(dev_error);
    dev_error = nullptr;
    cudaStreamDestroy(stream);
    stream = nullptr;
    is_open = false;
}

// Over-budget weights travel through transient buffers that live for one operator call: every
// transient upload of a call takes the next buffer of a grow-only pool (an operator that needs
// gate, up and down at once gets three distinct regions), and the pool's cursor returns to the
// start when the next call takes the state lock.
int State::transient_upload(const uint8_t *host, size_t len, const uint8_t **dev_out) {
    if (transient_used >= transient_pool.size()) transient_pool.emplace_back();
    DevBuf &buf = transient_pool[transient_used];
    RNB_TRY(buf.ensure(len + 16));
    RNB_CU(cudaMemcpyAsync(buf.p, host, len, cudaMemcpyHostToDevice, stream));
    transient_used++;
    ctr.transient_uploads++;
    ctr.h2d_bytes += len;
    *dev_out = buf.as<uint8_t>();
    return RNB_B200_OK;
}

// Resident lookup: exact (ptr,len) hit, or a slice of a larger resident range (stacked expert
// tensors registered once); miss -> budget check, LRU eviction, allocate, upload.  Over-budget
// weights are uploaded into a transient buffer of the current call
// (crates/rnb-backend/cuda/src/runtime/state/q4k_cache.rs:757-851).
// Weight slices that the calling thread's current operation must NOT admit into the residency cache (an expert
// bundle that failed the admission test): a miss on one of them is staged for the call only.
thread_local std::vector<std::pair<const uint8_t *, size_t>> tl_stage_only;

int State::resident_ptr(const uint8_t *host, size_t len, bool pin, const uint8_t **dev_out) {
    ctr.lookups++;
    epoch++;
    auto it = resident.upper_bound(std::make_pair((const void *)host, (size_t)-1));
    if (it != resident.begin()) {
        --it;
        const uint8_t *base = (const uint8_t *)it->first.first;
        if (host >= base && host + len <= base + it->first.second) {
            it->second.epoch = epoch;
            if (pin) it->second.pinned = true;
            ctr.hits++;
            *dev_out = it->second.dev + (host - base);
            return RNB_B200_OK;
        }
    }
    ctr.misses++;
    for (const auto &so : tl_stage_only)
        if (so.first == host && so.second == len) return transient_upload(host, len, dev_out);
    if (len > resident_limit) {
        if (pin) return fail(RNB_B200_OUT_OF_MEMORY, "resident weight of %zu bytes exceeds the residency limit %zu", len, resident_limit);
        return transient_upload(host, len, dev_out);
    }
    auto evict_lru = [&]() -> bool {
        auto victim = resident.end();
        for (auto j = resident.begin(); j != resident.end(); ++j)
            if (!j->second.pinned && (victim == resident.end() || j->second.epoch < victim->second.epoch)) victim = j;
        if (victim == resident.end()) return false;
        cudaFree(victim->second.dev);
        resident_bytes -= victim->second.bytes;
        ctr.evictions++;
        resident.erase(victim);
        return true;
    };
    while (resident_bytes + len > resident_limit)
        if (!evict_lru()) break;
    if (resident_bytes + len > resident_limit) {
        if (pin) return fail(RNB_B200_OUT_OF_MEMORY, "no room to pin %zu bytes (resident %zu, limit %zu)", len, resident_bytes, resident_limit);
        return transient_upload(host, len, dev_out);
    }
    uint8_t *dev = nullptr;
    for (;;) {
        cudaError_t e = cudaSuccess;
        if (fail_next_allocs > 0) {  // host-side fault injection: behave as if the driver said OOM
            fail_next_allocs--;
            e = cudaErrorMemoryAllocation;
        } else {
            e = cudaMalloc((void **)&dev, len + 16);  // +16: slack for the unaligned tile readers
        }
        if (e == cudaSuccess) break;
        cudaGetLastError();
        if (e != cudaErrorMemoryAllocation || !evict_lru()) return fail_cuda(e, "cudaMalloc(resident weight)");
    }
    cudaError_t e = cudaMemcpyAsync(dev, host, len, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) {
        cudaFree(dev);
        return fail_cuda(e, "cudaMemcpyAsync(resident weight)");
    }
    Resident r;
    r.dev = dev;
    r.bytes = len;
    r.epoch = epoch;
    r.pinned = pin;
    resident[std::make_pair((const void *)host, len)] = r;
    resident_bytes += len;
    ctr.uploads++;
    ctr.upload_bytes += len;
    ctr.h2d_bytes += len;
    *dev_out = dev;
    return RNB_B200_OK;
}

int State::h2d(void *dst, const void *src, size_t n, PinnedBuf &stage, size_t stage_off) {
    if (n == 0) return RNB_B200_OK;
    RNB_TRY(stage.ensure(stage_off + n));
    memcpy(stage.as<uint8_t>() + stage_off, src, n);
    RNB_CU(cudaMemcpyAsync(dst, stage.as<uint8_t>() + stage_off, n, cudaMemcpyHostToDevice, stream));
    ctr.h2d_bytes += n;
    return RNB_B200_OK;
}

int State::check_dev_error() {
    int flag = 0;
    RNB_CU(cudaMemcpyAsync(&flag, dev_error, sizeof(int), cudaMemcpyDeviceToHost, stream));
    RNB_CU(cudaStreamSynchronize(stream));
    if (flag != 0) {
        cudaMemsetAsync(dev_error, 0, sizeof(int), stream);
        return fail(RNB_B200_DEVICE_FAULT_FLAG, "device kernel reported error flag %d (%s)", flag,
                    flag == DEV_ERR_MBAR_TIMEOUT   ? "bounded mbarrier wait gave up"
                    : flag == DEV_ERR_GEMM_TIMEOUT ? "tensor-core matmul pipeline wait gave up"
                    : flag == DEV_ERR_PEER_TIMEOUT ? "a peer GPU's slice did not arrive in time"
                                                   : "inconsistent job table");
    }
    return RNB_B200_OK;
}

// D2H of results through pinned staging, then synchronise and surface device error flags.
static int finish_to_host(State &st, const void *dev_src, void *host_dst, size_t n) {
    RNB_TRY(st.pin_out.ensure(n + 16));
    RNB_CU(cudaMemcpyAsync(st.pin_out.p, dev_src, n, cudaMemcpyDeviceToHost, st.stream));
    int *flag = reinterpret_cast<int *>(st.pin_out.as<uint8_t>() + ((n + 3) & ~(size_t)3));
    RNB_CU(cudaMemcpyAsync(flag, st.dev_error, sizeof(int), cudaMemcpyDeviceToHost, st.stream));
    RNB_CU(cudaStreamSynchronize(st.stream));
    st.ctr.d2h_bytes += n;
    if (*flag != 0) {
        cudaMemsetAsync(st.dev_error, 0, sizeof(int), st.stream);
        return fail(RNB_B200_DEVICE_FAULT_FLAG, "device kernel reported error flag %d", *flag);
    }
    memcpy(host_dst, st.pin_out.p, n);
    return RNB_B200_OK;
}

struct Locked {
    std::lock_guard<std::mutex> g;
    State &st;
    Locked() : g(state_mutex()), st(state()) { st.transient_used = 0; }   // a new call: last call's transient uploads are dead
};

static const char *type_name(int t) {
    return t == TYPE_Q2_K ? "Q2_K" : t == TYPE_Q3_K ? "Q3_K" : t == TYPE_Q4_K ? "Q4_K" : t == TYPE_Q5_K ? "Q5_K" : t == TYPE_Q6_K ? "Q6_K" : t == TYPE_Q8_0 ? "Q8_0" : "?";
}

// Shape checks with the reference's wording (api/quant_api.rs:189-206).
static int validate_gemv(int type, size_t weights_len, size_t rows, size_t cols, size_t input_len,
                         size_t seq, size_t output_len, bool check_input) {
    const size_t blk = type == TYPE_Q8_0 ? 32 : 256;
    if (cols == 0 || cols % blk != 0)
        return fail(RNB_B200_VALIDATION_FAILED, "%s cols must be divisible by %zu, got %zu", type_name(type), blk, cols);
    const size_t expect = rows * row_bytes_of(type, cols);
    if (weights_len != expect)
        return fail(RNB_B200_VALIDATION_FAILED, "%s weight byte mismatch: got %zu, expected %zu", type_name(type), weights_len, expect);
    if (check_input && input_len != cols * seq)
        return fail(RNB_B200_VALIDATION_FAILED, "%s input length mismatch: got %zu, expected %zu", type_name(type), input_len, cols * seq);
    if (output_len < rows * seq)
        return fail(RNB_B200_VALIDATION_FAILED, "%s output too small: got %zu, expected >= %zu", type_name(type), output_len, rows * seq);
    if (rows == 0) return fail(RNB_B200_VALIDATION_FAILED, "%s rows must be non-zero", type_name(type));
    return RNB_B200_OK;
}

// Shared body of the host-buffer matvec entry points.
static int gemv_host(int type, const uint8_t *weights, size_t weights_len, size_t rows, size_t cols,
                     const float *input, size_t input_len, uint64_t input_dev, size_t seq,
                     float *output, size_t output_len, uint32_t *argmax_idx, float *argmax_val) {
    RNB_TRY(validate_gemv(type, weights_len, rows, cols, input_len, seq, argmax_idx ? rows * seq : output_len,
                          input_dev == 0));
    if (!weights || (!input && !input_dev)) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const uint8_t *w_dev = nullptr;
    RNB_TRY(st.resident_ptr(weights, weights_len, false, &w_dev));
    const float *x_dev = reinterpret_cast<const float *>(input_dev);
    if (!input_dev) {
        RNB_TRY(st.in_f32.ensure(cols * seq * sizeof(float)));
        RNB_TRY(st.h2d(st.in_f32.p, input, cols * seq * sizeof(float), st.pin_in));
        x_dev = st.in_f32.as<float>();
    }
    const void *act = x_dev;
    size_t x_stride = cols * sizeof(float);
    if (type != TYPE_Q8_0) {
        RNB_TRY(st.xq.ensure(q8k_dev_bytes(cols) * seq));
        RNB_TRY(launch_quantize_q8k(st.stream, x_dev, cols, seq, st.xq.as<uint8_t>(), nullptr));
        act = st.xq.p;
        x_stride = q8k_dev_bytes(cols);
    }
    RNB_TRY(st.out_f32.ensure(rows * seq * sizeof(float) + 16));
    if (type == TYPE_Q3_K) {
        RNB_CU(launch_k(gemv_q3k_kernel, dim3((unsigned)((rows + G5_WARPS - 1) / G5_WARPS)), dim3(G5_WARPS * 32), 0, st.stream, w_dev,
                        (const uint8_t *)act, x_stride, st.out_f32.as<float>(), (int)rows, (int)cols, (int)seq));
    } else if (type == TYPE_Q2_K) {
        RNB_CU(launch_k(gemv_q2k_kernel, dim3((unsigned)((rows + G5_WARPS - 1) / G5_WARPS)), dim3(G5_WARPS * 32), 0, st.stream, w_dev,
                        (const uint8_t *)act, x_stride, st.out_f32.as<float>(), (int)rows, (int)cols, (int)seq));
    } else if (type == TYPE_Q5_K) {
        // its own warp-per-row kernel (exact; seq-major output like the others)
        RNB_CU(launch_k(gemv_q5k_kernel, dim3((unsigned)((rows + G5_WARPS - 1) / G5_WARPS)), dim3(G5_WARPS * 32), 0, st.stream, w_dev,
                        (const uint8_t *)act, x_stride, st.out_f32.as<float>(), (int)rows, (int)cols, (int)seq));
    } else {
        GemvJob job = make_job(type, w_dev, act, st.out_f32.as<float>(), nullptr, rows, cols, 0, st.sm_count,
                               (int)seq, x_stride);
        RNB_TRY(launch_gemv_one(st.stream, job, cols, st.dev_error));
    }
    if (argmax_idx) {
        RNB_TRY(st.misc.ensure(16));
        RNB_CU(launch_k(argmax_last_kernel, dim3(1), dim3(1024), 0, st.stream, (const float *)st.out_f32.p,
                        (int)rows, st.misc.as<uint32_t>(), st.misc.as<float>() + 1));
        uint32_t pair[2];
        RNB_TRY(finish_to_host(st, st.misc.p, pair, 8));
        *argmax_idx = pair[0];
        if (argmax_val) memcpy(argmax_val, &pair[1], 4);
        return RNB_B200_OK;
    }
    return finish_to_host(st, st.out_f32.p, output, rows * seq * sizeof(float));
}

// Batched (prefill) matvec: each weight tile is staged once and applied to every token's
// Q8_K activations, so results are the ones rnb-cpu's gemv_quantized gives for seq_len > 1
// (crates/rnb-cpu/src/gemm/quant_gemv.rs:1145-1182), seq-major.
static int prefill_gemm_host(int type, const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in,
                             size_t seq, float *out, size_t ol) {
    if (seq == 0) return fail(RNB_B200_VALIDATION_FAILED, "%s batch needs at least one token", type_name(type));
    return gemv_host(type, w, wl, rows, cols, in, seq * cols, 0, seq, out, ol, nullptr, nullptr);
}

int prefill_gemm_setup() {
    static bool done = false;
    if (done) return RNB_B200_OK;
    RNB_CU(cudaFuncSetAttribute(prefill_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PG_SMEM));
    done = true;
    return RNB_B200_OK;
}

// Tensor-core prefill matmul from host buffers: bf16 x bf16 -> f32, weights dequantised in the
// kernel (the reference's q4k_f16_gemm_batch dequantises to f16 and calls cuBLAS).
static int prefill_tc_host(int type, const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    if (cols == 0 || il == 0 || il % cols != 0) return fail(RNB_B200_VALIDATION_FAILED, "%s batch input length %zu is not a multiple of cols %zu", type_name(type), il, cols);
    const size_t seq = il / cols;
    RNB_TRY(validate_gemv(type, wl, rows, cols, il, seq, ol, true));
    if (!w || !in || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const uint8_t *w_dev = nullptr;
    RNB_TRY(st.resident_ptr(w, wl, false, &w_dev));
    RNB_TRY(st.in_f32.ensure(il * sizeof(float)));
    RNB_TRY(st.h2d(st.in_f32.p, in, il * sizeof(float), st.pin_in));
    RNB_TRY(st.xb.ensure(il * 2));
    RNB_TRY(st.out_f32.ensure(rows * seq * sizeof(float) + 16));
    RNB_TRY(launch_prefill_gemm(st.stream, type, w_dev, rows, cols, st.in_f32.as<float>(), seq, st.xb.as<uint16_t>(), st.out_f32.as<float>(), st.dev_error));
    RNB_TRY(finish_to_host(st, st.out_f32.p, out, rows * seq * sizeof(float)));
    return st.check_dev_error();
}

// q / k / v of a token batch in one tensor-core launch (the reference's q4k_f16_qkv_gemm_batch)
static int prefill_tc_qkv_host(const uint8_t *qw, size_t qwl, const uint8_t *kw, size_t kwl, const uint8_t *vw, size_t vwl, size_t q_rows, size_t kv_rows,
                               size_t cols, const float *in, size_t il, float *q_out, size_t q_len, float *k_out, size_t k_len, float *v_out, size_t v_len) {
    if (cols == 0 || cols % 256 != 0) return fail(RNB_B200_VALIDATION_FAILED, "Q4_K QKV GEMM cols must be divisible by 256, got %zu", cols);
    if (il == 0 || il % cols != 0) return fail(RNB_B200_VALIDATION_FAILED, "Q4_K QKV GEMM batch input length %zu is not divisible by cols %zu", il, cols);
    const size_t seq = il / cols, rb = cols / 256 * Q4K_BYTES;
    if (qwl != q_rows * rb) return fail(RNB_B200_VALIDATION_FAILED, "Q4_K QKV GEMM q weight byte mismatch: got %zu, expected %zu", qwl, q_rows * rb);
    if (kwl != kv_rows * rb || vwl != kv_rows * rb)
        return fail(RNB_B200_VALIDATION_FAILED, "Q4_K QKV GEMM k/v weight byte mismatch: k=%zu v=%zu expected %zu", kwl, vwl, kv_rows * rb);
    if (q_rows == 0 || kv_rows == 0) return fail(RNB_B200_VALIDATION_FAILED, "Q4_K QKV GEMM needs rows");
    if (q_len < seq * q_rows || k_len < seq * kv_rows || v_len < seq * kv_rows) return fail(RNB_B200_VALIDATION_FAILED, "Q4_K QKV GEMM output too small");
    if (!qw || !kw || !vw || !in || !q_out || !k_out || !v_out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const uint8_t *w_dev[3] = {nullptr, nullptr, nullptr};
    RNB_TRY(st.resident_ptr(qw, qwl, false, &w_dev[0]));
    RNB_TRY(st.resident_ptr(kw, kwl, false, &w_dev[1]));
    RNB_TRY(st.resident_ptr(vw, vwl, false, &w_dev[2]));
    RNB_TRY(st.in_f32.ensure(il * sizeof(float)));
    RNB_TRY(st.h2d(st.in_f32.p, in, il * sizeof(float), st.pin_in));
    RNB_TRY(st.xb.ensure(il * 2));
    const size_t qn = seq * q_rows, kn = seq * kv_rows;
    const size_t qn_pad = (qn + 3) & ~(size_t)3, kn_pad = (kn + 3) & ~(size_t)3;   // 16-byte aligned outputs
    RNB_TRY(st.out_f32.ensure((qn_pad + 2 * kn_pad) * sizeof(float) + 16));
    float *y[3] = {st.out_f32.as<float>(), st.out_f32.as<float>() + qn_pad, st.out_f32.as<float>() + qn_pad + kn_pad};
    const int types[3] = {TYPE_Q4_K, TYPE_Q4_K, TYPE_Q4_K};
    const size_t rows[3] = {q_rows, kv_rows, kv_rows};
    RNB_TRY(launch_prefill_gemm_multi(st.stream, 3, types, w_dev, rows, y, cols, st.in_f32.as<float>(), seq, st.xb.as<uint16_t>(), st.dev_error));
    RNB_CU(cudaMemcpyAsync(q_out, y[0], qn * sizeof(float), cudaMemcpyDeviceToHost, st.stream));
    RNB_CU(cudaMemcpyAsync(k_out, y[1], kn * sizeof(float), cudaMemcpyDeviceToHost, st.stream));
    RNB_CU(cudaMemcpyAsync(v_out, y[2], kn * sizeof(float), cudaMemcpyDeviceToHost, st.stream));
    RNB_CU(cudaStreamSynchronize(st.stream));
    st.ctr.d2h_bytes += (qn + 2 * kn) * sizeof(float);
    return st.check_dev_error();
}

}  // namespace rnb

using namespace rnb;

// =============================================================================================
// extern "C"
// =============================================================================================
namespace rnb {
// defined with the rest of the boundary (boundary.inc): frees device tensors, decode carriers and the expert
// history; `all` = library close (false: engine re-init keeps handles a caller may still hold)
static void boundary_release(bool all);
// defined with the rest of the boundary (boundary.inc): brings a layer's device KV mirror up to kv_len rows
static int kv_mirror_sync(State &st, size_t layer, const uint16_t *k, const uint16_t *v, size_t kv_len, size_t kv_dim, const uint16_t *last_k_dev,
                          const uint16_t *last_v_dev);
}  // namespace rnb

extern "C" {

const char *rnb_b200_last_error(void) { return g_last_error.c_str(); }

int rnb_b200_open(void) {
    Locked L;
    return L.st.open();
}
void rnb_b200_close(void) {
    Locked L;
    if (L.st.is_open) {
        cudaSetDevice(L.st.device);
        cudaStreamSynchronize(L.st.stream);
        boundary_release(true);
    }
    L.st.close();
}
int rnb_b200_cuda_memory_info(size_t *free_bytes, size_t *total_bytes) {
    Locked L;
    RNB_TRY(L.st.open());
    RNB_CU(cudaSetDevice(L.st.device));
    size_t f = 0, t = 0;
    RNB_CU(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return RNB_B200_OK;
}
int rnb_b200_device_sm_count(int *sm_count) {
    Locked L;
    RNB_TRY(L.st.open());
    if (sm_count) *sm_count = L.st.sm_count;
    return RNB_B200_OK;
}
int rnb_b200_cuda_cache_snapshot(rnb_b200_cache_snapshot *out) {
    if (!out) return fail(RNB_B200_VALIDATION_FAILED, "null snapshot pointer");
    Locked L;
    *out = L.st.ctr;
    out->resident_entries = L.st.resident.size();
    out->resident_bytes = L.st.resident_bytes;
    out->resident_limit_bytes = L.st.resident_limit;
    return RNB_B200_OK;
}
int rnb_b200_clear_q4k_cache(void) {
    Locked L;
    if (!L.st.is_open) return RNB_B200_OK;
    RNB_CU(cudaSetDevice(L.st.device));
    RNB_CU(cudaStreamSynchronize(L.st.stream));
    L.st.evict_all(true);
    return RNB_B200_OK;
}
int rnb_b200_reset_state_for_engine_init(void) {
    Locked L;
    if (!L.st.is_open) return RNB_B200_OK;
    RNB_CU(cudaSetDevice(L.st.device));
    RNB_CU(cudaStreamSynchronize(L.st.stream));
    L.st.evict_all(true);
    for (auto &kv : L.st.kv_mirrors) {
        cudaFree(kv.second.dk);
        cudaFree(kv.second.dv);
    }
    L.st.kv_mirrors.clear();
    memset(&L.st.ctr, 0, sizeof(L.st.ctr));
    boundary_release(false);
    return RNB_B200_OK;
}
int rnb_b200_prewarm_q4k_weights(const uint8_t *const *slices, const size_t *lens, size_t n, size_t *n_resident) {
    if (n && (!slices || !lens)) return fail(RNB_B200_VALIDATION_FAILED, "null slice table");
    Locked L;
    RNB_TRY(L.st.open());
    RNB_CU(cudaSetDevice(L.st.device));
    size_t ok = 0;
    for (size_t i = 0; i < n; i++) {
        const uint8_t *dev = nullptr;
        const uint64_t before = L.st.ctr.transient_uploads;
        RNB_TRY(L.st.resident_ptr(slices[i], lens[i], false, &dev));
        if (L.st.ctr.transient_uploads == before) ok++;
    }
    RNB_CU(cudaStreamSynchronize(L.st.stream));
    if (n_resident) *n_resident = ok;
    return RNB_B200_OK;
}
int rnb_b200_set_resident_limit(size_t bytes) {
    Locked L;
    L.st.limit_override = bytes;
    if (L.st.is_open) {
        if (bytes) {
            L.st.resident_limit = bytes;
        } else {
            size_t f = 0, t = 0;
            RNB_CU(cudaMemGetInfo(&f, &t));
            L.st.resident_limit = (size_t)resident_limit_for(t, f + L.st.resident_bytes);
        }
    }
    return RNB_B200_OK;
}
int rnb_b200_inject_resident_alloc_ooms_for_test(size_t count) {
    Locked L;
    L.st.fail_next_allocs = (int)std::min<size_t>(count, 1u << 20);
    return RNB_B200_OK;
}
int rnb_b200_register_host_range(const void *ptr, size_t len) {
    if (!ptr || !len) return fail(RNB_B200_VALIDATION_FAILED, "empty host range");
    Locked L;
    RNB_TRY(L.st.open());
    RNB_CU(cudaSetDevice(L.st.device));
    // only whole pages strictly inside the range can be pinned
    const uintptr_t page = 4096, b = ((uintptr_t)ptr + page - 1) & ~(page - 1), e = ((uintptr_t)ptr + len) & ~(page - 1);
    if (e <= b) return RNB_B200_OK;
    cudaError_t err = cudaHostRegister((void *)b, e - b, cudaHostRegisterReadOnly);
    if (err == cudaErrorNotSupported || err == cudaErrorInvalidValue) {
        cudaGetLastError();
        err = cudaHostRegister((void *)b, e - b, cudaHostRegisterDefault);
    }
    if (err == cudaErrorHostMemoryAlreadyRegistered) {
        cudaGetLastError();
        return RNB_B200_OK;
    }
    if (err != cudaSuccess) return fail_cuda(err, "cudaHostRegister");
    L.st.registered.push_back(std::make_pair((void *)b, (size_t)(e - b)));
    return RNB_B200_OK;
}
int rnb_b200_clear_host_registered_ranges(void) {
    Locked L;
    if (!L.st.is_open) return RNB_B200_OK;
    RNB_CU(cudaSetDevice(L.st.device));
    RNB_CU(cudaStreamSynchronize(L.st.stream));
    for (auto &r : L.st.registered) cudaHostUnregister(r.first);
    L.st.registered.clear();
    return RNB_B200_OK;
}

int rnb_b200_quantize_q8k(const float *input, size_t n, void *blocks_out) {
    if (n % 256 != 0) return fail(RNB_B200_VALIDATION_FAILED, "Q8_K input length must be divisible by 256, got %zu", n);
    if (n == 0) return RNB_B200_OK;
    if (!input || !blocks_out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    RNB_TRY(st.in_f32.ensure(n * sizeof(float)));
    RNB_TRY(st.h2d(st.in_f32.p, input, n * sizeof(float), st.pin_in));
    const size_t out_bytes = n / 256 * Q8K_BYTES;
    RNB_TRY(st.out_f32.ensure(out_bytes));
    RNB_TRY(launch_quantize_q8k(st.stream, st.in_f32.as<float>(), n, 1, nullptr, st.out_f32.as<uint8_t>()));
    return finish_to_host(st, st.out_f32.p, blocks_out, out_bytes);
}

int rnb_b200_q4k_gemv(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    return gemv_host(TYPE_Q4_K, w, wl, rows, cols, in, il, 0, 1, out, ol, nullptr, nullptr);
}
int rnb_b200_q2k_gemv(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    return gemv_host(TYPE_Q2_K, w, wl, rows, cols, in, il, 0, 1, out, ol, nullptr, nullptr);
}
int rnb_b200_q2k_gemv_batch(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    if (cols == 0 || il % cols != 0) return fail(RNB_B200_VALIDATION_FAILED, "Q2_K input length mismatch: got %zu, not a multiple of cols %zu", il, cols);
    return prefill_gemm_host(TYPE_Q2_K, w, wl, rows, cols, in, il / cols, out, ol);
}
int rnb_b200_q3k_gemv(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    return gemv_host(TYPE_Q3_K, w, wl, rows, cols, in, il, 0, 1, out, ol, nullptr, nullptr);
}
int rnb_b200_q3k_gemv_batch(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    if (cols == 0 || il % cols != 0) return fail(RNB_B200_VALIDATION_FAILED, "Q3_K input length mismatch: got %zu, not a multiple of cols %zu", il, cols);
    return prefill_gemm_host(TYPE_Q3_K, w, wl, rows, cols, in, il / cols, out, ol);
}
int rnb_b200_q5k_gemv(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    return gemv_host(TYPE_Q5_K, w, wl, rows, cols, in, il, 0, 1, out, ol, nullptr, nullptr);
}
int rnb_b200_q5k_gemv_batch(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    if (cols == 0 || il % cols != 0) return fail(RNB_B200_VALIDATION_FAILED, "Q5_K input length mismatch: got %zu, not a multiple of cols %zu", il, cols);
    return prefill_gemm_host(TYPE_Q5_K, w, wl, rows, cols, in, il / cols, out, ol);
}
int rnb_b200_q6k_gemv(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    return gemv_host(TYPE_Q6_K, w, wl, rows, cols, in, il, 0, 1, out, ol, nullptr, nullptr);
}
int rnb_b200_q8_0_gemv(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    return gemv_host(TYPE_Q8_0, w, wl, rows, cols, in, il, 0, 1, out, ol, nullptr, nullptr);
}
int rnb_b200_q4k_gemv_with_device_input(const uint8_t *w, size_t wl, size_t rows, size_t cols, uint64_t in_dev, float *out, size_t ol) {
    if (!in_dev) return fail(RNB_B200_VALIDATION_FAILED, "Q4_K device input pointer is null");
    return gemv_host(TYPE_Q4_K, w, wl, rows, cols, nullptr, 0, in_dev, 1, out, ol, nullptr, nullptr);
}
int rnb_b200_q6k_gemv_with_device_input(const uint8_t *w, size_t wl, size_t rows, size_t cols, uint64_t in_dev, float *out, size_t ol) {
    if (!in_dev) return fail(RNB_B200_VALIDATION_FAILED, "Q6_K device input pointer is null");
    return gemv_host(TYPE_Q6_K, w, wl, rows, cols, nullptr, 0, in_dev, 1, out, ol, nullptr, nullptr);
}
int rnb_b200_q6k_gemv_argmax(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, uint32_t *idx, float *val) {
    if (!idx) return fail(RNB_B200_VALIDATION_FAILED, "null index output");
    return gemv_host(TYPE_Q6_K, w, wl, rows, cols, in, il, 0, 1, nullptr, 0, idx, val);
}
int rnb_b200_q8_0_gemv_argmax(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, uint32_t *idx, float *val) {
    if (!idx) return fail(RNB_B200_VALIDATION_FAILED, "null index output");
    return gemv_host(TYPE_Q8_0, w, wl, rows, cols, in, il, 0, 1, nullptr, 0, idx, val);
}
int rnb_b200_q8_0_gemv_batch(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    if (cols == 0 || il % cols != 0) return fail(RNB_B200_VALIDATION_FAILED, "Q8_0 batch input length %zu is not a multiple of cols %zu", il, cols);
    return prefill_gemm_host(TYPE_Q8_0, w, wl, rows, cols, in, il / cols, out, ol);
}
int rnb_b200_q4k_gemv_batch(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    if (cols == 0 || il % cols != 0) return fail(RNB_B200_VALIDATION_FAILED, "Q4_K batch input length %zu is not a multiple of cols %zu", il, cols);
    return prefill_gemm_host(TYPE_Q4_K, w, wl, rows, cols, in, il / cols, out, ol);
}
int rnb_b200_q6k_gemv_batch(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    if (cols == 0 || il % cols != 0) return fail(RNB_B200_VALIDATION_FAILED, "Q6_K batch input length %zu is not a multiple of cols %zu", il, cols);
    return prefill_gemm_host(TYPE_Q6_K, w, wl, rows, cols, in, il / cols, out, ol);
}
int rnb_b200_q4k_bf16_gemm_batch(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    return prefill_tc_host(TYPE_Q4_K, w, wl, rows, cols, in, il, out, ol);
}
int rnb_b200_q6k_bf16_gemm_batch(const uint8_t *w, size_t wl, size_t rows, size_t cols, const float *in, size_t il, float *out, size_t ol) {
    return prefill_tc_host(TYPE_Q6_K, w, wl, rows, cols, in, il, out, ol);
}
int rnb_b200_q4k_bf16_qkv_gemm_batch(const uint8_t *qw, size_t qwl, const uint8_t *kw, size_t kwl, const uint8_t *vw, size_t vwl, size_t q_rows,
                                     size_t kv_rows, size_t cols, const float *in, size_t il, float *q_out, size_t q_len, float *k_out, size_t k_len,
                                     float *v_out, size_t v_len) {
    return prefill_tc_qkv_host(qw, qwl, kw, kwl, vw, vwl, q_rows, kv_rows, cols, in, il, q_out, q_len, k_out, k_len, v_out, v_len);
}
int rnb_b200_dev_prefill_gemm(int type, const uint8_t *w_dev, size_t rows, size_t cols, const float *x_dev, size_t seq, uint16_t *xb_dev,
                              float *y_dev, void *stream) {
    if (!w_dev || !x_dev || !xb_dev || !y_dev) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    RNB_TRY(L.st.open());
    return launch_prefill_gemm((cudaStream_t)stream, type, w_dev, rows, cols, x_dev, seq, xb_dev, y_dev, L.st.dev_error);
}
int rnb_b200_dev_prefill_gemm_multi(int n, const int *types, const uint8_t *const *w_dev, const size_t *rows, float *const *y_dev, size_t cols,
                                    const float *x_dev, size_t seq, uint16_t *xb_dev, void *stream) {
    if (!types || !w_dev || !rows || !y_dev || !x_dev || !xb_dev) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    for (int i = 0; i < n && i < PG_MAX_JOBS; i++)
        if (!w_dev[i] || !y_dev[i]) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    RNB_TRY(L.st.open());
    return launch_prefill_gemm_multi((cudaStream_t)stream, n, types, w_dev, rows, y_dev, cols, x_dev, seq, xb_dev, L.st.dev_error);
}

int rnb_b200_dev_prefill_gemm_silu(int type, const uint8_t *gate_dev, const uint8_t *up_dev, size_t rows, size_t cols, const float *x_dev, size_t seq,
                                   uint16_t *xb_dev, uint16_t *act_dev, void *stream) {
    if (!gate_dev || !up_dev || !x_dev || !xb_dev || !act_dev) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    RNB_TRY(L.st.open());
    return launch_prefill_gemm_silu((cudaStream_t)stream, type, gate_dev, up_dev, rows, cols, x_dev, seq, xb_dev, act_dev, L.st.dev_error);
}

// ---- attention --------------------------------------------------------------------------------
static int validate_attn(size_t q_len, size_t kv_elems, size_t kv_len, size_t heads, size_t kv_heads, size_t head_dim, size_t out_len) {
    if (head_dim != 128) return fail(RNB_B200_UNSUPPORTED, "decode attention supports head_dim 128 only, got %zu", head_dim);
    if (kv_heads == 0 || heads == 0 || heads % kv_heads != 0)
        return fail(RNB_B200_VALIDATION_FAILED, "attention: num_heads(%zu) must be a multiple of num_kv_heads(%zu)", heads, kv_heads);
    if (q_len != heads * head_dim) return fail(RNB_B200_VALIDATION_FAILED, "attention q length mismatch: got %zu, expected %zu", q_len, heads * head_dim);
    if (kv_elems < kv_len * kv_heads * head_dim)
        return fail(RNB_B200_VALIDATION_FAILED, "attention kv length mismatch: got %zu, expected >= %zu", kv_elems, kv_len * kv_heads * head_dim);
    if (out_len < heads * head_dim) return fail(RNB_B200_VALIDATION_FAILED, "attention output too small: got %zu, expected >= %zu", out_len, heads * head_dim);
    if (kv_len == 0) return fail(RNB_B200_VALIDATION_FAILED, "attention kv_len must be non-zero");
    return RNB_B200_OK;
}

static int attention_run(State &st, const uint16_t *k_dev, const uint16_t *v_dev, const float *q, size_t kv_len,
                         size_t heads, size_t kv_heads, float scale, float *out) {
    RNB_TRY(st.in_f32.ensure(heads * HD * sizeof(float)));
    RNB_TRY(st.h2d(st.in_f32.p, q, heads * HD * sizeof(float), st.pin_in));
    const int n_chunks = flash_decode_default_chunks(kv_len, kv_heads, st.sm_count);
    RNB_TRY(st.partials.ensure(flash_decode_scratch_bytes(heads, n_chunks)));
    RNB_TRY(st.out_f32.ensure(heads * HD * sizeof(float)));
    RNB_TRY(launch_attention_decode(st.stream, st.in_f32.as<float>(), k_dev, v_dev, (int)kv_len, (int)heads, (int)kv_heads, scale,
                                    st.partials.as<float>(), n_chunks, st.out_f32.as<float>(), st.dev_error));
    return finish_to_host(st, st.out_f32.p, out, heads * HD * sizeof(float));
}

int rnb_b200_attention_decode_hd128(const float *q, size_t q_len, const uint16_t *k, const uint16_t *v, size_t kv_elems,
                                    size_t kv_len, size_t heads, size_t kv_heads, float scale, float *out, size_t out_len) {
    RNB_TRY(validate_attn(q_len, kv_elems, kv_len, heads, kv_heads, 128, out_len));
    if (!q || !k || !v || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const size_t bytes = kv_len * kv_heads * HD * sizeof(uint16_t);
    RNB_TRY(st.mid_a.ensure(bytes));
    RNB_TRY(st.mid_b.ensure(bytes));
    RNB_CU(cudaMemcpyAsync(st.mid_a.p, k, bytes, cudaMemcpyHostToDevice, st.stream));
    RNB_CU(cudaMemcpyAsync(st.mid_b.p, v, bytes, cudaMemcpyHostToDevice, st.stream));
    st.ctr.h2d_bytes += 2 * bytes;
    return attention_run(st, st.mid_a.as<uint16_t>(), st.mid_b.as<uint16_t>(), q, kv_len, heads, kv_heads, scale, out);
}

// head_dim 256 / 512: split-KV on CUDA cores (attention_wide.cuh)
static int attention_decode_wide(const size_t HD_, const float *q, size_t q_len, const uint16_t *k, const uint16_t *v, size_t kv_elems, size_t kv_len, size_t heads,
                                 size_t kv_heads, float scale, float *out, size_t out_len) {
    if (kv_heads == 0 || heads == 0 || heads % kv_heads != 0)
        return fail(RNB_B200_VALIDATION_FAILED, "attention: num_heads(%zu) must be a multiple of num_kv_heads(%zu)", heads, kv_heads);
    if (q_len != heads * HD_) return fail(RNB_B200_VALIDATION_FAILED, "decode attention q len mismatch: got %zu, expected %zu", q_len, heads * HD_);
    if (kv_elems < kv_len * kv_heads * HD_)
        return fail(RNB_B200_VALIDATION_FAILED, "decode attention k/v len mismatch: got %zu, expected >= %zu", kv_elems, kv_len * kv_heads * HD_);
    if (out_len < heads * HD_) return fail(RNB_B200_VALIDATION_FAILED, "attention output too small: got %zu, expected >= %zu", out_len, heads * HD_);
    if (kv_len == 0) return fail(RNB_B200_VALIDATION_FAILED, "attention kv_len must be non-zero");
    if (kv_len > (size_t)1 << 30) return fail(RNB_B200_VALIDATION_FAILED, "attention kv_len too large");
    if (!q || !k || !v || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const size_t bytes = kv_len * kv_heads * HD_ * sizeof(uint16_t), qb = heads * HD_ * sizeof(float);
    RNB_TRY(st.mid_a.ensure(bytes));
    RNB_TRY(st.mid_b.ensure(bytes));
    RNB_CU(cudaMemcpyAsync(st.mid_a.p, k, bytes, cudaMemcpyHostToDevice, st.stream));
    RNB_CU(cudaMemcpyAsync(st.mid_b.p, v, bytes, cudaMemcpyHostToDevice, st.stream));
    st.ctr.h2d_bytes += 2 * bytes;
    RNB_TRY(st.in_f32.ensure(qb));
    RNB_TRY(st.h2d(st.in_f32.p, q, qb, st.pin_in));
    const int n_chunks = attention_wide_chunks(kv_len, heads, st.sm_count);
    RNB_TRY(st.partials.ensure(attention_wide_scratch_bytes(heads, n_chunks, HD_)));
    RNB_TRY(st.out_f32.ensure(qb));
    const dim3 grid((unsigned)heads, (unsigned)n_chunks);
    const float *qd = st.in_f32.as<float>(), *pd = st.partials.as<float>();
    const uint16_t *kd = st.mid_a.as<uint16_t>(), *vd = st.mid_b.as<uint16_t>();
    if (HD_ == 256) {
        RNB_CU(launch_k(attention_wide_partials_kernel<256>, grid, dim3(AW_THREADS), 0, st.stream, qd, kd, vd, (int)kv_len, (int)heads, (int)kv_heads, scale, st.partials.as<float>()));
        RNB_CU(launch_k(attention_wide_merge_kernel<256>, dim3((unsigned)heads), dim3(128), 0, st.stream, pd, n_chunks, st.out_f32.as<float>()));
    } else {
        RNB_CU(launch_k(attention_wide_partials_kernel<512>, grid, dim3(AW_THREADS), 0, st.stream, qd, kd, vd, (int)kv_len, (int)heads, (int)kv_heads, scale, st.partials.as<float>()));
        RNB_CU(launch_k(attention_wide_merge_kernel<512>, dim3((unsigned)heads), dim3(256), 0, st.stream, pd, n_chunks, st.out_f32.as<float>()));
    }
    return finish_to_host(st, st.out_f32.p, out, qb);
}
int rnb_b200_attention_decode_hd256(const float *q, size_t q_len, const uint16_t *k, const uint16_t *v, size_t kv_elems, size_t kv_len, size_t heads,
                                    size_t kv_heads, float scale, float *out, size_t out_len) {
    return attention_decode_wide(256, q, q_len, k, v, kv_elems, kv_len, heads, kv_heads, scale, out, out_len);
}
int rnb_b200_attention_decode_hd512(const float *q, size_t q_len, const uint16_t *k, const uint16_t *v, size_t kv_elems, size_t kv_len, size_t heads,
                                    size_t kv_heads, float scale, float *out, size_t out_len) {
    return attention_decode_wide(512, q, q_len, k, v, kv_elems, kv_len, heads, kv_heads, scale, out, out_len);
}

int rnb_b200_attention_decode_cached(size_t layer, const float *q, size_t q_len, const uint16_t *k, const uint16_t *v,
                                     size_t kv_elems, size_t kv_len, size_t heads, size_t kv_heads, size_t head_dim,
                                     float scale, float *out, size_t out_len) {
    RNB_TRY(validate_attn(q_len, kv_elems, kv_len, heads, kv_heads, head_dim, out_len));
    if (!q || !k || !v || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    RNB_TRY(kv_mirror_sync(st, layer, k, v, kv_len, kv_heads * HD, nullptr, nullptr));
    KvMirror &m = st.kv_mirrors[layer];
    return attention_run(st, m.dk, m.dv, q, kv_len, heads, kv_heads, scale, out);
}

int rnb_b200_attention_decode_cached_window(size_t layer, const float *q, size_t q_len, const uint16_t *k, const uint16_t *v,
                                            size_t kv_elems, size_t kv_len, size_t window_start, size_t window_len, size_t heads,
                                            size_t kv_heads, size_t head_dim, float scale, float *out, size_t out_len) {
    RNB_TRY(validate_attn(q_len, kv_elems, kv_len, heads, kv_heads, head_dim, out_len));
    if (!q || !k || !v || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    if (window_len == 0 || window_start > kv_len || window_len > kv_len - window_start)
        return fail(RNB_B200_VALIDATION_FAILED, "cached window decode attention invalid window: kv_len=%zu start=%zu len=%zu", kv_len, window_start, window_len);
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    // the mirror holds every position (the next call may widen the window); attention runs over the window's rows only
    RNB_TRY(kv_mirror_sync(st, layer, k, v, kv_len, kv_heads * HD, nullptr, nullptr));
    KvMirror &m = st.kv_mirrors[layer];
    const size_t off = window_start * kv_heads * HD;
    return attention_run(st, m.dk + off, m.dv + off, q, window_len, heads, kv_heads, scale, out);
}

int rnb_b200_clear_decode_attention_kv_cache(void) {
    Locked L;
    if (!L.st.is_open) return RNB_B200_OK;
    RNB_CU(cudaSetDevice(L.st.device));
    RNB_CU(cudaStreamSynchronize(L.st.stream));
    for (auto &kv : L.st.kv_mirrors) {
        cudaFree(kv.second.dk);
        cudaFree(kv.second.dv);
    }
    L.st.kv_mirrors.clear();
    return RNB_B200_OK;
}

int rnb_b200_attention_prefill_flash_hd128(const float *q, const float *k, const float *v, size_t seq_len, size_t kv_len,
                                           size_t heads, size_t kv_heads, float scale, float *out) {
    if (kv_heads == 0 || heads == 0 || heads % kv_heads != 0)
        return fail(RNB_B200_VALIDATION_FAILED, "attention: num_heads(%zu) must be a multiple of num_kv_heads(%zu)", heads, kv_heads);
    if (seq_len == 0 || kv_len < seq_len) return fail(RNB_B200_VALIDATION_FAILED, "prefill attention needs 0 < seq_len <= kv_len, got %zu / %zu", seq_len, kv_len);
    if (!q || !k || !v || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const size_t qb = seq_len * heads * HD * 4, kb = kv_len * kv_heads * HD * 4;
    RNB_TRY(st.in_f32.ensure(qb));
    RNB_TRY(st.mid_a.ensure(kb));
    RNB_TRY(st.mid_b.ensure(kb));
    RNB_TRY(st.out_f32.ensure(qb));
    RNB_CU(cudaMemcpyAsync(st.in_f32.p, q, qb, cudaMemcpyHostToDevice, st.stream));
    RNB_CU(cudaMemcpyAsync(st.mid_a.p, k, kb, cudaMemcpyHostToDevice, st.stream));
    RNB_CU(cudaMemcpyAsync(st.mid_b.p, v, kb, cudaMemcpyHostToDevice, st.stream));
    st.ctr.h2d_bytes += qb + 2 * kb;
    RNB_TRY(launch_prefill_attention_f32kv(st.stream, st.in_f32.as<float>(), st.mid_a.as<float>(), st.mid_b.as<float>(),
                                           (int)seq_len, (int)kv_len, (int)heads, (int)kv_heads, scale, st.out_f32.as<float>()));
    return finish_to_host(st, st.out_f32.p, out, qb);
}

int rnb_b200_attention_prefill_flash_hd128_f16kv(const float *q, const uint16_t *k, const uint16_t *v, size_t seq_len, size_t kv_len,
                                                 size_t heads, size_t kv_heads, float scale, float *out) {
    if (kv_heads == 0 || heads == 0 || heads % kv_heads != 0)
        return fail(RNB_B200_VALIDATION_FAILED, "attention: num_heads(%zu) must be a multiple of num_kv_heads(%zu)", heads, kv_heads);
    if (seq_len == 0 || kv_len < seq_len) return fail(RNB_B200_VALIDATION_FAILED, "prefill attention needs 0 < seq_len <= kv_len, got %zu / %zu", seq_len, kv_len);
    if (!q || !k || !v || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const size_t qb = seq_len * heads * HD * 4, kb = kv_len * kv_heads * HD * 2;
    RNB_TRY(st.in_f32.ensure(qb));
    RNB_TRY(st.mid_a.ensure(kb));
    RNB_TRY(st.mid_b.ensure(kb));
    RNB_TRY(st.out_f32.ensure(qb));
    RNB_CU(cudaMemcpyAsync(st.in_f32.p, q, qb, cudaMemcpyHostToDevice, st.stream));
    RNB_CU(cudaMemcpyAsync(st.mid_a.p, k, kb, cudaMemcpyHostToDevice, st.stream));
    RNB_CU(cudaMemcpyAsync(st.mid_b.p, v, kb, cudaMemcpyHostToDevice, st.stream));
    st.ctr.h2d_bytes += qb + 2 * kb;
    RNB_TRY(launch_prefill_attention_f16kv(st.stream, st.in_f32.as<float>(), st.mid_a.as<uint16_t>(), st.mid_b.as<uint16_t>(), (int)seq_len, (int)kv_len,
                                           (int)heads, (int)kv_heads, scale, st.out_f32.as<float>(), st.dev_error));
    return finish_to_host(st, st.out_f32.p, out, qb);
}

// ---- glue ops -----------------------------------------------------------------------------------
static void host_rope_row(size_t pos, size_t head_dim, float theta, float *row /* [2][head_dim/2] */) {
    // CPU angle chain: crates/rnb-cpu/src/kernels/rope.rs:267-293
    const float theta_scale = powf(theta, -2.0f / (float)head_dim);
    float angle = (float)pos;
    for (size_t i = 0; i < head_dim / 2; i++) {
        row[i] = cosf(angle);
        row[head_dim / 2 + i] = sinf(angle);
        angle *= theta_scale;
    }
}

int rnb_b200_rms_norm_rows_f32(const float *input, const float *weight, size_t hidden, size_t rows, float eps, float *output) {
    if (hidden == 0 || hidden % 256 != 0) return fail(RNB_B200_VALIDATION_FAILED, "rms_norm hidden must be divisible by 256, got %zu", hidden);
    if (!input || !weight || !output) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    if (rows == 0) return RNB_B200_OK;
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    RNB_TRY(st.in_f32.ensure(rows * hidden * 4));
    RNB_TRY(st.mid_a.ensure(hidden * 4));
    RNB_TRY(st.out_f32.ensure(rows * hidden * 4));
    RNB_TRY(st.h2d(st.in_f32.p, input, rows * hidden * 4, st.pin_in));
    RNB_CU(cudaMemcpyAsync(st.mid_a.p, weight, hidden * 4, cudaMemcpyHostToDevice, st.stream));
    RNB_CU(launch_k(rmsnorm_q8k_kernel<512>, dim3((unsigned)rows), dim3(512), 0, st.stream, (const float *)st.in_f32.p,
                    (const float *)st.mid_a.p, eps, (int)hidden, st.out_f32.as<float>(), (uint8_t *)nullptr));
    return finish_to_host(st, st.out_f32.p, output, rows * hidden * 4);
}

int rnb_b200_rope_f32_inplace(float *data, size_t n, size_t pos_start, size_t head_dim, size_t dim, float theta, int neox) {
    if (head_dim != 128) return fail(RNB_B200_UNSUPPORTED, "rope supports head_dim 128 only, got %zu", head_dim);
    if (dim == 0 || dim % head_dim != 0 || n % dim != 0) return fail(RNB_B200_VALIDATION_FAILED, "rope shape mismatch: n=%zu dim=%zu head_dim=%zu", n, dim, head_dim);
    if (n == 0) return RNB_B200_OK;
    if (!data) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const size_t seq = n / dim, heads = dim / head_dim;
    RNB_TRY(st.in_f32.ensure(n * 4));
    RNB_TRY(st.mid_a.ensure(seq * 128 * 4));
    RNB_TRY(st.pin_jobs.ensure(seq * 128 * 4));
    for (size_t t = 0; t < seq; t++) host_rope_row(pos_start + t, 128, theta, st.pin_jobs.as<float>() + t * 128);
    RNB_CU(cudaMemcpyAsync(st.mid_a.p, st.pin_jobs.p, seq * 128 * 4, cudaMemcpyHostToDevice, st.stream));
    RNB_TRY(st.h2d(st.in_f32.p, data, n * 4, st.pin_in));
    for (size_t t = 0; t < seq; t++)  // rotate "q" heads only; no cache writes
        RNB_CU(launch_k(rope_kv_append_kernel, dim3((unsigned)heads), dim3(64), 0, st.stream, st.in_f32.as<float>() + t * dim,
                        (const float *)nullptr, (const float *)nullptr, (const float *)st.mid_a.p, (const int *)nullptr, (int)t, 1,
                        (int)heads, 0, neox, (uint16_t *)nullptr, (uint16_t *)nullptr, (uint16_t *)nullptr, (uint16_t *)nullptr));
    return finish_to_host(st, st.in_f32.p, data, n * 4);
}

int rnb_b200_activation_mul_f32_inplace(float *gate, const float *up, size_t n) {
    if (n % 256 != 0) return fail(RNB_B200_VALIDATION_FAILED, "activation length must be divisible by 256, got %zu", n);
    if (n == 0) return RNB_B200_OK;
    if (!gate || !up) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    RNB_TRY(st.in_f32.ensure(2 * n * 4));
    RNB_TRY(st.out_f32.ensure(n * 4));
    RNB_TRY(st.pin_in.ensure(2 * n * 4));
    memcpy(st.pin_in.p, gate, n * 4);
    memcpy(st.pin_in.as<float>() + n, up, n * 4);
    RNB_CU(cudaMemcpyAsync(st.in_f32.p, st.pin_in.p, 2 * n * 4, cudaMemcpyHostToDevice, st.stream));
    RNB_CU(launch_k(silu_mul_q8k_kernel, dim3((unsigned)((n / 256 + 3) / 4)), dim3(128), 0, st.stream, (const float *)st.in_f32.p,
                    (const float *)(st.in_f32.as<float>() + n), (int)n, 1, st.out_f32.as<float>(), (uint8_t *)nullptr));
    return finish_to_host(st, st.out_f32.p, gate, n * 4);
}

// ---- fused decode front half ---------------------------------------------------------------------
int rnb_b200_dense_attention_qkv_rope_hd128_decode(const uint8_t *q_w, size_t q_w_len, uint32_t q_type, const uint8_t *k_w,
                                                   size_t k_w_len, uint32_t k_type, const uint8_t *v_w, size_t v_w_len,
                                                   uint32_t v_type, size_t q_rows, size_t kv_rows, size_t n_embd,
                                                   size_t num_heads, size_t num_kv_heads, float rope_theta, size_t pos_start,
                                                   const float *input, float *q_rope, uint16_t *k_bits, uint16_t *v_bits) {
    if (q_rows != num_heads * 128 || kv_rows != num_kv_heads * 128)
        return fail(RNB_B200_VALIDATION_FAILED, "qkv rope hd128: rows (%zu, %zu) do not match heads (%zu, %zu) x 128", q_rows, kv_rows, num_heads, num_kv_heads);
    const uint32_t types[3] = {q_type, k_type, v_type};
    const size_t lens[3] = {q_w_len, k_w_len, v_w_len}, rows[3] = {q_rows, kv_rows, kv_rows};
    for (int i = 0; i < 3; i++) {
        if (types[i] != TYPE_Q4_K && types[i] != TYPE_Q6_K) return fail(RNB_B200_UNSUPPORTED, "qkv rope hd128: weight type %u not supported", types[i]);
        RNB_TRY(validate_gemv((int)types[i], lens[i], rows[i], n_embd, n_embd, 1, rows[i], true));
    }
    if (!q_w || !k_w || !v_w || !input || !q_rope || !k_bits || !v_bits) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const uint8_t *wd[3];
    const uint8_t *wh[3] = {q_w, k_w, v_w};
    for (int i = 0; i < 3; i++) RNB_TRY(st.resident_ptr(wh[i], lens[i], false, &wd[i]));
    RNB_TRY(st.in_f32.ensure(n_embd * 4));
    RNB_TRY(st.h2d(st.in_f32.p, input, n_embd * 4, st.pin_in));
    RNB_TRY(st.xq.ensure(q8k_dev_bytes(n_embd)));
    RNB_TRY(launch_quantize_q8k(st.stream, st.in_f32.as<float>(), n_embd, 1, st.xq.as<uint8_t>(), nullptr));
    const size_t out_floats = q_rows + 2 * kv_rows;
    RNB_TRY(st.out_f32.ensure(out_floats * 4 + 2 * kv_rows * 2));
    float *qd = st.out_f32.as<float>(), *kd = qd + q_rows, *vd = kd + kv_rows;
    uint16_t *kb = reinterpret_cast<uint16_t *>(vd + kv_rows), *vb = kb + kv_rows;
    GemvJob jobs[3];
    float *outs[3] = {qd, kd, vd};
    for (int i = 0; i < 3; i++) jobs[i] = make_job((int)types[i], wd[i], st.xq.p, outs[i], nullptr, rows[i], n_embd, 0, st.sm_count);
    gemv_finalize_group(jobs, 3, n_embd, st.sm_count);
    RNB_TRY(st.jobs.ensure(sizeof(jobs)));
    RNB_TRY(st.h2d(st.jobs.p, jobs, sizeof(jobs), st.pin_jobs));
    RNB_TRY(launch_gemv_jobs(st.stream, jobs, st.jobs.as<GemvJob>(), 3, n_embd, st.dev_error));
    RNB_TRY(st.mid_a.ensure(128 * 4));
    host_rope_row(pos_start, 128, rope_theta, st.pin_jobs.as<float>() + 256);
    RNB_CU(cudaMemcpyAsync(st.mid_a.p, st.pin_jobs.as<float>() + 256, 128 * 4, cudaMemcpyHostToDevice, st.stream));
    RNB_CU(launch_k(rope_kv_append_kernel, dim3((unsigned)(num_heads + 2 * num_kv_heads)), dim3(64), 0, st.stream, qd,
                    (const float *)kd, (const float *)vd, (const float *)st.mid_a.p, (const int *)nullptr, 0, 0, (int)num_heads,
                    (int)num_kv_heads, 0, (uint16_t *)nullptr, (uint16_t *)nullptr, kb, vb));
    RNB_TRY(st.pin_out.ensure(out_floats * 4 + 2 * kv_rows * 2 + 16));
    std::vector<uint8_t> tmp(out_floats * 4 + 2 * kv_rows * 2);
    RNB_TRY(finish_to_host(st, st.out_f32.p, tmp.data(), tmp.size()));
    memcpy(q_rope, tmp.data(), q_rows * 4);
    memcpy(k_bits, tmp.data() + out_floats * 4, kv_rows * 2);
    memcpy(v_bits, tmp.data() + out_floats * 4 + kv_rows * 2, kv_rows * 2);
    return RNB_B200_OK;
}

int rnb_b200_dense_attention_qkv(const uint8_t *q_w, size_t q_w_len, uint32_t q_type, const uint8_t *k_w, size_t k_w_len, uint32_t k_type,
                                 const uint8_t *v_w, size_t v_w_len, uint32_t v_type, size_t q_rows, size_t kv_rows, size_t n_embd, const float *input,
                                 size_t input_len, float *q, size_t q_len, float *k, size_t k_len, float *v, size_t v_len) {
    if (input_len != n_embd) return fail(RNB_B200_VALIDATION_FAILED, "dense QKV input length mismatch: got %zu, expected %zu", input_len, n_embd);
    if (n_embd == 0 || n_embd % 256 != 0) return fail(RNB_B200_VALIDATION_FAILED, "dense QKV cols must be divisible by 256, got %zu", n_embd);
    if (q_len < q_rows || k_len < kv_rows || v_len < kv_rows)
        return fail(RNB_B200_VALIDATION_FAILED, "dense QKV output length mismatch: q=%zu k=%zu v=%zu expected q>=%zu k/v>=%zu", q_len, k_len, v_len, q_rows, kv_rows);
    const uint32_t types[3] = {q_type, k_type, v_type};
    const size_t lens[3] = {q_w_len, k_w_len, v_w_len}, rows[3] = {q_rows, kv_rows, kv_rows};
    for (int i = 0; i < 3; i++) {
        if (types[i] != TYPE_Q4_K && types[i] != TYPE_Q6_K) return fail(RNB_B200_UNSUPPORTED, "dense QKV: weight type %u not supported", types[i]);
        RNB_TRY(validate_gemv((int)types[i], lens[i], rows[i], n_embd, n_embd, 1, rows[i], true));
    }
    if (!q_w || !k_w || !v_w || !input || !q || !k || !v) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const uint8_t *wd[3];
    const uint8_t *wh[3] = {q_w, k_w, v_w};
    for (int i = 0; i < 3; i++) RNB_TRY(st.resident_ptr(wh[i], lens[i], false, &wd[i]));
    RNB_TRY(st.in_f32.ensure(n_embd * 4));
    RNB_TRY(st.h2d(st.in_f32.p, input, n_embd * 4, st.pin_in));
    RNB_TRY(st.xq.ensure(q8k_dev_bytes(n_embd)));
    RNB_TRY(launch_quantize_q8k(st.stream, st.in_f32.as<float>(), n_embd, 1, st.xq.as<uint8_t>(), nullptr));
    const size_t out_floats = q_rows + 2 * kv_rows;
    RNB_TRY(st.out_f32.ensure(out_floats * 4));
    float *qd = st.out_f32.as<float>(), *kd = qd + q_rows, *vd = kd + kv_rows;
    GemvJob jobs[3];
    float *outs[3] = {qd, kd, vd};
    for (int i = 0; i < 3; i++) jobs[i] = make_job((int)types[i], wd[i], st.xq.p, outs[i], nullptr, rows[i], n_embd, 0, st.sm_count);
    gemv_finalize_group(jobs, 3, n_embd, st.sm_count);
    RNB_TRY(st.jobs.ensure(sizeof(jobs)));
    RNB_TRY(st.h2d(st.jobs.p, jobs, sizeof(jobs), st.pin_jobs));
    RNB_TRY(launch_gemv_jobs(st.stream, jobs, st.jobs.as<GemvJob>(), 3, n_embd, st.dev_error));
    std::vector<float> tmp(out_floats);
    RNB_TRY(finish_to_host(st, st.out_f32.p, tmp.data(), out_floats * 4));
    memcpy(q, tmp.data(), q_rows * 4);
    memcpy(k, tmp.data() + q_rows, kv_rows * 4);
    memcpy(v, tmp.data() + q_rows + kv_rows, kv_rows * 4);
    return RNB_B200_OK;
}

int rnb_b200_dense_q4k_silu_ffn_batch(const uint8_t *gate, size_t gate_len, const uint8_t *up, size_t up_len, const uint8_t *down,
                                      size_t down_len, uint32_t down_quant, size_t n_ff, size_t n_embd, size_t seq_len,
                                      const float *input, float *output) {
    if (down_quant != TYPE_Q4_K && down_quant != TYPE_Q5_K && down_quant != TYPE_Q6_K)
        return fail(RNB_B200_UNSUPPORTED, "dense FFN: down quant %u not supported", down_quant);
    if (seq_len == 0) return fail(RNB_B200_VALIDATION_FAILED, "dense FFN: seq_len must be non-zero");
    RNB_TRY(validate_gemv(TYPE_Q4_K, gate_len, n_ff, n_embd, n_embd * seq_len, seq_len, n_ff * seq_len, true));
    RNB_TRY(validate_gemv(TYPE_Q4_K, up_len, n_ff, n_embd, n_embd * seq_len, seq_len, n_ff * seq_len, true));
    RNB_TRY(validate_gemv((int)down_quant, down_len, n_embd, n_ff, n_ff * seq_len, seq_len, n_embd * seq_len, true));
    if (!gate || !up || !down || !input || !output) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const uint8_t *gd, *ud, *dd;
    RNB_TRY(st.resident_ptr(gate, gate_len, false, &gd));
    RNB_TRY(st.resident_ptr(up, up_len, false, &ud));
    RNB_TRY(st.resident_ptr(down, down_len, false, &dd));
    RNB_TRY(st.in_f32.ensure(n_embd * seq_len * 4));
    RNB_TRY(st.h2d(st.in_f32.p, input, n_embd * seq_len * 4, st.pin_in));
    RNB_TRY(st.xq.ensure(q8k_dev_bytes(n_embd) * seq_len));
    RNB_TRY(launch_quantize_q8k(st.stream, st.in_f32.as<float>(), n_embd, seq_len, st.xq.as<uint8_t>(), nullptr));
    RNB_TRY(st.mid_a.ensure(n_ff * seq_len * 4));
    RNB_TRY(st.mid_b.ensure(n_ff * seq_len * 4));
    GemvJob jobs[2];
    jobs[0] = make_job(TYPE_Q4_K, gd, st.xq.p, st.mid_a.as<float>(), nullptr, n_ff, n_embd, 0, st.sm_count, (int)seq_len, q8k_dev_bytes(n_embd));
    jobs[1] = make_job(TYPE_Q4_K, ud, st.xq.p, st.mid_b.as<float>(), nullptr, n_ff, n_embd, jobs[0].rows_per_tile, st.sm_count, (int)seq_len, q8k_dev_bytes(n_embd));
    gemv_finalize_group(jobs, 2, n_embd, st.sm_count);
    RNB_TRY(st.jobs.ensure(sizeof(jobs)));
    RNB_TRY(st.h2d(st.jobs.p, jobs, sizeof(jobs), st.pin_jobs));
    RNB_TRY(launch_gemv_jobs(st.stream, jobs, st.jobs.as<GemvJob>(), 2, n_embd, st.dev_error));
    RNB_TRY(st.xq2.ensure(q8k_dev_bytes(n_ff) * seq_len));
    RNB_CU(launch_k(silu_mul_q8k_kernel, dim3((unsigned)((n_ff / 256 * seq_len + 3) / 4)), dim3(128), 0, st.stream,
                    (const float *)st.mid_a.p, (const float *)st.mid_b.p, (int)n_ff, (int)seq_len, (float *)nullptr, st.xq2.as<uint8_t>()));
    RNB_TRY(st.out_f32.ensure(n_embd * seq_len * 4));
    if (down_quant == TYPE_Q5_K) {
        RNB_CU(launch_k(gemv_q5k_kernel, dim3((unsigned)((n_embd + G5_WARPS - 1) / G5_WARPS)), dim3(G5_WARPS * 32), 0, st.stream, dd,
                        (const uint8_t *)st.xq2.p, q8k_dev_bytes(n_ff), st.out_f32.as<float>(), (int)n_embd, (int)n_ff, (int)seq_len));
    } else {
        GemvJob dj = make_job((int)down_quant, dd, st.xq2.p, st.out_f32.as<float>(), nullptr, n_embd, n_ff, 0, st.sm_count, (int)seq_len, q8k_dev_bytes(n_ff));
        RNB_TRY(launch_gemv_one(st.stream, dj, n_ff, st.dev_error));
    }
    return finish_to_host(st, st.out_f32.p, output, n_embd * seq_len * 4);
}

// ---- MoE ---------------------------------------------------------------------------------------------
int rnb_b200_moe_route_topk_f32(const float *logits, size_t logits_len, const float *selection_bias, size_t seq_len, size_t n_expert,
                                size_t top_k, int sigmoid_mode, int normalize_selected, float scale, float adaptive_top_p,
                                uint32_t *ids_out, float *weights_out, uint32_t *retained_counts_out) {
    (void)normalize_selected;
    (void)adaptive_top_p;
    if (logits_len != seq_len * n_expert) return fail(RNB_B200_VALIDATION_FAILED, "CUDA MoE route logits mismatch: got=%zu expected=%zu", logits_len, seq_len * n_expert);
    if (n_expert == 0 || n_expert > 1024 || top_k == 0 || top_k > n_expert || top_k > 32)
        return fail(RNB_B200_VALIDATION_FAILED, "invalid CUDA MoE route shape: seq_len=%zu n_expert=%zu top_k=%zu", seq_len, n_expert, top_k);
    if (sigmoid_mode || selection_bias) return fail(RNB_B200_UNSUPPORTED, "sigmoid / biased routing is not on this path (softmax top-k only)");
    if (seq_len == 0) return RNB_B200_OK;
    if (!logits || !ids_out || !weights_out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    RNB_TRY(st.in_f32.ensure(logits_len * 4));
    RNB_TRY(st.h2d(st.in_f32.p, logits, logits_len * 4, st.pin_in));
    const size_t slots = seq_len * top_k;
    RNB_TRY(st.out_f32.ensure(slots * 8));
    uint32_t *ids_dev = st.out_f32.as<uint32_t>();
    float *w_dev = st.out_f32.as<float>() + slots;
    RNB_CU(launch_k(moe_route_topk_kernel, dim3((unsigned)seq_len), dim3(32), 0, st.stream, (const float *)st.in_f32.p, (int)n_expert,
                    (int)top_k, ids_dev, w_dev));
    std::vector<uint8_t> tmp(slots * 8);
    RNB_TRY(finish_to_host(st, st.out_f32.p, tmp.data(), tmp.size()));
    memcpy(ids_out, tmp.data(), slots * 4);
    const float *wsrc = reinterpret_cast<const float *>(tmp.data() + slots * 4);
    for (size_t i = 0; i < slots; i++) weights_out[i] = scale == 1.0f ? wsrc[i] : wsrc[i] * scale;
    if (retained_counts_out)
        for (size_t t = 0; t < seq_len; t++) retained_counts_out[t] = (uint32_t)top_k;
    return RNB_B200_OK;
}

int rnb_b200_router_logits_f32(const float *router_w, size_t n_expert, size_t hidden, const float *h, float *logits_out) {
    if (hidden == 0 || hidden % 16 != 0) return fail(RNB_B200_VALIDATION_FAILED, "router hidden must be divisible by 16, got %zu", hidden);
    if (n_expert == 0) return RNB_B200_OK;
    if (!router_w || !h || !logits_out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const uint8_t *wd = nullptr;
    RNB_TRY(st.resident_ptr(reinterpret_cast<const uint8_t *>(router_w), n_expert * hidden * 4, false, &wd));
    RNB_TRY(st.in_f32.ensure(hidden * 4));
    RNB_TRY(st.h2d(st.in_f32.p, h, hidden * 4, st.pin_in));
    RNB_TRY(st.out_f32.ensure(n_expert * 4));
    RNB_CU(launch_k(router_logits_kernel, dim3((unsigned)((n_expert + 7) / 8)), dim3(128), 0, st.stream, reinterpret_cast<const float *>(wd),
                    (const float *)st.in_f32.p, (int)n_expert, (int)hidden, st.out_f32.as<float>()));
    return finish_to_host(st, st.out_f32.p, logits_out, n_expert * 4);
}

int rnb_b200_qwen35_sparse_experts(const uint8_t *const *gate, const uint8_t *const *up, const uint8_t *const *down,
                                   size_t gate_slice_len, size_t down_slice_len, const float *route_weights, size_t n_selected,
                                   uint32_t down_quant, size_t n_ff, size_t n_embd, const float *input, float *output) {
    if (down_quant != TYPE_Q4_K && down_quant != TYPE_Q6_K) return fail(RNB_B200_UNSUPPORTED, "sparse experts: down quant %u not supported", down_quant);
    if (n_selected == 0 || n_selected > 32) return fail(RNB_B200_VALIDATION_FAILED, "sparse experts: selected count %zu out of range 1..32", n_selected);
    RNB_TRY(validate_gemv(TYPE_Q4_K, gate_slice_len, n_ff, n_embd, n_embd, 1, n_ff, true));
    RNB_TRY(validate_gemv((int)down_quant, down_slice_len, n_embd, n_ff, n_ff, 1, n_embd, true));
    if (!gate || !up || !down || !route_weights || !input || !output) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    const size_t k = n_selected;
    std::vector<const uint8_t *> gd(k), ud(k), dd(k);
    for (size_t e = 0; e < k; e++) {
        RNB_TRY(st.resident_ptr(gate[e], gate_slice_len, false, &gd[e]));
        RNB_TRY(st.resident_ptr(up[e], gate_slice_len, false, &ud[e]));
        RNB_TRY(st.resident_ptr(down[e], down_slice_len, false, &dd[e]));
    }
    RNB_TRY(st.in_f32.ensure(n_embd * 4 + k * 4));
    RNB_TRY(st.pin_in.ensure(n_embd * 4 + k * 4));
    memcpy(st.pin_in.p, input, n_embd * 4);
    memcpy(st.pin_in.as<uint8_t>() + n_embd * 4, route_weights, k * 4);
    RNB_CU(cudaMemcpyAsync(st.in_f32.p, st.pin_in.p, n_embd * 4 + k * 4, cudaMemcpyHostToDevice, st.stream));
    const float *rw_dev = st.in_f32.as<float>() + n_embd;
    RNB_TRY(st.xq.ensure(q8k_dev_bytes(n_embd)));
    RNB_TRY(launch_quantize_q8k(st.stream, st.in_f32.as<float>(), n_embd, 1, st.xq.as<uint8_t>(), nullptr));
    RNB_TRY(st.mid_a.ensure(k * n_ff * 4));
    RNB_TRY(st.mid_b.ensure(k * n_ff * 4));
    const size_t n_down_jobs = (k + GEMV_MAX_PARTS - 1) / GEMV_MAX_PARTS;
    std::vector<GemvJob> jobs(2 * k + n_down_jobs);
    for (size_t e = 0; e < 2 * k; e++) {
        const bool is_up = e >= k;
        const size_t ee = is_up ? e - k : e;
        jobs[e] = make_job(TYPE_Q4_K, is_up ? ud[ee] : gd[ee], st.xq.p, (is_up ? st.mid_b.as<float>() : st.mid_a.as<float>()) + ee * n_ff,
                           nullptr, n_ff, n_embd, 0, st.sm_count);
    }
    gemv_finalize_group(jobs.data(), (int)(2 * k), n_embd, st.sm_count);
    RNB_TRY(st.xq2.ensure(q8k_dev_bytes(n_ff) * k));
    RNB_TRY(st.out_f32.ensure(n_embd * 4));
    RNB_TRY(st.mid_c.ensure(n_embd * 4));
    // down: groups of up to 8 experts per job; later groups add onto the earlier partial sum
    for (size_t gi = 0; gi < n_down_jobs; gi++) {
        const size_t e0 = gi * GEMV_MAX_PARTS, ne = std::min<size_t>(GEMV_MAX_PARTS, k - e0);
        const bool last = gi + 1 == n_down_jobs;
        float *dst = ((n_down_jobs - 1 - gi) % 2 == 0) ? st.out_f32.as<float>() : st.mid_c.as<float>();
        const float *prev = gi == 0 ? nullptr : (((n_down_jobs - gi) % 2 == 0) ? st.out_f32.as<float>() : st.mid_c.as<float>());
        (void)last;
        GemvJob &dj = jobs[2 * k + gi];
        dj = make_job((int)down_quant, dd[e0], st.xq2.p, dst, prev, n_embd, n_ff, 0, st.sm_count, 1, 0, (int)ne);
        for (size_t p = 0; p < ne; p++) {
            dj.parts[p].w = dd[e0 + p];
            dj.parts[p].x = st.xq2.as<uint8_t>() + (e0 + p) * q8k_dev_bytes(n_ff);
            dj.parts[p].scale = rw_dev + e0 + p;
        }
    }
    RNB_TRY(st.jobs.ensure(jobs.size() * sizeof(GemvJob)));
    RNB_TRY(st.h2d(st.jobs.p, jobs.data(), jobs.size() * sizeof(GemvJob), st.pin_jobs));
    RNB_TRY(launch_gemv_jobs(st.stream, jobs.data(), st.jobs.as<GemvJob>(), (int)(2 * k), n_embd, st.dev_error));
    RNB_CU(launch_k(silu_mul_q8k_kernel, dim3((unsigned)((n_ff / 256 * k + 3) / 4)), dim3(128), 0, st.stream, (const float *)st.mid_a.p,
                    (const float *)st.mid_b.p, (int)n_ff, (int)k, (float *)nullptr, st.xq2.as<uint8_t>()));
    for (size_t gi = 0; gi < n_down_jobs; gi++)
        RNB_TRY(launch_gemv_jobs(st.stream, &jobs[2 * k + gi], st.jobs.as<GemvJob>() + 2 * k + gi, 1, n_ff, st.dev_error));
    return finish_to_host(st, st.out_f32.p, output, n_embd * 4);
}

int rnb_b200_qwen35_register_moe_layer(const uint8_t *gate_all, size_t gate_len, const uint8_t *up_all, size_t up_len,
                                       const uint8_t *down_all, size_t down_len, uint32_t down_quant, size_t n_ff, size_t n_embd,
                                       int *fitted) {
    if (down_quant != TYPE_Q4_K && down_quant != TYPE_Q6_K) return fail(RNB_B200_UNSUPPORTED, "register MoE layer: down quant %u not supported", down_quant);
    const size_t gslice = n_ff * row_bytes_of(TYPE_Q4_K, n_embd), dslice = n_embd * row_bytes_of((int)down_quant, n_ff);
    if (gslice == 0 || dslice == 0 || gate_len % gslice || up_len != gate_len || down_len % dslice || down_len / dslice != gate_len / gslice)
        return fail(RNB_B200_VALIDATION_FAILED, "register MoE layer: stacked tensor sizes (%zu, %zu, %zu) do not match n_ff=%zu n_embd=%zu", gate_len, up_len, down_len, n_ff, n_embd);
    if (!gate_all || !up_all || !down_all) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    Locked L;
    State &st = L.st;
    RNB_TRY(st.open());
    RNB_CU(cudaSetDevice(st.device));
    if (fitted) *fitted = 0;
    // "without evicting": only admit when everything fits beside what is already resident
    if (st.resident_bytes + gate_len + up_len + down_len > st.resident_limit) return RNB_B200_OK;
    const uint8_t *d = nullptr;
    RNB_TRY(st.resident_ptr(gate_all, gate_len, true, &d));
    RNB_TRY(st.resident_ptr(up_all, up_len, true, &d));
    RNB_TRY(st.resident_ptr(down_all, down_len, true, &d));
    RNB_CU(cudaStreamSynchronize(st.stream));
    if (fitted) *fitted = 1;
    return RNB_B200_OK;
}

// ---- host-only bookkeeping -----------------------------------------------------------------------
// admit iff missing_bytes * (predicted_future_reuses + [replaces a temp upload]) >
//           missing_bytes + eviction_reload_bytes   (strict)
// crates/rnb-memory/src/sparse_expert_cache.rs:221-245
int rnb_b200_evaluate_expert_bundle_admission(const rnb_b200_bundle_admission *a) {
    if (!a || a->missing_bytes == 0) return 0;
    const unsigned __int128 benefit = (unsigned __int128)a->missing_bytes * ((uint64_t)a->predicted_future_reuses + (a->replaces_temp_upload ? 1u : 0u));
    const unsigned __int128 cost = (unsigned __int128)a->missing_bytes + a->eviction_reload_bytes;
    return benefit > cost ? 1 : 0;
}
uint64_t rnb_b200_resident_limit_for(uint64_t total_bytes, uint64_t free_bytes) { return resident_limit_for(total_bytes, free_bytes); }

// ---- device-pointer tier ---------------------------------------------------------------------------
size_t rnb_b200_dev_q8k_bytes(size_t cols) { return q8k_dev_bytes(cols); }
int rnb_b200_dev_quantize_q8k(const float *x_dev, size_t cols, size_t seq, void *xq_dev, void *ref_blocks_dev, void *stream) {
    if (cols % 256 != 0) return fail(RNB_B200_VALIDATION_FAILED, "Q8_K input length must be divisible by 256, got %zu", cols);
    Locked L;
    RNB_TRY(L.st.open());
    return launch_quantize_q8k((cudaStream_t)stream, x_dev, cols, seq, (uint8_t *)xq_dev, (uint8_t *)ref_blocks_dev);
}
int rnb_b200_dev_gemv(uint32_t type, const uint8_t *w_dev, size_t rows, size_t cols, const void *x_dev, float *y_dev, int rows_per_tile, void *stream) {
    if (row_bytes_of((int)type, cols) == 0 || cols % (type == TYPE_Q8_0 ? 32 : 256) != 0)
        return fail(RNB_B200_VALIDATION_FAILED, "%s cols must be divisible by %d, got %zu", type_name((int)type), type == TYPE_Q8_0 ? 32 : 256, cols);
    Locked L;
    RNB_TRY(L.st.open());
    GemvJob job = make_job((int)type, w_dev, x_dev, y_dev, nullptr, rows, cols, rows_per_tile, L.st.sm_count);
    return launch_gemv_one((cudaStream_t)stream, job, cols, L.st.dev_error);
}
size_t rnb_b200_flash_decode_scratch_bytes(size_t num_heads, int n_chunks) { return flash_decode_scratch_bytes(num_heads, n_chunks); }
int rnb_b200_flash_decode_default_chunks(size_t kv_len, size_t num_kv_heads) {
    Locked L;
    return flash_decode_default_chunks(kv_len, num_kv_heads, L.st.is_open ? L.st.sm_count : 148);
}
int rnb_b200_dev_flash_decode(const float *q_dev, const uint16_t *k_dev, const uint16_t *v_dev, size_t kv_len, size_t num_heads,
                              size_t num_kv_heads, float scale, float *partials_dev, size_t partials_bytes, int n_chunks,
                              float *out_dev, void *stream) {
    if (!q_dev || !k_dev || !v_dev || !partials_dev || !out_dev) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    if (num_kv_heads == 0 || num_heads == 0 || num_heads % num_kv_heads != 0) return fail(RNB_B200_VALIDATION_FAILED, "attention: num_heads(%zu) must be a multiple of num_kv_heads(%zu)", num_heads, num_kv_heads);
    if (kv_len == 0 || kv_len > (size_t)0x7fffffff) return fail(RNB_B200_VALIDATION_FAILED, "attention kv_len must be in 1..2^31-1, got %zu", kv_len);
    // the merge kernels keep one rescale factor per chunk in a fixed shared-memory array
    if (n_chunks < 1 || n_chunks > FD_MAX_CHUNKS) return fail(RNB_B200_VALIDATION_FAILED, "flash decode n_chunks must be in 1..%d, got %d", FD_MAX_CHUNKS, n_chunks);
    if (partials_bytes < flash_decode_scratch_bytes(num_heads, n_chunks))
        return fail(RNB_B200_VALIDATION_FAILED, "flash decode scratch too small: got %zu, expected >= %zu", partials_bytes, flash_decode_scratch_bytes(num_heads, n_chunks));
    // vector loads: q 16 bytes, K/V 8 bytes (16 selects the tensor-core kernel), f32 records and output
    if (((uintptr_t)q_dev & 15u) || ((uintptr_t)k_dev & 7u) || ((uintptr_t)v_dev & 7u) || ((uintptr_t)out_dev & 3u) || ((uintptr_t)partials_dev & 15u))
        return fail(RNB_B200_VALIDATION_FAILED, "attention operands are not aligned: q and the scratch need 16 bytes, k and v 8 bytes, out 4 bytes");
    Locked L;
    RNB_TRY(L.st.open());
    return launch_attention_decode((cudaStream_t)stream, q_dev, k_dev, v_dev, (int)kv_len, (int)num_heads, (int)num_kv_heads, scale, partials_dev,
                                   n_chunks, out_dev, L.st.dev_error);
}
#ifdef GM_PROFILE
extern "C" int rnb_b200_debug_gm_profile(unsigned long long *out8, int reset) {
    cudaDeviceSynchronize();
    if (cudaMemcpyFromSymbol(out8, g_gm_prof, 8 * sizeof(unsigned long long)) != cudaSuccess) return 1;
    if (reset) {
        unsigned long long z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        cudaMemcpyToSymbol(g_gm_prof, z, sizeof(z));
    }
    return 0;
}
#endif
int rnb_b200_dev_error_flag(int *flag_out) {
    Locked L;
    RNB_TRY(L.st.open());
    RNB_CU(cudaSetDevice(L.st.device));
    int flag = 0;
    RNB_CU(cudaMemcpy(&flag, L.st.dev_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag) RNB_CU(cudaMemset(L.st.dev_error, 0, sizeof(int)));
    if (flag_out) *flag_out = flag;
    return RNB_B200_OK;
}

}  // extern "C"

#include "boundary.inc"
#include "decoder.inc"
