// Prefill-side kernels: causal attention over f32 K/V (the reference's prefill operator takes
// f32 tensors: crates/rnb-backend/cuda/src/runtime/api/attention_api.rs:661-700).
#pragma once
#include "attention.cuh"
#include "prefill_attention_tiled.cuh"
#include "state.hpp"

namespace rnb {

// grid = (seq_len, num_kv_heads), 128 threads: one CTA per (query, KV group); query i sees
// keys 0..(kv_len - seq_len + i).  q/out f32 [seq][heads][128]; k, v [kv_len][kv_heads][128].
template <typename KVT>
RNB_GLOBAL void __launch_bounds__(FD_THREADS)
prefill_attention_kernel(const float *__restrict__ q, const KVT *__restrict__ k,
                         const KVT *__restrict__ v, int seq_len, int kv_len, int num_heads,
                         int num_kv_heads, float scale, float *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_acc[(FD_THREADS / 32) * 4 * HD];
    __shared__ float s_ml[(FD_THREADS / 32) * 4 * 2];
    const int i = blockIdx.x, kv_h = blockIdx.y;
    const int visible = kv_len - seq_len + i + 1;
    const int group = num_heads / num_kv_heads;
    const size_t kv_dim = (size_t)num_kv_heads * HD;
    const float *qi = q + (size_t)i * num_heads * HD;
    float *oi = out + (size_t)i * num_heads * HD;
    for (int g0 = 0; g0 < group; g0 += 4) {
        const int here = min(4, group - g0);
        fd_process<4, KVT>(qi, k, v, kv_h, kv_h * group + g0, here, kv_dim, 0, visible, scale, 1, 0,
                           nullptr, s_acc, s_ml, oi);
        __syncthreads();
    }
}

inline int launch_prefill_attention_f32kv(cudaStream_t s, const float *q, const float *k,
                                          const float *v, int seq_len, int kv_len, int num_heads,
                                          int num_kv_heads, float scale, float *out) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(seq_len, num_kv_heads);
    cfg.blockDim = dim3(FD_THREADS);
    cfg.stream = s;
    RNB_CU(cudaLaunchKernelEx(&cfg, prefill_attention_kernel<float>, q, k, v, seq_len, kv_len,
                              num_heads, num_kv_heads, scale, out));
    return RNB_B200_OK;
}
// f16 caches on 16-byte boundaries take the tensor-core kernel, anything else the CUDA-core one.
inline int launch_prefill_attention_f16kv(cudaStream_t s, const float *q, const uint16_t *k,
                                          const uint16_t *v, int seq_len, int kv_len,
                                          int num_heads, int num_kv_heads, float scale,
                                          float *out, int *dev_error = nullptr) {
    const int group = num_heads / num_kv_heads;
    static const bool simt = [] {
        const char *e = getenv("RNB_B200_FD_SIMT");
        return e && *e == '1';
    }();
    // RNB_B200_PF_ATTN=split keeps the split-KV decode machinery (8 columns per CTA) for prefill
    static const bool tiled = [] {
        const char *e = getenv("RNB_B200_PF_ATTN");
        return !(e && !strcmp(e, "split"));
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.stream = s;
    const bool aligned = (((uintptr_t)k | (uintptr_t)v) & 15) == 0;
    if (!simt && tiled && aligned && group >= 1 && group <= PAT_ROWS && (group & (group - 1)) == 0 && num_heads == group * num_kv_heads &&
        ((uintptr_t)q & 7) == 0 && ((uintptr_t)out & 7) == 0 && kv_len >= seq_len) {
        static bool attr_set = false;
        if (!attr_set) {
            RNB_CU(cudaFuncSetAttribute(prefill_attention_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PAT_SMEM));
            attr_set = true;
        }
        const int qpc = PAT_ROWS / group;
        cfg.blockDim = dim3(PAT_THREADS);
        cfg.gridDim = dim3((seq_len + qpc - 1) / qpc, num_kv_heads);
        cfg.dynamicSmemBytes = PAT_SMEM;
        RNB_CU(cudaLaunchKernelEx(&cfg, prefill_attention_tiled_kernel, q, k, v, seq_len, kv_len, num_heads, num_kv_heads, scale, out));
        return RNB_B200_OK;
    }
    cfg.blockDim = dim3(FD_THREADS);
    if (!simt && aligned) {
        const int qpc = group >= 8 ? 1 : 8 / group;
        cfg.gridDim = dim3(num_kv_heads, (seq_len + qpc - 1) / qpc);
        RNB_CU(cudaLaunchKernelEx(&cfg, prefill_attention_mma_kernel, q, k, v, seq_len, kv_len, num_heads, num_kv_heads, scale, out, dev_error));
        return RNB_B200_OK;
    }
    cfg.gridDim = dim3(seq_len, num_kv_heads);
    RNB_CU(cudaLaunchKernelEx(&cfg, prefill_attention_kernel<uint16_t>, q, k, v, seq_len, kv_len,
                              num_heads, num_kv_heads, scale, out));
    return RNB_B200_OK;
}

}  // namespace rnb
