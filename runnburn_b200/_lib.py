"""Loads librnb_b200.so and declares its C ABI (include/rnb_b200.h) for ctypes.

The CUDA library is the product: if it is missing this module raises, there is no fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "librnb_b200.so"
HEADER = PKG.parent / "include" / "rnb_b200.h"

OK, UNSUPPORTED, VALIDATION_FAILED, OUT_OF_MEMORY, CUDA_ERROR, DEVICE_FAULT_FLAG = range(6)
TYPE_Q8_0, TYPE_Q4_K, TYPE_Q6_K = 8, 12, 14
TYPE_Q5_K = 13


class RnbError(RuntimeError):
    """A failing library call: `status` is the RNB_B200_* code, the message is the library's."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class CacheSnapshot(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "lookups", "hits", "misses", "evictions", "uploads", "upload_bytes", "transient_uploads",
        "resident_entries", "resident_bytes", "resident_limit_bytes", "h2d_bytes", "d2h_bytes")]


class BundleAdmission(C.Structure):
    _fields_ = [("missing_bytes", C.c_uint64), ("eviction_reload_bytes", C.c_uint64),
                ("predicted_future_reuses", C.c_uint32), ("replaces_temp_upload", C.c_uint32)]


class ModelCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "hidden", "n_head", "n_kv_head", "head_dim",
                                         "n_ff", "vocab", "rope_neox")] + \
               [("rms_eps", C.c_float), ("rope_theta", C.c_float)] + \
               [(n, C.c_int32) for n in ("n_expert", "n_expert_used", "n_ff_expert", "max_ctx",
                                         "world_size", "rank")]


class QWeight(C.Structure):
    _fields_ = [("type", C.c_uint32), ("data", C.c_void_p), ("len", C.c_size_t)]


class GgufTensorInfo(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("n_dims", C.c_uint32), ("ggml_type", C.c_uint32), ("dims", C.c_uint64 * 4),
                ("offset", C.c_uint64), ("n_elements", C.c_uint64), ("n_bytes", C.c_uint64), ("data", C.c_void_p)]


class LayerWeights(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p)] + \
               [(n, QWeight) for n in ("wq", "wk", "wv", "wo", "gate", "up", "down")] + \
               [("router", C.c_void_p)] + \
               [(n, QWeight) for n in ("gate_exps", "up_exps", "down_exps")]


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m runnburn_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this library.")
    L = C.CDLL(str(LIB_PATH))
    sz, vp, i32, u32, f32, u64 = C.c_size_t, C.c_void_p, C.c_int, C.c_uint32, C.c_float, C.c_uint64
    L.rnb_b200_last_error.restype = C.c_char_p
    L.rnb_b200_close.restype = None
    L.rnb_b200_gguf_close.restype = None
    L.rnb_b200_gguf_close.argtypes = [C.c_void_p]
    sig = {
        "rnb_b200_open": [],
        "rnb_b200_cuda_memory_info": [vp, vp],
        "rnb_b200_device_sm_count": [vp],
        "rnb_b200_cuda_cache_snapshot": [vp],
        "rnb_b200_clear_q4k_cache": [],
        "rnb_b200_reset_state_for_engine_init": [],
        "rnb_b200_prewarm_q4k_weights": [vp, vp, sz, vp],
        "rnb_b200_set_resident_limit": [sz],
        "rnb_b200_register_host_range": [vp, sz],
        "rnb_b200_clear_host_registered_ranges": [],
        "rnb_b200_quantize_q8k": [vp, sz, vp],
        "rnb_b200_q4k_gemv": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q6k_gemv": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q5k_gemv": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q2k_gemv": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q3k_gemv": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q3k_gemv_batch": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q2k_gemv_batch": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q5k_gemv_batch": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q8_0_gemv": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q4k_gemv_with_device_input": [vp, sz, sz, sz, u64, vp, sz],
        "rnb_b200_q6k_gemv_with_device_input": [vp, sz, sz, sz, u64, vp, sz],
        "rnb_b200_q6k_gemv_argmax": [vp, sz, sz, sz, vp, sz, vp, vp],
        "rnb_b200_q4k_bf16_qkv_gemm_batch": [vp, sz, vp, sz, vp, sz, sz, sz, sz, vp, sz, vp, sz, vp, sz, vp, sz],
        "rnb_b200_dense_attention_qkv": [vp, sz, u32, vp, sz, u32, vp, sz, u32, sz, sz, sz, vp, sz, vp, sz, vp, sz, vp, sz],
        "rnb_b200_q8_0_gemv_argmax": [vp, sz, sz, sz, vp, sz, vp, vp],
        "rnb_b200_q8_0_gemv_batch": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q4k_gemv_batch": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q6k_gemv_batch": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q4k_bf16_gemm_batch": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_q6k_bf16_gemm_batch": [vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_attention_decode_hd128": [vp, sz, vp, vp, sz, sz, sz, sz, f32, vp, sz],
        "rnb_b200_quant_embedding_gather": [u32, vp, sz, sz, sz, vp, sz, vp, sz],
        "rnb_b200_attention_decode_hd256": [vp, sz, vp, vp, sz, sz, sz, sz, f32, vp, sz],
        "rnb_b200_attention_decode_hd512": [vp, sz, vp, vp, sz, sz, sz, sz, f32, vp, sz],
        "rnb_b200_attention_decode_cached": [sz, vp, sz, vp, vp, sz, sz, sz, sz, sz, f32, vp, sz],
        "rnb_b200_attention_decode_cached_window": [sz, vp, sz, vp, vp, sz, sz, sz, sz, sz, sz, sz, f32, vp, sz],
        "rnb_b200_clear_decode_attention_kv_cache": [],
        "rnb_b200_attention_prefill_flash_hd128": [vp, vp, vp, sz, sz, sz, sz, f32, vp],
        "rnb_b200_attention_prefill_flash_hd128_f16kv": [vp, vp, vp, sz, sz, sz, sz, f32, vp],
        "rnb_b200_dense_attention_qkv_rope_hd128_decode": [
            vp, sz, u32, vp, sz, u32, vp, sz, u32, sz, sz, sz, sz, sz, f32, sz, vp, vp, vp, vp],
        "rnb_b200_dense_q4k_silu_ffn_batch": [vp, sz, vp, sz, vp, sz, u32, sz, sz, sz, vp, vp],
        "rnb_b200_moe_route_topk_f32": [vp, sz, vp, sz, sz, sz, i32, i32, f32, f32, vp, vp, vp],
        "rnb_b200_router_logits_f32": [vp, sz, sz, vp, vp],
        "rnb_b200_qwen35_expert": [vp, sz, vp, sz, vp, sz, u32, sz, sz, vp, sz, vp, sz],
        "rnb_b200_qwen35_sparse_experts_by_token": [vp, vp, vp, sz, sz, vp, vp, sz, sz, u32, sz, sz, vp, sz, vp, sz],
        "rnb_b200_qwen35_sparse_experts": [vp, vp, vp, sz, sz, vp, sz, u32, sz, sz, vp, vp],
        "rnb_b200_qwen35_register_moe_layer": [vp, sz, vp, sz, vp, sz, u32, sz, sz, vp],
        "rnb_b200_rms_norm_rows_f32": [vp, vp, sz, sz, f32, vp],
        "rnb_b200_rope_f32_inplace": [vp, sz, sz, sz, sz, f32, i32],
        "rnb_b200_activation_mul_f32_inplace": [vp, vp, sz],
        "rnb_b200_evaluate_expert_bundle_admission": [vp],
        "rnb_b200_add_f32_inplace": [vp, sz, vp, sz],
        "rnb_b200_upload_device_tensor_f32": [sz, sz, u32, vp, sz, vp],
        "rnb_b200_download_device_tensor_f32": [u64, vp, sz],
        "rnb_b200_download_device_tensor_f32_row": [u64, sz, vp, sz],
        "rnb_b200_release_device_tensor": [u64, vp],
        "rnb_b200_device_tensor_ptr": [u64, vp, vp, vp],
        "rnb_b200_acquire_decode_carrier": [u32, sz, vp],
        "rnb_b200_upload_to_decode_carrier": [vp, sz, u64],
        "rnb_b200_download_from_decode_carrier": [u64, vp, sz],
        "rnb_b200_sync_decode_stream": [],
        "rnb_b200_attention_decode_cached_to_device": [sz, vp, sz, vp, vp, sz, sz, sz, sz, sz, f32, u64, u64, u64, u64],
        "rnb_b200_dense_attention_qkv_rope_hd128_prefill": [
            vp, sz, u32, vp, sz, u32, vp, sz, u32, sz, sz, sz, sz, sz, f32, sz, sz, vp, sz, vp, vp, vp],
        "rnb_b200_qwen35_sparse_experts_into": [vp, vp, vp, sz, sz, vp, sz, C.c_int64, vp, vp, u32, sz, sz, vp, vp, sz],
        "rnb_b200_qwen35_sparse_experts_add_residual_into": [vp, vp, vp, sz, sz, vp, sz, C.c_int64, vp, vp, u32, sz, sz, vp, vp, sz],
        "rnb_b200_qwen35_expert_cache_stats": [vp],
        "rnb_b200_qwen35_configure_moe_layer_cache": [sz, sz, sz, vp],
        "rnb_b200_qwen35_admit_expert_misses_async": [vp, vp, sz, vp],
        "rnb_b200_qwen35_prefill_device_topk_route_slots": [vp, sz, sz, vp, sz, sz, vp, vp, vp],
        "rnb_b200_cuda_weight_residency_counters": [vp],
        "rnb_b200_prewarm_quant_resident_weights": [vp, vp, sz, vp],
        "rnb_b200_decoder_create": [vp, vp],
        "rnb_b200_decoder_set_layer": [vp, i32, vp],
        "rnb_b200_decoder_set_globals": [vp, QWeight, vp, QWeight],
        "rnb_b200_decoder_fill_synthetic": [vp, u64, f32],
        "rnb_b200_decoder_fill_kv_synthetic": [vp, i32, u64],
        "rnb_b200_decoder_step": [vp, u32, i32, vp, vp],
        "rnb_b200_decoder_step_dev": [vp, i32, i32],
        "rnb_b200_decoder_sync": [vp],
        "rnb_b200_decoder_read_kv": [vp, i32, i32, vp, vp],
        "rnb_b200_decoder_read_hidden": [vp, vp],
        "rnb_b200_decoder_read_expert_ids": [vp, i32, vp],
        "rnb_b200_decoder_stats": [vp, vp, vp, vp],
        "rnb_b200_decoder_time_steps": [vp, i32, i32, vp],
        "rnb_b200_decoder_time_matvecs": [vp, i32, vp, vp, vp],
        "rnb_b200_nccl_unique_id": [vp],
        "rnb_b200_decoder_attach_nccl": [vp, vp],
        "rnb_b200_decoder_prefill": [vp, vp, i32, i32, vp, vp],
        "rnb_b200_decoder_read_logits": [vp, vp, sz],
        "rnb_b200_decoder_exchange_handle": [vp, vp],
        "rnb_b200_decoder_attach_peers": [vp, vp],
        "rnb_b200_peer_exchange_timeout_selftest": [vp],
        "rnb_b200_dev_quantize_q8k": [vp, sz, sz, vp, vp, vp],
        "rnb_b200_dev_gemv": [u32, vp, sz, sz, vp, vp, i32, vp],
        "rnb_b200_dev_prefill_gemm": [i32, vp, sz, sz, vp, sz, vp, vp, vp],
        "rnb_b200_dev_prefill_gemm_multi": [i32, vp, vp, vp, vp, sz, vp, sz, vp, vp],
        "rnb_b200_dev_prefill_gemm_silu": [i32, vp, vp, sz, sz, vp, sz, vp, vp, vp],
        "rnb_b200_dev_flash_decode": [vp, vp, vp, sz, sz, sz, f32, vp, sz, i32, vp, vp],
        "rnb_b200_flash_decode_default_chunks": [sz, sz],
        "rnb_b200_attention_decode_hd128_noalloc": [vp, vp, vp, sz, sz, sz, f32, vp, vp],
        "rnb_b200_attention_decode_hd128_noalloc_status": [vp, vp],
        "rnb_b200_dev_error_flag": [vp],
        "rnb_b200_decoder_config": [vp, vp],
        "rnb_b200_decoder_set_exact_attention_max": [vp, C.c_int],
        "rnb_b200_gguf_open": [C.c_char_p, vp],
        "rnb_b200_gguf_parse": [vp, sz, vp],
        "rnb_b200_gguf_info": [vp, vp, vp, vp, vp, vp],
        "rnb_b200_gguf_get_u64": [vp, C.c_char_p, vp],
        "rnb_b200_gguf_get_f64": [vp, C.c_char_p, vp],
        "rnb_b200_gguf_get_str": [vp, C.c_char_p, vp, sz, vp],
        "rnb_b200_gguf_get_array_u64": [vp, C.c_char_p, vp, sz, vp],
        "rnb_b200_gguf_tensor": [vp, C.c_char_p, vp],
        "rnb_b200_gguf_tensor_at": [vp, sz, vp],
        "rnb_b200_gguf_model_config": [vp, i32, vp],
        "rnb_b200_decoder_load_gguf": [vp, vp, i32],
        "rnb_b200_inject_resident_alloc_ooms_for_test": [sz],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = i32
    L.rnb_b200_decoder_destroy.argtypes = [vp]
    L.rnb_b200_decoder_destroy.restype = None
    L.rnb_b200_decoder_stream.argtypes = [vp]
    L.rnb_b200_decoder_stream.restype = vp
    L.rnb_b200_resident_limit_for.argtypes = [u64, u64]
    L.rnb_b200_resident_limit_for.restype = u64
    L.rnb_b200_dev_q8k_bytes.argtypes = [sz]
    L.rnb_b200_dev_q8k_bytes.restype = sz
    L.rnb_b200_flash_decode_scratch_bytes.argtypes = [sz, i32]
    L.rnb_b200_flash_decode_scratch_bytes.restype = sz
    _lib = L
    return L


def check(status: int) -> None:
    if status != OK:
        raise RnbError(status, load().rnb_b200_last_error().decode("utf-8", "replace"))
