"""Python mirror of the operator functions of runNburn's `rnb_backend_cuda`
(crates/rnb-backend/cuda/src/runtime/api/*.rs), bound to the C ABI by ctypes.

Same names, argument order and error behaviour as the Rust functions: a failing call raises
`RnbError` carrying the message the Rust `Result::Err(String)` would carry.  Arrays are numpy;
weights are `uint8` views of GGUF block data and stay on the host (the library keeps its own
device-resident copies keyed by host address).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import TYPE_Q4_K, TYPE_Q6_K, TYPE_Q8_0, check, load

Q8K_DTYPE = np.dtype([("d", "<f4"), ("qs", "i1", (256,)), ("bsums", "<i2", (16,))])


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    a = np.asarray(a)
    if a.dtype != np.uint8 or not a.flags["C_CONTIGUOUS"]:
        a = np.ascontiguousarray(a, dtype=np.uint8)
    return a


def _u16(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint16)


# ---- state / cache -------------------------------------------------------------------------
def open() -> None:  # noqa: A001 - mirrors CudaState::open
    check(load().rnb_b200_open())


def close() -> None:
    load().rnb_b200_close()


def cuda_memory_info() -> tuple[int, int]:
    f, t = C.c_size_t(), C.c_size_t()
    check(load().rnb_b200_cuda_memory_info(C.byref(f), C.byref(t)))
    return f.value, t.value


def device_sm_count() -> int:
    n = C.c_int()
    check(load().rnb_b200_device_sm_count(C.byref(n)))
    return n.value


def cuda_cache_snapshot() -> dict:
    s = _lib.CacheSnapshot()
    check(load().rnb_b200_cuda_cache_snapshot(C.byref(s)))
    return {n: getattr(s, n) for n, _ in s._fields_}


def clear_q4k_cache() -> None:
    check(load().rnb_b200_clear_q4k_cache())


def reset_state_for_engine_init() -> None:
    check(load().rnb_b200_reset_state_for_engine_init())


def set_resident_limit(nbytes: int) -> None:
    check(load().rnb_b200_set_resident_limit(nbytes))


def prewarm_q4k_weights(slices) -> int:
    arrs = [_u8(s) for s in slices]
    n = len(arrs)
    ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in arrs])
    lens = (C.c_size_t * n)(*[a.size for a in arrs])
    got = C.c_size_t()
    check(load().rnb_b200_prewarm_q4k_weights(ptrs, lens, n, C.byref(got)))
    return got.value


def inject_resident_alloc_ooms_for_test(count: int) -> None:
    """The next `count` device allocations of the resident cache report out-of-memory (host-side
    fault injection, as the reference's test hook of the same name)."""
    check(load().rnb_b200_inject_resident_alloc_ooms_for_test(count))


def register_host_range(a: np.ndarray) -> None:
    check(load().rnb_b200_register_host_range(_p(a), a.nbytes))


def clear_host_registered_ranges() -> None:
    check(load().rnb_b200_clear_host_registered_ranges())


# ---- quantisation / matvec -----------------------------------------------------------------
def quantize_q8k(x) -> np.ndarray:
    """GGML Q8_K blocks of `x` (structured array, 292 bytes per 256 values), computed on the GPU."""
    x = _f32(x).ravel()
    out = np.zeros(x.size // 256 if x.size % 256 == 0 else 0, dtype=Q8K_DTYPE)
    check(load().rnb_b200_quantize_q8k(_p(x), x.size, _p(out)))
    return out


def _gemv(fn, weights, rows, cols, x, seq=1) -> np.ndarray:
    w, x = _u8(weights), _f32(x).ravel()
    out = np.empty(rows * seq, dtype=np.float32)
    check(fn(_p(w), w.size, rows, cols, _p(x), x.size, _p(out), out.size))
    return out


def q4k_gemv(weights, rows: int, cols: int, x) -> np.ndarray:
    return _gemv(load().rnb_b200_q4k_gemv, weights, rows, cols, x)


def q6k_gemv(weights, rows: int, cols: int, x) -> np.ndarray:
    return _gemv(load().rnb_b200_q6k_gemv, weights, rows, cols, x)


def q2k_gemv(weights, rows: int, cols: int, x) -> np.ndarray:
    """Q2_K matvec (QuantGemvType::Q2K, crates/rnb-cpu/src/gemm/quant_gemv.rs:94-101)"""
    return _gemv(load().rnb_b200_q2k_gemv, weights, rows, cols, x)


def q2k_gemv_batch(weights, rows: int, cols: int, x) -> np.ndarray:
    x = _f32(x)
    return _gemv(load().rnb_b200_q2k_gemv_batch, weights, rows, cols, x, seq=x.size // cols)


def q3k_gemv(weights, rows: int, cols: int, x) -> np.ndarray:
    """Q3_K matvec (QuantGemvType::Q3K, crates/rnb-cpu/src/gemm/quant_gemv.rs:94-101)"""
    return _gemv(load().rnb_b200_q3k_gemv, weights, rows, cols, x)


def q3k_gemv_batch(weights, rows: int, cols: int, x) -> np.ndarray:
    x = _f32(x)
    return _gemv(load().rnb_b200_q3k_gemv_batch, weights, rows, cols, x, seq=x.size // cols)


def q5k_gemv(weights, rows: int, cols: int, x) -> np.ndarray:
    """Q5_K matvec (QuantGemvType::Q5K, crates/rnb-cpu/src/gemm/quant_gemv.rs:94-101)"""
    return _gemv(load().rnb_b200_q5k_gemv, weights, rows, cols, x)


def q5k_gemv_batch(weights, rows: int, cols: int, x) -> np.ndarray:
    x = _f32(x)
    return _gemv(load().rnb_b200_q5k_gemv_batch, weights, rows, cols, x, seq=x.size // cols)


def q8_0_gemv(weights, rows: int, cols: int, x) -> np.ndarray:
    return _gemv(load().rnb_b200_q8_0_gemv, weights, rows, cols, x)


def gemv(ggml_type: int, weights, rows: int, cols: int, x) -> np.ndarray:
    return {TYPE_Q4_K: q4k_gemv, TYPE_Q6_K: q6k_gemv, TYPE_Q8_0: q8_0_gemv}[ggml_type](weights, rows, cols, x)


def q4k_gemv_with_device_input(weights, rows: int, cols: int, input_dev: int) -> np.ndarray:
    w = _u8(weights)
    out = np.empty(rows, dtype=np.float32)
    check(load().rnb_b200_q4k_gemv_with_device_input(_p(w), w.size, rows, cols, input_dev, _p(out), out.size))
    return out


def q6k_gemv_with_device_input(weights, rows: int, cols: int, input_dev: int) -> np.ndarray:
    w = _u8(weights)
    out = np.empty(rows, dtype=np.float32)
    check(load().rnb_b200_q6k_gemv_with_device_input(_p(w), w.size, rows, cols, input_dev, _p(out), out.size))
    return out


def q6k_gemv_argmax(weights, rows: int, cols: int, x) -> tuple[int, float]:
    w, x = _u8(weights), _f32(x).ravel()
    idx, val = C.c_uint32(), C.c_float()
    check(load().rnb_b200_q6k_gemv_argmax(_p(w), w.size, rows, cols, _p(x), x.size, C.byref(idx), C.byref(val)))
    return idx.value, val.value


def q8_0_gemv_argmax(weights, rows: int, cols: int, x) -> tuple[int, float]:
    """q8_0_gemv_argmax — api/quant_api.rs:733"""
    w, x = _u8(weights), _f32(x).ravel()
    idx, val = C.c_uint32(), C.c_float()
    check(load().rnb_b200_q8_0_gemv_argmax(_p(w), w.size, rows, cols, _p(x), x.size, C.byref(idx), C.byref(val)))
    return idx.value, val.value


def q8_0_gemv_batch(weights, rows: int, cols: int, x) -> np.ndarray:
    """q8_0_gemv_batch — api/quant_api.rs:807: input [seq][cols], output [seq][rows]"""
    x = _f32(x).ravel()
    return _gemv(load().rnb_b200_q8_0_gemv_batch, weights, rows, cols, x, seq=max(1, x.size // max(cols, 1)))


def q4k_gemv_batch(weights, rows: int, cols: int, x) -> np.ndarray:
    x = _f32(x).ravel()
    return _gemv(load().rnb_b200_q4k_gemv_batch, weights, rows, cols, x, seq=max(1, x.size // max(cols, 1)))


def q6k_gemv_batch(weights, rows: int, cols: int, x) -> np.ndarray:
    x = _f32(x).ravel()
    return _gemv(load().rnb_b200_q6k_gemv_batch, weights, rows, cols, x, seq=max(1, x.size // max(cols, 1)))


def q4k_bf16_qkv_gemm_batch(q_weights, k_weights, v_weights, q_rows: int, kv_rows: int, cols: int, x):
    """q4k_f16_qkv_gemm_batch — api/quant_api.rs:2405: (q [seq][q_rows], k [seq][kv_rows], v [seq][kv_rows]) of a
    token batch, the three Q4_K projections in one tensor-core launch."""
    qw, kw, vw, x = _u8(q_weights), _u8(k_weights), _u8(v_weights), _f32(x).ravel()
    seq = x.size // max(cols, 1)
    q = np.empty(seq * q_rows, dtype=np.float32)
    k = np.empty(seq * kv_rows, dtype=np.float32)
    v = np.empty(seq * kv_rows, dtype=np.float32)
    check(load().rnb_b200_q4k_bf16_qkv_gemm_batch(_p(qw), qw.size, _p(kw), kw.size, _p(vw), vw.size, q_rows, kv_rows, cols, _p(x), x.size,
                                                  _p(q), q.size, _p(k), k.size, _p(v), v.size))
    return q, k, v


def q4k_bf16_gemm_batch(weights, rows: int, cols: int, x) -> np.ndarray:
    """Tensor-core prefill matmul (reference: q4k_f16_gemm_batch, api/quant_api.rs:2364): bf16
    weights x bf16 tokens, f32 accumulate, output [seq][rows]."""
    x = _f32(x).ravel()
    return _gemv(load().rnb_b200_q4k_bf16_gemm_batch, weights, rows, cols, x, seq=max(1, x.size // max(cols, 1)))


def q6k_bf16_gemm_batch(weights, rows: int, cols: int, x) -> np.ndarray:
    x = _f32(x).ravel()
    return _gemv(load().rnb_b200_q6k_bf16_gemm_batch, weights, rows, cols, x, seq=max(1, x.size // max(cols, 1)))


# ---- attention -----------------------------------------------------------------------------
def attention_decode_hd128(q, k, v, kv_len: int, num_heads: int, num_kv_heads: int, scale: float) -> np.ndarray:
    q, k, v = _f32(q).ravel(), _u16(k).ravel(), _u16(v).ravel()
    out = np.empty(num_heads * 128, dtype=np.float32)
    check(load().rnb_b200_attention_decode_hd128(_p(q), q.size, _p(k), _p(v), min(k.size, v.size), kv_len,
                                                 num_heads, num_kv_heads, scale, _p(out), out.size))
    return out


def quant_embedding_gather(quant: int, weights, rows: int, cols: int, token_ids) -> np.ndarray:
    """quant_embedding_gather — api/quant_api.rs:1827: f32 [n_tokens][cols] rows of a quantised embedding table"""
    w = _u8(weights)
    ids = np.ascontiguousarray(token_ids, dtype=np.uint32).ravel()
    out = np.empty((ids.size, cols), dtype=np.float32)
    check(load().rnb_b200_quant_embedding_gather(quant, _p(w), w.size, rows, cols, _p(ids) if ids.size else None, ids.size,
                                                 _p(out) if ids.size else None, out.size))
    return out


def _attention_decode_wide(fn, head_dim: int, q, k, v, kv_len: int, num_heads: int, num_kv_heads: int, scale: float) -> np.ndarray:
    q, k, v = _f32(q).ravel(), _u16(k).ravel(), _u16(v).ravel()
    out = np.empty(num_heads * head_dim, dtype=np.float32)
    check(fn(_p(q), q.size, _p(k), _p(v), min(k.size, v.size), kv_len, num_heads, num_kv_heads, scale, _p(out), out.size))
    return out


def attention_decode_hd256(q, k, v, kv_len: int, num_heads: int, num_kv_heads: int, scale: float) -> np.ndarray:
    """attention_decode_hd256 — api/attention_api.rs:1906"""
    return _attention_decode_wide(load().rnb_b200_attention_decode_hd256, 256, q, k, v, kv_len, num_heads, num_kv_heads, scale)


def attention_decode_hd512(q, k, v, kv_len: int, num_heads: int, num_kv_heads: int, scale: float) -> np.ndarray:
    """attention_decode_hd512 — api/attention_api.rs:1980"""
    return _attention_decode_wide(load().rnb_b200_attention_decode_hd512, 512, q, k, v, kv_len, num_heads, num_kv_heads, scale)


def attention_decode_cached(layer_index: int, q, k, v, kv_len: int, num_heads: int, num_kv_heads: int,
                            head_dim: int, scale: float) -> np.ndarray:
    q = _f32(q).ravel()
    assert k.dtype == np.uint16 and v.dtype == np.uint16 and k.flags["C_CONTIGUOUS"] and v.flags["C_CONTIGUOUS"], \
        "the KV mirror is keyed by the host buffers' addresses: pass the cache arrays themselves"
    out = np.empty(num_heads * head_dim, dtype=np.float32)
    check(load().rnb_b200_attention_decode_cached(layer_index, _p(q), q.size, _p(k), _p(v), min(k.size, v.size),
                                                  kv_len, num_heads, num_kv_heads, head_dim, scale, _p(out), out.size))
    return out


def attention_decode_cached_window(layer_index: int, q, k, v, kv_len: int, window_start: int, window_len: int,
                                   num_heads: int, num_kv_heads: int, head_dim: int, scale: float) -> np.ndarray:
    """attention_decode_cached_window — api/attention_api.rs:2105: sliding-window decode over positions
    [window_start, window_start + window_len) of the mirrored cache; an empty or out-of-range window raises."""
    q = _f32(q).ravel()
    assert k.dtype == np.uint16 and v.dtype == np.uint16 and k.flags["C_CONTIGUOUS"] and v.flags["C_CONTIGUOUS"], \
        "the KV mirror is keyed by the host buffers' addresses: pass the cache arrays themselves"
    out = np.empty(num_heads * head_dim, dtype=np.float32)
    check(load().rnb_b200_attention_decode_cached_window(layer_index, _p(q), q.size, _p(k), _p(v), min(k.size, v.size), kv_len,
                                                         window_start, window_len, num_heads, num_kv_heads, head_dim, scale,
                                                         _p(out), out.size))
    return out


def clear_decode_attention_kv_cache() -> None:
    check(load().rnb_b200_clear_decode_attention_kv_cache())


def attention_prefill_flash_hd128(q, k, v, seq_len: int, kv_len: int, num_heads: int, num_kv_heads: int,
                                  scale: float) -> np.ndarray:
    q, k, v = _f32(q).ravel(), _f32(k).ravel(), _f32(v).ravel()
    out = np.empty(seq_len * num_heads * 128, dtype=np.float32)
    check(load().rnb_b200_attention_prefill_flash_hd128(_p(q), _p(k), _p(v), seq_len, kv_len, num_heads,
                                                        num_kv_heads, scale, _p(out)))
    return out


def attention_prefill_flash_hd128_f16kv(q, k_bits, v_bits, seq_len: int, kv_len: int, num_heads: int, num_kv_heads: int,
                                        scale: float) -> np.ndarray:
    """Causal prefill attention against an f16 cache (uint16 bit patterns, [kv_len][kv_heads][128])."""
    q = _f32(q).ravel()
    k = np.ascontiguousarray(k_bits, dtype=np.uint16).ravel()
    v = np.ascontiguousarray(v_bits, dtype=np.uint16).ravel()
    out = np.empty(seq_len * num_heads * 128, dtype=np.float32)
    check(load().rnb_b200_attention_prefill_flash_hd128_f16kv(_p(q), _p(k), _p(v), seq_len, kv_len, num_heads,
                                                              num_kv_heads, scale, _p(out)))
    return out


def dense_attention_qkv_rope_hd128_decode(q_w, k_w, v_w, q_rows, kv_rows, n_embd, num_heads, num_kv_heads,
                                          rope_theta, pos_start, x, q_type=TYPE_Q4_K, k_type=TYPE_Q4_K,
                                          v_type=TYPE_Q4_K):
    qw, kw, vw, x = _u8(q_w), _u8(k_w), _u8(v_w), _f32(x).ravel()
    q = np.empty(q_rows, np.float32)
    kb, vb = np.empty(kv_rows, np.uint16), np.empty(kv_rows, np.uint16)
    check(load().rnb_b200_dense_attention_qkv_rope_hd128_decode(
        _p(qw), qw.size, q_type, _p(kw), kw.size, k_type, _p(vw), vw.size, v_type, q_rows, kv_rows, n_embd,
        num_heads, num_kv_heads, rope_theta, pos_start, _p(x), _p(q), _p(kb), _p(vb)))
    return q, kb, vb


def dense_attention_qkv(q_w, k_w, v_w, q_rows, kv_rows, n_embd, x, q_type=TYPE_Q4_K, k_type=TYPE_Q4_K, v_type=TYPE_Q4_K):
    """dense_q4k_attention_qkv — api/dense_api.rs:916: q, k, v of one token in one launch, no RoPE"""
    qw, kw, vw, x = _u8(q_w), _u8(k_w), _u8(v_w), _f32(x).ravel()
    q, k, v = np.empty(q_rows, np.float32), np.empty(kv_rows, np.float32), np.empty(kv_rows, np.float32)
    check(load().rnb_b200_dense_attention_qkv(_p(qw), qw.size, q_type, _p(kw), kw.size, k_type, _p(vw), vw.size, v_type, q_rows, kv_rows, n_embd,
                                              _p(x), x.size, _p(q), q.size, _p(k), k.size, _p(v), v.size))
    return q, k, v


def dense_q4k_silu_ffn_batch(gate, up, down, down_quant, n_ff, n_embd, seq_len, x) -> np.ndarray:
    g, u, d, x = _u8(gate), _u8(up), _u8(down), _f32(x).ravel()
    out = np.empty(seq_len * n_embd, np.float32)
    check(load().rnb_b200_dense_q4k_silu_ffn_batch(_p(g), g.size, _p(u), u.size, _p(d), d.size, down_quant, n_ff,
                                                   n_embd, seq_len, _p(x), _p(out)))
    return out


# ---- MoE -----------------------------------------------------------------------------------
def moe_route_topk_f32(logits, selection_bias, seq_len, n_expert, top_k, sigmoid_mode=False,
                       normalize_selected=False, scale=1.0, adaptive_top_p=None):
    lg = _f32(logits).ravel()
    ids = np.zeros(seq_len * top_k, np.uint32)
    w = np.zeros(seq_len * top_k, np.float32)
    cnt = np.zeros(seq_len, np.uint32)
    bias = None if selection_bias is None else _f32(selection_bias)
    check(load().rnb_b200_moe_route_topk_f32(_p(lg), lg.size, None if bias is None else _p(bias), seq_len, n_expert,
                                             top_k, int(sigmoid_mode), int(normalize_selected), scale,
                                             0.0 if adaptive_top_p is None else adaptive_top_p, _p(ids), _p(w), _p(cnt)))
    return ids, w, cnt


def router_logits_f32(router_w, h) -> np.ndarray:
    w, h = _f32(router_w), _f32(h).ravel()
    out = np.empty(w.shape[0], np.float32)
    check(load().rnb_b200_router_logits_f32(_p(w), w.shape[0], w.shape[1], _p(h), _p(out)))
    return out


def qwen35_sparse_experts(gate, up, down, route_weights, down_quant, n_ff, n_embd, x) -> np.ndarray:
    n = len(gate)
    keep = [_u8(a) for a in list(gate) + list(up) + list(down)]
    arr = C.c_void_p * n
    g = arr(*[a.ctypes.data for a in keep[:n]])
    u = arr(*[a.ctypes.data for a in keep[n:2 * n]])
    d = arr(*[a.ctypes.data for a in keep[2 * n:]])
    rw, x = _f32(route_weights).ravel(), _f32(x).ravel()
    out = np.empty(n_embd, np.float32)
    check(load().rnb_b200_qwen35_sparse_experts(g, u, d, keep[0].size if n else 0, keep[2 * n].size if n else 0, _p(rw), n,
                                                down_quant, n_ff, n_embd, _p(x), _p(out)))
    return out


def qwen35_expert(gate, up, down, down_quant, n_ff, n_embd, x) -> np.ndarray:
    """qwen35_expert — api/qwen_moe_api.rs:1566: one expert's FFN"""
    g, u, d, x = _u8(gate), _u8(up), _u8(down), _f32(x).ravel()
    out = np.empty(n_embd, np.float32)
    check(load().rnb_b200_qwen35_expert(_p(g), g.size, _p(u), u.size, _p(d), d.size, down_quant, n_ff, n_embd, _p(x), x.size, _p(out), out.size))
    return out


def qwen35_sparse_experts_by_token(gate, up, down, route_weights, token_ids, token_count, down_quant, n_ff, n_embd, x) -> np.ndarray:
    """qwen35_sparse_experts_by_token — api/qwen_moe_api.rs:2477: output [token_count][n_embd]"""
    n = len(gate)
    rw, x = _f32(route_weights).ravel(), _f32(x).ravel()
    ids = np.ascontiguousarray(token_ids, dtype=np.uint32).ravel()
    assert len(up) == n and len(down) == n and rw.size == n and ids.size == n, "Qwen35 token-batch sparse expert length mismatch"
    out = np.empty((token_count, n_embd), np.float32)
    if n == 0:
        check(load().rnb_b200_qwen35_sparse_experts_by_token(None, None, None, 0, 0, None, None, 0, token_count, down_quant, n_ff, n_embd,
                                                             _p(x) if x.size else None, x.size, _p(out) if out.size else None, out.size))
        return out
    keep = [_u8(a) for a in list(gate) + list(up) + list(down)]
    arr = C.c_void_p * n
    g = arr(*[a.ctypes.data for a in keep[:n]])
    u = arr(*[a.ctypes.data for a in keep[n:2 * n]])
    d = arr(*[a.ctypes.data for a in keep[2 * n:]])
    check(load().rnb_b200_qwen35_sparse_experts_by_token(g, u, d, keep[0].size, keep[2 * n].size, _p(rw), _p(ids), n, token_count, down_quant, n_ff,
                                                         n_embd, _p(x), x.size, _p(out), out.size))
    return out


def qwen35_register_moe_layer(gate_all, up_all, down_all, down_quant, n_ff, n_embd) -> bool:
    g, u, d = _u8(gate_all), _u8(up_all), _u8(down_all)
    fitted = C.c_int()
    check(load().rnb_b200_qwen35_register_moe_layer(_p(g), g.size, _p(u), u.size, _p(d), d.size, down_quant, n_ff,
                                                    n_embd, C.byref(fitted)))
    return bool(fitted.value)


# ---- glue ----------------------------------------------------------------------------------
def rms_norm_rows_f32(x, weight, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(weight).ravel()
    out = np.empty_like(x)
    check(load().rnb_b200_rms_norm_rows_f32(_p(x), _p(w), w.size, x.size // max(w.size, 1), eps, _p(out)))
    return out


def rope_f32_inplace(data: np.ndarray, pos_start: int, head_dim: int, dim: int, theta: float, neox=False) -> None:
    assert data.dtype == np.float32 and data.flags["C_CONTIGUOUS"]
    check(load().rnb_b200_rope_f32_inplace(_p(data), data.size, pos_start, head_dim, dim, theta, int(neox)))


def activation_mul_f32_inplace(gate: np.ndarray, up) -> None:
    assert gate.dtype == np.float32 and gate.flags["C_CONTIGUOUS"]
    up = _f32(up).ravel()
    check(load().rnb_b200_activation_mul_f32_inplace(_p(gate), _p(up), gate.size))


# ---- expert-cache bookkeeping --------------------------------------------------------------
def evaluate_expert_bundle_admission(missing_bytes, eviction_reload_bytes, predicted_future_reuses,
                                     replaces_temp_upload) -> bool:
    a = _lib.BundleAdmission(missing_bytes, eviction_reload_bytes, predicted_future_reuses, int(replaces_temp_upload))
    return bool(load().rnb_b200_evaluate_expert_bundle_admission(C.byref(a)))


def resident_limit_for(total_bytes: int, free_bytes: int) -> int:
    return int(load().rnb_b200_resident_limit_for(total_bytes, free_bytes))


def dev_error_flag() -> int:
    f = C.c_int()
    check(load().rnb_b200_dev_error_flag(C.byref(f)))
    return f.value


# ---- the rest of the operator boundary --------------------------------------------------------
def add_f32_inplace(dst: np.ndarray, src) -> None:
    """add_f32_inplace — crates/rnb-backend/cuda/src/runtime/api/dense_api.rs:1389"""
    assert dst.dtype == np.float32 and dst.flags["C_CONTIGUOUS"]
    src = _f32(src).ravel()
    check(load().rnb_b200_add_f32_inplace(_p(dst), dst.size, _p(src), src.size))


class DeviceTensor:
    """upload_device_tensor_f32 / download_device_tensor_f32[_row] / release_device_tensor —
    api/sequence_api.rs:4-56"""

    def __init__(self, data, role: int = 0):
        a = _f32(data)
        a2 = a.reshape(1, -1) if a.ndim == 1 else a
        self.rows, self.cols = a2.shape
        ident = C.c_uint64()
        check(load().rnb_b200_upload_device_tensor_f32(self.rows, self.cols, role, _p(a2), a2.size, C.byref(ident)))
        self.id = ident.value

    @property
    def ptr(self) -> int:
        p = C.c_uint64()
        check(load().rnb_b200_device_tensor_ptr(self.id, C.byref(p), None, None))
        return p.value

    def download(self) -> np.ndarray:
        out = np.empty((self.rows, self.cols), np.float32)
        check(load().rnb_b200_download_device_tensor_f32(self.id, _p(out), out.size))
        return out

    def download_row(self, row: int) -> np.ndarray:
        out = np.empty(self.cols, np.float32)
        check(load().rnb_b200_download_device_tensor_f32_row(self.id, row, _p(out), out.size))
        return out

    def release(self) -> bool:
        r = C.c_int()
        check(load().rnb_b200_release_device_tensor(self.id, C.byref(r)))
        return bool(r.value)


CARRIER_HIDDEN, CARRIER_NORM_BUF, CARRIER_K, CARRIER_V, CARRIER_K_F16, CARRIER_V_F16, CARRIER_ATTN_OUT = range(7)


def acquire_decode_carrier(kind: int, nbytes: int) -> int:
    """acquire_decode_*_carrier — api/dense_api.rs:1176-1290"""
    p = C.c_uint64()
    check(load().rnb_b200_acquire_decode_carrier(kind, nbytes, C.byref(p)))
    return p.value


def upload_to_decode_carrier(host: np.ndarray, dev: int) -> None:
    check(load().rnb_b200_upload_to_decode_carrier(_p(host), host.nbytes, dev))


def download_from_decode_carrier(dev: int, host: np.ndarray) -> None:
    check(load().rnb_b200_download_from_decode_carrier(dev, _p(host), host.nbytes))


def sync_decode_stream() -> None:
    check(load().rnb_b200_sync_decode_stream())


def attention_decode_cached_to_device(layer_index: int, q, k, v, kv_len, num_heads, num_kv_heads, head_dim, scale, output_dev: int,
                                      last_token_k_dev: int = 0, last_token_v_dev: int = 0, q_dev_override: int = 0) -> None:
    """attention_decode_cached_to_device — api/attention_api.rs:1776 (0 stands for None)"""
    assert k.dtype == np.uint16 and v.dtype == np.uint16
    qa = _f32(q).ravel() if q is not None else None
    check(load().rnb_b200_attention_decode_cached_to_device(layer_index, _p(qa) if qa is not None else None, qa.size if qa is not None else 0,
                                                            _p(k), _p(v), min(k.size, v.size), kv_len, num_heads, num_kv_heads, head_dim, scale,
                                                            output_dev, last_token_k_dev, last_token_v_dev, q_dev_override))


def dense_attention_qkv_rope_hd128_prefill(q_w, k_w, v_w, q_rows, kv_rows, n_embd, num_heads, num_kv_heads, rope_theta, pos_start, seq_len, x):
    """dense_q4k_attention_qkv_rope_hd128_prefill — api/dense_api.rs:1075; weights are (type, bytes) pairs"""
    (qt, qw), (kt, kw), (vt, vw) = [(t, _u8(w)) for t, w in (q_w, k_w, v_w)]
    x = _f32(x).ravel()
    q = np.empty(seq_len * q_rows, np.float32)
    kb = np.empty(seq_len * kv_rows, np.uint16)
    vb = np.empty(seq_len * kv_rows, np.uint16)
    check(load().rnb_b200_dense_attention_qkv_rope_hd128_prefill(_p(qw), qw.size, qt, _p(kw), kw.size, kt, _p(vw), vw.size, vt, q_rows, kv_rows,
                                                                 n_embd, num_heads, num_kv_heads, rope_theta, pos_start, seq_len, _p(x), x.size,
                                                                 _p(q), _p(kb), _p(vb)))
    return q, kb, vb


class ExpertStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("bundle_lookups", "bundle_hits", "bundle_partial_hits", "bundle_misses", "bundle_admissions",
                                          "bundle_evictions", "admitted_bytes", "evicted_bytes", "h2d_bytes", "temp_h2d_bytes")]

    def as_dict(self) -> dict:
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


class ExpertReceipt(C.Structure):
    _fields_ = [("consumed", C.c_uint32), ("reserved", C.c_uint32), ("pending_stats", ExpertStats)]


def _expert_ptrs(gate, up, down):
    n = len(gate)
    keep = [_u8(a) for a in list(gate) + list(up) + list(down)]
    arr = C.c_void_p * n
    return keep, arr(*[a.ctypes.data for a in keep[:n]]), arr(*[a.ctypes.data for a in keep[n:2 * n]]), arr(*[a.ctypes.data for a in keep[2 * n:]])


def qwen35_sparse_experts_into(gate, up, down, route_weights, layer_idx, selected_expert_ids, receipt, down_quant, n_ff, n_embd, x,
                               residual=None) -> np.ndarray:
    """qwen35_sparse_experts_into / _add_residual_into — api/qwen_moe_api.rs:1918,2163.  layer_idx None -> -1."""
    n = len(gate)
    keep, g, u, d = _expert_ptrs(gate, up, down)
    rw, x = _f32(route_weights).ravel(), _f32(x).ravel()
    ids = (C.c_size_t * n)(*[int(i) for i in selected_expert_ids]) if selected_expert_ids is not None else None
    li = -1 if layer_idx is None else int(layer_idx)
    rc = C.byref(receipt) if receipt is not None else None
    if residual is None:
        out = np.empty(n_embd, np.float32)
        check(load().rnb_b200_qwen35_sparse_experts_into(g, u, d, keep[0].size, keep[2 * n].size, _p(rw), n, li, ids, rc, down_quant, n_ff, n_embd,
                                                         _p(x), _p(out), out.size))
        return out
    out = _f32(residual).ravel().copy()
    check(load().rnb_b200_qwen35_sparse_experts_add_residual_into(g, u, d, keep[0].size, keep[2 * n].size, _p(rw), n, li, ids, rc, down_quant, n_ff,
                                                                  n_embd, _p(x), _p(out), out.size))
    return out


def qwen35_expert_cache_stats() -> dict:
    s = ExpertStats()
    check(load().rnb_b200_qwen35_expert_cache_stats(C.byref(s)))
    return s.as_dict()


def qwen35_configure_moe_layer_cache(model_moe_bytes: int, runtime_headroom_bytes: int, min_layer_bytes: int) -> int:
    out = C.c_size_t()
    check(load().rnb_b200_qwen35_configure_moe_layer_cache(model_moe_bytes, runtime_headroom_bytes, min_layer_bytes, C.byref(out)))
    return out.value


def qwen35_admit_expert_misses_async(slices) -> int:
    keep = [_u8(a) for a in slices]
    n = len(keep)
    ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in keep])
    lens = (C.c_size_t * n)(*[a.size for a in keep])
    out = C.c_size_t()
    check(load().rnb_b200_qwen35_admit_expert_misses_async(ptrs, lens, n, C.byref(out)))
    return out.value


def qwen35_prefill_device_topk_route_slots(router_w, norm_all, n_expert_used: int):
    w, h = _f32(router_w), _f32(norm_all)
    n_expert, hidden = w.shape
    seq = h.size // hidden
    ids = np.empty(seq * n_expert_used, np.uint32)
    wts = np.empty(seq * n_expert_used, np.float32)
    toks = np.empty(seq * n_expert_used, np.uint32)
    check(load().rnb_b200_qwen35_prefill_device_topk_route_slots(_p(w), n_expert, hidden, _p(h), seq, n_expert_used, _p(ids), _p(wts), _p(toks)))
    return ids, wts, toks


def cuda_weight_residency_counters() -> dict:
    names = ("expanded_diag_bytes", "native_f32_bytes", "packed_q8dot_bytes", "raw_quant_bytes", "transient_quant_upload_bytes",
             "q4_expanded_f16_bytes", "q4_expanded_f32_bytes", "q6_expanded_f16_bytes", "q6_expanded_f32_bytes", "q4_raw_quant_bytes",
             "q6_raw_quant_bytes", "q4_transient_quant_upload_bytes", "q6_transient_quant_upload_bytes")
    buf = (C.c_uint64 * len(names))()
    check(load().rnb_b200_cuda_weight_residency_counters(buf))
    return dict(zip(names, [int(v) for v in buf]))


def prewarm_quant_resident_weights(slices) -> int:
    keep = [_u8(a) for a in slices]
    n = len(keep)
    ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in keep])
    lens = (C.c_size_t * n)(*[a.size for a in keep])
    out = C.c_size_t()
    check(load().rnb_b200_prewarm_quant_resident_weights(ptrs, lens, n, C.byref(out)))
    return out.value
