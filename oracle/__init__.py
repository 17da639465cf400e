"""ctypes binding of the CPU oracle (`oracle/rnb_oracle.c`).

TEST INFRASTRUCTURE ONLY.  Importers are the test-suite, the smoke check and the bench's
CPU-baseline leg; the shipped package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "librnb_oracle.so"

TYPE_Q8_0 = 8
TYPE_Q2_K = 10
TYPE_Q3_K = 11
TYPE_Q4_K = 12
TYPE_Q5_K = 13
TYPE_Q6_K = 14
Q8K_DTYPE = np.dtype([("d", "<f4"), ("qs", "i1", (256,)), ("bsums", "<i2", (16,))])
assert Q8K_DTYPE.itemsize == 292


def build(force: bool = False) -> Path:
    """Compile the oracle with the committed Makefile (gcc only)."""
    src_mtime = max((_HERE / n).stat().st_mtime for n in ("rnb_oracle.c", "rnb_oracle.h"))
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        _lib = C.CDLL(str(_LIB_PATH))
        _declare(_lib)
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _declare(L):
    sz, vp, i32, f32 = C.c_size_t, C.c_void_p, C.c_int, C.c_float
    L.orc_f16_to_f32.restype = f32
    L.orc_f16_to_f32.argtypes = [C.c_uint16]
    L.orc_f32_to_f16.restype = C.c_uint16
    L.orc_f32_to_f16.argtypes = [f32]
    L.orc_f32_to_f16_row.argtypes = [vp, vp, sz]
    L.orc_quantize_q8k.argtypes = [vp, sz, vp]
    L.orc_dequantize_row.argtypes = [i32, vp, sz, vp]
    L.orc_dequantize_row.restype = i32
    L.orc_quantize_matrix.argtypes = [i32, vp, sz, sz, vp, i32]
    L.orc_quantize_matrix.restype = i32
    L.orc_synth_matrix.argtypes = [i32, sz, sz, C.c_uint64, C.c_float, vp, i32]
    L.orc_synth_matrix.restype = i32
    for n in ("orc_dot_q2k_q8k", "orc_dot_q3k_q8k", "orc_dot_q4k_q8k", "orc_dot_q5k_q8k", "orc_dot_q6k_q8k", "orc_dot_q4k_q8k_lanes", "orc_dot_q6k_q8k_lanes"):
        getattr(L, n).restype = f32
        getattr(L, n).argtypes = [vp, vp, sz]
    L.orc_dot_q8_0_row.restype = f32
    L.orc_dot_q8_0_row.argtypes = [vp, vp, sz]
    L.orc_dot_dequant_row.restype = f32
    L.orc_dot_dequant_row.argtypes = [i32, vp, vp, sz]
    L.orc_have_avx2.restype = i32
    L.orc_force_scalar.argtypes = [i32]
    L.orc_gemv.restype = i32
    L.orc_gemv.argtypes = [i32, vp, vp, vp, sz, sz, sz, i32]
    L.orc_row_bytes.restype = sz
    L.orc_row_bytes.argtypes = [i32, sz]
    L.orc_attention_decode.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, f32]
    L.orc_attention_decode_window.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, f32, sz]
    L.orc_attention_decode_online.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, f32]
    L.orc_attention_decode_mt.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, f32, i32]
    L.orc_attention_prefill.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, sz, f32]
    L.orc_attention_prefill_f16kv.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, sz, f32]
    L.orc_moe_route_topk.restype = sz
    L.orc_moe_route_topk.argtypes = [vp, sz, sz, vp, vp]
    L.orc_gemv_f32.argtypes = [vp, vp, vp, sz, sz]
    L.orc_moe_experts.restype = i32
    L.orc_moe_experts.argtypes = [vp, vp, vp, vp, sz, i32, sz, sz, vp, vp, i32]
    L.orc_rms_norm.argtypes = [vp, vp, f32, vp, sz, sz]
    L.orc_rope_inplace.argtypes = [vp, sz, sz, sz, sz, f32]
    L.orc_rope_neox_inplace.argtypes = [vp, sz, sz, sz, sz, f32]
    L.orc_rope_table.argtypes = [sz, sz, f32, vp, vp]
    L.orc_silu_mul_inplace.argtypes = [vp, vp, sz]
    L.orc_argmax_last.restype = C.c_uint32
    L.orc_argmax_last.argtypes = [vp, sz]
    L.orc_model_create.restype = vp
    L.orc_model_create.argtypes = [vp, vp, _QWeight, vp, _QWeight, sz, i32]
    L.orc_model_free.argtypes = [vp]
    L.orc_model_reset.argtypes = [vp]
    L.orc_model_decode.restype = C.POINTER(C.c_float)
    L.orc_model_decode.argtypes = [vp, C.c_uint32, sz]
    L.orc_model_k_cache.restype = C.POINTER(C.c_uint16)
    L.orc_model_k_cache.argtypes = [vp, i32]
    L.orc_model_v_cache.restype = C.POINTER(C.c_uint16)
    L.orc_model_v_cache.argtypes = [vp, i32]
    L.orc_model_hidden.restype = C.POINTER(C.c_float)
    L.orc_model_hidden.argtypes = [vp]
    L.orc_model_last_expert_ids.restype = C.POINTER(C.c_uint32)
    L.orc_model_last_expert_ids.argtypes = [vp, i32]


def n_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


def row_bytes(ggml_type: int, cols: int) -> int:
    return int(lib().orc_row_bytes(ggml_type, cols))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


# ---- conversions ---------------------------------------------------------------------------
def f32_to_f16_bits(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_f16_row(_p(x), _p(out), x.size)
    return out


def f16_bits_to_f32(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    f = lib().orc_f16_to_f32
    return np.array([f(int(v)) for v in h.ravel()], dtype=np.float32).reshape(h.shape)


# ---- quantisation --------------------------------------------------------------------------
def quantize_q8k(x) -> np.ndarray:
    """f32[n] (n % 256 == 0) → structured array of Q8_K blocks (292 bytes each)."""
    x = _f32(x).ravel()
    assert x.size % 256 == 0
    out = np.zeros(x.size // 256, dtype=Q8K_DTYPE)
    lib().orc_quantize_q8k(_p(x), x.size, _p(out))
    return out


def quantize_matrix(ggml_type: int, w, threads: int | None = None) -> np.ndarray:
    w = _f32(w)
    rows, cols = w.shape
    out = np.zeros(rows * row_bytes(ggml_type, cols), dtype=np.uint8)
    rc = lib().orc_quantize_matrix(ggml_type, _p(w), rows, cols, _p(out), threads or n_threads())
    assert rc == 0
    return out


def synth_matrix(ggml_type: int, rows: int, cols: int, seed: int, sigma: float = 0.02,
                 threads: int | None = None) -> np.ndarray:
    """Seeded N(0, sigma) weights as GGUF blocks, quantised with a plain per-block fit: a fast
    harness utility for full-width test models (not a restatement of reference code)."""
    out = np.zeros(rows * row_bytes(ggml_type, cols), dtype=np.uint8)
    rc = lib().orc_synth_matrix(ggml_type, rows, cols, seed, sigma, _p(out), threads or n_threads())
    assert rc == 0
    return out


def dequantize_matrix(ggml_type: int, data, rows: int, cols: int) -> np.ndarray:
    data = _u8(data)
    rb = row_bytes(ggml_type, cols)
    out = np.empty((rows, cols), dtype=np.float32)
    for r in range(rows):
        rc = lib().orc_dequantize_row(ggml_type, _p(data[r * rb:(r + 1) * rb]), cols, _p(out[r]))
        assert rc == 0
    return out


# ---- dots / GEMV ---------------------------------------------------------------------------
def dot_row(ggml_type: int, row, xq: np.ndarray, lanes: bool = False) -> float:
    row = _u8(row)
    name = {TYPE_Q2_K: "orc_dot_q2k_q8k", TYPE_Q3_K: "orc_dot_q3k_q8k", TYPE_Q4_K: "orc_dot_q4k_q8k", TYPE_Q5_K: "orc_dot_q5k_q8k", TYPE_Q6_K: "orc_dot_q6k_q8k"}[ggml_type]
    if lanes:
        name += "_lanes"
    return float(getattr(lib(), name)(_p(row), _p(xq), xq.size))


def dot_q8_0_row(row, x) -> float:
    row, x = _u8(row), _f32(x)
    return float(lib().orc_dot_q8_0_row(_p(row), _p(x), x.size // 32))


def dot_dequant_row(ggml_type: int, row, x) -> float:
    row, x = _u8(row), _f32(x)
    return float(lib().orc_dot_dequant_row(ggml_type, _p(row), _p(x), x.size))


def gemv(ggml_type: int, w, x, rows: int, cols: int, seq_len: int = 1,
         threads: int | None = None) -> np.ndarray:
    """Seq-major output `out[s*rows + row]`, Q8_K activations for K-quants, f32 for Q8_0."""
    w, x = _u8(w), _f32(x).ravel()
    assert w.size == rows * row_bytes(ggml_type, cols), "weight byte mismatch"
    assert x.size == seq_len * cols
    out = np.empty(seq_len * rows, dtype=np.float32)
    rc = lib().orc_gemv(ggml_type, _p(w), _p(x), _p(out), rows, cols, seq_len,
                        threads or n_threads())
    assert rc == 0
    return out


# ---- attention -----------------------------------------------------------------------------
def attention_decode(q, k_bits, v_bits, num_heads, num_kv_heads, head_dim, kv_len, scale,
                     online: bool = False, threads: int = 1) -> np.ndarray:
    q = _f32(q).ravel()
    k = np.ascontiguousarray(k_bits, dtype=np.uint16)
    v = np.ascontiguousarray(v_bits, dtype=np.uint16)
    out = np.empty(num_heads * head_dim, dtype=np.float32)
    if threads > 1 and not online:
        lib().orc_attention_decode_mt(_p(q), _p(k), _p(v), _p(out), num_heads, num_kv_heads,
                                      head_dim, kv_len, scale, threads)
        return out
    fn = lib().orc_attention_decode_online if online else lib().orc_attention_decode
    fn(_p(q), _p(k), _p(v), _p(out), num_heads, num_kv_heads, head_dim, kv_len, scale)
    return out


def attention_decode_window(q, k_bits, v_bits, num_heads, num_kv_heads, head_dim, kv_len, scale, window: int) -> np.ndarray:
    """The CPU routine with sliding_window = Some(window): every position walked, masked ones with weight zero."""
    q = _f32(q).ravel()
    k = np.ascontiguousarray(k_bits, dtype=np.uint16)
    v = np.ascontiguousarray(v_bits, dtype=np.uint16)
    out = np.empty(num_heads * head_dim, dtype=np.float32)
    lib().orc_attention_decode_window(_p(q), _p(k), _p(v), _p(out), num_heads, num_kv_heads, head_dim, kv_len, scale, window)
    return out


def attention_prefill(q, k, v, seq_len, kv_len, num_heads, num_kv_heads, head_dim, scale):
    q = _f32(q).ravel()
    out = np.empty(seq_len * num_heads * head_dim, dtype=np.float32)
    if np.asarray(k).dtype == np.uint16:
        k = np.ascontiguousarray(k, dtype=np.uint16)
        v = np.ascontiguousarray(v, dtype=np.uint16)
        lib().orc_attention_prefill_f16kv(_p(q), _p(k), _p(v), _p(out), seq_len, kv_len,
                                          num_heads, num_kv_heads, head_dim, scale)
    else:
        k, v = _f32(k), _f32(v)
        lib().orc_attention_prefill(_p(q), _p(k), _p(v), _p(out), seq_len, kv_len, num_heads,
                                    num_kv_heads, head_dim, scale)
    return out


# ---- MoE -----------------------------------------------------------------------------------
def moe_route_topk(logits, top_k: int):
    logits = _f32(logits).ravel()
    ids = np.zeros(32, dtype=np.uint32)
    w = np.zeros(32, dtype=np.float32)
    n = lib().orc_moe_route_topk(_p(logits), logits.size, top_k, _p(ids), _p(w))
    return ids[:n].copy(), w[:n].copy()


def gemv_f32(w, x) -> np.ndarray:
    w, x = _f32(w), _f32(x).ravel()
    out = np.empty(w.shape[0], dtype=np.float32)
    lib().orc_gemv_f32(_p(w), _p(x), _p(out), w.shape[0], w.shape[1])
    return out


def moe_experts(gate_list, up_list, down_list, route_weights, down_type, n_ff, n_embd, x,
                threads: int | None = None) -> np.ndarray:
    n = len(gate_list)
    keep = [_u8(a) for a in list(gate_list) + list(up_list) + list(down_list)]
    arr = (C.c_void_p * n)
    g = arr(*[a.ctypes.data for a in keep[:n]])
    u = arr(*[a.ctypes.data for a in keep[n:2 * n]])
    d = arr(*[a.ctypes.data for a in keep[2 * n:]])
    rw, x = _f32(route_weights), _f32(x)
    out = np.empty(n_embd, dtype=np.float32)
    rc = lib().orc_moe_experts(g, u, d, _p(rw), n, down_type, n_ff, n_embd, _p(x), _p(out),
                               threads or n_threads())
    assert rc == 0
    return out


# ---- glue ----------------------------------------------------------------------------------
def rms_norm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    hidden = w.size
    out = np.empty_like(x)
    lib().orc_rms_norm(_p(x), _p(w), eps, _p(out), hidden, x.size // hidden)
    return out


def rope(x, pos_start: int, head_dim: int, dim: int, theta: float, neox: bool = False):
    x = _f32(x).copy()
    fn = lib().orc_rope_neox_inplace if neox else lib().orc_rope_inplace
    fn(_p(x), x.size, pos_start, head_dim, dim, theta)
    return x


def rope_table(pos: int, head_dim: int, theta: float):
    c = np.empty(head_dim // 2, dtype=np.float32)
    s = np.empty(head_dim // 2, dtype=np.float32)
    lib().orc_rope_table(pos, head_dim, theta, _p(c), _p(s))
    return c, s


def silu_mul(gate, up) -> np.ndarray:
    g, u = _f32(gate).copy(), _f32(up)
    lib().orc_silu_mul_inplace(_p(g), _p(u), g.size)
    return g


def argmax_last(x) -> int:
    x = _f32(x)
    return int(lib().orc_argmax_last(_p(x), x.size))


# ---- token-level model ---------------------------------------------------------------------
class _QWeight(C.Structure):
    _fields_ = [("type", C.c_int32), ("data", C.c_void_p)]


class _Cfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "hidden", "n_head", "n_kv_head", "head_dim",
                                         "n_ff", "vocab", "rope_neox")] + \
               [("rms_eps", C.c_float), ("rope_theta", C.c_float)] + \
               [(n, C.c_int32) for n in ("n_expert", "n_expert_used", "n_ff_expert")]


class _Layer(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p),
                ("wq", _QWeight), ("wk", _QWeight), ("wv", _QWeight), ("wo", _QWeight),
                ("gate", _QWeight), ("up", _QWeight), ("down", _QWeight),
                ("router", C.c_void_p),
                ("gate_exps", _QWeight), ("up_exps", _QWeight), ("down_exps", _QWeight)]


class Model:
    """Oracle decode of a synthetic model description (see `runnburn_b200.synth`)."""

    def __init__(self, desc: dict, max_ctx: int, threads: int | None = None):
        cfg = desc["cfg"]
        self._keep = []
        c = _Cfg()
        for name, _ in _Cfg._fields_:
            setattr(c, name, cfg.get(name, 0))
        layers = (_Layer * cfg["n_layer"])()

        def qw(pair):
            if pair is None:
                return _QWeight(0, None)
            t, a = pair
            a = _u8(a)
            self._keep.append(a)
            return _QWeight(t, a.ctypes.data)

        def fp(a):
            if a is None:
                return None
            a = _f32(a)
            self._keep.append(a)
            return a.ctypes.data

        for i, ld in enumerate(desc["layers"]):
            L = layers[i]
            L.attn_norm, L.ffn_norm = fp(ld["attn_norm"]), fp(ld["ffn_norm"])
            for k in ("wq", "wk", "wv", "wo", "gate", "up", "down", "gate_exps", "up_exps",
                      "down_exps"):
                setattr(L, k, qw(ld.get(k)))
            L.router = fp(ld.get("router"))
        self.cfg = cfg
        self.vocab = cfg["vocab"]
        self._h = lib().orc_model_create(C.byref(c), layers, qw(desc["token_embd"]),
                                         fp(desc["out_norm"]), qw(desc["output"]), max_ctx,
                                         threads or n_threads())
        self._layers = layers
        self.max_ctx = max_ctx

    def decode(self, token: int, pos: int) -> np.ndarray:
        p = lib().orc_model_decode(self._h, int(token), int(pos))
        assert p, "position beyond max_ctx"
        return np.ctypeslib.as_array(p, shape=(self.vocab,)).copy()

    def kv_cache(self, layer: int, kv_len: int):
        kv_dim = self.cfg["n_kv_head"] * self.cfg["head_dim"]
        k = np.ctypeslib.as_array(lib().orc_model_k_cache(self._h, layer), shape=(self.max_ctx * kv_dim,))
        v = np.ctypeslib.as_array(lib().orc_model_v_cache(self._h, layer), shape=(self.max_ctx * kv_dim,))
        return k[:kv_len * kv_dim].copy(), v[:kv_len * kv_dim].copy()

    def hidden(self) -> np.ndarray:
        return np.ctypeslib.as_array(lib().orc_model_hidden(self._h), shape=(self.cfg["hidden"],)).copy()

    def expert_ids(self, layer: int) -> np.ndarray:
        p = lib().orc_model_last_expert_ids(self._h, layer)
        return np.ctypeslib.as_array(p, shape=(32,))[: self.cfg["n_expert_used"]].copy()

    def reset(self):
        lib().orc_model_reset(self._h)

    def close(self):
        if self._h:
            lib().orc_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
