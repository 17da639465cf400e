"""Parity of the CUDA operators with the CPU oracle, through the C ABI, on seeded inputs.

Bars (BASELINE north star): Q8_K activation quantisation and MoE routing bit-exact;
matvec and attention within max relative error 1e-3 (fp32 accumulate).  The matvec kernels
go further: they replay the accumulation order of rnb-cpu's AVX2 dots, so their outputs are
compared bit for bit; the 1e-3 bar is kept for attention and for chains through exp().
"""
import numpy as np
import pytest

import oracle as orc
from synth import Q4_K, Q6_K, Q8_0, max_rel_err, max_err_vs_norm, quantized, random_blocks

pytestmark = pytest.mark.gpu

TOL = 1e-3  # max relative error, matvec and attention


def bits_equal(a, b) -> bool:
    a, b = np.ascontiguousarray(a, np.float32), np.ascontiguousarray(b, np.float32)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.fixture(scope="module")
def ops():
    from runnburn_b200 import build, ops
    build.build_library()
    ops.open()
    return ops


@pytest.fixture(autouse=True)
def _fresh_weight_cache(ops):
    """The resident cache is keyed by host address (weights are borrowed, immutable mmap pages
    in the reference's contract).  numpy reuses freed addresses for new arrays, so every test
    starts from an empty cache."""
    ops.reset_state_for_engine_init()
    yield


# ---- Q8_K -------------------------------------------------------------------------------------
def _q8k_equal(a, b):
    return a.tobytes() == b.tobytes()


def test_q8k_reference_fixtures_on_device(ops):
    x = np.zeros((5, 256), np.float32)
    x[1, 0] = 127.0
    x[1, 1:7] = [-0.5, -1.5, -2.5, 0.5, 1.5, 2.5]
    x[2, 0], x[2, 1] = 127.0, -127.0
    x[3, 0], x[3, 1] = -127.0, 127.0
    x[4, 15], x[4, 16], x[4, 255] = -1.0, -2.0, 127.0
    got = ops.quantize_q8k(x.ravel())
    assert _q8k_equal(got, orc.quantize_q8k(x.ravel()))
    assert got[0]["d"] == 0.0 and got[1]["d"] == -1.0 and got[1]["qs"][1:7].tolist() == [0, 2, 2, 0, -2, -2]
    assert got[2]["qs"][:2].tolist() == [-127, 127] and got[3]["d"] == 1.0
    assert got[4]["bsums"][0] == 1 and got[4]["bsums"][1] == 2 and got[4]["bsums"][15] == -127


@pytest.mark.parametrize("n", [256, 4096, 14336, 28672])
def test_q8k_bit_exact(ops, n):
    rng = np.random.default_rng(n)
    for scale in (1.0, 1e-6, 3e4):
        x = (rng.standard_normal(n) * scale).astype(np.float32)
        x[rng.integers(0, n, 16)] = 0.0
        assert _q8k_equal(ops.quantize_q8k(x), orc.quantize_q8k(x))
    idx = np.arange(n)
    x = (((idx * 73 + 19) % 2001).astype(np.float32) - 1000.0)   # many ties and repeated maxima
    assert _q8k_equal(ops.quantize_q8k(x), orc.quantize_q8k(x))
    x = np.repeat(np.float32([2.5, -2.5]), n // 2)               # |x| all equal: first element decides the sign
    assert _q8k_equal(ops.quantize_q8k(x), orc.quantize_q8k(x))


def test_q8k_empty_and_ragged(ops):
    import runnburn_b200 as r
    assert ops.quantize_q8k(np.zeros(0, np.float32)).size == 0
    with pytest.raises(r.RnbError, match="divisible by 256"):
        ops.quantize_q8k(np.zeros(255, np.float32))


# ---- matvec -------------------------------------------------------------------------------------
CONFIG1 = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)]


@pytest.mark.parametrize("rows,cols", CONFIG1)
def test_q4k_gemv_config1_shapes(ops, rows, cols):
    """BASELINE config 1: Llama-3-8B layer shapes, uniform quants/scales, |N(0,1e-3)| d/dmin, seed 0."""
    rng = np.random.default_rng(0)
    w = random_blocks(rng, Q4_K, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    ref = orc.gemv(Q4_K, w, x, rows, cols)
    got = ops.q4k_gemv(w, rows, cols, x)
    assert max_rel_err(got, ref) <= TOL
    assert bits_equal(got, ref)
    # linearity in the activation scale is exact for powers of two (Q8_K d scales, qs unchanged)
    got2 = ops.q4k_gemv(w, rows, cols, x * np.float32(4.0))
    assert np.array_equal(got2, got * np.float32(4.0))


@pytest.mark.parametrize("t,rows,cols", [
    (Q4_K, 1, 256), (Q4_K, 3, 256), (Q4_K, 130, 512), (Q4_K, 257, 768), (Q4_K, 2048, 768), (Q4_K, 768, 2048),
    (Q6_K, 1, 256), (Q6_K, 5, 256), (Q6_K, 7, 768), (Q6_K, 130, 512), (Q6_K, 1024, 4096), (Q6_K, 4096, 14336),
    (Q6_K, 515, 2048), (Q4_K, 16400, 512), (Q4_K, 20000, 1024), (Q4_K, 16385, 256),   # >= 16384 rows: two-threads-per-row kernel
    (Q8_0, 1, 32), (Q8_0, 3, 96), (Q8_0, 129, 256), (Q8_0, 1000, 4096),
])
def test_gemv_shapes_and_ragged_tiles(ops, t, rows, cols):
    rng = np.random.default_rng(rows * 131 + cols)
    w = random_blocks(rng, t, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    ref = orc.gemv(t, w, x, rows, cols)
    got = ops.gemv(t, w, rows, cols, x)
    assert max_rel_err(got, ref) <= TOL
    assert bits_equal(got, ref)


@pytest.mark.parametrize("t", [Q4_K, Q6_K, Q8_0])
def test_gemv_on_quantised_gaussian_weights(ops, t):
    rng = np.random.default_rng(7)
    rows, cols = 384, 1024
    _, w = quantized(rng, t, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    assert bits_equal(ops.gemv(t, w, rows, cols, x), orc.gemv(t, w, x, rows, cols))


def test_gemv_misaligned_weight_slice_takes_the_plain_load_path(ops):
    """Weights that start at an odd byte inside a resident range are not 16-byte aligned on the
    device either; the kernel must fall back to plain loads (reference: odd-offset rows are
    bit-identical, crates/rnb-cpu/src/gemm/quant_gemv.rs:1257-1296)."""
    rng = np.random.default_rng(3)
    rows, cols = 64, 512
    for t in (Q4_K, Q6_K, Q8_0):
        w = random_blocks(rng, t, rows, cols)
        x = rng.standard_normal(cols).astype(np.float32)
        aligned = ops.gemv(t, w, rows, cols, x)
        ops.clear_q4k_cache()
        backing = np.zeros(w.size + 64, np.uint8)
        backing[2:2 + w.size] = w
        ops.prewarm_q4k_weights([backing])            # one resident range; the slice below lives inside it
        shifted = ops.gemv(t, backing[2:2 + w.size], rows, cols, x)
        assert np.array_equal(aligned, shifted)


def test_gemv_batch_is_seq_major_and_matches_single_token_bits(ops):
    rng = np.random.default_rng(5)
    rows, cols, seq = 300, 512, 5
    for t, batch in ((Q4_K, ops.q4k_gemv_batch), (Q6_K, ops.q6k_gemv_batch)):
        w = random_blocks(rng, t, rows, cols)
        x = rng.standard_normal((seq, cols)).astype(np.float32)
        got = batch(w, rows, cols, x)
        ref = orc.gemv(t, w, x, rows, cols, seq_len=seq)
        assert bits_equal(got, ref)
        for s in range(seq):   # one accumulation order for decode and prefill-of-1
            assert np.array_equal(got[s * rows:(s + 1) * rows], ops.gemv(t, w, rows, cols, x[s]))


def test_q6k_gemv_argmax_tie_rule(ops):
    rng = np.random.default_rng(11)
    rows, cols = 1000, 512
    w = random_blocks(rng, Q6_K, rows, cols).reshape(rows, -1)
    w[777] = w[123]                      # two identical rows -> exact tie if they are the maximum
    x = rng.standard_normal(cols).astype(np.float32)
    y = orc.gemv(Q6_K, w.ravel(), x, rows, cols)
    w[123] = w[int(np.argmax(y))]
    w[777] = w[123]
    y = ops.q6k_gemv(w.ravel(), rows, cols, x)
    idx, val = ops.q6k_gemv_argmax(w.ravel(), rows, cols, x)
    assert idx == orc.argmax_last(y) and val == y[idx]
    assert idx == max(i for i in range(rows) if y[i] == y.max())


def test_q8_0_gemv_argmax_and_batch(ops):
    # the Q8_0 LM-head form (argmax with the sampler's tie rule) and the batched Q8_0 matvec: same bits as the
    # single-token call
    rng = np.random.default_rng(12)
    rows, cols, seq = 500, 256, 4
    w = random_blocks(rng, Q8_0, rows, cols).reshape(rows, -1)
    x = rng.standard_normal((seq, cols)).astype(np.float32)
    y0 = orc.gemv(Q8_0, w.ravel(), x[0], rows, cols)
    w[400] = w[int(np.argmax(y0))]       # the maximum twice: the later row wins
    w[77] = w[400]
    y = ops.q8_0_gemv(w.ravel(), rows, cols, x[0])
    assert bits_equal(y, orc.gemv(Q8_0, w.ravel(), x[0], rows, cols))
    idx, val = ops.q8_0_gemv_argmax(w.ravel(), rows, cols, x[0])
    assert idx == orc.argmax_last(y) and val == y[idx] and idx == max(i for i in range(rows) if y[i] == y.max())
    got = ops.q8_0_gemv_batch(w.ravel(), rows, cols, x)
    for s in range(seq):
        assert np.array_equal(got[s * rows:(s + 1) * rows], ops.q8_0_gemv(w.ravel(), rows, cols, x[s]))


def test_resident_cache_counters_and_eviction(ops):
    ops.reset_state_for_engine_init()
    rng = np.random.default_rng(1)
    rows, cols = 256, 512
    ws = [random_blocks(rng, Q4_K, rows, cols) for _ in range(3)]
    x = rng.standard_normal(cols).astype(np.float32)
    refs = [orc.gemv(Q4_K, w, x, rows, cols) for w in ws]
    ops.set_resident_limit(2 * ws[0].size + 100)          # room for two of the three
    try:
        for rnd in range(2):
            for w, ref in zip(ws, refs):
                assert max_rel_err(ops.q4k_gemv(w, rows, cols, x), ref) <= TOL
        s = ops.cuda_cache_snapshot()
        assert s["lookups"] == 6 and s["hits"] == 0 and s["misses"] == 6 and s["evictions"] >= 4
        assert s["resident_entries"] == 2 and s["resident_bytes"] == 2 * ws[0].size
        ops.q4k_gemv(ws[2], rows, cols, x)
        assert ops.cuda_cache_snapshot()["hits"] == 1
        ops.set_resident_limit(100)                        # nothing fits: transient uploads still compute
        ops.clear_q4k_cache()
        assert max_rel_err(ops.q4k_gemv(ws[0], rows, cols, x), refs[0]) <= TOL
        assert ops.cuda_cache_snapshot()["transient_uploads"] >= 1
    finally:
        ops.set_resident_limit(0)
        ops.reset_state_for_engine_init()


# ---- attention ----------------------------------------------------------------------------------
@pytest.mark.parametrize("heads,kvh,kv_len", [(32, 8, 1), (32, 8, 7), (32, 8, 333), (32, 8, 4096), (32, 4, 1025),
                                              (64, 8, 2000), (8, 8, 65), (6, 2, 100), (32, 2, 300), (16, 8, 20000), (24, 2, 17),
                                              (5, 5, 9), (7, 1, 500), (32, 8, 511), (32, 8, 512), (3, 1, 2),
                                              # the headline configurations' own shapes: MoE at 8192, a 70B 8-GPU shard and the whole 70B at 32768
                                              (32, 4, 8192), (8, 1, 32768), (64, 8, 32768)])
def test_attention_decode_hd128(ops, heads, kvh, kv_len):
    rng = np.random.default_rng(heads * 1000 + kv_len)
    q = rng.standard_normal(heads * 128).astype(np.float32)
    k = orc.f32_to_f16_bits(rng.standard_normal(kv_len * kvh * 128))
    v = orc.f32_to_f16_bits(rng.standard_normal(kv_len * kvh * 128))
    scale = 1.0 / np.sqrt(128.0)
    ref = orc.attention_decode(q, k, v, heads, kvh, 128, kv_len, scale)
    got = ops.attention_decode_hd128(q, k, v, kv_len, heads, kvh, scale)
    if kv_len <= 512:
        # the reference-order kernel serves these: same operations in the same order as the CPU
        assert np.array_equal(got, ref), f"not bit-identical: {np.max(np.abs(got - ref)):.3e}"
    elif kv_len <= 4096:
        assert max_rel_err(got, ref) <= TOL
    else:
        # Over 20000 positions the f32 running sums of either side carry ~1e-8 of absolute noise,
        # which is more than 1e-3 of the few outputs that lie 1000x below the vector's scale:
        # bound the error against the vector's scale instead, ten times tighter.
        assert max_err_vs_norm(got, ref) <= TOL / 10
    assert np.max(np.abs(got - ref)) < 1e-4        # the reference's own CUDA tests: max_diff < 1e-4


def test_attention_decode_cached_appends_only_new_rows(ops):
    rng = np.random.default_rng(21)
    heads, kvh, cap = 8, 2, 600
    k = orc.f32_to_f16_bits(rng.standard_normal(cap * kvh * 128))
    v = orc.f32_to_f16_bits(rng.standard_normal(cap * kvh * 128))
    scale = 1.0 / np.sqrt(128.0)
    ops.clear_decode_attention_kv_cache()
    before = ops.cuda_cache_snapshot()["h2d_bytes"]
    for kv_len in (1, 2, 3, 300, 301, 600):
        q = rng.standard_normal(heads * 128).astype(np.float32)
        got = ops.attention_decode_cached(3, q, k, v, kv_len, heads, kvh, 128, scale)
        ref = orc.attention_decode(q, k, v, heads, kvh, 128, kv_len, scale)
        if kv_len <= 512:
            assert np.array_equal(got, ref)
        else:
            assert max_rel_err(got, ref) <= TOL
    moved = ops.cuda_cache_snapshot()["h2d_bytes"] - before
    assert moved == 2 * 600 * kvh * 128 * 2 + 6 * heads * 128 * 4   # each KV row crossed PCIe once
    ops.clear_decode_attention_kv_cache()


@pytest.mark.parametrize("ggml_type", [Q4_K, Q6_K, Q8_0])
def test_quant_embedding_gather_bit_exact(ops, ggml_type):
    # quant_embedding_gather: the selected rows of a quantised table, dequantised on the device, equal the CPU
    # dequantiser's bit for bit; ragged cases: no tokens, repeated ids, the last row, an id out of range
    rng = np.random.default_rng(40 + ggml_type)
    rows, cols = 300, 512
    _, w = quantized(rng, ggml_type, rows, cols)
    table = orc.dequantize_matrix(ggml_type, w, rows, cols)
    ids = np.array([0, 299, 17, 17, 255, 1], dtype=np.uint32)
    got = ops.quant_embedding_gather(ggml_type, w, rows, cols, ids)
    assert got.shape == (6, cols) and np.array_equal(got, table[ids])
    assert ops.quant_embedding_gather(ggml_type, w, rows, cols, []).shape == (0, cols)
    import runnburn_b200 as r
    with pytest.raises(r.RnbError, match="out of range"):
        ops.quant_embedding_gather(ggml_type, w, rows, cols, [300])
    with pytest.raises(r.RnbError, match="byte mismatch"):
        ops.quant_embedding_gather(ggml_type, w[:-1], rows, cols, [0])


@pytest.mark.parametrize("head_dim", [256, 512])
def test_attention_decode_wide_heads(ops, head_dim):
    # head_dim 256 / 512 (attention_decode_hd256 / _hd512): fp32 split-KV against the CPU routine, the bounds of the
    # long-context hd128 path
    rng = np.random.default_rng(23 + head_dim)
    fn = ops.attention_decode_hd256 if head_dim == 256 else ops.attention_decode_hd512
    scale = 1.0 / np.sqrt(float(head_dim))
    for heads, kvh, kv_len in ((8, 2, 1), (8, 2, 37), (4, 4, 300), (16, 2, 2051), (1, 1, 5000)):
        q = rng.standard_normal(heads * head_dim).astype(np.float32)
        k = orc.f32_to_f16_bits(rng.standard_normal(kv_len * kvh * head_dim))
        v = orc.f32_to_f16_bits(rng.standard_normal(kv_len * kvh * head_dim))
        got = fn(q, k, v, kv_len, heads, kvh, scale)
        ref = orc.attention_decode(q, k, v, heads, kvh, head_dim, kv_len, scale)
        assert max_err_vs_norm(got, ref) <= TOL / 10 and np.max(np.abs(got - ref)) < 1e-4, (heads, kvh, kv_len)
    import runnburn_b200 as r
    with pytest.raises(r.RnbError):
        fn(q[:-1], k, v, kv_len, heads, kvh, scale)
    with pytest.raises(r.RnbError):
        fn(q, k, v, 0, heads, kvh, scale)


def test_attention_decode_cached_window(ops):
    # sliding-window decode over the mirrored cache: equal to the CPU routine with sliding_window = window_len when the
    # window ends at kv_len (bit for bit up to 512 positions), and attention over the range for any other start
    rng = np.random.default_rng(22)
    heads, kvh, cap = 8, 2, 1500
    k = orc.f32_to_f16_bits(rng.standard_normal(cap * kvh * 128))
    v = orc.f32_to_f16_bits(rng.standard_normal(cap * kvh * 128))
    scale = 1.0 / np.sqrt(128.0)
    ops.clear_decode_attention_kv_cache()
    for kv_len, window in ((1, 1), (40, 8), (300, 300), (700, 512), (701, 33), (1500, 1024)):
        q = rng.standard_normal(heads * 128).astype(np.float32)
        got = ops.attention_decode_cached_window(4, q, k, v, kv_len, kv_len - window, window, heads, kvh, 128, scale)
        ref = orc.attention_decode_window(q, k, v, heads, kvh, 128, kv_len, scale, window)
        if window <= 512:
            assert np.array_equal(got, ref), (kv_len, window)
        else:
            assert max_rel_err(got, ref) <= TOL and np.max(np.abs(got - ref)) < 1e-4
    # a window in the middle of the cache: attention over those rows alone
    q = rng.standard_normal(heads * 128).astype(np.float32)
    got = ops.attention_decode_cached_window(4, q, k, v, 1500, 100, 200, heads, kvh, 128, scale)
    lo, hi = 100 * kvh * 128, 300 * kvh * 128
    assert np.array_equal(got, orc.attention_decode(q, k[lo:hi], v[lo:hi], heads, kvh, 128, 200, scale))
    import runnburn_b200 as r
    for start, length in ((0, 0), (1501, 1), (1400, 101)):
        with pytest.raises(r.RnbError):
            ops.attention_decode_cached_window(4, q, k, v, 1500, start, length, heads, kvh, 128, scale)
    ops.clear_decode_attention_kv_cache()


def test_attention_prefill_causal(ops):
    rng = np.random.default_rng(8)
    heads, kvh, seq, kv_len = 8, 2, 37, 50
    q = rng.standard_normal(seq * heads * 128).astype(np.float32)
    k = rng.standard_normal(kv_len * kvh * 128).astype(np.float32)
    v = rng.standard_normal(kv_len * kvh * 128).astype(np.float32)
    scale = 1.0 / np.sqrt(128.0)
    ref = orc.attention_prefill(q, k, v, seq, kv_len, heads, kvh, 128, scale)
    got = ops.attention_prefill_flash_hd128(q, k, v, seq, kv_len, heads, kvh, scale)
    assert max_rel_err(got, ref) <= TOL


@pytest.mark.parametrize("heads,kvh,seq,kv_len", [
    (32, 8, 300, 300),    # Llama-3-8B head layout, ragged last query block and key tile
    (8, 1, 70, 1000),     # group 8, a cache much longer than the batch (later piece of a prompt)
    (4, 4, 129, 129),     # no grouping: 128 queries per CTA + one more
    (16, 4, 1, 65),       # a single query
    (6, 2, 33, 64),       # group 3 does not divide 128: the split-KV kernel takes it
])
def test_attention_prefill_causal_f16_cache(ops, heads, kvh, seq, kv_len):
    rng = np.random.default_rng(heads * 1000 + seq)
    q = rng.standard_normal(seq * heads * 128).astype(np.float32)
    k16 = rng.standard_normal(kv_len * kvh * 128).astype(np.float16)
    v16 = rng.standard_normal(kv_len * kvh * 128).astype(np.float16)
    scale = 1.0 / np.sqrt(128.0)
    ref = orc.attention_prefill(q, k16.astype(np.float32), v16.astype(np.float32), seq, kv_len, heads, kvh, 128, scale)
    got = ops.attention_prefill_flash_hd128_f16kv(q, k16.view(np.uint16), v16.view(np.uint16), seq, kv_len, heads, kvh, scale)
    assert max_rel_err(got, ref) <= TOL


# ---- glue ---------------------------------------------------------------------------------------
def test_rms_norm_rope_silu(ops):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, 4096)).astype(np.float32) * 3
    w = rng.standard_normal(4096).astype(np.float32)
    got = ops.rms_norm_rows_f32(x, w, 1e-5)
    ref = orc.rms_norm(x, w, 1e-5)
    assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-6)) <= 2e-7     # <= 1 ulp of the rms
    for neox in (False, True):
        d = rng.standard_normal(2 * 1024).astype(np.float32)
        ref = orc.rope(d, 4095, 128, 1024, 5e5, neox=neox)
        ops.rope_f32_inplace(d, 4095, 128, 1024, 5e5, neox=neox)
        assert np.array_equal(d, ref)                                           # same table, same mul/add order
    g = rng.standard_normal(1024).astype(np.float32) * 4
    u = rng.standard_normal(1024).astype(np.float32)
    ref = orc.silu_mul(g, u)
    ops.activation_mul_f32_inplace(g, u)
    assert np.max(np.abs(g - ref) / np.maximum(np.abs(ref), 1e-12)) <= 2.4e-7    # 2 ulp


def test_fused_qkv_rope_decode(ops):
    rng = np.random.default_rng(6)
    n_embd, heads, kvh, pos = 1024, 8, 2, 77
    tq, wq = quantized(rng, Q4_K, heads * 128, n_embd)
    tk, wk = quantized(rng, Q4_K, kvh * 128, n_embd)
    tv, wv = quantized(rng, Q6_K, kvh * 128, n_embd)
    x = rng.standard_normal(n_embd).astype(np.float32)
    q, kb, vb = ops.dense_attention_qkv_rope_hd128_decode(wq, wk, wv, heads * 128, kvh * 128, n_embd, heads, kvh,
                                                          5e5, pos, x, tq, tk, tv)
    q_ref = orc.rope(orc.gemv(Q4_K, wq, x, heads * 128, n_embd), pos, 128, heads * 128, 5e5)
    k_ref = orc.rope(orc.gemv(Q4_K, wk, x, kvh * 128, n_embd), pos, 128, kvh * 128, 5e5)
    v_ref = orc.gemv(Q6_K, wv, x, kvh * 128, n_embd)
    assert bits_equal(q, q_ref)
    assert np.array_equal(kb, orc.f32_to_f16_bits(k_ref)) and np.array_equal(vb, orc.f32_to_f16_bits(v_ref))
    # exactness of the rotation + rounding given the device's own matvec output
    qd = ops.q4k_gemv(wq, heads * 128, n_embd, x)
    assert np.array_equal(q, orc.rope(qd, pos, 128, heads * 128, 5e5))
    kd = ops.q4k_gemv(wk, kvh * 128, n_embd, x)
    assert np.array_equal(kb, orc.f32_to_f16_bits(orc.rope(kd, pos, 128, kvh * 128, 5e5)))
    assert np.array_equal(vb, orc.f32_to_f16_bits(ops.q6k_gemv(wv, kvh * 128, n_embd, x)))


def test_dense_attention_qkv_without_rope(ops):
    # dense_q4k_attention_qkv: the three projections of one token in one launch, bit-identical to the CPU matvecs;
    # ragged row counts, mixed Q4_K / Q6_K, and the reference's length checks
    rng = np.random.default_rng(16)
    n_embd, q_rows, kv_rows = 768, 520, 130
    tq, wq = quantized(rng, Q4_K, q_rows, n_embd)
    tk, wk = quantized(rng, Q4_K, kv_rows, n_embd)
    tv, wv = quantized(rng, Q6_K, kv_rows, n_embd)
    x = rng.standard_normal(n_embd).astype(np.float32)
    q, k, v = ops.dense_attention_qkv(wq, wk, wv, q_rows, kv_rows, n_embd, x, tq, tk, tv)
    assert bits_equal(q, orc.gemv(Q4_K, wq, x, q_rows, n_embd))
    assert bits_equal(k, orc.gemv(Q4_K, wk, x, kv_rows, n_embd))
    assert bits_equal(v, orc.gemv(Q6_K, wv, x, kv_rows, n_embd))
    import runnburn_b200 as r
    with pytest.raises(r.RnbError, match="input length mismatch"):
        ops.dense_attention_qkv(wq, wk, wv, q_rows, kv_rows, n_embd, x[:-1], tq, tk, tv)


def test_dense_silu_ffn(ops):
    rng = np.random.default_rng(9)
    n_embd, n_ff, seq = 512, 1024, 3
    _, g = quantized(rng, Q4_K, n_ff, n_embd)
    _, u = quantized(rng, Q4_K, n_ff, n_embd)
    for dt in (Q4_K, Q6_K):
        _, d = quantized(rng, dt, n_embd, n_ff)
        x = rng.standard_normal((seq, n_embd)).astype(np.float32)
        got = ops.dense_q4k_silu_ffn_batch(g, u, d, dt, n_ff, n_embd, seq, x)
        for s in range(seq):
            act = orc.silu_mul(orc.gemv(Q4_K, g, x[s], n_ff, n_embd), orc.gemv(Q4_K, u, x[s], n_ff, n_embd))
            ref = orc.gemv(dt, d, act, n_embd, n_ff)
            assert max_rel_err(got[s * n_embd:(s + 1) * n_embd], ref) <= 2 * TOL   # two chained matvecs


# ---- MoE ----------------------------------------------------------------------------------------
def test_moe_routing_bit_exact(ops):
    ids, w, cnt = ops.moe_route_topk_f32(np.float32([1.0, 4.0, 4.0, -2.0, 3.0]), None, 1, 5, 3)
    assert ids.tolist() == [1, 2, 4] and cnt.tolist() == [3]
    rng = np.random.default_rng(12)
    for n_expert, k, seq in ((128, 8, 9), (16, 4, 3), (256, 8, 2), (8, 8, 2), (60, 1, 4)):
        lg = rng.standard_normal((seq, n_expert)).astype(np.float32)
        lg[0, :] = np.round(lg[0, :] * 2) / 2                  # many exact ties
        lg[-1, :] = 0.25                                        # all tied
        ids, w, cnt = ops.moe_route_topk_f32(lg, None, seq, n_expert, k)
        for s in range(seq):
            rid, rw = orc.moe_route_topk(lg[s], k)
            assert np.array_equal(ids[s * k:(s + 1) * k], rid)
            assert np.array_equal(w[s * k:(s + 1) * k].view(np.uint32), rw.view(np.uint32))
    import runnburn_b200 as r
    with pytest.raises(r.RnbError) as e:
        ops.moe_route_topk_f32(np.zeros(8, np.float32), None, 1, 8, 2, sigmoid_mode=True)
    assert e.value.status == 1


def test_router_logits_bit_exact(ops):
    rng = np.random.default_rng(13)
    for n_expert, hidden in ((128, 2048), (16, 512), (5, 256)):
        w = rng.standard_normal((n_expert, hidden)).astype(np.float32)
        h = rng.standard_normal(hidden).astype(np.float32)
        assert np.array_equal(ops.router_logits_f32(w, h).view(np.uint32), orc.gemv_f32(w, h).view(np.uint32))


def test_single_expert_and_token_batch_experts(ops):
    # qwen35_expert (one expert, no route weight) and qwen35_sparse_experts_by_token (slots -> tokens): both equal the
    # decode call's results bit for bit; a token without slots is zero; the reference's length checks
    rng = np.random.default_rng(19)
    n_embd, n_ff, n_expert, tokens = 512, 256, 5, 4
    gs, ds = n_ff * orc.row_bytes(Q4_K, n_embd), n_embd * orc.row_bytes(Q6_K, n_ff)
    _, gate_all = quantized(rng, Q4_K, n_expert * n_ff, n_embd)
    _, up_all = quantized(rng, Q4_K, n_expert * n_ff, n_embd)
    _, down_all = quantized(rng, Q6_K, n_expert * n_embd, n_ff)
    sl = lambda a, e, n: a[e * n:(e + 1) * n]
    x = rng.standard_normal((tokens, n_embd)).astype(np.float32)
    one = ops.qwen35_expert(sl(gate_all, 2, gs), sl(up_all, 2, gs), sl(down_all, 2, ds), Q6_K, n_ff, n_embd, x[0])
    ref = orc.moe_experts([sl(gate_all, 2, gs)], [sl(up_all, 2, gs)], [sl(down_all, 2, ds)], np.float32([1.0]), Q6_K, n_ff, n_embd, x[0])
    assert max_rel_err(one, ref) <= 2 * TOL
    assert np.array_equal(one, ops.qwen35_sparse_experts([sl(gate_all, 2, gs)], [sl(up_all, 2, gs)], [sl(down_all, 2, ds)], np.float32([1.0]), Q6_K,
                                                         n_ff, n_embd, x[0]))
    # slots: token 0 <- experts 1, 3; token 1 <- none; token 2 <- expert 4; token 3 <- experts 0, 2, 4 (interleaved order)
    slot_expert = [1, 0, 4, 3, 2, 4]
    slot_token = [0, 3, 2, 0, 3, 3]
    rw = rng.random(len(slot_expert)).astype(np.float32)
    gate = [sl(gate_all, e, gs) for e in slot_expert]
    up = [sl(up_all, e, gs) for e in slot_expert]
    down = [sl(down_all, e, ds) for e in slot_expert]
    got = ops.qwen35_sparse_experts_by_token(gate, up, down, rw, slot_token, tokens, Q6_K, n_ff, n_embd, x)
    assert got.shape == (tokens, n_embd) and not got[1].any()
    for t in (0, 2, 3):
        mine = [s for s in range(len(slot_token)) if slot_token[s] == t]
        ref_t = orc.moe_experts([gate[s] for s in mine], [up[s] for s in mine], [down[s] for s in mine], rw[mine], Q6_K, n_ff, n_embd, x[t])
        assert max_rel_err(got[t], ref_t) <= 2 * TOL
        assert np.array_equal(got[t], ops.qwen35_sparse_experts([gate[s] for s in mine], [up[s] for s in mine], [down[s] for s in mine], rw[mine], Q6_K,
                                                                n_ff, n_embd, x[t]))
    assert not ops.qwen35_sparse_experts_by_token([], [], [], [], [], tokens, Q6_K, n_ff, n_embd, x).any()
    import runnburn_b200 as r
    with pytest.raises(r.RnbError, match="token id out of range"):
        ops.qwen35_sparse_experts_by_token(gate, up, down, rw, [0, 3, 2, 0, 3, 4], tokens, Q6_K, n_ff, n_embd, x)
    with pytest.raises(r.RnbError, match="input length mismatch"):
        ops.qwen35_expert(gate[0], up[0], down[0], Q6_K, n_ff, n_embd, x[0][:-1])


def test_sparse_experts(ops):
    rng = np.random.default_rng(14)
    n_embd, n_ff, n_expert, k = 512, 256, 12, 4
    _, gate_all = quantized(rng, Q4_K, n_expert * n_ff, n_embd)
    _, up_all = quantized(rng, Q4_K, n_expert * n_ff, n_embd)
    gs = n_ff * orc.row_bytes(Q4_K, n_embd)
    x = rng.standard_normal(n_embd).astype(np.float32)
    lg = rng.standard_normal(n_expert).astype(np.float32)
    ids, rw = orc.moe_route_topk(lg, k)
    for dt in (Q4_K, Q6_K):
        ops.reset_state_for_engine_init()
        _, down_all = quantized(rng, dt, n_expert * n_embd, n_ff)
        ds = n_embd * orc.row_bytes(dt, n_ff)
        assert ops.qwen35_register_moe_layer(gate_all, up_all, down_all, dt, n_ff, n_embd)
        before = ops.cuda_cache_snapshot()
        gate = [gate_all[e * gs:(e + 1) * gs] for e in ids]
        up = [up_all[e * gs:(e + 1) * gs] for e in ids]
        down = [down_all[e * ds:(e + 1) * ds] for e in ids]
        ref = orc.moe_experts(gate, up, down, rw, dt, n_ff, n_embd, x)
        got = ops.qwen35_sparse_experts(gate, up, down, rw, dt, n_ff, n_embd, x)
        assert max_rel_err(got, ref) <= 2 * TOL
        after = ops.cuda_cache_snapshot()
        assert after["uploads"] == before["uploads"] and after["hits"] - before["hits"] == 3 * k   # slices of the registered layer
    ops.reset_state_for_engine_init()
