"""The rest of the reference's operator boundary through the C ABI: device tensors, decode carriers,
cached decode attention with the output left on the device, the batched q/k/v + RoPE call, the MoE
entry points that carry layer index / expert ids / receipt through the expert-bundle accounting, and
the residency reports.  Results are compared with the oracle (bit for bit where the path is exact)."""
import ctypes as C

import numpy as np
import pytest

import oracle as orc
from synth import max_rel_err

pytestmark = pytest.mark.gpu
Q4_K, Q6_K = 12, 14


@pytest.fixture(scope="module")
def ops():
    from runnburn_b200 import ops as o
    o.open()
    return o


@pytest.fixture(autouse=True)
def _fresh_weight_cache(ops):
    """The resident cache is keyed by host address (weights are borrowed, immutable mmap pages in the
    reference's contract); numpy reuses freed addresses, so every test starts from an empty cache."""
    ops.reset_state_for_engine_init()
    yield


def quantized(rng, t, rows, cols):
    return orc.quantize_matrix(t, rng.standard_normal((rows, cols)).astype(np.float32) * 0.05)


def test_add_f32_inplace_and_its_messages(ops):
    import runnburn_b200 as r
    rng = np.random.default_rng(1)
    a, b = rng.standard_normal(5000).astype(np.float32), rng.standard_normal(5000).astype(np.float32)
    want = a + b
    ops.add_f32_inplace(a, b)
    assert np.array_equal(a, want)
    with pytest.raises(r.RnbError, match="CUDA add shape mismatch: dst=4 src=3"):
        ops.add_f32_inplace(np.zeros(4, np.float32), np.zeros(3, np.float32))
    ops.add_f32_inplace(np.zeros(0, np.float32), np.zeros(0, np.float32))   # empty: nothing to do


def test_device_tensor_round_trip_rows_and_release(ops):
    import runnburn_b200 as r
    data = np.arange(3 * 700, dtype=np.float32).reshape(3, 700)
    t = ops.DeviceTensor(data, role=2)
    assert t.ptr != 0
    assert np.array_equal(t.download(), data)
    assert np.array_equal(t.download_row(2), data[2])
    with pytest.raises(r.RnbError, match="out of range"):
        t.download_row(3)
    assert t.release() is True
    assert t.release() is False           # Ok(false): already gone
    with pytest.raises(r.RnbError, match="unknown device tensor id"):
        t.download()


def test_decode_carriers_hold_their_bytes_across_calls(ops):
    h = ops.acquire_decode_carrier(ops.CARRIER_HIDDEN, 4096 * 4)
    n = ops.acquire_decode_carrier(ops.CARRIER_NORM_BUF, 4096 * 4)
    assert h != 0 and n != 0 and h != n
    assert ops.acquire_decode_carrier(ops.CARRIER_HIDDEN, 1024) == h      # no regrowth for a smaller request
    x = np.linspace(-3, 3, 4096, dtype=np.float32)
    ops.upload_to_decode_carrier(x, h)
    back = np.zeros_like(x)
    ops.download_from_decode_carrier(h, back)
    ops.sync_decode_stream()
    assert np.array_equal(back, x)
    import runnburn_b200 as r
    with pytest.raises(r.RnbError):
        ops.acquire_decode_carrier(99, 16)


def test_attention_decode_cached_to_device_with_device_side_last_row(ops):
    rng = np.random.default_rng(2)
    heads, kvh, cap = 8, 2, 64
    kv_dim = kvh * 128
    k = orc.f32_to_f16_bits(rng.standard_normal(cap * kv_dim))
    v = orc.f32_to_f16_bits(rng.standard_normal(cap * kv_dim))
    scale = float(1.0 / np.sqrt(128.0))
    ops.clear_decode_attention_kv_cache()
    out_dev = ops.acquire_decode_carrier(ops.CARRIER_ATTN_OUT, heads * 128 * 4)
    out = np.zeros(heads * 128, np.float32)
    # host rows up to 40, output read back from the device buffer
    q = rng.standard_normal(heads * 128).astype(np.float32)
    ops.attention_decode_cached_to_device(5, q, k, v, 40, heads, kvh, 128, scale, out_dev)
    ops.download_from_decode_carrier(out_dev, out)
    ops.sync_decode_stream()
    assert np.array_equal(out, orc.attention_decode(q, k, v, heads, kvh, 128, 40, scale))
    # row 40 arrives from device buffers (the host arrays hold something else there), q from the device too
    k_new = orc.f32_to_f16_bits(rng.standard_normal(kv_dim))
    v_new = orc.f32_to_f16_bits(rng.standard_normal(kv_dim))
    kd = ops.acquire_decode_carrier(ops.CARRIER_K_F16, kv_dim * 2)
    vd = ops.acquire_decode_carrier(ops.CARRIER_V_F16, kv_dim * 2)
    ops.upload_to_decode_carrier(k_new, kd)
    ops.upload_to_decode_carrier(v_new, vd)
    q2 = rng.standard_normal(heads * 128).astype(np.float32)
    qt = ops.DeviceTensor(q2)
    before = ops.cuda_cache_snapshot()["h2d_bytes"]
    ops.attention_decode_cached_to_device(5, None, k, v, 41, heads, kvh, 128, scale, out_dev, kd, vd, qt.ptr)
    ops.download_from_decode_carrier(out_dev, out)
    ops.sync_decode_stream()
    assert ops.cuda_cache_snapshot()["h2d_bytes"] == before          # nothing crossed PCIe for this step
    k_ref, v_ref = k.copy(), v.copy()
    k_ref[40 * kv_dim:41 * kv_dim] = k_new
    v_ref[40 * kv_dim:41 * kv_dim] = v_new
    assert np.array_equal(out, orc.attention_decode(q2, k_ref, v_ref, heads, kvh, 128, 41, scale))
    qt.release()
    ops.clear_decode_attention_kv_cache()


def test_qkv_rope_prefill_equals_the_oracle_token_by_token(ops):
    rng = np.random.default_rng(3)
    n_embd, heads, kvh, pos0, seq = 512, 4, 2, 9, 5
    wq, wk, wv = quantized(rng, Q4_K, heads * 128, n_embd), quantized(rng, Q4_K, kvh * 128, n_embd), quantized(rng, Q6_K, kvh * 128, n_embd)
    x = rng.standard_normal((seq, n_embd)).astype(np.float32)
    q, kb, vb = ops.dense_attention_qkv_rope_hd128_prefill((Q4_K, wq), (Q4_K, wk), (Q6_K, wv), heads * 128, kvh * 128, n_embd, heads, kvh, 5e5, pos0, seq, x)
    for s in range(seq):
        q_ref = orc.rope(orc.gemv(Q4_K, wq, x[s], heads * 128, n_embd), pos0 + s, 128, heads * 128, 5e5)
        k_ref = orc.rope(orc.gemv(Q4_K, wk, x[s], kvh * 128, n_embd), pos0 + s, 128, kvh * 128, 5e5)
        v_ref = orc.gemv(Q6_K, wv, x[s], kvh * 128, n_embd)
        assert np.array_equal(q[s * heads * 128:(s + 1) * heads * 128], q_ref)
        assert np.array_equal(kb[s * kvh * 128:(s + 1) * kvh * 128], orc.f32_to_f16_bits(k_ref))
        assert np.array_equal(vb[s * kvh * 128:(s + 1) * kvh * 128], orc.f32_to_f16_bits(v_ref))


def test_sparse_experts_into_miss_path_accounting_and_receipt(ops):
    """A layer that is NOT registered.  First sighting of a bundle: full miss, reuse history says 0, and under
    the reference's rule (saved = missing x (reuses + 1) must EXCEED missing + reload) admission does not pay,
    so the bytes are staged for the call only.  Second sighting: still a miss, history says 1, admitted.
    Third: full hit, nothing crosses PCIe.  Every call's receipt carries its own stats delta and the result
    equals the oracle's."""
    rng = np.random.default_rng(4)
    n_embd, n_ff, n_expert, k = 512, 256, 6, 2
    gate_all, up_all = quantized(rng, Q4_K, n_expert * n_ff, n_embd), quantized(rng, Q4_K, n_expert * n_ff, n_embd)
    down_all = quantized(rng, Q4_K, n_expert * n_embd, n_ff)
    gs, ds = n_ff * orc.row_bytes(Q4_K, n_embd), n_embd * orc.row_bytes(Q4_K, n_ff)
    bundle = 2 * gs + ds
    x = rng.standard_normal(n_embd).astype(np.float32)
    ids = [4, 1]
    rw = np.array([0.7, 0.3], np.float32)
    gate = [gate_all[e * gs:(e + 1) * gs] for e in ids]
    up = [up_all[e * gs:(e + 1) * gs] for e in ids]
    down = [down_all[e * ds:(e + 1) * ds] for e in ids]
    ref = orc.moe_experts(gate, up, down, rw, Q4_K, n_ff, n_embd, x)
    before = ops.qwen35_expert_cache_stats()
    snap0 = ops.cuda_cache_snapshot()
    r1 = ops.ExpertReceipt()
    got = ops.qwen35_sparse_experts_into(gate, up, down, rw, 3, ids, r1, Q4_K, n_ff, n_embd, x)
    assert max_rel_err(got, ref) <= 2e-3
    d1 = r1.pending_stats.as_dict()
    assert r1.consumed == 0 and d1["bundle_lookups"] == k and d1["bundle_misses"] == k and d1["bundle_hits"] == 0
    assert d1["bundle_admissions"] == 0 and d1["temp_h2d_bytes"] == k * bundle and d1["h2d_bytes"] == 0
    snap1 = ops.cuda_cache_snapshot()
    assert snap1["resident_bytes"] == snap0["resident_bytes"] and snap1["transient_uploads"] - snap0["transient_uploads"] == 3 * k
    r2 = ops.ExpertReceipt()
    res = rng.standard_normal(n_embd).astype(np.float32)
    got2 = ops.qwen35_sparse_experts_into(gate, up, down, rw, 3, ids, r2, Q4_K, n_ff, n_embd, x, residual=res)
    d2 = r2.pending_stats.as_dict()
    assert d2["bundle_misses"] == k and d2["bundle_admissions"] == k and d2["admitted_bytes"] == k * bundle and d2["temp_h2d_bytes"] == 0
    assert np.array_equal(got2, res + got)                     # residual + experts, f32
    assert ops.cuda_cache_snapshot()["resident_bytes"] - snap1["resident_bytes"] == k * bundle
    r3 = ops.ExpertReceipt()
    h2d = ops.cuda_cache_snapshot()["upload_bytes"]
    got3 = ops.qwen35_sparse_experts_into(gate, up, down, rw, 3, ids, r3, Q4_K, n_ff, n_embd, x)
    d3 = r3.pending_stats.as_dict()
    assert d3["bundle_hits"] == k and d3["bundle_misses"] == 0 and d3["h2d_bytes"] == 0 and d3["temp_h2d_bytes"] == 0
    assert ops.cuda_cache_snapshot()["upload_bytes"] == h2d and np.array_equal(got3, got)
    after = ops.qwen35_expert_cache_stats()
    assert after["bundle_lookups"] - before["bundle_lookups"] == 3 * k
    # no layer index: no history is kept, the lookups are still accounted
    got4 = ops.qwen35_sparse_experts_into(gate, up, down, rw, None, None, None, Q4_K, n_ff, n_embd, x)
    assert np.array_equal(got4, got)
    import runnburn_b200 as r
    with pytest.raises(r.RnbError, match="needs the selected expert ids"):
        ops.qwen35_sparse_experts_into(gate, up, down, rw, 3, None, None, Q4_K, n_ff, n_embd, x)


def test_admit_misses_async_configure_cache_and_residency_counters(ops):
    rng = np.random.default_rng(5)
    ops.reset_state_for_engine_init()
    a, b = quantized(rng, Q4_K, 256, 512), quantized(rng, Q6_K, 128, 512)
    c0 = ops.cuda_weight_residency_counters()
    assert ops.qwen35_admit_expert_misses_async([a, b]) == 2
    assert ops.qwen35_admit_expert_misses_async([a, b]) == 0          # already resident
    ops.sync_decode_stream()
    c1 = ops.cuda_weight_residency_counters()
    assert c1["raw_quant_bytes"] - c0["raw_quant_bytes"] == a.size + b.size
    assert c1["q4_expanded_f16_bytes"] == 0 and c1["native_f32_bytes"] == 0
    assert ops.prewarm_quant_resident_weights([a, b]) == 2
    free_b, total_b = ops.cuda_memory_info()
    lim = ops.qwen35_configure_moe_layer_cache(10 << 20, 1 << 30, 1 << 20)
    assert lim == 10 << 20                                            # the model's expert bytes fit beside the head-room
    assert ops.qwen35_configure_moe_layer_cache(10 << 20, total_b, 1 << 20) == 0   # head-room swallows everything
    assert ops.qwen35_configure_moe_layer_cache(1 << 10, 0, 1 << 20) == 0          # less than one layer: nothing kept
    ops.reset_state_for_engine_init()


def test_prefill_route_slots_equal_the_oracle_router(ops):
    rng = np.random.default_rng(6)
    n_expert, hidden, seq, k = 16, 512, 7, 4
    w = rng.standard_normal((n_expert, hidden)).astype(np.float32)
    h = rng.standard_normal((seq, hidden)).astype(np.float32)
    ids, wts, toks = ops.qwen35_prefill_device_topk_route_slots(w, h, k)
    for s in range(seq):
        lg = orc.gemv_f32(w, h[s])
        ri, rw = orc.moe_route_topk(lg, k)
        assert np.array_equal(ids[s * k:(s + 1) * k], np.asarray(ri, np.uint32))
        assert np.array_equal(wts[s * k:(s + 1) * k], np.asarray(rw, np.float32))
        assert np.all(toks[s * k:(s + 1) * k] == s)


Q5_K = 13


@pytest.mark.parametrize("rows,cols", [(1, 256), (5, 512), (130, 1024), (1024, 4096), (4096, 14336), (33, 768)])
def test_q5k_matvec_bit_exact(ops, rows, cols):
    """Q5_K x Q8_K (crates/rnb-cpu/src/gemm/avx2_dot.rs:698-789): the device result equals the oracle's bit for
    bit, on quantised N(0, 0.05) weights and on random block bytes (all scale / high-bit patterns)."""
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.standard_normal(cols).astype(np.float32)
    w = orc.quantize_matrix(Q5_K, (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32))
    assert np.array_equal(ops.q5k_gemv(w, rows, cols, x).view(np.uint32), orc.gemv(Q5_K, w, x, rows, cols).view(np.uint32))
    ops.clear_q4k_cache()        # `raw` may land on a freed array's address
    raw = rng.integers(0, 256, size=(rows, cols // 256, 176), dtype=np.uint8)
    raw[..., 1] = 0x10
    raw[..., 3] = 0x10
    raw = raw.reshape(-1)
    assert np.array_equal(ops.q5k_gemv(raw, rows, cols, x).view(np.uint32), orc.gemv(Q5_K, raw, x, rows, cols).view(np.uint32))


def test_q5k_batch_and_ffn_down_quant_13(ops):
    import runnburn_b200 as r
    rng = np.random.default_rng(77)
    rows, cols, seq = 96, 1024, 3
    w = orc.quantize_matrix(Q5_K, (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32))
    x = rng.standard_normal((seq, cols)).astype(np.float32)
    got = ops.q5k_gemv_batch(w, rows, cols, x)
    want = orc.gemv(Q5_K, w, x, rows, cols, seq_len=seq)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # dense FFN with a Q5_K down matrix (ggml type id 13 of dense_q4k_silu_ffn_batch)
    n_embd, n_ff = 512, 1024
    g = orc.quantize_matrix(Q4_K, (rng.standard_normal((n_ff, n_embd)) * 0.05).astype(np.float32))
    u = orc.quantize_matrix(Q4_K, (rng.standard_normal((n_ff, n_embd)) * 0.05).astype(np.float32))
    d = orc.quantize_matrix(Q5_K, (rng.standard_normal((n_embd, n_ff)) * 0.05).astype(np.float32))
    xs = rng.standard_normal((2, n_embd)).astype(np.float32)
    out = ops.dense_q4k_silu_ffn_batch(g, u, d, Q5_K, n_ff, n_embd, 2, xs)
    for s in range(2):
        act = orc.silu_mul(orc.gemv(Q4_K, g, xs[s], n_ff, n_embd), orc.gemv(Q4_K, u, xs[s], n_ff, n_embd))
        ref = orc.gemv(Q5_K, d, act, n_embd, n_ff)
        assert np.array_equal(out[s * n_embd:(s + 1) * n_embd].view(np.uint32), ref.view(np.uint32))
    with pytest.raises(r.RnbError, match="Q5_K cols must be divisible by 256"):
        ops.q5k_gemv(np.zeros(176, np.uint8), 1, 100, np.zeros(100, np.float32))
    with pytest.raises(r.RnbError, match="Q5_K weight byte mismatch"):
        ops.q5k_gemv(np.zeros(100, np.uint8), 1, 256, np.zeros(256, np.float32))


Q2_K = 10


@pytest.mark.parametrize("rows,cols", [(1, 256), (5, 512), (33, 768), (130, 1024), (1024, 4096), (2048, 768)])
def test_q2k_matvec_bit_exact(ops, rows, cols):
    """Q2_K x Q8_K (crates/rnb-cpu/src/gemm/avx2_dot.rs:169-245): bit for bit the oracle's, on fitted weights
    and on random block bytes; the batched form likewise."""
    rng = np.random.default_rng(rows * 11 + cols)
    x = rng.standard_normal(cols).astype(np.float32)
    w = orc.quantize_matrix(Q2_K, (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32))
    assert np.array_equal(ops.q2k_gemv(w, rows, cols, x).view(np.uint32), orc.gemv(Q2_K, w, x, rows, cols).view(np.uint32))
    ops.clear_q4k_cache()
    raw = rng.integers(0, 256, size=(rows, cols // 256, 84), dtype=np.uint8)
    raw[..., 81] = 0x10
    raw[..., 83] = 0x10
    raw = raw.reshape(-1)
    assert np.array_equal(ops.q2k_gemv(raw, rows, cols, x).view(np.uint32), orc.gemv(Q2_K, raw, x, rows, cols).view(np.uint32))
    xs = rng.standard_normal((2, cols)).astype(np.float32)
    got = ops.q2k_gemv_batch(raw, rows, cols, xs)
    assert np.array_equal(got.view(np.uint32), orc.gemv(Q2_K, raw, xs, rows, cols, seq_len=2).view(np.uint32))


Q3_K = 11


@pytest.mark.parametrize("rows,cols", [(1, 256), (5, 512), (33, 768), (130, 1024), (1024, 4096), (2048, 768)])
def test_q3k_matvec_bit_exact(ops, rows, cols):
    """Q3_K x Q8_K (crates/rnb-cpu/src/gemm/avx2_dot.rs:247-378): bit for bit the oracle's, on fitted weights and
    on random block bytes (odd block indices sit on 2-byte boundaries); the batched form likewise."""
    rng = np.random.default_rng(rows * 13 + cols)
    x = rng.standard_normal(cols).astype(np.float32)
    w = orc.quantize_matrix(Q3_K, (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32))
    assert np.array_equal(ops.q3k_gemv(w, rows, cols, x).view(np.uint32), orc.gemv(Q3_K, w, x, rows, cols).view(np.uint32))
    ops.clear_q4k_cache()
    raw = rng.integers(0, 256, size=(rows, cols // 256, 110), dtype=np.uint8)
    raw[..., 109] = 0x10
    raw = raw.reshape(-1)
    assert np.array_equal(ops.q3k_gemv(raw, rows, cols, x).view(np.uint32), orc.gemv(Q3_K, raw, x, rows, cols).view(np.uint32))
    xs = rng.standard_normal((2, cols)).astype(np.float32)
    got = ops.q3k_gemv_batch(raw, rows, cols, xs)
    assert np.array_equal(got.view(np.uint32), orc.gemv(Q3_K, raw, xs, rows, cols, seq_len=2).view(np.uint32))
