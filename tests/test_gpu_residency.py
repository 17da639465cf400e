"""Resident weight cache under pressure, through the C ABI: over-budget operands of one call,
the evict-and-retry ladder after an (injected) allocation failure, host-range registration.

Reference behaviour: crates/rnb-backend/cuda/src/runtime/state/q4k_cache.rs:757-851 (miss ->
budget check -> LRU eviction -> allocate, evict and retry on OOM, transient upload when over
budget), :1040-1053 (the test hook that fakes OOM), state/host_register.rs:45-190.
"""
import numpy as np
import pytest

import oracle as orc
from synth import Q4_K, Q6_K, max_rel_err, quantized, random_blocks

pytestmark = pytest.mark.gpu
TOL = 1e-3


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
def _fresh(ops):
    ops.reset_state_for_engine_init()
    ops.set_resident_limit(0)
    yield
    ops.inject_resident_alloc_ooms_for_test(0)
    ops.set_resident_limit(0)
    ops.reset_state_for_engine_init()


def test_over_budget_operands_of_one_call_do_not_alias(ops):
    """With a residency limit that fits nothing, every weight of a call is a transient upload;
    gate, up and down (or q, k and v) must each get their own region."""
    rng = np.random.default_rng(21)
    n_embd, n_ff, seq = 512, 1024, 2
    _, g = quantized(rng, Q4_K, n_ff, n_embd)
    _, u = quantized(rng, Q4_K, n_ff, n_embd)
    _, d = quantized(rng, Q6_K, n_embd, n_ff)
    x = rng.standard_normal((seq, n_embd)).astype(np.float32)
    ops.set_resident_limit(100)
    got = ops.dense_q4k_silu_ffn_batch(g, u, d, Q6_K, n_ff, n_embd, seq, x)
    assert ops.cuda_cache_snapshot()["transient_uploads"] == 3
    for s in range(seq):
        act = orc.silu_mul(orc.gemv(Q4_K, g, x[s], n_ff, n_embd), orc.gemv(Q4_K, u, x[s], n_ff, n_embd))
        assert max_rel_err(got[s * n_embd:(s + 1) * n_embd], orc.gemv(Q6_K, d, act, n_embd, n_ff)) <= 2 * TOL
    # fused q/k/v
    heads, kvh, pos = 4, 2, 9
    tq, wq = quantized(rng, Q4_K, heads * 128, n_embd)
    tk, wk = quantized(rng, Q4_K, kvh * 128, n_embd)
    tv, wv = quantized(rng, Q6_K, kvh * 128, n_embd)
    q, kb, vb = ops.dense_attention_qkv_rope_hd128_decode(wq, wk, wv, heads * 128, kvh * 128, n_embd, heads, kvh, 5e5, pos, x[0], tq, tk, tv)
    assert bits_equal(q, orc.rope(orc.gemv(Q4_K, wq, x[0], heads * 128, n_embd), pos, 128, heads * 128, 5e5))
    assert np.array_equal(kb, orc.f32_to_f16_bits(orc.rope(orc.gemv(Q4_K, wk, x[0], kvh * 128, n_embd), pos, 128, kvh * 128, 5e5)))
    assert np.array_equal(vb, orc.f32_to_f16_bits(orc.gemv(Q6_K, wv, x[0], kvh * 128, n_embd)))
    # expert-gathered matvec: 3 roles x k experts, all transient
    n_ffe, n_expert, k = 256, 6, 3
    _, gate_all = quantized(rng, Q4_K, n_expert * n_ffe, n_embd)
    _, up_all = quantized(rng, Q4_K, n_expert * n_ffe, n_embd)
    _, down_all = quantized(rng, Q4_K, n_expert * n_embd, n_ffe)
    gs, ds = n_ffe * orc.row_bytes(Q4_K, n_embd), n_embd * orc.row_bytes(Q4_K, n_ffe)
    ids, rw = orc.moe_route_topk(rng.standard_normal(n_expert).astype(np.float32), k)
    gate = [gate_all[e * gs:(e + 1) * gs] for e in ids]
    up = [up_all[e * gs:(e + 1) * gs] for e in ids]
    down = [down_all[e * ds:(e + 1) * ds] for e in ids]
    before = ops.cuda_cache_snapshot()["transient_uploads"]
    got = ops.qwen35_sparse_experts(gate, up, down, rw, Q4_K, n_ffe, n_embd, x[0])
    assert ops.cuda_cache_snapshot()["transient_uploads"] - before == 3 * k
    assert max_rel_err(got, orc.moe_experts(gate, up, down, rw, Q4_K, n_ffe, n_embd, x[0])) <= 2 * TOL


def test_injected_oom_evicts_least_recently_used_and_retries(ops):
    import runnburn_b200 as r
    rng = np.random.default_rng(22)
    rows, cols = 256, 512
    ws = [random_blocks(rng, Q4_K, rows, cols) for _ in range(3)]
    x = rng.standard_normal(cols).astype(np.float32)
    refs = [orc.gemv(Q4_K, w, x, rows, cols) for w in ws]
    for w, ref in zip(ws[:2], refs[:2]):
        assert bits_equal(ops.q4k_gemv(w, rows, cols, x), ref)
    s0 = ops.cuda_cache_snapshot()
    assert s0["resident_entries"] == 2 and s0["evictions"] == 0
    # one fake OOM: the oldest entry (ws[0]) goes, the allocation is retried and succeeds
    ops.inject_resident_alloc_ooms_for_test(1)
    assert bits_equal(ops.q4k_gemv(ws[2], rows, cols, x), refs[2])
    s1 = ops.cuda_cache_snapshot()
    assert s1["evictions"] == 1 and s1["resident_entries"] == 2
    assert bits_equal(ops.q4k_gemv(ws[1], rows, cols, x), refs[1])
    assert ops.cuda_cache_snapshot()["hits"] == s1["hits"] + 1          # ws[1] survived: it was used more recently
    # more failures than entries to evict: the call reports out-of-memory instead of looping
    ops.clear_q4k_cache()
    assert bits_equal(ops.q4k_gemv(ws[0], rows, cols, x), refs[0])
    ops.inject_resident_alloc_ooms_for_test(5)
    with pytest.raises(r.RnbError) as e:
        ops.q4k_gemv(ws[1], rows, cols, x)
    assert e.value.status == 3 and "cudaMalloc(resident weight)" in str(e.value)
    ops.inject_resident_alloc_ooms_for_test(0)
    assert bits_equal(ops.q4k_gemv(ws[1], rows, cols, x), refs[1])     # the context is still usable


def test_registered_host_range_feeds_uploads(ops):
    """Weights that sit in a registered (pinned) host range upload and compute as before; a range
    registered twice or cleared twice is not an error."""
    rng = np.random.default_rng(23)
    rows, cols = 512, 1024
    page = 4096
    raw = np.zeros(rows * orc.row_bytes(Q4_K, cols) + 2 * page, np.uint8)
    off = (-raw.ctypes.data) % page                                     # page-aligned start, like an mmap
    w = raw[off:off + rows * orc.row_bytes(Q4_K, cols)]
    w[:] = random_blocks(rng, Q4_K, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    ops.register_host_range(w)
    ops.register_host_range(w)
    assert bits_equal(ops.q4k_gemv(w, rows, cols, x), orc.gemv(Q4_K, w, x, rows, cols))
    assert ops.prewarm_q4k_weights([w]) == 1
    ops.clear_host_registered_ranges()
    ops.clear_host_registered_ranges()
    assert bits_equal(ops.q4k_gemv(w, rows, cols, x), orc.gemv(Q4_K, w, x, rows, cols))
