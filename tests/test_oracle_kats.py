"""Pins the CPU oracle against the reference's own unit-test fixtures, restated here, and
against an independent dequantiser (committed fixtures made with the `gguf` package).

Reference fixtures restated (paths relative to the reference project):
  crates/rnb-cpu/src/gemm/activation_q8.rs:179-241      Q8_K ties / sign rule / bsums / batch
  crates/rnb-cpu/src/quantize/blocks.rs:114-132         block sizes
  crates/rnb-cpu/src/quantize/dequant.rs:843-856,995-1033   zero blocks, Q8_0 known values
  crates/rnb-cpu/src/quantize/quant.rs:766-798          Q4_K quantise→dequantise cosine
  crates/rnb-cpu/src/gemm/quant_gemv.rs:1222-1296       odd byte offsets, bit-identical
  crates/rnb-cpu/src/gemm/quant_gemv.rs:1448-1464       seq-major Q8_0 output
  crates/rnb-cpu/src/gemm/avx2_dot.rs:941-983           int dot vs scalar on dequantised Q8_K
  crates/rnb-llm/src/engine/models/shared_expert_moe/routing.rs:250-298   routing
"""
from pathlib import Path

import numpy as np
import pytest

GOLD = Path(__file__).parent / "golden"


def test_block_sizes(orc):
    assert orc.row_bytes(orc.TYPE_Q4_K, 256) == 144
    assert orc.row_bytes(orc.TYPE_Q6_K, 256) == 210
    assert orc.row_bytes(orc.TYPE_Q8_0, 32) == 34
    assert orc.Q8K_DTYPE.itemsize == 292
    assert orc.Q8K_DTYPE.fields["qs"][1] == 4 and orc.Q8K_DTYPE.fields["bsums"][1] == 260


def test_f16_conversions_match_ieee(orc):
    allh = np.arange(65536, dtype=np.uint16)
    ours = orc.f16_bits_to_f32(allh)
    ref = allh.view(np.float16).astype(np.float32)
    nan = np.isnan(ref)
    assert np.array_equal(ours[~nan].view(np.uint32), ref[~nan].view(np.uint32))
    assert np.all(np.isnan(ours[nan]))
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 200000),
        ref[~nan],                                             # exact halves
        np.nextafter(ref[~nan], np.float32(np.inf)),           # just above a half
        ((ref[~nan][:-1].astype(np.float64) + ref[~nan][1:]) / 2).astype(np.float32),  # ties
        np.array([65504, 65519.99, 65520, 1e9, -1e9, 5.96e-8, 2.98e-8, 2.9802322e-8, 0.0, -0.0],
                 dtype=np.float32),
    ]).astype(np.float32)
    x = x[np.isfinite(x)]
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(orc.f32_to_f16_bits(x), want)


def test_q8k_reference_fixtures(orc):
    z = orc.quantize_q8k(np.zeros(256, np.float32))[0]
    assert z["d"] == 0.0 and not z["qs"].any() and not z["bsums"].any()

    ties = np.zeros(256, np.float32)
    ties[0] = 127.0
    ties[1:7] = [-0.5, -1.5, -2.5, 0.5, 1.5, 2.5]
    b = orc.quantize_q8k(ties)[0]
    assert b["d"] == -1.0
    assert b["qs"][1:7].tolist() == [0, 2, 2, 0, -2, -2]

    fp = np.zeros(256, np.float32)
    fp[0], fp[1] = 127.0, -127.0
    b = orc.quantize_q8k(fp)[0]
    assert b["d"] == -1.0 and b["qs"][:2].tolist() == [-127, 127]

    fn = np.zeros(256, np.float32)
    fn[0], fn[1] = -127.0, 127.0
    b = orc.quantize_q8k(fn)[0]
    assert b["d"] == 1.0 and b["qs"][:2].tolist() == [-127, 127]

    bd = np.zeros(256, np.float32)
    bd[15], bd[16], bd[255] = -1.0, -2.0, 127.0
    b = orc.quantize_q8k(bd)[0]
    assert b["bsums"][0] == 1 and b["bsums"][1] == 2
    assert not b["bsums"][2:15].any() and b["bsums"][15] == -127


def test_q8k_batch_equals_blockwise(orc):
    idx = np.arange(16 * 256)
    x = ((idx * 73 + 19) % 2001).astype(np.float32) - 1000.0
    whole = orc.quantize_q8k(x)
    for i in range(16):
        one = orc.quantize_q8k(x[i * 256:(i + 1) * 256])[0]
        assert whole[i].tobytes() == one.tobytes()
    # python restatement of the block rule, independent of the C code
    for i in (0, 7, 15):
        c = x[i * 256:(i + 1) * 256]
        j = int(np.argmax(np.abs(c)))  # first index of the maximum
        iscale = np.float32(-127.0) / c[j]
        q = np.minimum(np.rint(iscale * c), 127).astype(np.int8)
        assert np.array_equal(whole[i]["qs"], q)
        assert whole[i]["d"] == np.float32(1.0) / iscale
        assert np.array_equal(whole[i]["bsums"], q.reshape(16, 16).sum(1).astype(np.int16))


def test_dequant_zero_blocks_and_q8_0_known(orc):
    for t, nbytes, cols in ((orc.TYPE_Q4_K, 144, 256), (orc.TYPE_Q6_K, 210, 256)):
        out = orc.dequantize_matrix(t, np.zeros(nbytes, np.uint8), 1, cols)
        assert np.all(out == 0.0)
    blk = np.zeros(34, np.uint8)
    blk[0:2] = [0x00, 0x3C]
    blk[2], blk[3] = 5, np.uint8(np.int8(-3))
    out = orc.dequantize_matrix(orc.TYPE_Q8_0, blk, 1, 32)[0]
    assert out[0] == 5.0 and out[1] == -3.0 and out[2] == 0.0


def test_dequant_matches_gguf_package(orc):
    g = np.load(GOLD / "gguf_dequant.npz")
    for name, t, cols in (("q4k", orc.TYPE_Q4_K, 256), ("q6k", orc.TYPE_Q6_K, 256),
                          ("q8_0", orc.TYPE_Q8_0, 32)):
        raw, want = g[f"{name}_bytes"], g[f"{name}_f32"]
        got = orc.dequantize_matrix(t, raw.ravel(), raw.shape[0], cols)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name
    x = g["q8_0_quant_in"]
    got = orc.quantize_matrix(orc.TYPE_Q8_0, x)
    assert np.array_equal(got, g["q8_0_quant_bytes"].ravel())


def _cos(a, b):
    return float(np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-10))


def test_q4k_quantize_roundtrip_reference_fixture(orc):
    t = np.arange(1024, dtype=np.float32) * np.float32(0.017)
    x = (np.sin(t) * (1.0 + 0.25 * np.cos(t * 0.9))).astype(np.float32)
    q = orc.quantize_matrix(orc.TYPE_Q4_K, x.reshape(1, -1))
    assert q.size == 4 * 144
    back = orc.dequantize_matrix(orc.TYPE_Q4_K, q, 1, 1024)[0]
    assert _cos(x, back) >= 0.97


def test_harness_quantisers_roundtrip(orc):
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((8, 512)) * 0.02).astype(np.float32)
    for t, lo in ((orc.TYPE_Q4_K, 0.99), (orc.TYPE_Q6_K, 0.999), (orc.TYPE_Q8_0, 0.9999)):
        q = orc.quantize_matrix(t, w)
        back = orc.dequantize_matrix(t, q, 8, 512)
        assert _cos(w.ravel(), back.ravel()) >= lo, t
    assert not orc.quantize_matrix(orc.TYPE_Q6_K, np.zeros((1, 256), np.float32)).any()


def _fixture_block(orc, t):
    n = {orc.TYPE_Q4_K: 144, orc.TYPE_Q6_K: 210, orc.TYPE_Q8_0: 34}[t]
    blk = ((np.arange(n) * 37 + 11) & 0xFF).astype(np.uint8)
    if t == orc.TYPE_Q4_K:
        blk[0:2], blk[2:4] = [0x00, 0x3C], [0x00, 0x38]
    elif t == orc.TYPE_Q6_K:
        blk[208:210] = [0x00, 0x3C]
    else:
        blk[0:2] = [0x00, 0x3C]
    return blk


def test_rows_accept_odd_byte_offsets(orc):
    for t, elems in ((orc.TYPE_Q4_K, 256), (orc.TYPE_Q6_K, 256), (orc.TYPE_Q8_0, 32)):
        blk = _fixture_block(orc, t)
        x = ((np.arange(elems) % 17).astype(np.float32) * 0.125 - 1.0)
        want = orc.dot_dequant_row(t, blk, x)
        assert np.isfinite(want)
        backing = np.zeros(blk.size + 3, np.uint8)
        odd = backing[1:1 + blk.size]
        odd[:] = blk
        assert odd.ctypes.data % 2 == 1
        got = orc.lib().orc_dot_dequant_row(t, odd.ctypes.data, x.ctypes.data, elems)
        assert np.float32(got).tobytes() == np.float32(want).tobytes()
        if t != orc.TYPE_Q8_0:
            xq = orc.quantize_q8k(x)
            name = "orc_dot_q4k_q8k" if t == orc.TYPE_Q4_K else "orc_dot_q6k_q8k"
            a = getattr(orc.lib(), name)(blk.ctypes.data, xq.ctypes.data, 1)
            b = getattr(orc.lib(), name)(odd.ctypes.data, xq.ctypes.data, 1)
            assert np.float32(a).tobytes() == np.float32(b).tobytes()


def test_q8_0_gemv_writes_seq_major_output(orc):
    blocks = bytes([0x00, 0x3C] + list(range(1, 33)) + [0x00, 0x3C] + list(range(32, 0, -1)))
    w = np.frombuffer(blocks, np.uint8)
    x = np.ones(64, np.float32)
    out = orc.gemv(orc.TYPE_Q8_0, w, x, rows=2, cols=32, seq_len=2)
    assert out[0] == orc.dot_q8_0_row(w[:34], x[:32])
    assert out[1] == orc.dot_q8_0_row(w[34:], x[:32])
    assert out[2] == orc.dot_q8_0_row(w[:34], x[32:])
    assert out[3] == orc.dot_q8_0_row(w[34:], x[32:])
    assert out[0] == 528.0


def _random_rows(orc, rng, t, rows, nb):
    """Config-1 style blocks: uniform quants/scales, small positive f16 super-scales."""
    if t == orc.TYPE_Q4_K:
        w = rng.integers(0, 256, size=(rows, nb, 144), dtype=np.uint8)
        d = np.abs(rng.standard_normal((rows, nb, 2)) * 1e-3).astype(np.float16)
        w[:, :, 0:4] = d.view(np.uint8).reshape(rows, nb, 4)
    else:
        w = rng.integers(0, 256, size=(rows, nb, 210), dtype=np.uint8)
        d = (rng.standard_normal((rows, nb, 1)) * 1e-3).astype(np.float16)
        w[:, :, 208:210] = d.view(np.uint8).reshape(rows, nb, 2)
    return w.reshape(rows, -1)


@pytest.mark.parametrize("tname", ["Q4_K", "Q6_K"])
def test_int_dot_avx2_equals_lane_restatement_and_scalar(orc, tname):
    t = getattr(orc, f"TYPE_{tname}")
    rng = np.random.default_rng(11)
    nb = 5
    w = _random_rows(orc, rng, t, 33, nb)
    x = rng.standard_normal(nb * 256).astype(np.float32)
    xq = orc.quantize_q8k(x)
    x_deq = (xq["qs"].astype(np.float32) * xq["d"][:, None]).ravel()
    for r in range(w.shape[0]):
        lanes = orc.dot_row(t, w[r], xq, lanes=True)
        if orc.lib().orc_have_avx2():
            fast = orc.dot_row(t, w[r], xq)
            assert np.float32(fast).tobytes() == np.float32(lanes).tobytes()
        scalar = orc.dot_dequant_row(t, w[r], x_deq)
        assert abs(lanes - scalar) <= 1e-3 + 2e-4 * abs(scalar)
    # exact integer identity: with d = dmin = 1, unit scales, the dot is an integer sum
    wd = orc.dequantize_matrix(t, w.ravel(), w.shape[0], nb * 256).astype(np.float64)
    want = wd @ x_deq.astype(np.float64)
    got = np.array([orc.dot_row(t, w[r], xq, lanes=True) for r in range(w.shape[0])])
    assert np.allclose(got, want, rtol=2e-5, atol=1e-6)


def test_gemv_seq_major_and_threads(orc):
    rng = np.random.default_rng(5)
    rows, nb, seq = 130, 2, 3
    w = _random_rows(orc, rng, orc.TYPE_Q4_K, rows, nb)
    x = rng.standard_normal(seq * nb * 256).astype(np.float32)
    out1 = orc.gemv(orc.TYPE_Q4_K, w.ravel(), x, rows, nb * 256, seq, threads=1)
    out4 = orc.gemv(orc.TYPE_Q4_K, w.ravel(), x, rows, nb * 256, seq, threads=4)
    assert np.array_equal(out1, out4)
    for s in range(seq):
        xq = orc.quantize_q8k(x[s * nb * 256:(s + 1) * nb * 256])
        for r in (0, 64, 129):
            assert out1[s * rows + r] == np.float32(orc.dot_row(orc.TYPE_Q4_K, w[r], xq))


def test_routing_reference_fixtures(orc):
    ids, w = orc.moe_route_topk([0.0, 4.0, 3.0, 2.0], 2)
    assert ids.tolist() == [1, 2]
    assert abs(w.sum() - 1.0) < 1e-6 and w[0] > w[1]
    ids, w = orc.moe_route_topk([1.0, 4.0, 4.0, -2.0, 3.0], 3)
    assert ids.tolist() == [1, 2, 4]
    e3 = np.exp(np.float32(-1.0))
    s = 1.0 + 1.0 + e3
    assert abs(w[0] - 1.0 / s) < 1e-6 and abs(w[1] - 1.0 / s) < 1e-6 and abs(w[2] - e3 / s) < 1e-6
    ids, w = orc.moe_route_topk([0.5, 0.5, 0.5], 8)  # k > n_expert, all tied
    assert ids.tolist() == [0, 1, 2]


def test_decode_attention_4pass_online_and_numpy_agree(orc):
    rng = np.random.default_rng(9)
    heads, kvh, hd, kv_len = 8, 2, 128, 77
    q = rng.standard_normal(heads * hd).astype(np.float32)
    k = orc.f32_to_f16_bits(rng.standard_normal(kv_len * kvh * hd))
    v = orc.f32_to_f16_bits(rng.standard_normal(kv_len * kvh * hd))
    scale = 1.0 / np.sqrt(hd)
    a = orc.attention_decode(q, k, v, heads, kvh, hd, kv_len, scale)
    b = orc.attention_decode(q, k, v, heads, kvh, hd, kv_len, scale, online=True)
    kf = k.view(np.float16).astype(np.float64).reshape(kv_len, kvh, hd)
    vf = v.view(np.float16).astype(np.float64).reshape(kv_len, kvh, hd)
    want = np.empty((heads, hd))
    for h in range(heads):
        s = kf[:, h // (heads // kvh), :] @ q[h * hd:(h + 1) * hd].astype(np.float64) * scale
        p = np.exp(s - s.max())
        want[h] = (p / p.sum()) @ vf[:, h // (heads // kvh), :]
    assert np.max(np.abs(a - want.ravel())) < 1e-4   # reference CUDA tests: max_diff < 1e-4
    assert np.max(np.abs(b - want.ravel())) < 1e-4
    # prefill with seq_len == 1 equals decode
    c = orc.attention_prefill(q, k, v, 1, kv_len, heads, kvh, hd, scale)
    assert np.max(np.abs(c - a)) < 1e-5


def test_glue_formulas(orc):
    rng = np.random.default_rng(2)
    x = rng.standard_normal(512).astype(np.float32)
    w = rng.standard_normal(512).astype(np.float32)
    got = orc.rms_norm(x, w, 1e-5)
    rms = np.float32(np.sqrt(np.mean(x.astype(np.float64) ** 2) + np.float64(np.float32(1e-5))))
    assert np.array_equal(got, (x / rms) * w)
    r = orc.rope(np.ones(8, np.float32), 3, 4, 8, 10000.0)
    ts = np.float32(10000.0) ** np.float32(-0.5)
    a0, a1 = np.float32(3.0), np.float32(3.0) * ts
    want = [np.cos(a0) - np.sin(a0), np.sin(a0) + np.cos(a0), np.cos(a1) - np.sin(a1),
            np.sin(a1) + np.cos(a1)]
    assert np.allclose(r[:4], want, atol=1e-6) and np.array_equal(r[:4], r[4:])
    assert orc.argmax_last(np.array([1, 5, 5, 2], np.float32)) == 2
    g = orc.silu_mul(np.array([0.0, 1.0, -2.0], np.float32), np.array([3.0, 2.0, 1.0], np.float32))
    assert np.allclose(g, [0.0, 2.0 / (1 + np.exp(-1.0)), -2.0 / (1 + np.exp(2.0))], atol=1e-6)
