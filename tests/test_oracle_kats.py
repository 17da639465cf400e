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
    for name, t, cols in (("q2k", orc.TYPE_Q2_K, 256), ("q3k", orc.TYPE_Q3_K, 256), ("q4k", orc.TYPE_Q4_K, 256), ("q5k", orc.TYPE_Q5_K, 256), ("q6k", orc.TYPE_Q6_K, 256),
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


# ---- the reference's own attention / RoPE / RMSNorm fixtures, restated -------------------------
def _lcg_f32(seed: int, n: int) -> np.ndarray:
    """The generator of the reference's attention tests (kernels/attention/mod.rs:213-221):
    a 64-bit LCG whose top 31 bits map to [-1, 1)."""
    out = np.empty(n, np.float32)
    s = seed
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = np.float32(np.float32(s >> 33) / np.float32(1 << 31)) * np.float32(2.0) - np.float32(1.0)
    return out


def _naive_attention(q, k, v, seq, kv, nh, nkv, hd):
    """naive_attention of kernels/attention/mod.rs:146-201 (f32 throughout, causal by global position)."""
    out = np.zeros(seq * nh * hd, np.float32)
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    for h in range(nh):
        kvh = h // (nh // nkv)
        for i in range(seq):
            qr = q[i * nh * hd + h * hd:][:hd]
            gp = (kv - seq) + i
            n_vis = min(gp, kv - 1) + 1
            sc = np.full(kv, -np.inf, np.float32)
            for j in range(n_vis):
                kr = k[j * nkv * hd + kvh * hd:][:hd]
                dot = np.float32(0.0)
                for d in range(hd):
                    dot = np.float32(dot + qr[d] * kr[d])
                sc[j] = dot * scale
            p = np.exp((sc - sc.max()).astype(np.float32)).astype(np.float32)
            p = (p / p.sum(dtype=np.float32)).astype(np.float32)
            acc = np.zeros(hd, np.float32)
            for j in range(kv):
                acc = (acc + p[j] * v[j * nkv * hd + kvh * hd:][:hd]).astype(np.float32)
            out[i * nh * hd + h * hd:][:hd] = acc
    return out


def test_reference_attention_fixtures(orc):
    # test_attention_decode_into_matches_tensor (kernels/attention/mod.rs:32-88): sin/cos ramps,
    # 4 heads over 2 KV heads, head_dim 4, 3 cached rows; f16 cache vs f32 attention within 1e-2
    nh, nkv, hd, kv = 4, 2, 4, 3
    q = np.sin(np.arange(nh * hd, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    kf = np.cos(np.arange(kv * nkv * hd, dtype=np.float32) * np.float32(0.2)).astype(np.float32)
    vf = np.sin(np.arange(kv * nkv * hd, dtype=np.float32) * np.float32(0.3)).astype(np.float32)
    scale = 1.0 / np.sqrt(np.float32(hd))
    want = orc.attention_prefill(q, kf, vf, 1, kv, nh, nkv, hd, scale)
    got = orc.attention_decode(q, orc.f32_to_f16_bits(kf), orc.f32_to_f16_bits(vf), nh, nkv, hd, kv, scale)
    assert np.max(np.abs(got - want)) < 1e-2
    assert np.max(np.abs(want - _naive_attention(q, kf, vf, 1, kv, nh, nkv, hd))) < 1e-5
    # test_attention_single_token (:112-127): one query, one key -> the value row itself
    out = orc.attention_prefill(np.float32([1, 0]), np.float32([1, 0]), np.float32([3, 7]), 1, 1, 1, 1, 2, 1.0 / np.sqrt(2.0))
    assert abs(out[0] - 3.0) < 1e-4 and abs(out[1] - 7.0) < 1e-4
    # test_attention_long_seq_matches_naive (:203-266), at a quarter of its sequence length so that
    # the pure-Python naive loop stays in seconds: LCG seed 42, 4 heads, head_dim 64, causal
    seq, nh, nkv, hd = 32, 4, 4, 64
    g = _lcg_f32(42, seq * nh * hd + 2 * seq * nkv * hd)
    q, k, v = g[:seq * nh * hd], g[seq * nh * hd:][:seq * nkv * hd], g[seq * nh * hd + seq * nkv * hd:]
    flash = orc.attention_prefill(q, k, v, seq, seq, nh, nkv, hd, 1.0 / np.sqrt(np.float32(hd)))
    assert np.max(np.abs(flash - _naive_attention(q, k, v, seq, seq, nh, nkv, hd))) < 1e-4
    # test_attention_decode_flash_matches_legacy (:346-428): LCG seed 12345, 8 heads over 4 KV heads,
    # head_dim 64, 128 rows; the online form against the 4-pass form: cos >= 0.9999, max abs < 1e-3
    nh, nkv, hd, kv = 8, 4, 64, 128
    g = _lcg_f32(12345, nh * hd + 2 * kv * nkv * hd)
    q, k, v = g[:nh * hd], g[nh * hd:][:kv * nkv * hd], g[nh * hd + kv * nkv * hd:]
    kb, vb = orc.f32_to_f16_bits(k), orc.f32_to_f16_bits(v)
    legacy = orc.attention_decode(q, kb, vb, nh, nkv, hd, kv, 1.0 / np.sqrt(np.float32(hd)))
    flash = orc.attention_decode(q, kb, vb, nh, nkv, hd, kv, 1.0 / np.sqrt(np.float32(hd)), online=True)
    cos = float(np.dot(legacy.astype(np.float64), flash.astype(np.float64)) /
                (np.linalg.norm(legacy.astype(np.float64)) * np.linalg.norm(flash.astype(np.float64))))
    assert cos >= 0.9999 and np.max(np.abs(legacy - flash)) < 1e-3
    # the f16 conversion the fixtures rely on is IEEE round-to-nearest-even (half::f16::from_f32)
    assert np.array_equal(kb, k.astype(np.float16).view(np.uint16))


def test_reference_rope_fixtures(orc):
    """kernels/rope.rs:725-790: position 0 is the identity, position 1 rotates, the in-place form
    equals the tensor form, positions advance per token, and the closed form of the first pairs
    (pair 0 turns by `pos` radians, pair 1 by pos * theta^(-2/head_dim))."""
    x = np.float32([1, 2, 3, 4])
    assert np.max(np.abs(orc.rope(x, 0, 4, 4, 10000.0) - x)) < 1e-5
    r = orc.rope(np.float32([1, 0, 0, 0]), 1, 4, 4, 10000.0)
    assert abs(r[0] - 1.0) > 1e-3 or abs(r[1]) > 1e-3
    assert abs(r[0] - np.cos(np.float32(1.0))) < 1e-5 and abs(r[1] - np.sin(np.float32(1.0))) < 1e-5
    r = orc.rope(np.float32([1, 0, 0, 1]), 1, 4, 4, 10000.0)
    a1 = np.float32(0.01)                                      # 1 * 10000^(-2/4)
    assert abs(r[2] + np.sin(a1)) < 1e-6 and abs(r[3] - np.cos(a1)) < 1e-6
    # two heads of one token share the angles (test_rope_inplace_matches_tensor, pos 5)
    r = orc.rope(np.float32([1, 0, 0, 1, 2, 0, 0, 2]), 5, 4, 8, 10000.0)
    assert np.allclose(r[4:], 2 * r[:4], atol=1e-6)
    assert abs(r[0] - np.cos(np.float32(5.0))) < 1e-5 and abs(r[1] - np.sin(np.float32(5.0))) < 1e-5
    # test_rope_per_token_position: token 0 at pos 0 unchanged, token 1 at pos 1 rotated
    two = np.float32([1, 2, 3, 4, 1, 2, 3, 4])
    r = orc.rope(two, 0, 4, 4, 10000.0)
    assert np.max(np.abs(r[:4] - two[:4])) < 1e-5 and (abs(r[4] - 1.0) > 1e-3 or abs(r[5] - 2.0) > 1e-3)


def test_reference_rms_norm_fixtures(orc):
    """kernels/norm.rs:339-415: [1,2,3,4] with unit weights divides by sqrt(7.5 + eps); weighted
    rows follow (x / rms) * w bit for bit; the f64 reduce stays within 2e-5 of the f32 scalar
    formula on the 1536-wide pattern rows of the reference's AVX2 test."""
    x = np.float32([1, 2, 3, 4])
    got = orc.rms_norm(x, np.ones(4, np.float32), 1e-5)
    rms = np.sqrt(np.float32(7.5) + np.float32(1e-5))
    assert abs(got[0] - 1.0 / rms) < 1e-4 and abs(got[1] - 2.0 / rms) < 1e-4
    w = np.float32([1.0, 0.5, 2.0, 0.25])
    rms64 = np.float32(np.sqrt(np.float64(7.5) + np.float64(np.float32(1e-5))))
    assert np.array_equal(orc.rms_norm(x, w, 1e-5).view(np.uint32), ((x / rms64) * w).astype(np.float32).view(np.uint32))
    hidden, rows = 1536, 3
    i = np.arange(hidden * rows)
    inp = (((i * 37 % 251).astype(np.float32) - np.float32(125.0)) / np.float32(31.0)).astype(np.float32)
    j = np.arange(hidden)
    wt = (((j * 19 % 127).astype(np.float32) - np.float32(63.0)) / np.float32(97.0)).astype(np.float32)
    got = orc.rms_norm(inp, wt, 1e-5).reshape(rows, hidden)
    for s in range(rows):
        xs = inp[s * hidden:(s + 1) * hidden]
        acc = np.float32(0.0)
        for vv in xs:                                           # rms_norm_into_scalar: sequential f32 sum
            acc = np.float32(acc + vv * vv)
        rms32 = np.sqrt(np.float32(acc / np.float32(hidden)) + np.float32(1e-5))
        assert np.max(np.abs(got[s] - (xs / rms32) * wt)) < 2e-5


def test_q5k_block_size_zero_block_and_dot_against_dequantised_q8k(orc):
    """Q5_K (crates/rnb-cpu/src/quantize/blocks.rs:90-98: 176 bytes; dequant.rs test_dequant_q5_k_zero).
    The integer dot equals the scalar dot over the dequantised weights and the dequantised Q8_K
    activation to f32 rounding (the bound the reference uses for its int-dot tests), and the harness
    quantiser round-trips through the reference's dequantiser."""
    assert orc.row_bytes(orc.TYPE_Q5_K, 256) == 176
    assert np.all(orc.dequantize_matrix(orc.TYPE_Q5_K, np.zeros(176, np.uint8), 1, 256) == 0.0)
    rng = np.random.default_rng(55)
    rows, cols = 6, 1024
    w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
    q = orc.quantize_matrix(orc.TYPE_Q5_K, w)
    back = orc.dequantize_matrix(orc.TYPE_Q5_K, q, rows, cols)
    assert _cos(w.ravel(), back.ravel()) >= 0.999
    x = rng.standard_normal(cols).astype(np.float32)
    xq = orc.quantize_q8k(x)
    blocks = xq.view(np.uint8).reshape(-1, 292)
    xd = np.concatenate([blocks[b, :4].view(np.float32)[0] * blocks[b, 4:260].view(np.int8).astype(np.float32) for b in range(cols // 256)])
    got = orc.gemv(orc.TYPE_Q5_K, q, x, rows, cols)
    want = back.astype(np.float64) @ xd.astype(np.float64)
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) < 1e-4
    # random blocks (all bit patterns of scales and high bits) as well
    raw = rng.integers(0, 256, size=(rows, cols // 256, 176), dtype=np.uint8)
    raw[..., 1] = 0x10
    raw[..., 3] = 0x10
    raw = raw.reshape(-1)
    back = orc.dequantize_matrix(orc.TYPE_Q5_K, raw, rows, cols)
    got = orc.gemv(orc.TYPE_Q5_K, raw, x, rows, cols)
    want = back.astype(np.float64) @ xd.astype(np.float64)
    assert np.max(np.abs(got - want)) < 1e-4 * np.max(np.abs(want))


def test_q2k_block_size_and_dot_against_dequantised_q8k(orc):
    """Q2_K (crates/rnb-cpu/src/quantize/blocks.rs:63-69: 84 bytes).  The integer dot
    (crates/rnb-cpu/src/gemm/avx2_dot.rs:169-245) equals the scalar dot over the dequantised weights and
    the dequantised Q8_K activation to f32 rounding, on fitted weights and on random block bytes."""
    assert orc.row_bytes(orc.TYPE_Q2_K, 256) == 84
    assert np.all(orc.dequantize_matrix(orc.TYPE_Q2_K, np.zeros(84, np.uint8), 1, 256) == 0.0)
    rng = np.random.default_rng(22)
    rows, cols = 6, 1024
    x = rng.standard_normal(cols).astype(np.float32)
    blocks = orc.quantize_q8k(x).view(np.uint8).reshape(-1, 292)
    xd = np.concatenate([blocks[b, :4].view(np.float32)[0] * blocks[b, 4:260].view(np.int8).astype(np.float32) for b in range(cols // 256)])
    w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
    q = orc.quantize_matrix(orc.TYPE_Q2_K, w)
    raw = rng.integers(0, 256, size=(rows, cols // 256, 84), dtype=np.uint8)
    raw[..., 81] = 0x10
    raw[..., 83] = 0x10
    for data in (q, raw.reshape(-1)):
        back = orc.dequantize_matrix(orc.TYPE_Q2_K, data, rows, cols)
        got = orc.gemv(orc.TYPE_Q2_K, data, x, rows, cols)
        want = back.astype(np.float64) @ xd.astype(np.float64)
        assert np.max(np.abs(got - want)) < 1e-4 * np.max(np.abs(want))
    assert _cos(w.ravel(), orc.dequantize_matrix(orc.TYPE_Q2_K, q, rows, cols).ravel()) >= 0.9


def test_q3k_block_size_and_dot_against_dequantised_q8k(orc):
    """Q3_K (crates/rnb-cpu/src/quantize/blocks.rs:72-78: 110 bytes, 2-byte aligned only).  The integer dot
    (crates/rnb-cpu/src/gemm/avx2_dot.rs:247-378) equals the scalar dot over the dequantised weights and the
    dequantised Q8_K activation to f32 rounding, on fitted weights and on random block bytes."""
    assert orc.row_bytes(orc.TYPE_Q3_K, 256) == 110
    rng = np.random.default_rng(33)
    rows, cols = 6, 1024
    x = rng.standard_normal(cols).astype(np.float32)
    blocks = orc.quantize_q8k(x).view(np.uint8).reshape(-1, 292)
    xd = np.concatenate([blocks[b, :4].view(np.float32)[0] * blocks[b, 4:260].view(np.int8).astype(np.float32) for b in range(cols // 256)])
    w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
    q = orc.quantize_matrix(orc.TYPE_Q3_K, w)
    raw = rng.integers(0, 256, size=(rows, cols // 256, 110), dtype=np.uint8)
    raw[..., 109] = 0x10
    for data in (q, raw.reshape(-1)):
        back = orc.dequantize_matrix(orc.TYPE_Q3_K, data, rows, cols)
        got = orc.gemv(orc.TYPE_Q3_K, data, x, rows, cols)
        want = back.astype(np.float64) @ xd.astype(np.float64)
        assert np.max(np.abs(got - want)) < 1e-4 * np.max(np.abs(want))
    assert _cos(w.ravel(), orc.dequantize_matrix(orc.TYPE_Q3_K, q, rows, cols).ravel()) >= 0.97


def test_sliding_window_equals_attention_over_the_last_rows(orc):
    # the literal routine (every position walked, masked ones scoring -inf) equals plain attention over the
    # window's rows bit for bit: the masked weights are exact zeros
    rng = np.random.default_rng(31)
    heads, kvh, kv_len = 4, 2, 90
    k = orc.f32_to_f16_bits(rng.standard_normal(kv_len * kvh * 128))
    v = orc.f32_to_f16_bits(rng.standard_normal(kv_len * kvh * 128))
    q = rng.standard_normal(heads * 128).astype(np.float32)
    scale = 1.0 / np.sqrt(128.0)
    for window in (1, 7, 64, 90, 200):
        w = min(window, kv_len)
        lo = (kv_len - w) * kvh * 128
        full = orc.attention_decode_window(q, k, v, heads, kvh, 128, kv_len, scale, window)
        assert np.array_equal(full, orc.attention_decode(q, k[lo:], v[lo:], heads, kvh, 128, w, scale))
