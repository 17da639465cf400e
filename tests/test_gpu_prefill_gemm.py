"""Tensor-core prefill matmul (tcgen05, bf16 x bf16 -> f32) against the oracle.

The oracle side is rnb-cpu's dequantisation (f32) rounded once to bf16, tokens rounded to bf16,
products summed in float64: the GPU result differs only by its f32 accumulation (a random walk
of about sqrt(K) * 2^-24 of the partial sums, 1e-5 absolute at K = 4096), so errors are bounded
relative to the size of a dot product, sqrt(sum (x*w)^2): 1e-4 of it, ten times tighter than
the path's 1e-3.  A second check bounds the distance to the exact (unrounded) rnb-cpu matmul by
what bf16 inputs allow."""
import numpy as np
import pytest

import oracle as orc
from synth import Q4_K, Q6_K, max_err_vs_norm, max_rel_err, quantized, random_blocks

pytestmark = pytest.mark.gpu
TOL = 1e-3


def bf16_round(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32)


@pytest.fixture()
def ops():
    import runnburn_b200.ops as o
    o.reset_state_for_engine_init()
    return o


@pytest.mark.parametrize("t,rows,cols,seq", [
    (Q4_K, 256, 256, 1), (Q4_K, 256, 256, 256), (Q4_K, 300, 512, 37), (Q4_K, 1024, 4096, 273), (Q4_K, 4096, 4096, 512),
    (Q6_K, 256, 256, 5), (Q6_K, 515, 1024, 100), (Q6_K, 1024, 4096, 300), (Q6_K, 4096, 2048, 512),
])
def test_bf16_gemm_matches_bf16_rounded_oracle(ops, t, rows, cols, seq):
    rng = np.random.default_rng(rows * 31 + cols + seq)
    _, w = quantized(rng, t, rows, cols)
    x = rng.standard_normal((seq, cols)).astype(np.float32)
    wd = orc.dequantize_matrix(t, w, rows, cols).reshape(rows, cols)
    ref = bf16_round(x).astype(np.float64) @ bf16_round(wd).astype(np.float64).T
    fn = ops.q4k_bf16_gemm_batch if t == Q4_K else ops.q6k_bf16_gemm_batch
    got = fn(w, rows, cols, x).reshape(seq, rows)
    scale = np.sqrt((x.astype(np.float64) ** 2) @ (wd.astype(np.float64) ** 2).T)
    assert np.max(np.abs(got - ref) / np.maximum(scale, 1e-30)) <= TOL / 10
    assert max_err_vs_norm(got, ref) <= TOL / 10
    # distance to the exact matmul: two bf16 roundings per product, averaged over K terms
    exact = x.astype(np.float64) @ wd.astype(np.float64).T
    assert np.max(np.abs(got - exact) / np.maximum(scale, 1e-30)) <= 3e-2


def test_bf16_gemm_uniform_quant_blocks_config1_shape(ops):
    """BASELINE config 1 style blocks (uniform quants and scales) at a Llama layer shape."""
    rng = np.random.default_rng(0)
    rows, cols, seq = 4096, 4096, 256
    w = random_blocks(rng, Q4_K, rows, cols)
    x = rng.standard_normal((seq, cols)).astype(np.float32)
    wd = orc.dequantize_matrix(Q4_K, w, rows, cols).reshape(rows, cols)
    ref = bf16_round(x).astype(np.float64) @ bf16_round(wd).astype(np.float64).T
    got = ops.q4k_bf16_gemm_batch(w, rows, cols, x).reshape(seq, rows)
    assert max_err_vs_norm(got, ref) <= TOL / 10


def test_bf16_qkv_gemm_batch_equals_the_single_matrix_calls(ops):
    # q4k_f16_qkv_gemm_batch: three Q4_K projections of one token batch; each output equals the single-matrix call's
    # (same kernel, same tiles) and so inherits its bound against the oracle
    rng = np.random.default_rng(17)
    q_rows, kv_rows, cols, seq = 512, 130, 1024, 45
    ws = [quantized(rng, Q4_K, r, cols)[1] for r in (q_rows, kv_rows, kv_rows)]
    x = rng.standard_normal((seq, cols)).astype(np.float32)
    q, k, v = ops.q4k_bf16_qkv_gemm_batch(ws[0], ws[1], ws[2], q_rows, kv_rows, cols, x)
    for got, w, rows in ((q, ws[0], q_rows), (k, ws[1], kv_rows), (v, ws[2], kv_rows)):
        assert np.array_equal(got, ops.q4k_bf16_gemm_batch(w, rows, cols, x))
        wd = orc.dequantize_matrix(Q4_K, w, rows, cols).reshape(rows, cols)
        ref = bf16_round(x).astype(np.float64) @ bf16_round(wd).astype(np.float64).T
        assert max_err_vs_norm(got.reshape(seq, rows), ref) <= TOL / 10
    import runnburn_b200 as r
    with pytest.raises(r.RnbError, match="byte mismatch"):
        ops.q4k_bf16_qkv_gemm_batch(ws[0], ws[1][:-1], ws[2], q_rows, kv_rows, cols, x)


def test_bf16_gemm_three_matrices_one_launch(ops):
    """q/k/v style: three matrices (mixed Q4_K / Q6_K, different row counts) behind one token tile."""
    import ctypes as C

    import torch

    import runnburn_b200 as r
    L = r.load()
    rng = np.random.default_rng(11)
    cols, seq = 1024, 70
    specs = [(Q4_K, 512), (Q4_K, 130), (Q6_K, 256)]
    ws = [quantized(rng, t, rows, cols)[1] for t, rows in specs]
    x = rng.standard_normal((seq, cols)).astype(np.float32)
    wt = [torch.from_numpy(np.ascontiguousarray(w)).cuda() for w in ws]
    xt = torch.from_numpy(x).cuda()
    xb = torch.empty(seq * cols, dtype=torch.int16, device="cuda")
    ys = [torch.zeros(seq, rows, device="cuda") for _, rows in specs]
    n = len(specs)
    rc = L.rnb_b200_dev_prefill_gemm_multi(n, (C.c_int * n)(*[t for t, _ in specs]), (C.c_void_p * n)(*[w.data_ptr() for w in wt]),
                                           (C.c_size_t * n)(*[rows for _, rows in specs]), (C.c_void_p * n)(*[y.data_ptr() for y in ys]),
                                           cols, xt.data_ptr(), seq, xb.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.rnb_b200_last_error()
    torch.cuda.synchronize()
    assert ops.dev_error_flag() == 0
    for (t, rows), w, y in zip(specs, ws, ys):
        wd = orc.dequantize_matrix(t, w, rows, cols).reshape(rows, cols)
        ref = bf16_round(x).astype(np.float64) @ bf16_round(wd).astype(np.float64).T
        assert max_err_vs_norm(y.cpu().numpy(), ref) <= TOL / 10


@pytest.mark.parametrize("t,rows,cols,seq", [(Q4_K, 256, 512, 70), (Q4_K, 1000, 1024, 600), (Q6_K, 192, 1024, 33), (Q4_K, 14336, 4096, 512)])
def test_bf16_gate_up_silu_epilogue(ops, t, rows, cols, seq):
    """gate + up in one launch (64 rows of each per tile) with silu(gate) * up written as bf16 by the epilogue: equal to
    the two single-matrix products pushed through the same formula, up to the bf16 rounding of the result; ragged
    row and token counts."""
    import torch

    import runnburn_b200 as r
    L = r.load()
    rng = np.random.default_rng(rows + seq)
    wg = quantized(rng, t, rows, cols)[1] if rows < 4096 else random_blocks(rng, t, rows, cols)
    wu = quantized(rng, t, rows, cols)[1] if rows < 4096 else random_blocks(rng, t, rows, cols)
    x = (rng.standard_normal((seq, cols)) * (1.0 if rows < 4096 else 0.05)).astype(np.float32)
    fn = ops.q4k_bf16_gemm_batch if t == Q4_K else ops.q6k_bf16_gemm_batch
    g = fn(wg, rows, cols, x).reshape(seq, rows).astype(np.float64)
    u = fn(wu, rows, cols, x).reshape(seq, rows).astype(np.float64)
    ref = g / (1.0 + np.exp(-g)) * u
    gt, ut = torch.from_numpy(np.ascontiguousarray(wg)).cuda(), torch.from_numpy(np.ascontiguousarray(wu)).cuda()
    xt = torch.from_numpy(x).cuda()
    xb = torch.empty(seq * cols, dtype=torch.int16, device="cuda")
    act = torch.zeros(seq, rows, dtype=torch.bfloat16, device="cuda")
    rc = L.rnb_b200_dev_prefill_gemm_silu(t, gt.data_ptr(), ut.data_ptr(), rows, cols, xt.data_ptr(), seq, xb.data_ptr(), act.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.rnb_b200_last_error()
    torch.cuda.synchronize()
    assert ops.dev_error_flag() == 0
    got = act.float().cpu().numpy().astype(np.float64)
    # one bf16 rounding of the result (2^-9 relative) on top of the f32 evaluation
    assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-3 * np.max(np.abs(ref)))) <= 2.0 ** -8


def test_bf16_gemm_rejects_bad_shapes(ops):
    import runnburn_b200 as r
    w = np.zeros(144, np.uint8)
    with pytest.raises(r.RnbError):
        ops.q4k_bf16_gemm_batch(w, 1, 256, np.zeros(255, np.float32))
