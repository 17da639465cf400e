"""Generates tests/golden/gguf_dequant.npz.

Independent pin for the oracle's dequantisers: seeded random GGUF blocks are expanded by
the third-party `gguf` Python package (its own numpy implementation of the GGML block
formats) and stored next to the input bytes.  The oracle must reproduce the floats
bit for bit (tests/test_oracle_kats.py).  Run from the repository root:

    python tests/golden/make_gguf_dequant_golden.py
"""
from pathlib import Path

import numpy as np
from gguf import GGMLQuantizationType as T
from gguf import quants


def f16_bits(rng, n, lo=1e-4, hi=2e-2):
    return rng.uniform(lo, hi, size=n).astype(np.float16).view(np.uint16)


def main():
    rng = np.random.default_rng(20240607)
    n = 24
    out = {}
    q4 = rng.integers(0, 256, size=(n, 144), dtype=np.uint8)
    q4[:, 0:2] = f16_bits(rng, n).view(np.uint8).reshape(n, 2)
    q4[:, 2:4] = f16_bits(rng, n).view(np.uint8).reshape(n, 2)
    out["q4k_bytes"] = q4
    out["q4k_f32"] = quants.dequantize(q4, T.Q4_K).astype(np.float32)
    q6 = rng.integers(0, 256, size=(n, 210), dtype=np.uint8)
    d = f16_bits(rng, n)
    d[::3] |= 0x8000  # negative super-scales occur in real files
    q6[:, 208:210] = d.view(np.uint8).reshape(n, 2)
    out["q6k_bytes"] = q6
    out["q6k_f32"] = quants.dequantize(q6, T.Q6_K).astype(np.float32)
    q8 = rng.integers(0, 256, size=(n * 8, 34), dtype=np.uint8)
    q8[:, 0:2] = f16_bits(rng, n * 8).view(np.uint8).reshape(n * 8, 2)
    out["q8_0_bytes"] = q8
    out["q8_0_f32"] = quants.dequantize(q8, T.Q8_0).astype(np.float32)
    # Q8_0 quantiser cross-check (gguf implements this one)
    x = rng.standard_normal((16, 64)).astype(np.float32)
    out["q8_0_quant_in"] = x
    out["q8_0_quant_bytes"] = quants.quantize(x, T.Q8_0)
    # drawn after everything else so that the earlier vectors keep their bytes
    q5 = rng.integers(0, 256, size=(n, 176), dtype=np.uint8)
    q5[:, 0:2] = f16_bits(rng, n).view(np.uint8).reshape(n, 2)
    q5[:, 2:4] = f16_bits(rng, n).view(np.uint8).reshape(n, 2)
    out["q5k_bytes"] = q5
    out["q5k_f32"] = quants.dequantize(q5, T.Q5_K).astype(np.float32)
    q2 = rng.integers(0, 256, size=(n, 84), dtype=np.uint8)
    q2[:, 80:82] = f16_bits(rng, n).view(np.uint8).reshape(n, 2)
    q2[:, 82:84] = f16_bits(rng, n).view(np.uint8).reshape(n, 2)
    out["q2k_bytes"] = q2
    out["q2k_f32"] = quants.dequantize(q2, T.Q2_K).astype(np.float32)
    q3 = rng.integers(0, 256, size=(n, 110), dtype=np.uint8)
    q3[:, 108:110] = f16_bits(rng, n).view(np.uint8).reshape(n, 2)
    out["q3k_bytes"] = q3
    out["q3k_f32"] = quants.dequantize(q3, T.Q3_K).astype(np.float32)
    np.savez_compressed(Path(__file__).with_name("gguf_dequant.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
