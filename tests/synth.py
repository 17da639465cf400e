"""Seeded synthetic inputs shared by the tests (weights in GGUF block formats, small models)."""
from __future__ import annotations

import numpy as np

import oracle as orc

Q4_K, Q6_K, Q8_0 = orc.TYPE_Q4_K, orc.TYPE_Q6_K, orc.TYPE_Q8_0


def random_blocks(rng, ggml_type: int, rows: int, cols: int) -> np.ndarray:
    """Config-1 style blocks: uniform quants and 6-bit scales, |N(0,1e-3)| f16 super-scales."""
    if ggml_type == Q4_K:
        nb = cols // 256
        w = rng.integers(0, 256, size=(rows, nb, 144), dtype=np.uint8)
        d = np.abs(rng.standard_normal((rows, nb, 2)) * 1e-3).astype(np.float16)
        w[:, :, 0:4] = d.view(np.uint8).reshape(rows, nb, 4)
    elif ggml_type == Q6_K:
        nb = cols // 256
        w = rng.integers(0, 256, size=(rows, nb, 210), dtype=np.uint8)
        d = (rng.standard_normal((rows, nb, 1)) * 1e-3).astype(np.float16)
        w[:, :, 208:210] = d.view(np.uint8).reshape(rows, nb, 2)
    else:
        nb = cols // 32
        w = rng.integers(0, 256, size=(rows, nb, 34), dtype=np.uint8)
        d = np.abs(rng.standard_normal((rows, nb, 1)) * 1e-2).astype(np.float16)
        w[:, :, 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
    return np.ascontiguousarray(w.reshape(-1))


def quantized(rng, ggml_type: int, rows: int, cols: int, sigma: float = 0.02):
    w = (rng.standard_normal((rows, cols)) * sigma).astype(np.float32)
    return ggml_type, orc.quantize_matrix(ggml_type, w)


def max_rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """max |got - ref| / max(|ref|, eps * ||ref||_inf): relative error that tolerates zeros."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    floor = 1e-3 * max(np.max(np.abs(ref)), 1e-30)
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), floor)))


def max_err_vs_norm(got: np.ndarray, ref: np.ndarray) -> float:
    """max |got - ref| / max |ref|: error of a whole vector (logits) relative to its scale."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30))


def llama_description(seed: int, n_layer=2, hidden=512, n_head=4, n_kv_head=2, n_ff=1024, vocab=1024,
                      rope_theta=5e5, rms_eps=1e-5, sigma=0.02):
    """Random-init Llama-style stack in the Q4_K_M convention: attn_v, ffn_down and the LM
    head in Q6_K, everything else Q4_K; N(0, sigma) weights quantised by the oracle."""
    rng = np.random.default_rng(seed)
    hd = 128
    layers = []
    for _ in range(n_layer):
        layers.append(dict(
            attn_norm=np.ones(hidden, np.float32), ffn_norm=np.ones(hidden, np.float32),
            wq=quantized(rng, Q4_K, n_head * hd, hidden, sigma), wk=quantized(rng, Q4_K, n_kv_head * hd, hidden, sigma),
            wv=quantized(rng, Q6_K, n_kv_head * hd, hidden, sigma), wo=quantized(rng, Q4_K, hidden, n_head * hd, sigma),
            gate=quantized(rng, Q4_K, n_ff, hidden, sigma), up=quantized(rng, Q4_K, n_ff, hidden, sigma),
            down=quantized(rng, Q6_K, hidden, n_ff, sigma)))
    cfg = dict(n_layer=n_layer, hidden=hidden, n_head=n_head, n_kv_head=n_kv_head, head_dim=hd, n_ff=n_ff,
               vocab=vocab, rope_neox=0, rms_eps=rms_eps, rope_theta=rope_theta, n_expert=0, n_expert_used=0,
               n_ff_expert=0)
    return dict(cfg=cfg, layers=layers, token_embd=quantized(rng, Q4_K, vocab, hidden, 1.0),
                out_norm=np.ones(hidden, np.float32), output=quantized(rng, Q6_K, vocab, hidden, sigma))


def moe_description(seed: int, n_layer=2, hidden=512, n_head=4, n_kv_head=2, vocab=1024, n_expert=16,
                    n_expert_used=4, n_ff_expert=256, rope_theta=1e6, rms_eps=1e-6, sigma=0.02, down_type=Q4_K):
    """Qwen3-MoE-shaped stack: Q6_K attention, Q4_K experts (down experts: down_type), f32 N(0,1) router, half-split RoPE."""
    rng = np.random.default_rng(seed)
    hd = 128
    layers = []
    for _ in range(n_layer):
        layers.append(dict(
            attn_norm=np.ones(hidden, np.float32), ffn_norm=np.ones(hidden, np.float32),
            wq=quantized(rng, Q6_K, n_head * hd, hidden, sigma), wk=quantized(rng, Q6_K, n_kv_head * hd, hidden, sigma),
            wv=quantized(rng, Q6_K, n_kv_head * hd, hidden, sigma), wo=quantized(rng, Q6_K, hidden, n_head * hd, sigma),
            router=rng.standard_normal((n_expert, hidden)).astype(np.float32),
            gate_exps=quantized(rng, Q4_K, n_expert * n_ff_expert, hidden, sigma),
            up_exps=quantized(rng, Q4_K, n_expert * n_ff_expert, hidden, sigma),
            down_exps=quantized(rng, down_type, n_expert * hidden, n_ff_expert, sigma)))
    cfg = dict(n_layer=n_layer, hidden=hidden, n_head=n_head, n_kv_head=n_kv_head, head_dim=hd, n_ff=0, vocab=vocab,
               rope_neox=1, rms_eps=rms_eps, rope_theta=rope_theta, n_expert=n_expert, n_expert_used=n_expert_used,
               n_ff_expert=n_ff_expert)
    return dict(cfg=cfg, layers=layers, token_embd=quantized(rng, Q4_K, vocab, hidden, 1.0),
                out_norm=np.ones(hidden, np.float32), output=quantized(rng, Q6_K, vocab, hidden, sigma))


def synth(ggml_type: int, rows: int, cols: int, seed: int, sigma: float = 0.02):
    """(type, blocks) of a seeded N(0, sigma) matrix from the oracle's fast generator."""
    return ggml_type, orc.synth_matrix(ggml_type, rows, cols, seed, sigma)


def llama_description_fast(seed: int, n_layer=2, hidden=4096, n_head=32, n_kv_head=8, n_ff=14336, vocab=128256,
                           rope_theta=5e5, rms_eps=1e-5, sigma=0.02):
    """Llama-style stack in the Q4_K_M convention at full width (Llama-3-8B by default) with few
    layers: weights come from the oracle's fast seeded generator instead of numpy + the
    reference quantiser, which would take minutes at these sizes."""
    hd = 128
    layers = []
    for l in range(n_layer):
        b = seed * 1000 + l * 16
        layers.append(dict(
            attn_norm=np.ones(hidden, np.float32), ffn_norm=np.ones(hidden, np.float32),
            wq=synth(Q4_K, n_head * hd, hidden, b + 1, sigma), wk=synth(Q4_K, n_kv_head * hd, hidden, b + 2, sigma),
            wv=synth(Q6_K, n_kv_head * hd, hidden, b + 3, sigma), wo=synth(Q4_K, hidden, n_head * hd, b + 4, sigma),
            gate=synth(Q4_K, n_ff, hidden, b + 5, sigma), up=synth(Q4_K, n_ff, hidden, b + 6, sigma),
            down=synth(Q6_K, hidden, n_ff, b + 7, sigma)))
    cfg = dict(n_layer=n_layer, hidden=hidden, n_head=n_head, n_kv_head=n_kv_head, head_dim=hd, n_ff=n_ff,
               vocab=vocab, rope_neox=0, rms_eps=rms_eps, rope_theta=rope_theta, n_expert=0, n_expert_used=0,
               n_ff_expert=0)
    return dict(cfg=cfg, layers=layers, token_embd=synth(Q4_K, vocab, hidden, seed * 1000 + 900, 1.0),
                out_norm=np.ones(hidden, np.float32), output=synth(Q6_K, vocab, hidden, seed * 1000 + 901, sigma))


def moe_description_fast(seed: int, n_layer=2, hidden=2048, n_head=32, n_kv_head=4, vocab=32768, n_expert=128,
                         n_expert_used=8, n_ff_expert=768, rope_theta=1e6, rms_eps=1e-6, sigma=0.02):
    """Qwen3-30B-A3B-shaped stack (Q6_K attention, Q4_K experts, f32 N(0,1) router, half-split
    RoPE) at full width with few layers, weights from the oracle's fast generator."""
    rng = np.random.default_rng(seed)
    hd = 128
    layers = []
    for l in range(n_layer):
        b = seed * 1000 + l * 16
        layers.append(dict(
            attn_norm=np.ones(hidden, np.float32), ffn_norm=np.ones(hidden, np.float32),
            wq=synth(Q6_K, n_head * hd, hidden, b + 1, sigma), wk=synth(Q6_K, n_kv_head * hd, hidden, b + 2, sigma),
            wv=synth(Q6_K, n_kv_head * hd, hidden, b + 3, sigma), wo=synth(Q6_K, hidden, n_head * hd, b + 4, sigma),
            router=rng.standard_normal((n_expert, hidden)).astype(np.float32),
            gate_exps=synth(Q4_K, n_expert * n_ff_expert, hidden, b + 5, sigma),
            up_exps=synth(Q4_K, n_expert * n_ff_expert, hidden, b + 6, sigma),
            down_exps=synth(Q4_K, n_expert * hidden, n_ff_expert, b + 7, sigma)))
    cfg = dict(n_layer=n_layer, hidden=hidden, n_head=n_head, n_kv_head=n_kv_head, head_dim=hd, n_ff=0, vocab=vocab,
               rope_neox=1, rms_eps=rms_eps, rope_theta=rope_theta, n_expert=n_expert, n_expert_used=n_expert_used,
               n_ff_expert=n_ff_expert)
    return dict(cfg=cfg, layers=layers, token_embd=synth(Q4_K, vocab, hidden, seed * 1000 + 900, 1.0),
                out_norm=np.ones(hidden, np.float32), output=synth(Q6_K, vocab, hidden, seed * 1000 + 901, sigma))
