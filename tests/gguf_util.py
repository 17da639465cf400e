"""Writes small GGUF files for the tests with the third-party `gguf` package (used as a file
writer only): a random-init Llama-style stack in the Q4_K_M convention from a synth description."""
from __future__ import annotations

import numpy as np


def write_llama_gguf(path, desc: dict, arch: str = "llama", context_length: int = 256) -> None:
    import gguf
    from gguf import GGMLQuantizationType as T
    cfg = desc["cfg"]
    w = gguf.GGUFWriter(str(path), arch)
    w.add_context_length(context_length)
    w.add_embedding_length(cfg["hidden"])
    w.add_block_count(cfg["n_layer"])
    w.add_feed_forward_length(cfg["n_ff"])
    w.add_head_count(cfg["n_head"])
    w.add_head_count_kv(cfg["n_kv_head"])
    w.add_rope_freq_base(cfg["rope_theta"])
    w.add_layer_norm_rms_eps(cfg["rms_eps"])
    w.add_vocab_size(cfg["vocab"])

    def quant(name, pair, rows, cols):
        t, data = pair
        qt = T(t)
        w.add_tensor(name, np.ascontiguousarray(data, np.uint8).reshape(rows, -1), raw_dtype=qt)   # byte shape: the writer derives (rows, cols)

    hd = cfg["head_dim"]
    quant("token_embd.weight", desc["token_embd"], cfg["vocab"], cfg["hidden"])
    for i, L in enumerate(desc["layers"]):
        p = f"blk.{i}."
        w.add_tensor(p + "attn_norm.weight", np.asarray(L["attn_norm"], np.float32))
        quant(p + "attn_q.weight", L["wq"], cfg["n_head"] * hd, cfg["hidden"])
        quant(p + "attn_k.weight", L["wk"], cfg["n_kv_head"] * hd, cfg["hidden"])
        quant(p + "attn_v.weight", L["wv"], cfg["n_kv_head"] * hd, cfg["hidden"])
        quant(p + "attn_output.weight", L["wo"], cfg["hidden"], cfg["n_head"] * hd)
        w.add_tensor(p + "ffn_norm.weight", np.asarray(L["ffn_norm"], np.float32))
        quant(p + "ffn_gate.weight", L["gate"], cfg["n_ff"], cfg["hidden"])
        quant(p + "ffn_up.weight", L["up"], cfg["n_ff"], cfg["hidden"])
        quant(p + "ffn_down.weight", L["down"], cfg["hidden"], cfg["n_ff"])
    w.add_tensor("output_norm.weight", np.asarray(desc["out_norm"], np.float32))
    quant("output.weight", desc["output"], cfg["vocab"], cfg["hidden"])
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
