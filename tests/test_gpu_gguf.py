"""A small random-init Q4_K_M Llama file written with the `gguf` package, loaded through
rnb_b200_gguf_open / rnb_b200_decoder_load_gguf (mmap, page registration, upload from the mapped
pages) and decoded greedily against the oracle fed the same tensors."""
import numpy as np
import pytest

import oracle as orc
from synth import llama_description, max_err_vs_norm
from gguf_util import write_llama_gguf

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("register_pages", [True, False])
def test_decoder_loaded_from_gguf_matches_oracle(tmp_path, register_pages):
    from runnburn_b200 import build, ops
    from runnburn_b200.gguf import load_decoder
    build.build_library()
    ops.open()
    desc = llama_description(seed=8, n_layer=2, hidden=512, n_head=4, n_kv_head=2, n_ff=1024, vocab=1024)
    path = tmp_path / "model.gguf"
    write_llama_gguf(path, desc, context_length=64)
    dec, f = load_decoder(str(path), register_pages=register_pages)
    assert dec.cfg.n_layer == 2 and dec.cfg.hidden == 512 and dec.cfg.vocab == 1024 and dec.cfg.max_ctx == 64
    ref = orc.Model(desc, 64)
    tok_g = tok_c = None
    prompt = np.random.default_rng(2).integers(0, 1024, 6).tolist()
    pos = 0
    for t in prompt + [None] * 24:
        if t is None:
            assert tok_g == tok_c, f"greedy ids diverge at position {pos}"
            t = tok_g
        tok_g, lg = dec.step(t, pos, want_logits=True)
        lc = ref.decode(t, pos)
        tok_c = orc.argmax_last(lc)
        assert max_err_vs_norm(lg, lc) <= 1e-3
        pos += 1
    dec.close()
    f.close()
    ops.clear_host_registered_ranges()
    ref.close()
