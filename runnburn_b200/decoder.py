"""Device-resident greedy decoder over the C ABI (`rnb_b200_decoder_*`).

One decode step is one CUDA-graph launch; only the token id crosses PCIe.  The operator order
is the reference engine's (crates/rnb-llm/src/engine/decode.rs:199-564, decode_ffn.rs:294-366,
logits.rs).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, asdict

import numpy as np

from . import _lib
from ._lib import check, load


@dataclass
class ModelConfig:
    n_layer: int
    hidden: int
    n_head: int
    n_kv_head: int
    n_ff: int
    vocab: int
    max_ctx: int
    head_dim: int = 128
    rope_neox: int = 0
    rms_eps: float = 1e-5
    rope_theta: float = 5e5
    n_expert: int = 0
    n_expert_used: int = 0
    n_ff_expert: int = 0
    world_size: int = 1
    rank: int = 0

    def to_c(self) -> _lib.ModelCfg:
        c = _lib.ModelCfg()
        for k, v in asdict(self).items():
            setattr(c, k, v)
        return c


# Published shapes of the configurations the bench and tests use (random-init, synthetic).
LLAMA3_8B = dict(n_layer=32, hidden=4096, n_head=32, n_kv_head=8, n_ff=14336, vocab=128256)
LLAMA3_70B = dict(n_layer=80, hidden=8192, n_head=64, n_kv_head=8, n_ff=28672, vocab=128256)
QWEN3_30B_A3B = dict(n_layer=48, hidden=2048, n_head=32, n_kv_head=4, n_ff=0, vocab=128256,
                     n_expert=128, n_expert_used=8, n_ff_expert=768, rope_neox=1)


def _qw(pair, keep):
    if pair is None:
        return _lib.QWeight(0, None, 0)
    t, a = pair
    a = np.ascontiguousarray(a, dtype=np.uint8)
    keep.append(a)
    return _lib.QWeight(t, a.ctypes.data, a.size)


def _fp(a, keep):
    if a is None:
        return None
    a = np.ascontiguousarray(a, dtype=np.float32)
    keep.append(a)
    return a.ctypes.data


class Decoder:
    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg
        self._h = C.c_void_p()
        c = cfg.to_c()
        check(load().rnb_b200_decoder_create(C.byref(c), C.byref(self._h)))

    # -- weights --
    def load_description(self, desc: dict) -> None:
        """`desc`: {'layers': [{'attn_norm', 'ffn_norm', 'wq': (type, bytes), ...}], 'token_embd',
        'out_norm', 'output'} with full (unsharded) host arrays; row shards are cut here."""
        for i, ld in enumerate(desc["layers"]):
            keep = []
            w = _lib.LayerWeights()
            w.attn_norm, w.ffn_norm = _fp(ld["attn_norm"], keep), _fp(ld["ffn_norm"], keep)
            for k in ("wq", "wk", "wv", "wo", "gate", "up", "down", "gate_exps", "up_exps", "down_exps"):
                setattr(w, k, _qw(ld.get(k), keep))
            w.router = _fp(ld.get("router"), keep)
            check(load().rnb_b200_decoder_set_layer(self._h, i, C.byref(w)))
        keep = []
        check(load().rnb_b200_decoder_set_globals(self._h, _qw(desc["token_embd"], keep), _fp(desc["out_norm"], keep),
                                                  _qw(desc["output"], keep)))

    def set_exact_attention_max(self, max_positions: int) -> None:
        """Contexts up to `max_positions` use the reference-order attention kernel (bit-identical to
        the CPU's); 0 turns it off.  Only before the first step."""
        check(load().rnb_b200_decoder_set_exact_attention_max(self._h, int(max_positions)))

    def fill_synthetic(self, seed: int = 0, sigma: float = 0.02) -> None:
        check(load().rnb_b200_decoder_fill_synthetic(self._h, seed, sigma))

    def fill_kv_synthetic(self, n_pos: int, seed: int = 0) -> None:
        check(load().rnb_b200_decoder_fill_kv_synthetic(self._h, n_pos, seed))

    def attach_nccl(self, unique_id: bytes) -> None:
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        check(load().rnb_b200_decoder_attach_nccl(self._h, buf))

    # -- stepping --
    def exchange_handle(self) -> bytes:
        """CUDA IPC handle of this rank's exchange arena (64 bytes), to be all-gathered by the host."""
        buf = (C.c_uint8 * 64)()
        check(load().rnb_b200_decoder_exchange_handle(self._h, buf))
        return bytes(buf)

    def attach_peers(self, handles: list) -> None:
        """`handles`: every rank's exchange handle in rank order; switches the all-gathers to peer stores."""
        blob = b"".join(handles)
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        check(load().rnb_b200_decoder_attach_peers(self._h, buf))

    def prefill(self, tokens, pos0: int = 0, timed: bool = False):
        """Runs the prompt through the tensor-core prefill path, appends its K/V rows and returns the
        greedy next token (and the device milliseconds when `timed`)."""
        t = np.ascontiguousarray(np.asarray(tokens, dtype=np.uint32))
        nxt, ms = C.c_uint32(), C.c_float()
        check(load().rnb_b200_decoder_prefill(self._h, t.ctypes.data_as(C.c_void_p), int(t.size), int(pos0), C.byref(nxt),
                                              C.byref(ms) if timed else None))
        return (nxt.value, ms.value) if timed else nxt.value

    def read_logits(self) -> np.ndarray:
        out = np.empty(self.cfg.vocab // self.cfg.world_size, np.float32)
        check(load().rnb_b200_decoder_read_logits(self._h, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def step(self, token: int, pos: int, want_logits: bool = False):
        nxt = C.c_uint32()
        logits = np.empty(self.cfg.vocab, np.float32) if want_logits else None
        check(load().rnb_b200_decoder_step(self._h, int(token), int(pos), C.byref(nxt),
                                           None if logits is None else logits.ctypes.data_as(C.c_void_p)))
        return (nxt.value, logits) if want_logits else nxt.value

    def step_dev(self, pos: int = -1, chain: bool = True) -> None:
        check(load().rnb_b200_decoder_step_dev(self._h, pos, int(chain)))

    def sync(self) -> None:
        check(load().rnb_b200_decoder_sync(self._h))

    def time_steps(self, pos: int, steps: int) -> float:
        """Milliseconds (CUDA events) for `steps` chained device-resident steps from `pos`."""
        ms = C.c_float()
        check(load().rnb_b200_decoder_time_steps(self._h, pos, steps, C.byref(ms)))
        return ms.value

    def time_matvecs(self, iters: int = 1) -> dict:
        ms, b, n = C.c_float(), C.c_uint64(), C.c_uint64()
        check(load().rnb_b200_decoder_time_matvecs(self._h, iters, C.byref(ms), C.byref(b), C.byref(n)))
        return {"ms": ms.value, "bytes_per_iter": b.value, "launches_per_iter": n.value, "iters": iters}

    @property
    def stream(self) -> int:
        return load().rnb_b200_decoder_stream(self._h) or 0

    # -- inspection --
    def read_kv(self, layer: int, n_pos: int):
        kv_dim = self.cfg.n_kv_head // self.cfg.world_size * self.cfg.head_dim
        k = np.empty(n_pos * kv_dim, np.uint16)
        v = np.empty(n_pos * kv_dim, np.uint16)
        check(load().rnb_b200_decoder_read_kv(self._h, layer, n_pos, k.ctypes.data_as(C.c_void_p),
                                              v.ctypes.data_as(C.c_void_p)))
        return k, v

    def read_hidden(self) -> np.ndarray:
        h = np.empty(self.cfg.hidden, np.float32)
        check(load().rnb_b200_decoder_read_hidden(self._h, h.ctypes.data_as(C.c_void_p)))
        return h

    def read_expert_ids(self, layer: int) -> np.ndarray:
        ids = np.empty(self.cfg.n_expert_used, np.uint32)
        check(load().rnb_b200_decoder_read_expert_ids(self._h, layer, ids.ctypes.data_as(C.c_void_p)))
        return ids

    def stats(self) -> dict:
        a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint64()
        check(load().rnb_b200_decoder_stats(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return {"launches_per_step": a.value, "weight_bytes": b.value, "kv_bytes_per_pos": c.value}

    def close(self) -> None:
        if self._h:
            load().rnb_b200_decoder_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def nccl_unique_id() -> bytes:
    buf = (C.c_uint8 * 128)()
    check(load().rnb_b200_nccl_unique_id(buf))
    return bytes(buf)
