"""The GGUF container reader against files written by the third-party `gguf` package and against
hand-built byte strings for the error paths the reference's parser tests cover
(crates/rnb-loader/src/gguf/parser.rs: magic, versions, big-endian detection, counts that cannot
fit, duplicate keys, alignment rule, tensor-name and dimension limits).  No GPU involved."""
import struct

import numpy as np
import pytest

from synth import llama_description
from gguf_util import write_llama_gguf


@pytest.fixture(scope="module")
def r():
    from runnburn_b200 import build
    build.build_library()
    import runnburn_b200
    runnburn_b200.load()
    return runnburn_b200


def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def _header(version=3, n_tensors=0, n_kv=0, magic=b"GGUF") -> bytes:
    return magic + struct.pack("<I", version) + struct.pack("<QQ", n_tensors, n_kv)


def _kv_u32(key: bytes, v: int) -> bytes:
    return _s(key) + struct.pack("<I", 4) + struct.pack("<I", v)


def _tensor(name: bytes, dims, type_id: int, offset: int) -> bytes:
    return _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", type_id, offset)


def test_reads_a_file_written_by_the_gguf_package(r, tmp_path):
    from runnburn_b200.gguf import GgufFile
    desc = llama_description(seed=4, n_layer=2, hidden=256, n_head=2, n_kv_head=1, n_ff=512, vocab=512)
    path = tmp_path / "tiny.gguf"
    write_llama_gguf(path, desc, context_length=128)
    f = GgufFile(str(path))
    info = f.info()
    assert info["version"] == 3 and info["alignment"] == 32 and info["n_tensors"] == 3 + 2 * 9
    assert info["data_start"] % 32 == 0
    assert f.get_str("general.architecture") == "llama"
    assert f.get_int("llama.block_count") == 2 and f.get_int("llama.attention.head_count_kv") == 1
    assert abs(f.get_float("llama.rope.freq_base") - 5e5) < 1e-3
    with pytest.raises(r.RnbError) as e:
        f.get_int("llama.no_such_key")
    assert e.value.status == 1 and "missing GGUF metadata key" in str(e.value)
    with pytest.raises(r.RnbError) as e:
        f.get_int("general.architecture")
    assert e.value.status == 2
    cfg = f.model_config()
    want = desc["cfg"]
    for k in ("n_layer", "hidden", "n_head", "n_kv_head", "head_dim", "n_ff", "vocab", "rope_neox", "n_expert"):
        assert getattr(cfg, k) == want[k], k
    assert cfg.max_ctx == 128 and abs(cfg.rms_eps - 1e-5) < 1e-12 and cfg.rope_theta == 5e5
    assert f.model_config(max_ctx=64).max_ctx == 64
    # shapes come back outermost first; bytes are the writer's bytes
    t = f.tensor("blk.1.ffn_down.weight")
    assert t["shape"] == [256, 512] and t["ggml_type"] == 14 and t["n_bytes"] == 256 * 2 * 210 and t["offset"] % 32 == 0
    assert np.array_equal(f.tensor_bytes("blk.1.ffn_down.weight"), desc["layers"][1]["down"][1])
    assert np.array_equal(f.tensor_bytes("token_embd.weight"), desc["token_embd"][1])
    assert np.array_equal(f.tensor_bytes("blk.0.attn_norm.weight").view(np.float32), desc["layers"][0]["attn_norm"])
    names = [t["name"] for t in f.tensors()]
    assert names[0] == "token_embd.weight" and "output.weight" in names and len(set(names)) == len(names)
    with pytest.raises(r.RnbError) as e:
        f.tensor("blk.9.attn_q.weight")
    assert e.value.status == 1
    f.close()


def test_parser_error_paths(r):
    from runnburn_b200.gguf import GgufFile

    def err(data: bytes):
        with pytest.raises(r.RnbError) as e:
            GgufFile(data=data)
        return e.value.status, str(e.value)

    assert err(_header(magic=b"GGML") + b"\0" * 8) == (2, "invalid GGUF magic")
    st, msg = err(_header(version=1))
    assert st == 1 and msg == "unsupported GGUF version 1"
    st, msg = err(b"GGUF" + struct.pack(">I", 3) + struct.pack(">QQ", 0, 0))
    assert st == 1 and "big-endian GGUF is not supported" in msg
    st, msg = err(b"GGUF" + struct.pack("<I", 3) + b"\x01\x00")
    assert st == 2 and "need 8 bytes, only 2 remain" in msg
    st, msg = err(_header(n_tensors=1 << 40, n_kv=5))
    assert st == 2 and "cannot fit in 0 remaining bytes" in msg
    st, msg = err(_header(n_kv=2) + _kv_u32(b"a.b", 1) + _kv_u32(b"a.b", 2))
    assert st == 2 and "duplicate metadata key 'a.b'" in msg
    st, msg = err(_header(n_kv=1) + _s(b"") + struct.pack("<II", 4, 1) + b"\0" * 16)
    assert st == 2 and "metadata key must be non-empty ASCII" in msg
    st, msg = err(_header(n_kv=1) + _s(b"k") + struct.pack("<I", 13) + b"\0" * 16)
    assert st == 2 and "unknown GGUF value type: 13" in msg
    st, msg = err(_header(n_kv=1) + _s(b"flag") + struct.pack("<I", 7) + b"\x02" + b"\0" * 16)
    assert st == 2 and "invalid GGUF boolean value 2" in msg
    st, msg = err(_header(n_kv=1) + _kv_u32(b"general.alignment", 24) + b"\0" * 8)
    assert st == 2 and "general.alignment 24 must be a positive power of two" in msg
    st, msg = err(_header(n_tensors=1) + _tensor(b"t", [4], 0, 8))
    assert st == 2 and "tensor 't' offset 8 is not aligned to 32 bytes" in msg
    st, msg = err(_header(n_tensors=1) + _tensor(b"x" * 64, [4], 0, 0))
    assert st == 2 and "tensor name is 64 bytes; GGML requires fewer than 64" in msg
    st, msg = err(_header(n_tensors=1) + _tensor(b"t", [1, 1, 1, 1, 1], 0, 0))
    assert st == 2 and "has 5 dimensions; GGUF supports at most 4" in msg
    st, msg = err(_header(n_tensors=1) + _tensor(b"t", [4], 99, 0))
    assert st == 1 and "unsupported GGML type 99" in msg
    st, msg = err(_header(n_tensors=2) + _tensor(b"t", [4], 0, 0) + _tensor(b"t", [4], 0, 32))
    assert st == 2 and "duplicate tensor name 't'" in msg


def test_alignment_key_and_version_2(r):
    """`general.alignment` moves the data section; dims are stored innermost first; version 2 parses."""
    from runnburn_b200.gguf import GgufFile
    head = _header(version=2, n_tensors=1, n_kv=2) + _kv_u32(b"general.alignment", 64) + \
        _s(b"general.architecture") + struct.pack("<I", 8) + _s(b"llama") + _tensor(b"w", [8, 3], 0, 64)
    pad = (-len(head)) % 64
    payload = np.arange(64 + 24 * 4, dtype=np.uint8).tobytes()
    f = GgufFile(data=head + b"\0" * pad + payload)
    info = f.info()
    assert info == dict(version=2, alignment=64, data_start=len(head) + pad, n_tensors=1, n_metadata=2)
    t = f.tensor("w")
    assert t["shape"] == [3, 8] and t["n_elements"] == 24 and t["n_bytes"] == 96 and t["offset"] == 64
    assert f.tensor_bytes("w").tobytes() == payload[64:64 + 96]
    # a tensor that would run past the end of the buffer is refused when it is asked for
    g = GgufFile(data=head + b"\0" * pad + payload[:100])
    with pytest.raises(r.RnbError) as e:
        g.tensor("w")
    assert e.value.status == 2 and "extends beyond the file" in str(e.value)
