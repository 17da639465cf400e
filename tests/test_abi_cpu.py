"""CPU-side checks of the drop-in boundary: the library loads, exports every symbol the
header declares, validates shapes with the reference's messages before touching CUDA, and
fails loudly (no fallback) when no GPU is present.  No compute runs here."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from runnburn_b200 import build
    build.build_library()
    import runnburn_b200
    return runnburn_b200.load()


def test_library_exports_every_declared_symbol(lib):
    header = (ROOT / "include" / "rnb_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = sorted(set(re.findall(r"\b(rnb_b200_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) >= 50
    exported = subprocess.run(["nm", "-D", "--defined-only", str(ROOT / "runnburn_b200" / "librnb_b200.so")],
                              capture_output=True, text=True, check=True).stdout
    have = set(re.findall(r" T (rnb_b200_[a-z0-9_]+)", exported))
    missing = [s for s in declared if s not in have]
    assert not missing, f"declared in include/rnb_b200.h but not exported: {missing}"
    for s in declared:
        assert hasattr(lib, s)


def test_library_does_not_link_the_oracle(lib):
    deps = subprocess.run(["ldd", str(ROOT / "runnburn_b200" / "librnb_b200.so")], capture_output=True, text=True).stdout
    assert "oracle" not in deps
    for f in (ROOT / "runnburn_b200").rglob("*"):
        if f.suffix in (".py", ".cu", ".cuh", ".hpp", ".inc"):
            text = f.read_text()
            assert "import oracle" not in text and "rnb_oracle" not in text, f


def test_shape_errors_use_the_reference_messages(lib):
    import runnburn_b200 as r
    from runnburn_b200 import ops
    z = np.zeros
    cases = [
        (lambda: ops.q4k_gemv(z(144, np.uint8), 1, 255, z(255, np.float32)), "Q4_K cols must be divisible by 256, got 255"),
        (lambda: ops.q4k_gemv(z(100, np.uint8), 1, 256, z(256, np.float32)), "Q4_K weight byte mismatch: got 100, expected 144"),
        (lambda: ops.q4k_gemv(z(144, np.uint8), 1, 256, z(128, np.float32)), "Q4_K input length mismatch: got 128, expected 256"),
        (lambda: ops.q6k_gemv(z(209, np.uint8), 1, 256, z(256, np.float32)), "Q6_K weight byte mismatch: got 209, expected 210"),
        (lambda: ops.q8_0_gemv(z(34, np.uint8), 1, 33, z(33, np.float32)), "Q8_0 cols must be divisible by 32, got 33"),
        (lambda: ops.moe_route_topk_f32(z(7, np.float32), None, 1, 8, 2), "CUDA MoE route logits mismatch: got=7 expected=8"),
        (lambda: ops.moe_route_topk_f32(z(8, np.float32), None, 1, 8, 9), "invalid CUDA MoE route shape: seq_len=1 n_expert=8 top_k=9"),
        (lambda: ops.attention_decode_hd128(z(256, np.float32), z(128, np.uint16), z(128, np.uint16), 1, 3, 2, 1.0),
         "attention: num_heads(3) must be a multiple of num_kv_heads(2)"),
    ]
    for call, msg in cases:
        with pytest.raises(r.RnbError) as e:
            call()
        assert e.value.status == 2 and str(e.value) == msg


def test_residency_budget_rule(lib):
    """DeviceResidencyPlan / default_device_dynamic_reserve_bytes
    (crates/rnb-memory/src/device_residency.rs:40-96)."""
    from runnburn_b200 import ops
    MiB, GiB = 1 << 20, 1 << 30
    assert ops.resident_limit_for(24 * GiB, 23 * GiB) == 23 * GiB - 1536 * MiB    # 24/16 = 1.5 GiB
    assert ops.resident_limit_for(4 * GiB, 4 * GiB) == 4 * GiB - 512 * MiB         # floor 512 MiB
    assert ops.resident_limit_for(192 * GiB, 180 * GiB) == 178 * GiB               # cap 2 GiB
    assert ops.resident_limit_for(8 * GiB, 256 * MiB) == 0                         # saturating
    assert ops.resident_limit_for(17 * GiB, 17 * GiB) == 17 * GiB - 1280 * MiB     # 1.0625 GiB -> 1.25 GiB


def test_expert_bundle_admission_rule(lib):
    """admit iff missing*(reuses + [replaces temp upload]) > missing + eviction_reload, strictly
    (crates/rnb-memory/src/sparse_expert_cache.rs:221-245)."""
    from runnburn_b200 import ops
    adm = ops.evaluate_expert_bundle_admission
    assert not adm(100, 0, 1, False)      # 100 > 100 is false: strict
    assert adm(100, 0, 2, False)
    assert adm(100, 0, 1, True)           # the current lookup's temp upload counts as one reuse
    assert not adm(100, 100, 1, True)     # 200 > 200 false
    assert adm(100, 99, 1, True)
    assert not adm(0, 0, 10, True)        # nothing missing: nothing to admit
    assert adm(2 ** 63, 2 ** 63, 4, False)  # 128-bit arithmetic, no wrap


def test_compute_fails_loudly_without_a_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import runnburn_b200 as r
    from runnburn_b200 import ops
    with pytest.raises(r.RnbError) as e:
        ops.q4k_gemv(np.zeros(144, np.uint8), 1, 256, np.zeros(256, np.float32))
    assert e.value.status == 4 and "no CPU fallback" in str(e.value)
    with pytest.raises(r.RnbError):
        r.Decoder(r.ModelConfig(n_layer=1, hidden=256, n_head=2, n_kv_head=1, n_ff=256, vocab=32, max_ctx=8))


def test_split_kv_chunk_rule(lib):
    """Chunks per KV head of the split-KV decode attention (148 SMs assumed without a device):
    4 CTAs per SM spread over the KV heads, at most one chunk per 32 positions, and with four or
    more KV heads at most max(74, kv_len / 128) so that the merge stays short."""
    f = lib.rnb_b200_flash_decode_default_chunks
    assert f(4096, 8) == 74          # Llama-3-8B, ctx 4096
    assert f(8192, 4) == 74          # 4-KV-head MoE shape, ctx 8192 (148 without the cap)
    assert f(32768, 4) == 148        # 70B two-GPU shard: long chunks keep the full count
    assert f(32768, 1) == 592        # one KV head per GPU: no cap
    assert f(100, 8) == 4            # short cache: one chunk per 32 positions
    assert f(0, 8) == 1


def test_device_pointer_attention_rejects_bad_arguments_before_any_launch(lib):
    """rnb_b200_dev_flash_decode and the allocation-free entry point validate chunk count,
    cache length, null pointers and pointer alignment on the host: an out-of-range chunk count
    would index past the merge kernel's shared array, a misaligned pointer would fault on the
    device.  No GPU is needed to be refused."""
    f = lib.rnb_b200_dev_flash_decode
    err = lambda: lib.rnb_b200_last_error().decode()
    big = 1 << 40
    q, k, v, part, out = 0x10000, 0x20000, 0x30000, 0x40000, 0x50000   # never dereferenced: every call is refused
    assert f(q, k, v, 128, 32, 8, 0.1, part, big, 1025, out, None) == 2 and "n_chunks must be in 1..1024" in err()
    assert f(q, k, v, 128, 32, 8, 0.1, part, big, 0, out, None) == 2
    assert f(q, k, v, 0, 32, 8, 0.1, part, big, 4, out, None) == 2 and "kv_len" in err()
    assert f(q, k, v, 1 << 31, 32, 8, 0.1, part, big, 4, out, None) == 2 and "kv_len" in err()
    assert f(None, k, v, 128, 32, 8, 0.1, part, big, 4, out, None) == 2 and "null pointer" in err()
    assert f(q, k, v, 128, 32, 8, 0.1, None, big, 4, out, None) == 2 and "null pointer" in err()
    assert f(q + 4, k, v, 128, 32, 8, 0.1, part, big, 4, out, None) == 2 and "not aligned" in err()
    assert f(q, k + 2, v, 128, 32, 8, 0.1, part, big, 4, out, None) == 2 and "not aligned" in err()
    assert f(q, k, v + 4, 128, 32, 8, 0.1, part, big, 4, out, None) == 2 and "not aligned" in err()
    assert f(q, k, v, 128, 32, 8, 0.1, part, big, 4, out + 2, None) == 2 and "not aligned" in err()
    assert f(q, k, v, 128, 32, 8, 0.1, part, 16, 4, out, None) == 2 and "scratch too small" in err()
    assert f(q, k, v, 128, 33, 8, 0.1, part, big, 4, out, None) == 2 and "multiple of num_kv_heads" in err()
    g = lib.rnb_b200_attention_decode_hd128_noalloc
    assert g(q + 8, k, v, 128, 32, 8, 0.1, out, None) == 2 and "not aligned" in err()
    assert g(q, k + 4, v, 128, 32, 8, 0.1, out, None) == 2 and "not aligned" in err()
    assert g(q, k, v, 0, 32, 8, 0.1, out, None) == 2 and "kv_len" in err()
    assert g(q, k, v, 128, 65, 1, 0.1, out, None) == 2 and "at most 64 query heads" in err()
    assert g(None, k, v, 128, 32, 8, 0.1, out, None) == 2 and "null pointer" in err()


def test_static_archive_defines_every_declared_symbol_and_links_into_a_c_program(tmp_path):
    """The form a Rust build.rs links: `nvcc -lib` archive + the CUDA runtime.  A plain C program that
    binds the header links against it and runs (it only asks for the last error string: no GPU needed)."""
    from runnburn_b200 import build
    archive = build.build_static_library()
    header = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / "rnb_b200.h").read_text(), flags=re.S)
    declared = sorted(set(re.findall(r"\b(rnb_b200_[a-z0-9_]+)\s*\(", header)))
    have = set(re.findall(r" T (rnb_b200_[a-z0-9_]+)", subprocess.run(["nm", "-g", "--defined-only", str(archive)], capture_output=True, text=True,
                                                                       check=True).stdout))
    missing = [s for s in declared if s not in have]
    assert not missing, f"declared but not defined in the archive: {missing}"
    src = tmp_path / "main.c"
    src.write_text('#include <stdio.h>\n#include "rnb_b200.h"\nint main(void) { const char *e = rnb_b200_last_error(); '
                   'int rc = rnb_b200_q4k_gemv(0, 0, 3, 100, 0, 0, 0, 0); printf("%d|%s|%s\\n", rc, e ? "ok" : "null", rnb_b200_last_error()); return 0; }\n')
    exe = tmp_path / "main"
    cuda_lib = "/usr/local/cuda/lib64"
    r = subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), str(archive), "-L", cuda_lib, "-Wl,-rpath," + cuda_lib, "-lcudart", "-ldl",
                        "-lstdc++", "-lm", "-lpthread", "-lrt", "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr[-2000:]
    rc, first, msg = out.stdout.strip().split("|", 2)
    assert int(rc) != 0 and "256" in msg          # the reference's shape message: cols must be divisible by 256
