"""The allocation-free decode-attention entry point against the regular one.

Some callers of the library may not allocate device memory once they are running (a plug-in
in a server with a frozen pool, a sandbox that aborts on late allocations, a real-time loop).
For them `rnb_b200_attention_decode_hd128_noalloc` keeps the split-KV scratch in a fixed array
inside the library.  This test drives it through the C ABI with caller-owned device buffers,
twice in a row on the same array, and compares with `attention_decode_hd128`.  The file name
sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest

import oracle as orc
from synth import max_rel_err

pytestmark = pytest.mark.gpu

TOL = 1e-3  # the attention tolerance of tests/test_gpu_ops.py


def test_noalloc_attention_matches_regular_entry_point_twice():
    import torch

    import runnburn_b200 as r
    from runnburn_b200 import build, ops
    build.build_library()
    L = r.load()
    ops.open()
    rng = np.random.default_rng(77)
    heads, kvh = 32, 8
    scale = 1.0 / np.sqrt(128.0)
    out_dev = torch.empty(heads * 128, dtype=torch.float32, device="cuda")
    for call, kv_len in enumerate((4096, 333)):      # long first, then short: stale records must not leak
        q = rng.standard_normal(heads * 128).astype(np.float32)
        k = orc.f32_to_f16_bits(rng.standard_normal(kv_len * kvh * 128))
        v = orc.f32_to_f16_bits(rng.standard_normal(kv_len * kvh * 128))
        want = ops.attention_decode_hd128(q, k, v, kv_len, heads, kvh, scale)
        q_dev = torch.from_numpy(q).cuda()
        k_dev = torch.from_numpy(k.view(np.int16)).cuda()
        v_dev = torch.from_numpy(v.view(np.int16)).cuda()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        stream = torch.cuda.current_stream().cuda_stream
        rc = L.rnb_b200_attention_decode_hd128_noalloc(q_dev.data_ptr(), k_dev.data_ptr(), v_dev.data_ptr(), kv_len, heads, kvh,
                                                       scale, out_dev.data_ptr(), C.c_void_p(stream))
        assert rc == 0, L.rnb_b200_last_error()
        torch.cuda.synchronize()
        if call > 0:                                  # the first call may load the module lazily
            assert torch.cuda.mem_get_info()[0] == free_before
        got = out_dev.cpu().numpy()
        assert max_rel_err(got, want) <= TOL
        assert max_rel_err(got, orc.attention_decode(q, k, v, heads, kvh, 128, kv_len, scale)) <= TOL
    # sizes beyond the fixed array are rejected with a clear message, before any launch
    rc = L.rnb_b200_attention_decode_hd128_noalloc(q_dev.data_ptr(), k_dev.data_ptr(), v_dev.data_ptr(), 16, 128, 8, scale,
                                                   out_dev.data_ptr(), None)
    assert rc == 2 and b"at most 64 query heads" in L.rnb_b200_last_error()
    # a pointer the kernels' vector loads could not take is refused too, not left to fault
    rc = L.rnb_b200_attention_decode_hd128_noalloc(q_dev.data_ptr() + 4, k_dev.data_ptr(), v_dev.data_ptr(), 16, heads, kvh, scale,
                                                   out_dev.data_ptr(), None)
    assert rc == 2 and b"not aligned" in L.rnb_b200_last_error()
    # the entry point reports its kernels' bounded waits through its own fixed status word
    status = C.c_int(-1)
    assert L.rnb_b200_attention_decode_hd128_noalloc_status(C.byref(status), C.c_void_p(stream)) == 0
    assert status.value == 0
    assert ops.dev_error_flag() == 0
