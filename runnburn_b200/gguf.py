"""GGUF files over the C ABI (`rnb_b200_gguf_*`): the container reader and the decoder loader.

Mirrors crates/rnb-loader/src/gguf/parser.rs (GGUFFile::parse), arch/mod.rs (metadata
extraction) and arch/llama.rs (tensor names) of the reference.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, load
from .decoder import Decoder, ModelConfig


class GgufFile:
    """A parsed GGUF container.  `path` is mapped read-only; `data` (bytes-like) is parsed in place
    and kept alive by this object."""

    def __init__(self, path: str | None = None, data=None):
        self._h = C.c_void_p()
        self._keep = None
        L = load()
        if path is not None:
            check(L.rnb_b200_gguf_open(str(path).encode(), C.byref(self._h)))
        else:
            buf = np.frombuffer(data, dtype=np.uint8)
            self._keep = buf
            check(L.rnb_b200_gguf_parse(buf.ctypes.data, buf.size, C.byref(self._h)))

    def close(self):
        if self._h:
            load().rnb_b200_gguf_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def info(self) -> dict:
        v, a, d, t, m = C.c_uint32(), C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_uint64()
        check(load().rnb_b200_gguf_info(self._h, C.byref(v), C.byref(a), C.byref(d), C.byref(t), C.byref(m)))
        return dict(version=v.value, alignment=a.value, data_start=d.value, n_tensors=t.value, n_metadata=m.value)

    def get_int(self, key: str) -> int:
        v = C.c_uint64()
        check(load().rnb_b200_gguf_get_u64(self._h, key.encode(), C.byref(v)))
        return v.value

    def get_float(self, key: str) -> float:
        v = C.c_double()
        check(load().rnb_b200_gguf_get_f64(self._h, key.encode(), C.byref(v)))
        return v.value

    def get_str(self, key: str) -> str:
        n = C.c_size_t()
        check(load().rnb_b200_gguf_get_str(self._h, key.encode(), None, 0, C.byref(n)))
        buf = C.create_string_buffer(n.value + 1)
        check(load().rnb_b200_gguf_get_str(self._h, key.encode(), buf, n.value + 1, None))
        return buf.value.decode()

    def get_int_array(self, key: str) -> list[int]:
        n = C.c_size_t()
        check(load().rnb_b200_gguf_get_array_u64(self._h, key.encode(), None, 0, C.byref(n)))
        out = (C.c_uint64 * max(n.value, 1))()
        check(load().rnb_b200_gguf_get_array_u64(self._h, key.encode(), out, n.value, None))
        return list(out)[:n.value]

    def _tensor_dict(self, ti: _lib.GgufTensorInfo) -> dict:
        return dict(name=ti.name.decode(), shape=[int(ti.dims[i]) for i in range(ti.n_dims)], ggml_type=int(ti.ggml_type),
                    offset=int(ti.offset), n_elements=int(ti.n_elements), n_bytes=int(ti.n_bytes), data=ti.data)

    def tensor(self, name: str) -> dict:
        ti = _lib.GgufTensorInfo()
        check(load().rnb_b200_gguf_tensor(self._h, name.encode(), C.byref(ti)))
        return self._tensor_dict(ti)

    def tensors(self) -> list[dict]:
        out = []
        for i in range(self.info()["n_tensors"]):
            ti = _lib.GgufTensorInfo()
            check(load().rnb_b200_gguf_tensor_at(self._h, i, C.byref(ti)))
            out.append(self._tensor_dict(ti))
        return out

    def tensor_bytes(self, name: str) -> np.ndarray:
        """A copy of the tensor's bytes (tests; the loader itself never copies on the host)."""
        t = self.tensor(name)
        return np.ctypeslib.as_array((C.c_uint8 * t["n_bytes"]).from_address(t["data"])).copy()

    def model_config(self, max_ctx: int = 0) -> ModelConfig:
        c = _lib.ModelCfg()
        check(load().rnb_b200_gguf_model_config(self._h, max_ctx, C.byref(c)))
        return ModelConfig(**{n: getattr(c, n) for n, _ in c._fields_})


def load_decoder(path: str, max_ctx: int = 0, register_pages: bool = True) -> tuple[Decoder, GgufFile]:
    """Opens a Llama-style GGUF, creates the decoder its metadata describes and uploads the weights
    from the mapped pages.  Keep the returned file object alive as long as the decoder is loading."""
    f = GgufFile(path)
    dec = Decoder(f.model_config(max_ctx))
    check(load().rnb_b200_decoder_load_gguf(dec._h, f._h, 1 if register_pages else 0))
    return dec, f
