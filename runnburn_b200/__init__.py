"""B200-native batch-1 decode/prefill operator set (runNburn `rnb-backend-cuda` drop-in path).

`runnburn_b200.ops` mirrors the reference's operator functions over the C ABI in
`include/rnb_b200.h`; `runnburn_b200.Decoder` is the device-resident token loop.
"""
from ._lib import (TYPE_Q4_K, TYPE_Q6_K, TYPE_Q8_0, RnbError, load)  # noqa: F401
from . import ops  # noqa: F401
from .decoder import Decoder, ModelConfig  # noqa: F401

__all__ = ["ops", "Decoder", "ModelConfig", "RnbError", "load", "TYPE_Q4_K", "TYPE_Q6_K", "TYPE_Q8_0"]
