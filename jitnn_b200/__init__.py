"""jitnn_b200: the B200 (sm_100a) quantised linear operator for GGUF block formats.

The compute lives in ``libjitnn_b200.so`` (CUDA, C ABI in ``include/jitnn_b200.h``); this package is
the thin host-side mirror of the reference's operator interface plus the build helper.
"""
from ._lib import JitnnError, load  # noqa: F401
from .decoder import LlamaDecoder  # noqa: F401
from .ops import DType, F, Gguf, Quant, Tensor, device_status  # noqa: F401

__all__ = ["DType", "F", "Gguf", "Quant", "Tensor", "JitnnError", "load", "device_status", "LlamaDecoder"]
