"""ctypes front end of the CPU oracle (``jq_oracle.c``).

Test infrastructure only: the test-suite, the smoke check and the CPU-baseline leg of the benchmark
import this module; the product package never does. ``build()`` compiles the C file with the
Makefile beside it when the shared object is missing or older than its source.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libjq_oracle.so")
_SRC = os.path.join(_HERE, "jq_oracle.c")

# ggml type ids (GgmlType.java:27-51 of the reference's jitnn-gguf module)
TYPES = {"Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14}

_lib = None


def build(force=False):
    stale = not os.path.exists(_SO) or (os.path.exists(_SRC) and os.path.getmtime(_SRC) > os.path.getmtime(_SO))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True, capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        c_i64, c_int, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.jqo_block_values.argtypes = [c_int]
        L.jqo_block_bytes.argtypes = [c_int]
        L.jqo_dequantize.argtypes = [c_int, vp, c_i64, vp]
        L.jqo_matvec.argtypes = [c_int, vp, vp, c_i64, c_i64, c_i64, vp, c_int]
        L.jqo_linear_q8_0.argtypes = [vp, vp, vp, c_i64, c_i64, c_i64, vp, c_int]
        L.jqo_linear.argtypes = [c_int, vp, vp, vp, c_i64, c_i64, c_i64, vp, c_int]
        L.jqo_quantize_q8_0.argtypes = [vp, c_i64, vp]
        L.jqo_half_to_float.argtypes = [ctypes.c_uint16]
        L.jqo_half_to_float.restype = ctypes.c_float
        L.jqo_float_to_half.argtypes = [ctypes.c_float]
        L.jqo_float_to_half.restype = ctypes.c_uint16
        _lib = L
    return _lib


def _type(t):
    return TYPES[t] if isinstance(t, str) else int(t)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def block_values(t):
    return lib().jqo_block_values(_type(t))


def block_bytes(t):
    return lib().jqo_block_bytes(_type(t))


def dequantize(t, blocks, count=None):
    """Blocks (uint8, any shape) of format ``t`` to a flat float32 array."""
    t = _type(t)
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    full = blocks.size // block_bytes(t) * block_values(t)
    count = full if count is None else count
    out = np.empty(count, dtype=np.float32)
    if lib().jqo_dequantize(t, _ptr(blocks), count, _ptr(out)) != 0:
        raise ValueError("unsupported type %d" % t)
    return out


def linear(t, blocks, x, bias=None, n=None, threads=1):
    """y = x W^T (+ bias) with the reference's host arithmetic; x [m, k] float32, returns [m, n]."""
    t = _type(t)
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    row_bytes = k // block_values(t) * block_bytes(t)
    n = blocks.size // row_bytes if n is None else n
    assert blocks.size == n * row_bytes, "block bytes do not match [n, k]"
    y = np.empty((m, n), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    rc = lib().jqo_linear(t, _ptr(blocks), _ptr(x), None if b is None else _ptr(b), m, n, k, _ptr(y), threads)
    if rc != 0:
        raise ValueError("jqo_linear failed")
    return y


def quantize_q8_0(x):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    out = np.empty(x.size // 32 * 34, dtype=np.uint8)
    if lib().jqo_quantize_q8_0(_ptr(x), x.size, _ptr(out)) != 0:
        raise ValueError("count must be a multiple of 32")
    return out


def max_threads():
    return lib().jqo_max_threads()
