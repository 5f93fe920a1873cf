"""The C-ABI library loads and exports every symbol the header declares (no GPU, no compute)."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT
import jitnn_b200
from jitnn_b200 import _lib
from jitnn_b200.build import build

HEADER = os.path.join(ROOT, "include", "jitnn_b200.h")


@pytest.fixture(scope="module")
def lib():
    build()
    return _lib.load()


def declared_symbols():
    text = open(HEADER).read()
    return re.findall(r"JQ_API\s+[\w\s\*]+?\b(jq_\w+)\s*\(", text)


def test_header_symbols_all_exported(lib):
    names = declared_symbols()
    assert len(names) >= 19
    assert set(names) == set(_lib.SIGNATURES), "binding table and header disagree"
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in names:
        assert hasattr(raw, name), name


def test_block_geometry_matches_reference_dtype(lib):
    # DType.java:75-98
    expect = {"Q8_0": (32, 34), "Q4_0": (32, 18), "Q4_1": (32, 20), "Q4_K": (256, 144), "Q5_K": (256, 176), "Q6_K": (256, 210),
              "Q5_0": (32, 22), "Q5_1": (32, 24), "Q2_K": (256, 84), "Q3_K": (256, 110)}
    for name, (qk, nb) in expect.items():
        t = jitnn_b200.DType[name]
        assert (lib.jq_block_values(t.value), lib.jq_block_bytes(t.value)) == (qk, nb)
        assert (t.blockValues(), t.blockBytes()) == (qk, nb)
    assert lib.jq_block_values(0) == 0 and lib.jq_block_bytes(15) == 0


def test_version_and_options(lib):
    assert lib.jq_version() >= 100
    v = ctypes.c_int64(-1)
    assert lib.jq_get_option(b"prefill_min_rows", ctypes.byref(v)) == 0 and v.value == 0
    assert lib.jq_set_option(b"no_such_option", 1) == _lib.JQ_ERR_INVALID
    assert "no_such_option" in _lib.last_error()


def test_shape_errors_are_reported_before_any_device_work(lib):
    """Tensor.persistent's checks (Tensor.java:266-276): block multiple and exact byte length."""
    with pytest.raises(ValueError, match="last axis not a multiple of its block of 256"):
        jitnn_b200.Tensor.quantized("Q4_K", np.zeros(144, np.uint8), 1, 255)
    with pytest.raises(ValueError, match="needs 288 bytes, got 144"):
        jitnn_b200.Tensor.quantized("Q4_K", np.zeros(144, np.uint8), 2, 256)
    with pytest.raises(ValueError, match="not a GGUF block format"):
        out = ctypes.c_void_p()
        _lib.check(lib.jq_weight_upload(0, 15, None, 0, 1, 256, 0, ctypes.byref(out)))
    with pytest.raises(ValueError, match="rank-2"):
        jitnn_b200.Tensor.quantized("Q8_0", np.zeros(34, np.uint8), 32)
    with pytest.raises(ValueError, match="multiple of 32"):
        jitnn_b200.Quant.quantizeQ8Blocks(np.zeros((2, 33), np.float32))
    assert lib.jq_weight_free(None) == 0
    bogus = (ctypes.c_int64 * 16)()
    assert lib.jq_weight_info(ctypes.addressof(bogus), (ctypes.c_int64 * 8)()) == _lib.JQ_ERR_INVALID


def test_no_silent_cpu_fallback_without_a_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(jitnn_b200.JitnnError):
        jitnn_b200.Tensor.quantized("Q4_K", np.zeros(144, np.uint8), 1, 256)
