import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")

# formats on the hot path, and the extra formats of the dequantiser
LINEAR_TYPES = ["Q8_0", "Q4_0", "Q4_1", "Q4_K", "Q5_K", "Q6_K"]
EXTRA_TYPES = ["Q5_0", "Q5_1", "Q2_K", "Q3_K"]
GOLDEN_FORMATS = ["q4_0", "q4_1", "q4_k", "q5_k", "q6_k"]  # format codes 0..4 of the golden cases


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 machine)")


@pytest.fixture(scope="session")
def fixture_gguf():
    return np.load(os.path.join(GOLDEN, "gguf_fixture.npz"))


@pytest.fixture(scope="session")
def golden_cases():
    return np.load(os.path.join(GOLDEN, "golden_gguf_cases.npz"))


def close_like_reference(expect, actual, what=""):
    """GgufChecks.close of the reference's tests: |diff| <= 2e-4 * max|expect|."""
    expect = np.asarray(expect, dtype=np.float32).reshape(-1)
    actual = np.asarray(actual, dtype=np.float32).reshape(-1)
    assert expect.shape == actual.shape, what + ": length"
    scale = max(1e-6, float(np.abs(expect).max()))
    diff = np.abs(expect - actual)
    bad = int(np.argmax(diff))
    assert diff[bad] <= 2e-4 * scale, "%s[%d]: expected %r, got %r" % (what, bad, expect[bad], actual[bad])


def golden_close(expect, actual, rtol=1e-4, atol=1e-3, what=""):
    """Golden.java's comparison for the gguf cases: |diff| <= atol + rtol * |expect|."""
    expect = np.asarray(expect, dtype=np.float64).reshape(-1)
    actual = np.asarray(actual, dtype=np.float64).reshape(-1)
    diff = np.abs(expect - actual)
    lim = atol + rtol * np.abs(expect)
    bad = int(np.argmax(diff - lim))
    assert diff[bad] <= lim[bad], "%s[%d]: expected %r, got %r" % (what, bad, expect[bad], actual[bad])
