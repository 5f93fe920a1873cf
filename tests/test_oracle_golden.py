"""Pins the CPU oracle to the reference's own test vectors (no GPU needed).

Mirrors GgufChecks.check (jitnn-gguf tests) and the gguf_* golden cases (jitnn-core tests).
"""
import numpy as np
import pytest

from conftest import EXTRA_TYPES, GOLDEN_FORMATS, LINEAR_TYPES, close_like_reference, golden_close
from oracle import oracle

CODE_TO_TYPE = {0: "Q4_0", 1: "Q4_1", 2: "Q4_K", 3: "Q5_K", 4: "Q6_K"}


@pytest.mark.parametrize("t", LINEAR_TYPES + EXTRA_TYPES)
def test_fixture_dequantize_bit_exact(fixture_gguf, t):
    got = oracle.dequantize(t, fixture_gguf["w." + t])
    expect = fixture_gguf["expect." + t].reshape(-1)
    assert got.view(np.uint32).tolist() == expect.view(np.uint32).tolist()


@pytest.mark.parametrize("fmt", GOLDEN_FORMATS)
def test_golden_dequantize_bit_exact(golden_cases, fmt):
    name = "gguf_dequant_" + fmt
    code, rows = golden_cases[name + ".attrs"]
    got = oracle.dequantize(CODE_TO_TYPE[int(code)], golden_cases[name + ".in0"])
    expect = golden_cases[name + ".out"].reshape(-1)
    assert rows == 3
    assert np.array_equal(got.view(np.uint32), expect.view(np.uint32))


@pytest.mark.parametrize("rows", [1, 5, 40])
@pytest.mark.parametrize("fmt", GOLDEN_FORMATS)
def test_golden_linear(golden_cases, fmt, rows):
    name = "gguf_linear_%s_r%d" % (fmt, rows)
    code, n = golden_cases[name + ".attrs"]
    x = golden_cases[name + ".in0"]
    y = oracle.linear(CODE_TO_TYPE[int(code)], golden_cases[name + ".in1"], x, golden_cases[name + ".in2"], n=int(n))
    golden_close(golden_cases[name + ".out"], y, what=name)


@pytest.mark.parametrize("rows", [1, 5, 40])
@pytest.mark.parametrize("fmt", GOLDEN_FORMATS)
def test_golden_linear_gradients(golden_cases, fmt, rows):
    """The golden cases differentiate sum(w * out): grad0 = w . dequant(W) (the operator's input gradient,
    ops/Gguf.java:208-212) and grad2 = the column sums of w (the bias gradient); there is no weight gradient."""
    name = "gguf_linear_%s_r%d" % (fmt, rows)
    code, n = golden_cases[name + ".attrs"]
    W = oracle.dequantize(CODE_TO_TYPE[int(code)], golden_cases[name + ".in1"]).reshape(int(n), 512).astype(np.float64)
    g = golden_cases[name + ".w"].astype(np.float64)
    golden_close(golden_cases[name + ".grad0"], g @ W, what=name + ".grad0")
    golden_close(golden_cases[name + ".grad2"], g.sum(axis=0), what=name + ".grad2")
    assert name + ".grad1" not in golden_cases


@pytest.mark.parametrize("t", LINEAR_TYPES)
def test_fixture_linear_like_gguf_checks(fixture_gguf, t):
    """y = x W^T + b for 1, 5 and 40 rows against a double-precision product with expect.<T>."""
    rng = np.random.default_rng(abs(hash(t)) % (2 ** 31))
    expect = fixture_gguf["expect." + t].astype(np.float64)
    bias = np.array([0.25, -0.5, 1.0], dtype=np.float32)
    for rows in (1, 5, 40):
        x = (rng.random((rows, 512), dtype=np.float32) * 2 - 1).astype(np.float32)
        ref = (bias.astype(np.float64) + x.astype(np.float64) @ expect.T).astype(np.float32)
        y = oracle.linear(t, fixture_gguf["w." + t], x, bias)
        close_like_reference(ref, y, "%s linear, %d rows" % (t, rows))


def test_threads_do_not_change_results(fixture_gguf):
    x = np.random.default_rng(3).standard_normal((4, 512)).astype(np.float32)
    a = oracle.linear("Q4_K", fixture_gguf["w.Q4_K"], x, threads=1)
    b = oracle.linear("Q4_K", fixture_gguf["w.Q4_K"], x, threads=4)
    assert np.array_equal(a, b)


def test_half_conversions_round_trip():
    L = oracle.lib()
    for h in range(0, 0x7c00):  # every finite non-negative half
        f = L.jqo_half_to_float(h)
        assert L.jqo_float_to_half(f) == h
        assert np.float32(f) == np.array([h], dtype=np.uint16).view(np.float16)[0].astype(np.float32)
    vals = np.random.default_rng(5).uniform(-70000, 70000, 2000).astype(np.float32)
    vals = np.concatenate([vals, np.random.default_rng(6).uniform(-1e-4, 1e-4, 2000).astype(np.float32)])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([L.jqo_float_to_half(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(want, got)


def test_quantize_q8_0_matches_procedure():
    """OpsAccelTest.q8: round trip within one quantisation step; zero blocks give d = 0, q = 0."""
    rng = np.random.default_rng(41)
    x = rng.uniform(-1, 1, (6, 256)).astype(np.float32)
    x[2, 32:64] = 0
    q = oracle.quantize_q8_0(x)
    back = oracle.dequantize("Q8_0", q).reshape(6, 256)
    assert np.abs(back - x).max() <= 1.0 / 127 + 1e-6
    assert not q[(2 * 8 + 1) * 34:(2 * 8 + 2) * 34].any()
    # the stored scale is half(max|x| / 127) and every q is within [-127, 127]
    blocks = q.reshape(-1, 34)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32).reshape(-1)
    amax = np.abs(x.reshape(-1, 32)).max(axis=1)
    assert np.array_equal(d, (amax.astype(np.float64) / 127.0).astype(np.float32).astype(np.float16).astype(np.float32))
    assert blocks[:, 2:].view(np.int8).min() >= -127
