"""The arithmetic of the tcgen05 decode GEMV (jitnn_b200/csrc/jq_gemv_umma.cu, jq_umma_image.cuh) restated in numpy and
checked against the CPU oracle (ops/Gguf.java:187-205 semantics): the claims the kernel rests on are facts about numbers,
which a machine without a GPU can check.

  * a Q4_K / Q5_K quant times its 6-bit scale is an integer below 2048, so half precision holds it exactly, and the
    one-instruction forms the unpack uses give exactly that integer: (1024 + q) sc - 1024 sc, and for Q4_K's high nibbles
    left in place (1024 + 16 q) (sc / 16) - 64 sc;
  * x scaled by a power of two to 22-bit fixed point splits into two signed 11-bit digits that half precision holds exactly;
  * with exact products and exact sums per super-block the result differs from the oracle only by the rounding of x to 22 bits
    relative to the largest magnitude of its super-block: far inside the 1e-3 the operator's tests allow.
"""
import numpy as np

from jitnn_b200 import synth
from oracle import oracle


def halves_exact(v):
    return np.array_equal(np.asarray(v, np.float64), np.asarray(v, np.float64).astype(np.float16).astype(np.float64))


def test_quant_times_scale_is_exact_in_half_precision():
    q = np.arange(32, dtype=np.float64)[:, None]      # Q5_K quants 0..31 (Q4_K: 0..15)
    sc = np.arange(64, dtype=np.float64)[None, :]     # 6-bit scales
    prod = q * sc
    assert prod.max() == 1953 and halves_exact(prod)
    # the operands of the fused multiply-adds are exact halves too, and the fused result (one rounding) is the product itself
    assert halves_exact(1024 + q) and halves_exact(-1024 * sc) and halves_exact(sc / 16) and halves_exact(-64 * sc)
    assert np.array_equal((1024 + q) * sc - 1024 * sc, prod)
    q4 = np.arange(16, dtype=np.float64)[:, None]
    assert halves_exact(1024 + 16 * q4)
    assert np.array_equal((1024 + 16 * q4) * (sc / 16) - 64 * sc, q4 * sc)


def digits_of(x):
    """x [m, 256] -> (Xh, Xl, weight of the low digit) as the image builder makes them."""
    amax = np.abs(x).max(axis=1, keepdims=True)
    e = np.floor(np.log2(np.maximum(amax, 2.0 ** -100)))
    s = 2.0 ** e
    X = np.rint(x.astype(np.float64) / s * 2.0 ** 21)
    Xh = np.floor((X + 1024) / 2048)
    Xl = X - 2048 * Xh
    return Xh, Xl, s * 2.0 ** -21


def test_the_two_digits_are_exact_halves():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((64, 256)).astype(np.float32) * np.exp(rng.uniform(-20, 20, (64, 1))).astype(np.float32)
    x[0, :] = 0.0
    x[1, 5] = np.abs(x[1]).max() * 1.999  # close to twice the power of two below it
    Xh, Xl, w = digits_of(x)
    assert np.abs(Xh).max() <= 2048 and Xl.min() >= -1024 and Xl.max() < 1024
    assert halves_exact(Xh) and halves_exact(Xl)
    back = (2048 * Xh + Xl) * w
    s = 2.0 ** np.floor(np.log2(np.maximum(np.abs(x).max(axis=1, keepdims=True), 2.0 ** -100)))
    assert np.all(np.abs(back - x) <= 2.0 ** -22 * s)  # half a step of s 2^-21, s being the power of two at or below the largest magnitude


def q4k_fields(raw, n, kb):
    """Per block: d, dmin, 8 scales, 8 mins, 256 quants (GgufKernels.java:113-135)."""
    b = raw.reshape(n, kb, 144)
    d = b[:, :, 0:2].copy().view(np.float16).astype(np.float64)[..., 0]
    dmin = b[:, :, 2:4].copy().view(np.float16).astype(np.float64)[..., 0]
    s = b[:, :, 4:16].astype(np.int64)
    sc = np.empty((n, kb, 8), np.int64)
    mn = np.empty((n, kb, 8), np.int64)
    for j in range(8):
        if j < 4:
            sc[..., j] = s[..., j] & 63
            mn[..., j] = s[..., j + 4] & 63
        else:
            sc[..., j] = (s[..., j + 4] & 15) | ((s[..., j - 4] >> 6) << 4)
            mn[..., j] = (s[..., j + 4] >> 4) | ((s[..., j] >> 6) << 4)
    qs = b[:, :, 16:144].astype(np.int64).reshape(n, kb, 4, 32)
    q = np.empty((n, kb, 8, 32), np.int64)
    q[:, :, 0::2] = qs & 15
    q[:, :, 1::2] = qs >> 4
    return d, dmin, sc, mn, q


def test_the_scheme_against_the_oracle():
    n, k, m = 24, 1024, 5
    kb = k // 256
    raw = synth.random_valid_blocks("Q4_K", n, k, seed=7).numpy()
    x = np.random.default_rng(8).standard_normal((m, k)).astype(np.float32)
    x[2] *= 1e-3
    x[3, 100] = 40.0  # an outlier: its super-block's other values keep fewer bits
    d, dmin, sc, mn, q = q4k_fields(raw, n, kb)
    y = np.zeros((m, n))
    for b in range(kb):
        Xh, Xl, w = digits_of(x[:, 256 * b:256 * b + 256])            # [m, 256]
        A = (q[:, b] * sc[:, b, :, None]).reshape(n, 256)             # quant x scale, exact halves
        assert halves_exact(A)
        Dh, Dl = Xh @ A.T, Xl @ A.T                                    # the two accumulators of a unit, exact here
        sums = ((2048 * Xh + Xl) * w).reshape(m, 8, 32).sum(axis=2)    # the sub-blocks' sums of x as rounded
        y += d[None, :, b] * (w * 2048 * Dh + w * Dl) - dmin[None, :, b] * (sums @ mn[:, b].T)
    expect = oracle.linear("Q4_K", raw, x, None, threads=1)
    err = np.abs(y - expect).max() / np.abs(expect).max()
    assert err <= 2e-6, err
