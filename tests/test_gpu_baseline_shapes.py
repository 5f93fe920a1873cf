"""The decode kernels at the benchmark's own shapes, against the CPU oracle (ops/Gguf.java:187-205 semantics).

At these sizes a kernel takes paths that small shapes never reach (several tiles per CTA, tiles whose super-blocks
are split between CTAs and added up afterwards, sliced activation images), so every measured configuration is
compared with the oracle here: the GPU multiplies the whole weight, the oracle a sample of rows (the first and
the last tile, rows on both sides of 128-row tile borders, and rows spread over the middle), which takes
milliseconds. Tolerance: max |diff| <= 1e-3 max |expect| (FP32 accumulation) and the reference's own
|diff| <= 2e-4 max |expect| (GgufChecks.java:110-120).
"""
import numpy as np
import pytest
import torch

from conftest import close_like_reference
from jitnn_b200 import Gguf, Quant, Tensor, synth
from oracle import oracle

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3


def sample_rows(n, seed):
    rows = set(range(0, min(16, n))) | set(range(max(0, n - 16), n))
    for border in range(128, n, max(128, (n // 7) // 128 * 128)):
        rows |= {border - 1, border, border + 1}
    rows |= set(int(r) for r in np.random.default_rng(seed).integers(0, n, 24))
    return np.array(sorted(r for r in rows if 0 <= r < n))


def weights(t, n, k, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    wf = torch.randn(n, k, generator=g, device="cuda") * 0.02
    if t == "Q8_0":
        return Quant.quantizeQ8Blocks(wf).cpu().numpy().reshape(n, -1)
    return synth.QUANTIZERS[t](wf).cpu().numpy()


def check(t, n, k, ms, seed):
    raw = weights(t, n, k, seed)
    w = Tensor.quantized(t, raw, n, k)
    rows = sample_rows(n, seed)
    rng = np.random.default_rng(seed + 1)
    for m in ms:
        x = rng.standard_normal((m, k)).astype(np.float32)
        got = Gguf.linear(torch.from_numpy(x).cuda(), w, None).cpu().numpy()
        expect = oracle.linear(t, raw[rows], x, None, threads=8)
        assert np.isfinite(got).all()
        rel = float(np.abs(expect - got[:, rows]).max() / np.abs(expect).max())
        assert rel <= REL_TOL, (t, n, k, m, rel)
        close_like_reference(expect, got[:, rows], "%s [%d, %d] m=%d" % (t, n, k, m))
    w.release()


# BASELINE configs[1]: the Q4_K sweep, M = 1 and 8 (and 16, the largest decode batch)
@pytest.mark.parametrize("n,k", [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)])
def test_q4k_sweep_shapes(n, k):
    check("Q4_K", n, k, (1, 8, 16), seed=n + k)


# BASELINE configs[0]
def test_q8_0_config0_shape():
    check("Q8_0", 4096, 4096, (1, 2), seed=5)


# the shapes of the benchmark's per-format leg
@pytest.mark.parametrize("t,n,k", [("Q6_K", 4096, 11008), ("Q6_K", 32000, 4096), ("Q5_K", 32000, 4096), ("Q4_0", 32000, 4096),
                                   ("Q4_1", 32000, 4096), ("Q8_0", 32000, 4096)])
def test_format_leg_shapes(t, n, k):
    check(t, n, k, (1, 4), seed=n // 7 + k)


# the 70B shapes of BASELINE configs[4], whole and as the row shards of 8 GPUs
@pytest.mark.parametrize("n,k", [(8192, 8192), (28672, 8192), (8192, 28672), (1024, 8192), (3584, 8192), (1024, 28672)])
def test_q4k_70b_shapes(n, k):
    check("Q4_K", n, k, (1, 16), seed=n + 3 * k)


@pytest.mark.parametrize("t", ["Q4_K", "Q5_K", "Q6_K", "Q8_0", "Q4_0", "Q4_1"])
@pytest.mark.parametrize("m", [9, 12, 16])
def test_nine_to_sixteen_rows(t, m):
    """One call with 9 to 16 rows of x (the reference tiles up to 32 rows over one decode of the weights, ops/Gguf.java:170-183)."""
    n, k = 300, 2816
    raw = synth.random_valid_blocks(t, n, k, seed=m).numpy()
    x = np.random.default_rng(m).standard_normal((m, k)).astype(np.float32)
    bias = np.random.default_rng(m + 1).standard_normal(n).astype(np.float32)
    w = Tensor.quantized(t, raw, n, k)
    got = Gguf.linear(x, w, bias)
    expect = oracle.linear(t, raw, x, bias, threads=8)
    assert float(np.abs(expect - got).max() / np.abs(expect).max()) <= REL_TOL
    close_like_reference(expect, got, "%s m=%d" % (t, m))


@pytest.mark.parametrize("t", ["Q4_K", "Q5_K", "Q6_K", "Q8_0"])
def test_rows_of_a_large_weight_equal_their_own_shard_bitwise(t):
    """The same rows as a weight of their own and as part of a large weight (where a thread block walks several tiles) give
    bitwise the same outputs: the sum over k has one order, whatever the number of rows."""
    n, k = 4096, 4096
    raw = synth.random_valid_blocks(t, n, k, seed=77).numpy()
    x = np.random.default_rng(78).standard_normal((5, k)).astype(np.float32)
    whole = Gguf.linear(x, Tensor.quantized(t, raw, n, k), None)
    for lo, hi in [(0, 128), (1000, 1100), (4000, 4096)]:
        part = Gguf.linear(x, Tensor.quantized(t, raw, n, k, rows=(lo, hi)), None)
        assert np.array_equal(part.view(np.uint32), whole[:, lo:hi].view(np.uint32)), (lo, hi)


@pytest.mark.parametrize("t", ["Q4_K", "Q5_K", "Q6_K", "Q8_0", "Q4_0", "Q4_1"])
def test_non_finite_activations_give_non_finite_outputs(t):
    """A NaN or Inf in x reaches every output row in the reference (each row multiplies every x); the fixed-point image
    must not turn it into a finite number."""
    n, k = 64, 1024
    raw = synth.random_valid_blocks(t, n, k, seed=3).numpy()
    w = Tensor.quantized(t, raw, n, k)
    x = np.random.default_rng(3).standard_normal((3, k)).astype(np.float32)
    x[0, 300] = np.nan
    x[2, 900] = np.inf
    got = Gguf.linear(x, w, None)
    expect = oracle.linear(t, raw, x, None)
    assert not np.isfinite(expect[0]).any() and not np.isfinite(expect[2]).any()
    assert not np.isfinite(got[0]).any() and not np.isfinite(got[2]).any()
    close_like_reference(expect[1], got[1], t + " finite row")
