"""The tcgen05 decode GEMV (option "gemv_tcgen05"; Q4_K and Q5_K, 1 to 16 rows of x in one pass over the weights) against the
CPU oracle (ops/Gguf.java:187-205 semantics) and against the default kernel.

The kernel is not the default (the mma.sync kernel is faster on nearly every measured shape), so these tests switch it on. They
cover what is particular to it: every column count of the MMA (up to 4, 8 and 16 rows), tiles shared by several thread blocks
(few output rows), tiles split between two (many output rows), the activation image built inside the kernel (small k) and
streamed from a scratch buffer (large k or many rows), the pair of weights in one launch is covered by the decoder tests of
the default kernel only. Tolerance: max |diff| <= 1e-3 max |expect| (FP32 accumulation) and the reference's 2e-4 bound.
"""
import numpy as np
import pytest
import torch

import jitnn_b200
from conftest import close_like_reference
from jitnn_b200 import Gguf, Tensor, synth
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def tcgen05_kernel():
    L = jitnn_b200.load()
    L.jq_set_option(b"gemv_tcgen05", 1)
    yield
    L.jq_set_option(b"gemv_tcgen05", 0)


def check(t, n, k, m, seed, rows=None):
    raw = synth.random_valid_blocks(t, n, k, seed=seed).numpy()
    x = np.random.default_rng(seed + 1).standard_normal((m, k)).astype(np.float32)
    bias = np.random.default_rng(seed + 2).standard_normal(n).astype(np.float32)
    w = Tensor.quantized(t, raw, n, k)
    got = Gguf.linear(torch.from_numpy(x).cuda(), w, torch.from_numpy(bias).cuda()).cpu().numpy()
    rows = np.arange(n) if rows is None else rows
    expect = oracle.linear(t, raw[rows], x, bias[rows], threads=8)
    assert float(np.abs(expect - got[:, rows]).max() / np.abs(expect).max()) <= 1e-3
    close_like_reference(expect, got[:, rows], "%s [%d, %d] m=%d" % (t, n, k, m))
    w.release()
    return got


@pytest.mark.parametrize("t", ["Q4_K", "Q5_K"])
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 10, 16])
def test_small_shapes(t, m):
    check(t, 300, 2816, m, seed=m)
    check(t, 100, 256, m, seed=m + 20)


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 1), (4096, 4096, 8), (4096, 11008, 2), (11008, 4096, 16), (32000, 4096, 1), (32000, 4096, 5),
                                   (8192, 28672, 1), (28672, 8192, 16)])
def test_benchmark_shapes(n, k, m):
    rows = np.unique(np.concatenate([np.arange(130), np.arange(n - 130, n), np.random.default_rng(n).integers(0, n, 48)]))
    check("Q4_K", n, k, m, seed=n + k + m, rows=rows)


@pytest.mark.parametrize("t", ["Q4_K", "Q5_K"])
def test_row_shards_and_repeats_are_bitwise_stable(t):
    """A row shard gives bitwise the rows of the whole weight (the sum over k has one fixed order, however the tiles are dealt to
    the thread blocks), and a second call gives bitwise the first call's result (the hand-off words between thread blocks are
    back at zero after every launch)."""
    n, k = 4096, 4096
    raw = synth.random_valid_blocks(t, n, k, seed=77).numpy()
    x = np.random.default_rng(78).standard_normal((5, k)).astype(np.float32)
    w = Tensor.quantized(t, raw, n, k)
    whole = Gguf.linear(x, w, None)
    assert np.array_equal(Gguf.linear(x, w, None).view(np.uint32), whole.view(np.uint32))
    for lo, hi in [(0, 128), (1000, 1100), (4000, 4096)]:
        part = Gguf.linear(x, Tensor.quantized(t, raw, n, k, rows=(lo, hi)), None)
        assert np.array_equal(part.view(np.uint32), whole[:, lo:hi].view(np.uint32)), (lo, hi)


def test_non_finite_activations_give_nan():
    n, k = 64, 1024
    raw = synth.random_valid_blocks("Q4_K", n, k, seed=3).numpy()
    w = Tensor.quantized("Q4_K", raw, n, k)
    x = np.random.default_rng(3).standard_normal((3, k)).astype(np.float32)
    x[0, 300] = np.nan
    x[2, 900] = np.inf
    got = Gguf.linear(x, w, None)
    assert np.isnan(got[0]).all() and np.isnan(got[2]).all()
    close_like_reference(oracle.linear("Q4_K", raw, x[1:2]), got[1:2], "finite row")


@pytest.mark.parametrize("t,n,k,m", [("Q4_K", 32000, 4096, 12), ("Q5_K", 20480, 5120, 16), ("Q4_K", 32000, 4096, 27), ("Q5_K", 49152, 8192, 8),
                                     ("Q4_K", 8192, 8192, 16), ("Q4_K", 5120, 5120, 11), ("Q5_K", 8192, 28672, 13)])
def test_shapes_that_reach_the_kernel_without_the_option(t, n, k, m):
    """With the option at its default the kernel takes 11 to 16 rows of x on weights of at least one 128-row tile per SM (27 rows:
    16 through it, 11 more through it), on weights of fewer tiles with k cut into 2 to 8 equal ranges whose sums a second kernel
    adds in order (the last three cases: 4, 4 and 4 ranges), and stands in where the mma.sync kernel declines (Q5_K, k = 8192, 3 to
    8 rows of x and more 16-row tiles per thread block than that kernel can carry sums for)."""
    L = jitnn_b200.load()
    L.jq_set_option(b"gemv_tcgen05", 0)
    rows = np.unique(np.concatenate([np.arange(130), np.arange(n - 130, n), np.random.default_rng(n).integers(0, n, 48)]))
    got = check(t, n, k, m, seed=n + m, rows=rows)
    L.jq_set_option(b"gemv_tcgen05", 2)  # never: the same call through the mma.sync kernel (or, where that declines, the CUDA-core one)
    raw = synth.random_valid_blocks(t, n, k, seed=n + m).numpy()
    x = np.random.default_rng(n + m + 1).standard_normal((m, k)).astype(np.float32)
    bias = np.random.default_rng(n + m + 2).standard_normal(n).astype(np.float32)
    w = Tensor.quantized(t, raw, n, k)
    other = Gguf.linear(torch.from_numpy(x).cuda(), w, torch.from_numpy(bias).cuda()).cpu().numpy()
    w.release()
    assert float(np.abs(other - got).max() / np.abs(other).max()) <= 1e-5


def test_option_values():
    L = jitnn_b200.load()
    assert L.jq_set_option(b"gemv_tcgen05", 3) != 0
    assert L.jq_set_option(b"gemv_tcgen05", 2) == 0
    assert L.jq_set_option(b"gemv_tcgen05", 0) == 0


def test_launches_of_different_shapes_share_the_scratch():
    """The hand-off words between thread blocks must be all zero when a launch starts, whatever ran before it: a launch with few rows
    of x whose thread blocks keep floats aside (a tile shared by three or more of them) between two launches with many rows, whose
    hand-off words cover more of the scratch buffer."""
    rows = np.unique(np.concatenate([np.arange(130), np.arange(11008 - 130, 11008)]))
    check("Q4_K", 11008, 4096, 16, seed=1, rows=rows)
    check("Q4_K", 4096, 11008, 2, seed=2, rows=rows[:130])
    check("Q4_K", 11008, 4096, 16, seed=3, rows=rows)
    check("Q5_K", 4096, 11008, 5, seed=4, rows=rows[:130])
    check("Q4_K", 11008, 4096, 9, seed=5, rows=rows)
