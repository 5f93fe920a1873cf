"""The synthetic-weight quantisers emit valid blocks that dequantise (oracle) close to their input."""
import numpy as np
import pytest
import torch

from jitnn_b200 import synth
from oracle import oracle


@pytest.mark.parametrize("name,tol", [("Q4_0", 0.15), ("Q4_1", 0.12), ("Q4_K", 0.12), ("Q5_K", 0.06), ("Q6_K", 0.03)])
def test_quantiser_round_trip(name, tol):
    g = torch.Generator().manual_seed(7)
    w = torch.randn(6, 1024, generator=g) * 0.02
    w[1, 256:512] = 0  # an all-zero super-block
    w[2] = w[2].abs()  # no negative values: the K-quant min stays 0
    blocks = synth.QUANTIZERS[name](w).numpy()
    assert blocks.dtype == np.uint8 and blocks.shape == (6, 1024 // oracle.block_values(name) * oracle.block_bytes(name))
    back = oracle.dequantize(name, blocks).reshape(6, 1024)
    assert np.isfinite(back).all()
    assert not back[1, 256:512].any()
    rel = np.sqrt(((back - w.numpy()) ** 2).mean()) / w.numpy().std()
    assert rel < tol, rel


def test_random_valid_blocks_shape_and_scales():
    for name in ["Q8_0", "Q4_0", "Q4_1", "Q4_K", "Q5_K", "Q6_K", "Q5_0", "Q5_1", "Q2_K", "Q3_K"]:
        b = synth.random_valid_blocks(name, 3, 512, seed=1).numpy()
        assert b.shape == (3, 512 // oracle.block_values(name) * oracle.block_bytes(name))
        v = oracle.dequantize(name, b)
        assert np.isfinite(v).all() and np.abs(v).max() < 200
