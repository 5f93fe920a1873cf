"""The decoder oracle's operators against the reference's own golden vectors.

oracle/llama_oracle.py restates the block math of jitnn-nn/.../nn/models/Llama.java:167-222; every operator it is made of has
golden cases in the reference (jitnn-core/src/test/resources/golden/manifest.txt: rms_norm* :191-194, rope_heads :144,
sdpa_bthd_causal :142, silu* and swiglu :113-115, embedding* :125-127, argmax :64), extracted by tests/golden/make_golden.py.
Tolerances are the reference's (Golden.java:483-498): rtol = atol = 1e-4 for the accumulating operators (rms_norm, sdpa_bthd,
embedding), rtol 2e-6 / atol 1e-6 for the element-wise ones (rope_heads, silu, swiglu); argmax exact.
"""
import os

import numpy as np
import pytest

from conftest import GOLDEN, golden_close
from oracle import llama_oracle


@pytest.fixture(scope="module")
def ops():
    return np.load(os.path.join(GOLDEN, "golden_decoder_ops.npz"))


@pytest.mark.parametrize("name", ["rms_norm", "rms_norm_3d", "rms_norm_long", "rms_norm_rows"])
def test_rmsnorm(ops, name):
    x, w, eps = ops[name + ".in0"], ops[name + ".in1"], float(ops[name + ".attrs"][0])
    golden_close(ops[name + ".out"], llama_oracle.rmsnorm(x, w, eps), rtol=1e-4, atol=1e-4, what=name)


def test_rope_rotate_half(ops):
    x = ops["rope_heads.in0"]  # [batch, positions, heads, head_dim]
    base, offset, interleaved = ops["rope_heads.attrs"]
    assert interleaved == 0
    cfg = llama_oracle.Config(layers=1, dim=x.shape[2] * x.shape[3], heads=x.shape[2], kv_heads=x.shape[2], hidden=1, vocab=1, max_seq=x.shape[1] + int(offset),
                              rope_base=float(base))
    cos, sin = llama_oracle.rope_tables(cfg)
    got = np.stack([np.stack([llama_oracle.rope(x[b, t], cos, sin, t + int(offset)) for t in range(x.shape[1])]) for b in range(x.shape[0])])
    golden_close(ops["rope_heads.out"], got, rtol=2e-6, atol=1e-6, what="rope_heads")


def test_causal_attention(ops):
    q, k, v = ops["sdpa_bthd_causal.in0"], ops["sdpa_bthd_causal.in1"], ops["sdpa_bthd_causal.in2"]  # [batch, positions, heads, head_dim]
    causal, scale_attr = ops["sdpa_bthd_causal.attrs"]
    assert causal == 1 and scale_attr < 0
    B, T, H, D = q.shape
    scale = np.float64(np.float32(1.0 / np.sqrt(D)))
    got = np.empty_like(q)
    for b in range(B):
        keys, values = k[b].reshape(T, H * D), v[b].reshape(T, H * D)
        for t in range(T):
            got[b, t] = llama_oracle.attend(q[b, t], keys[:t + 1], values[:t + 1], 1, scale)
    golden_close(ops["sdpa_bthd_causal.out"], got, rtol=1e-4, atol=1e-4, what="sdpa_bthd_causal")


@pytest.mark.parametrize("name", ["silu", "silu_tails"])
def test_silu(ops, name):
    golden_close(ops[name + ".out"], llama_oracle.silu(ops[name + ".in0"]), rtol=2e-6, atol=1e-6, what=name)


def test_swiglu(ops):
    golden_close(ops["swiglu.out"], llama_oracle.swiglu(ops["swiglu.in0"], ops["swiglu.in1"]), rtol=2e-6, atol=1e-6, what="swiglu")


@pytest.mark.parametrize("name", ["embedding", "embedding_wide"])
def test_embedding(ops, name):
    ids, table = ops[name + ".in0"], ops[name + ".in1"]
    got = np.stack([llama_oracle.embedding(table, int(i)) for i in ids.reshape(-1)]).reshape(ids.shape + (table.shape[1],))
    assert np.array_equal(got, ops[name + ".out"])


def test_greedy_is_first_index_of_the_maximum(ops):
    x, want = ops["argmax.in0"], ops["argmax.out"]
    assert int(ops["argmax.attrs"][0]) == 1
    assert [llama_oracle.greedy(row) for row in x] == [int(v) for v in want]
    assert llama_oracle.greedy(np.array([1.0, 3.0, 3.0, 2.0], np.float32)) == 1
