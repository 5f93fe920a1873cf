"""The decoder's prompt path (jq_decoder_prompt): a long run of tokens in one pass over the weights, every linear on the
tensor-core prefill kernel with its input rounded to bfloat16.

The reference's block math (models/Llama.java:192-222) is the oracle's (oracle/llama_oracle.py, FP32 operands); bfloat16
keeps 8 bits of an activation, so the bar here is the one the prefill kernel's own tests use: 1e-2 of the largest logit
(tests/test_gpu_prefill.py), with the greedy token equal wherever the oracle's top-1/top-2 margin is wider than that.
The path's own consistency is checked more tightly: a prompt run in two calls equals the same prompt in one call (a
row of a linear does not depend on how many other rows ride along), and decoding on from the cache it left agrees with
the oracle to the same 1e-2.
"""
import numpy as np
import pytest

from jitnn_b200 import LlamaDecoder
from oracle import llama_oracle

pytestmark = pytest.mark.gpu

TOL = 1e-2


def build(cfg, seed):
    weights = llama_oracle.random_model(cfg, seed)
    dec = LlamaDecoder(cfg.layers, cfg.dim, cfg.heads, cfg.kv_heads, cfg.hidden, cfg.vocab, cfg.max_seq, cfg.eps, cfg.rope_base)
    dec.load(weights)
    return weights, dec


# head sizes 128 and 64, multi-head and grouped-query attention; 150 tokens: ragged against the kernel's 128-token tiles, the
# 64-key tiles and the 8-query groups of the attention
@pytest.mark.parametrize("dim,heads,kv_heads,prompt_len", [(512, 4, 4, 150), (512, 4, 2, 150), (256, 4, 2, 131), (512, 4, 1, 9)])
def test_prompt_against_the_oracle(dim, heads, kv_heads, prompt_len):
    cfg = llama_oracle.Config(layers=2, dim=dim, heads=heads, kv_heads=kv_heads, hidden=2 * dim, vocab=700, max_seq=prompt_len + 8)
    weights, dec = build(cfg, seed=3 * heads + kv_heads)
    ref = llama_oracle.Decoder(cfg, weights, threads=8)
    prompt = np.random.default_rng(prompt_len).integers(0, cfg.vocab, prompt_len).astype(np.int32)
    lr = None
    for i, t in enumerate(prompt):
        lr = ref.forward(int(t), i)
    got, nxt = dec.prompt(prompt, 0)
    scale = float(np.abs(lr).max())
    err = float(np.abs(got - lr).max() / scale)
    assert err <= TOL, err
    assert nxt == int(np.argmax(got))
    top = np.sort(lr)[-2:]
    if top[1] - top[0] > 2 * TOL * scale:
        assert nxt == llama_oracle.greedy(lr)
    # decoding on from the cache the prompt path wrote (FP32 single-token steps), on the oracle's tokens
    tok, pos = llama_oracle.greedy(lr), prompt_len
    for _ in range(4):
        lr = ref.forward(tok, pos)
        lg, _ = dec.forward([tok], pos)
        assert float(np.abs(lg[0] - lr).max() / max(scale, float(np.abs(lr).max()))) <= TOL
        tok, pos = llama_oracle.greedy(lr), pos + 1
    dec.close()


def test_a_prompt_in_two_calls_equals_the_prompt_in_one():
    cfg = llama_oracle.Config(layers=2, dim=512, heads=4, kv_heads=2, hidden=1024, vocab=700, max_seq=200)
    weights, dec = build(cfg, seed=11)
    prompt = np.random.default_rng(5).integers(0, cfg.vocab, 170).astype(np.int32)
    whole, nxt_whole = dec.prompt(prompt, 0)
    dec.prompt(prompt[:67], 0, want_logits=False)
    parts, nxt_parts = dec.prompt(prompt[67:], 67)
    assert float(np.abs(whole - parts).max()) <= 1e-5 * float(np.abs(whole).max())
    assert nxt_whole == nxt_parts
    # and against the FP32 path in groups of 16 tokens: the same model, two operand precisions
    dec2 = LlamaDecoder(cfg.layers, cfg.dim, cfg.heads, cfg.kv_heads, cfg.hidden, cfg.vocab, cfg.max_seq, cfg.eps, cfg.rope_base)
    dec2.load(weights)
    for i in range(0, len(prompt), 16):
        lg, _ = dec2.forward(prompt[i:i + 16], i)
    assert float(np.abs(whole - lg[-1]).max() / np.abs(lg[-1]).max()) <= TOL
    dec.close()
    dec2.close()


def test_what_the_prompt_path_refuses():
    from jitnn_b200 import _lib
    cfg = llama_oracle.Config(layers=1, dim=256, heads=8, kv_heads=8, hidden=512, vocab=300, max_seq=32)  # head size 32
    weights, dec = build(cfg, seed=2)
    with pytest.raises(Exception) as exc:
        dec.prompt(np.arange(8, dtype=np.int32), 0)
    assert "head size" in str(exc.value)
    dec.close()
    cfg = llama_oracle.Config(layers=1, dim=256, heads=4, kv_heads=4, hidden=512, vocab=300, max_seq=32)
    weights, dec = build(cfg, seed=2)
    with pytest.raises(Exception):
        dec.prompt(np.arange(40, dtype=np.int32), 0)  # more positions than the cache holds
    logits, nxt = dec.prompt(np.arange(32, dtype=np.int32), 0)
    assert np.isfinite(logits).all() and 0 <= nxt < cfg.vocab
    dec.close()
    assert _lib.load().jq_decoder_prompt is not None
