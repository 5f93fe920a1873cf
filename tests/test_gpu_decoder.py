"""The decoder (glue kernels + key/value cache + quantised linears) against the CPU oracle of the reference's
Llama block math (oracle/llama_oracle.py): logits within the tolerance the reference's own Hugging Face logit check
uses (2e-4 of the largest magnitude, HfAccelTest.llamaLogits), and the same greedy tokens wherever the oracle's
top-1/top-2 margin is not within rounding distance."""
import numpy as np
import pytest

from jitnn_b200 import LlamaDecoder
from oracle import llama_oracle

pytestmark = pytest.mark.gpu

MARGIN = 1e-4  # relative top-1/top-2 margin below which a different greedy token is not counted as an error


def build(cfg, seed):
    weights = llama_oracle.random_model(cfg, seed)
    dec = LlamaDecoder(cfg.layers, cfg.dim, cfg.heads, cfg.kv_heads, cfg.hidden, cfg.vocab, cfg.max_seq, cfg.eps, cfg.rope_base)
    dec.load(weights)
    return weights, dec


@pytest.mark.parametrize("heads,kv_heads", [(4, 4), (4, 2)])
def test_prompt_logits_and_greedy_tokens(heads, kv_heads):
    cfg = llama_oracle.Config(layers=2, dim=256, heads=heads, kv_heads=kv_heads, hidden=512, vocab=512, max_seq=48)
    weights, dec = build(cfg, seed=heads * 10 + kv_heads)
    ref = llama_oracle.Decoder(cfg, weights)
    rng = np.random.default_rng(7)
    prompt = rng.integers(0, cfg.vocab, 13).astype(np.int32)

    # prompt in chunks of 8 + 5 tokens on the GPU, token by token in the oracle
    ref_logits = np.stack([ref.forward(int(t), i) for i, t in enumerate(prompt)])
    got = np.concatenate([dec.forward(prompt[:8], 0)[0], dec.forward(prompt[8:], 8)[0]])
    scale = np.abs(ref_logits).max()
    assert np.abs(got - ref_logits).max() <= 2e-4 * scale, float(np.abs(got - ref_logits).max() / scale)

    # greedy decode
    tok_ref = llama_oracle.greedy(ref_logits[-1])
    tok_gpu = int(np.argmax(got[-1]))
    pos, checked, skipped = len(prompt), 0, 0
    for _ in range(16):
        top = np.sort(ref_logits[-1] if pos == len(prompt) else lr)[-2:]
        decisive = (top[1] - top[0]) > MARGIN * scale
        if decisive:
            assert tok_gpu == tok_ref, "greedy tokens diverge at position %d" % pos
            checked += 1
        else:
            skipped += 1
            tok_gpu = tok_ref  # stay on the oracle's path so that later positions remain comparable
        lr = ref.forward(tok_ref, pos)
        lg, nxt = dec.forward([tok_gpu], pos)
        assert np.abs(lg[0] - lr).max() <= 2e-4 * max(scale, np.abs(lr).max())
        assert int(nxt[0]) == int(np.argmax(lg[0]))  # the device argmax is the first index of the maximum
        tok_ref, tok_gpu = llama_oracle.greedy(lr), int(nxt[0])
        pos += 1
    assert checked >= 8, (checked, skipped)
    dec.close()


def test_forward_argument_checks():
    cfg = llama_oracle.Config(layers=1, dim=256, heads=4, kv_heads=4, hidden=256, vocab=64, max_seq=8)
    dec = LlamaDecoder(cfg.layers, cfg.dim, cfg.heads, cfg.kv_heads, cfg.hidden, cfg.vocab, cfg.max_seq)
    with pytest.raises(ValueError, match="not set"):
        dec.forward([1], 0)
    weights = llama_oracle.random_model(cfg, 3)
    dec.load(weights)
    with pytest.raises(ValueError, match="at most 8 per call"):
        dec.forward(list(range(9)), 0)
    with pytest.raises(ValueError, match="8 positions"):
        dec.forward([1, 2], 7)
    with pytest.raises(ValueError, match="inconsistent sizes"):
        LlamaDecoder(1, 250, 4, 3, 256, 64, 8)
    dec.close()
