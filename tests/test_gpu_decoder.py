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


# head_dim 64 takes the general kernels; head_dim 128 takes the fused single-token step (and, with the option off,
# the general kernels again); 61 prompt tokens put the decoded positions across the 64-key chunk boundary
@pytest.mark.parametrize("dim,heads,kv_heads,prompt_len,fused", [(256, 4, 4, 13, 1), (256, 4, 2, 13, 1), (512, 4, 4, 61, 1), (512, 4, 2, 13, 1),
                                                                 (512, 4, 2, 61, 0)])
def test_prompt_logits_and_greedy_tokens(dim, heads, kv_heads, prompt_len, fused):
    import jitnn_b200
    jitnn_b200.load().jq_set_option(b"decoder_fused", fused)
    try:
        run_prompt_and_greedy(dim, heads, kv_heads, prompt_len)
    finally:
        jitnn_b200.load().jq_set_option(b"decoder_fused", 1)


def run_prompt_and_greedy(dim, heads, kv_heads, prompt_len):
    cfg = llama_oracle.Config(layers=2, dim=dim, heads=heads, kv_heads=kv_heads, hidden=2 * dim, vocab=512, max_seq=prompt_len + 24)
    weights, dec = build(cfg, seed=heads * 10 + kv_heads)
    ref = llama_oracle.Decoder(cfg, weights)
    rng = np.random.default_rng(7)
    prompt = rng.integers(0, cfg.vocab, prompt_len).astype(np.int32)

    # prompt in chunks of up to 8 tokens on the GPU, token by token in the oracle
    ref_logits = np.stack([ref.forward(int(t), i) for i, t in enumerate(prompt)])
    got = np.concatenate([dec.forward(prompt[i:i + 8], i)[0] for i in range(0, prompt_len, 8)])
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


@pytest.mark.parametrize("dim,heads,kv_heads,n_seqs", [(512, 4, 2, 3), (256, 4, 4, 16)])
def test_batched_decode_matches_the_sequences_run_alone(dim, heads, kv_heads, n_seqs):
    """One token of each of several sequences per step (one pass over the weights) against the same sequences decoded
    one at a time: logits within the decoder tolerance, same greedy tokens where the margin is decisive."""
    prompt_len, steps = 13, 6
    cfg = llama_oracle.Config(layers=2, dim=dim, heads=heads, kv_heads=kv_heads, hidden=2 * dim, vocab=512, max_seq=prompt_len + steps + 2)
    weights, dec = build(cfg, seed=77)
    dec.set_sequences(n_seqs)
    rng = np.random.default_rng(3)
    prompts = rng.integers(0, cfg.vocab, (n_seqs, prompt_len)).astype(np.int32)
    # alone: sequence b lives in cache slot b and advances with single-token calls
    alone_logits = np.zeros((steps, n_seqs, cfg.vocab), np.float32)
    first = np.zeros(n_seqs, np.int32)
    for b in range(n_seqs):
        for i in range(0, prompt_len, 8):
            _, nxt = dec.forward(prompts[b, i:i + 8], i, seq=b)
        first[b] = nxt[-1]
        tok = int(first[b])
        for t in range(steps):
            lg, nxt = dec.forward([tok], prompt_len + t, seq=b)
            alone_logits[t, b] = lg[0]
            tok = int(nxt[0])
    # batched: the prompts again (the caches are rewritten position by position), then lockstep steps
    for b in range(n_seqs):
        for i in range(0, prompt_len, 8):
            dec.forward(prompts[b, i:i + 8], i, seq=b)
    toks = first.copy()
    scale = np.abs(alone_logits).max()
    for t in range(steps):
        lg, nxt = dec.forward_batch(toks, prompt_len + t)
        assert np.abs(lg - alone_logits[t]).max() <= 2e-4 * scale, (t, float(np.abs(lg - alone_logits[t]).max() / scale))
        assert np.array_equal(nxt, np.argmax(lg, axis=1))
        ref_next = np.argmax(alone_logits[t], axis=1)
        top = np.sort(alone_logits[t], axis=1)[:, -2:]
        decisive = (top[:, 1] - top[:, 0]) > MARGIN * scale
        assert np.array_equal(nxt[decisive], ref_next[decisive])
        toks = ref_next.astype(np.int32)  # stay on the path of the sequences run alone
    with pytest.raises(ValueError, match="holds %d sequence" % n_seqs):
        dec.forward([1], 0, seq=n_seqs)
    dec.close()


def test_forward_argument_checks():
    cfg = llama_oracle.Config(layers=1, dim=256, heads=4, kv_heads=4, hidden=256, vocab=64, max_seq=8)
    dec = LlamaDecoder(cfg.layers, cfg.dim, cfg.heads, cfg.kv_heads, cfg.hidden, cfg.vocab, cfg.max_seq)
    with pytest.raises(ValueError, match="not set"):
        dec.forward([1], 0)
    weights = llama_oracle.random_model(cfg, 3)
    dec.load(weights)
    with pytest.raises(ValueError, match="at most 16 per call"):
        dec.forward(list(range(17)), 0)
    with pytest.raises(ValueError, match="8 positions"):
        dec.forward([1, 2], 7)
    with pytest.raises(ValueError, match="inconsistent sizes"):
        LlamaDecoder(1, 250, 4, 3, 256, 64, 8)
    dec.close()


def test_shard_and_sequence_argument_checks():
    """jq_decoder_set_shard and jq_decoder_set_sequences refuse what they cannot serve, with a message."""
    import ctypes
    import jitnn_b200
    from jitnn_b200._lib import check
    L = jitnn_b200.load()
    cfg = llama_oracle.Config(layers=1, dim=256, heads=4, kv_heads=2, hidden=256, vocab=64, max_seq=8)
    dec = LlamaDecoder(cfg.layers, cfg.dim, cfg.heads, cfg.kv_heads, cfg.hidden, cfg.vocab, cfg.max_seq)
    nbytes = ctypes.c_int64()
    check(L.jq_decoder_peer_bytes(dec._h, ctypes.byref(nbytes)))
    assert nbytes.value > 16 * (2 * cfg.dim + cfg.hidden + cfg.dim + cfg.vocab) * 4
    fake = (ctypes.c_void_p * 4)(1, 1, 1, 1)  # never dereferenced by the checks below
    with pytest.raises(ValueError, match="do not divide"):
        check(L.jq_decoder_set_shard(dec._h, 0, 3, fake))  # 3 ranks, 4 heads
    with pytest.raises(ValueError, match="do not divide"):
        check(L.jq_decoder_set_shard(dec._h, 0, 4, fake))  # 4 ranks, 2 key/value heads
    with pytest.raises(ValueError, match="rank 2 of 2"):
        check(L.jq_decoder_set_shard(dec._h, 2, 2, fake))
    check(L.jq_decoder_set_shard(dec._h, 0, 1, None))  # one rank: the ordinary decoder
    with pytest.raises(ValueError, match="1 to 16"):
        dec.set_sequences(17)
    dec.load(llama_oracle.random_model(cfg, 5))
    with pytest.raises(ValueError, match="before the linears are set"):
        check(L.jq_decoder_set_shard(dec._h, 0, 2, fake))
    dec.set_sequences(2)
    with pytest.raises(ValueError, match="batch of 3"):
        dec.forward_batch([1, 2, 3], 0)
    lg, nxt = dec.forward_batch([1, 2], 0)
    assert lg.shape == (2, cfg.vocab) and nxt.shape == (2,)
    dec.close()


# ---- the benchmark's own widths: sliced activation images (k = 11008, 28672), the 32000-row argmax, grouped-query heads of the
# 70B shape, the Q4_K + Q6_K mix; a prompt of a few tokens and four greedy steps against the oracle, fused and general kernels
@pytest.mark.parametrize("fused", [1, 0])
@pytest.mark.parametrize("layers,dim,heads,kv_heads,hidden,formats", [(2, 4096, 32, 32, 11008, None),
                                                                      (1, 8192, 64, 8, 28672, {"wv": "Q4_K", "w2": "Q4_K", "output": "Q4_K"})])
def test_full_width_decoder(layers, dim, heads, kv_heads, hidden, formats, fused):
    import jitnn_b200
    cfg = llama_oracle.Config(layers=layers, dim=dim, heads=heads, kv_heads=kv_heads, hidden=hidden, vocab=32000, max_seq=16)
    weights = llama_oracle.random_model(cfg, seed=dim // 64, formats=formats)
    jitnn_b200.load().jq_set_option(b"decoder_fused", fused)
    try:
        dec = LlamaDecoder(cfg.layers, cfg.dim, cfg.heads, cfg.kv_heads, cfg.hidden, cfg.vocab, cfg.max_seq, cfg.eps, cfg.rope_base)
        dec.load(weights)
        ref = llama_oracle.Decoder(cfg, weights, threads=8)
        prompt = np.random.default_rng(dim).integers(0, cfg.vocab, 3).astype(np.int32)
        ref_logits = np.stack([ref.forward(int(t), i) for i, t in enumerate(prompt)])
        got, nxt = dec.forward(prompt, 0)
        scale = np.abs(ref_logits).max()
        assert np.abs(got - ref_logits).max() <= 2e-4 * scale, float(np.abs(got - ref_logits).max() / scale)
        tok, pos, lr = llama_oracle.greedy(ref_logits[-1]), len(prompt), ref_logits[-1]
        for _ in range(4):
            top = np.sort(lr)[-2:]
            if (top[1] - top[0]) > MARGIN * scale:
                assert int(nxt[-1]) == tok, "greedy tokens diverge at position %d" % pos
            lr = ref.forward(tok, pos)
            lg, nxt = dec.forward([tok], pos)  # on the oracle's path, so that later positions stay comparable
            assert np.abs(lg[0] - lr).max() <= 2e-4 * max(scale, np.abs(lr).max())
            assert int(nxt[0]) == int(np.argmax(lg[0]))
            tok, pos = llama_oracle.greedy(lr), pos + 1
        dec.close()
    finally:
        jitnn_b200.load().jq_set_option(b"decoder_fused", 1)


@pytest.mark.parametrize("layers,dim,heads,kv_heads,hidden", [(2, 4096, 32, 32, 11008), (1, 8192, 64, 8, 28672)])
def test_full_width_decoder_twelve_tokens_per_call(layers, dim, heads, kv_heads, hidden):
    """Twelve tokens in one call at the benchmark's widths, all Q4_K: from eleven rows on the linears whose weights have enough rows
    go through the tcgen05 GEMV in one pass, wq / wk / wv and w1 / w3 as one launch each on one activation image, weights of few
    128-row tiles with k cut into ranges; the others through the mma.sync kernel in two passes. Against the oracle, token by token."""
    all_q4k = {"wv": "Q4_K", "w2": "Q4_K", "output": "Q4_K"}
    cfg = llama_oracle.Config(layers=layers, dim=dim, heads=heads, kv_heads=kv_heads, hidden=hidden, vocab=32000, max_seq=16)
    weights = llama_oracle.random_model(cfg, seed=dim // 32, formats=all_q4k)
    dec = LlamaDecoder(cfg.layers, cfg.dim, cfg.heads, cfg.kv_heads, cfg.hidden, cfg.vocab, cfg.max_seq, cfg.eps, cfg.rope_base)
    dec.load(weights)
    ref = llama_oracle.Decoder(cfg, weights, threads=8)
    prompt = np.random.default_rng(dim + 1).integers(0, cfg.vocab, 12).astype(np.int32)
    ref_logits = np.stack([ref.forward(int(t), i) for i, t in enumerate(prompt)])
    got, nxt = dec.forward(prompt, 0)
    scale = np.abs(ref_logits).max()
    assert np.abs(got - ref_logits).max() <= 2e-4 * scale, float(np.abs(got - ref_logits).max() / scale)
    assert np.array_equal(nxt, np.argmax(got, axis=1))
    # the same tokens in groups of at most eight (mma.sync kernels only): the two routes agree far inside the tolerance
    dec.forward(prompt[:8], 0)
    tail, _ = dec.forward(prompt[8:], 8)
    assert np.abs(tail - got[8:]).max() <= 2e-5 * scale
    dec.close()
