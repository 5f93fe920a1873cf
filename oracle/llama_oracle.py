"""CPU oracle of the Llama-style decoder whose linears hold GGUF-quantised weights.

TEST INFRASTRUCTURE ONLY (see the header of jq_oracle.c). It restates, with numpy in double precision,
the forward pass of the reference's decoder, with every nn.Linear replaced by the semantics of
Gguf.linear on a quantised weight (the reference's own Llama uses FP32 linears and has no key/value
cache or generation loop; the cached decode below computes exactly what its full recompute would):

  * block structure        jitnn-nn/.../nn/models/Llama.java:209-222 (Block.forward), :167-174 (forward)
  * RMSNorm                jitnn-core/.../ops/RowNorm.java:266-306: y = x * (1 / sqrt(mean(x^2) + eps)) * w, in double
  * RoPE                   jitnn-core/.../ops/Rope.java:84-101 (cos/sin tables in double, stored as float),
                           :125-149 (rotate-half pairs (p, p + D/2), products in double)
  * attention              jitnn-core/.../ops/FlashAttention.java:538-578,594-626 (scores * scale, causal, softmax and
                           PV in double), F.java:588-599 (scale = (float)(1 / sqrt(head_dim))), F.java:606-... (query
                           head h reads key/value head h / group)
  * SwiGLU                 F.java:1158-1161, ops/RefMath.java:114 (silu = x / (1 + exp(-x)) in double, then a float multiply)
  * linears                oracle.linear: ops/Gguf.java:187-205 (double accumulation, float result)
  * greedy token           ops/Reduce.java:201 (first index of the maximum)

Every operator's result is rounded to float32 before the next one uses it, as the reference's engine does.
Parity status: every operator function below (rmsnorm, rope, attend, silu / swiglu, embedding, greedy) is pinned by
the reference's own golden vectors for it (rms_norm*, rope_heads, sdpa_bthd_causal, silu*, swiglu, embedding*,
argmax of jitnn-core/src/test/resources/golden, extracted into tests/golden/golden_decoder_ops.npz and checked by
tests/test_decoder_oracle_golden.py within Golden.java:483-498's tolerances), and the linears by the gguf_linear
vectors; the composition follows Llama.java:167-222 line by line. What stays unpinned is an end-to-end run of
the reference's GGUF decode loop, which lives in the un-vendored jitllm (no JVM here either).
"""
import numpy as np

from . import oracle


class Config:
    def __init__(self, layers, dim, heads, kv_heads, hidden, vocab, max_seq, eps=1e-5, rope_base=10000.0):
        self.layers, self.dim, self.heads, self.kv_heads = layers, dim, heads, kv_heads
        self.hidden, self.vocab, self.max_seq, self.eps, self.rope_base = hidden, vocab, max_seq, eps, rope_base
        self.head_dim = dim // heads


def rope_tables(cfg):
    half = cfg.head_dim // 2
    t = np.arange(cfg.max_seq, dtype=np.float64)[:, None]
    i = np.arange(half, dtype=np.float64)[None, :]
    freq = np.power(np.float64(np.float32(cfg.rope_base)), -2.0 * i / cfg.head_dim)
    angle = t * freq
    return np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)


def rmsnorm(x, w, eps):
    xd = x.astype(np.float64)
    inv = 1.0 / np.sqrt((xd * xd).mean(axis=-1, keepdims=True) + np.float64(np.float32(eps)))
    return (xd * inv * w.astype(np.float64)).astype(np.float32)


def rope(x, cos, sin, pos):
    """x [heads, head_dim] float32 at position pos."""
    half = x.shape[-1] // 2
    a, b = x[:, :half].astype(np.float64), x[:, half:].astype(np.float64)
    c, s = cos[pos].astype(np.float64), sin[pos].astype(np.float64)
    return np.concatenate([(a * c - b * s), (a * s + b * c)], axis=-1).astype(np.float32)


def attend(q, keys, values, group, scale):
    """Causal attention of one position: q [heads, head_dim]; keys, values [positions so far, kv_heads * head_dim];
    query head h reads key/value head h // group. Scores, softmax and the weighted sum in double."""
    heads, hd = q.shape
    y = np.empty((heads, hd), dtype=np.float32)
    for h in range(heads):
        kh = keys[:, (h // group) * hd:(h // group + 1) * hd].astype(np.float64)
        vh = values[:, (h // group) * hd:(h // group + 1) * hd].astype(np.float64)
        s = (kh @ q[h].astype(np.float64)) * scale
        pr = np.exp(s - s.max())
        pr /= pr.sum()
        y[h] = (pr @ vh).astype(np.float32)
    return y


def silu(x):
    xd = x.astype(np.float64)
    return (xd / (1.0 + np.exp(-xd))).astype(np.float32)


def swiglu(gate, up):
    return (silu(gate) * up.astype(np.float32)).astype(np.float32)


def embedding(table, token):
    return table[token].astype(np.float32)


class Decoder:
    """weights: dict name -> (type name, raw blocks uint8, n, k) for the linears, float32 arrays for norms and embeddings.

    Names: tok_embeddings, output, norm, layers.<l>.{attention_norm, ffn_norm, wq, wk, wv, wo, w1, w2, w3}.
    """

    def __init__(self, cfg, weights, threads=4):
        self.cfg, self.w, self.threads = cfg, weights, threads
        self.cos, self.sin = rope_tables(cfg)
        kv = cfg.kv_heads * cfg.head_dim
        self.k_cache = np.zeros((cfg.layers, cfg.max_seq, kv), dtype=np.float32)
        self.v_cache = np.zeros((cfg.layers, cfg.max_seq, kv), dtype=np.float32)

    def linear(self, name, x):
        t, raw, n, k = self.w[name]
        return oracle.linear(t, raw, x.reshape(1, k), None, n=n, threads=self.threads)[0]

    def forward(self, token, pos):
        """Logits (float32 [vocab]) for `token` at position `pos`; appends its key/value to the cache."""
        cfg = self.cfg
        hd, group = cfg.head_dim, cfg.heads // cfg.kv_heads
        scale = np.float64(np.float32(1.0 / np.sqrt(hd)))
        x = embedding(self.w["tok_embeddings"], token)
        for l in range(cfg.layers):
            p = "layers.%d." % l
            n = rmsnorm(x, self.w[p + "attention_norm"], cfg.eps)
            q = rope(self.linear(p + "wq", n).reshape(cfg.heads, hd), self.cos, self.sin, pos)
            k = rope(self.linear(p + "wk", n).reshape(cfg.kv_heads, hd), self.cos, self.sin, pos)
            v = self.linear(p + "wv", n)
            self.k_cache[l, pos] = k.reshape(-1)
            self.v_cache[l, pos] = v
            y = attend(q, self.k_cache[l, :pos + 1], self.v_cache[l, :pos + 1], group, scale)
            x = (x + self.linear(p + "wo", y.reshape(-1))).astype(np.float32)
            m = rmsnorm(x, self.w[p + "ffn_norm"], cfg.eps)
            act = swiglu(self.linear(p + "w1", m), self.linear(p + "w3", m))
            x = (x + self.linear(p + "w2", act)).astype(np.float32)
        h = rmsnorm(x, self.w["norm"], cfg.eps)
        return self.linear("output", h)


def greedy(logits):
    return int(np.argmax(logits))  # first index of the maximum


def random_model(cfg, seed, formats=None):
    """Seeded N(0, 0.02) weights quantised with the project's synthetic quantisers: Q6_K for wv, w2 and output,
    Q4_K elsewhere (the Q4_K_M-style mix of the benchmark), unless `formats` overrides per linear name suffix."""
    import torch
    from jitnn_b200 import synth
    g = torch.Generator().manual_seed(seed)
    formats = formats or {}
    w = {}

    def lin(name, n, k, default):
        t = formats.get(name.split(".")[-1], default)
        wf = torch.randn(n, k, generator=g) * 0.02
        raw = oracle.quantize_q8_0(wf.numpy()) if t == "Q8_0" else synth.QUANTIZERS[t](wf).numpy().reshape(-1)
        w[name] = (t, raw, n, k)

    kv = cfg.kv_heads * cfg.head_dim
    w["tok_embeddings"] = (torch.randn(cfg.vocab, cfg.dim, generator=g) * 0.02).numpy()
    for l in range(cfg.layers):
        p = "layers.%d." % l
        w[p + "attention_norm"] = (1.0 + 0.1 * torch.randn(cfg.dim, generator=g)).numpy()
        w[p + "ffn_norm"] = (1.0 + 0.1 * torch.randn(cfg.dim, generator=g)).numpy()
        lin(p + "wq", cfg.dim, cfg.dim, "Q4_K")
        lin(p + "wk", kv, cfg.dim, "Q4_K")
        lin(p + "wv", kv, cfg.dim, "Q6_K")
        lin(p + "wo", cfg.dim, cfg.dim, "Q4_K")
        lin(p + "w1", cfg.hidden, cfg.dim, "Q4_K")
        lin(p + "w3", cfg.hidden, cfg.dim, "Q4_K")
        lin(p + "w2", cfg.dim, cfg.hidden, "Q6_K")
    w["norm"] = (1.0 + 0.1 * torch.randn(cfg.dim, generator=g)).numpy()
    lin("output", cfg.vocab, cfg.dim, "Q6_K")
    return w
