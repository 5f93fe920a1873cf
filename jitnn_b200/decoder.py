"""Host-side mirror of the Llama-style decoder (jq_decoder_* of the C ABI).

Constructor arguments follow the reference's model class (jitnn-nn/.../nn/models/Llama.java: dim, heads,
kvHeads, hidden, vocab, layers, ropeBase, eps). Weight names follow its checkpoint loader: tok_embeddings,
layers.<l>.{attention_norm, ffn_norm, wq, wk, wv, wo, w1, w2, w3}, norm, output.
"""
import ctypes

import numpy as np

from . import _lib
from ._lib import check
from .ops import Tensor

_SLOT = {"wq": 0, "wk": 1, "wv": 2, "wo": 3, "w1": 4, "w3": 5, "w2": 6}


class LlamaDecoder:
    def __init__(self, layers, dim, heads, kv_heads, hidden, vocab, max_seq, eps=1e-5, rope_base=10000.0, device=0):
        self.layers, self.dim, self.vocab, self.max_seq, self.device = layers, dim, vocab, max_seq, device
        self._weights = []  # keeps the borrowed weights alive
        h = ctypes.c_void_p()
        check(_lib.load().jq_decoder_create(device, layers, dim, heads, kv_heads, hidden, vocab, max_seq, eps, rope_base, ctypes.byref(h)))
        self._h = h

    def load(self, weights):
        """weights: name -> (type name, raw blocks, n, k) for linears, float32 arrays for norms and the embedding table."""
        L = _lib.load()
        for name, value in weights.items():
            parts = name.split(".")
            if isinstance(value, tuple):
                t, raw, n, k = value
                w = Tensor.quantized(t, raw, n, k, device=self.device)
                self._weights.append(w)
                if name == "output":
                    check(L.jq_decoder_set_linear(self._h, -1, 7, w._handle()))
                else:
                    check(L.jq_decoder_set_linear(self._h, int(parts[1]), _SLOT[parts[2]], w._handle()))
            else:
                a = np.ascontiguousarray(value, dtype=np.float32)
                if name == "tok_embeddings":
                    check(L.jq_decoder_set_embedding(self._h, a.ctypes.data))
                elif name == "norm":
                    check(L.jq_decoder_set_norm(self._h, -1, 0, a.ctypes.data))
                else:
                    check(L.jq_decoder_set_norm(self._h, int(parts[1]), 0 if parts[2] == "attention_norm" else 1, a.ctypes.data))

    def forward(self, tokens, pos0, want_logits=True, stream=None):
        """Runs up to 8 tokens starting at position pos0; returns (logits [n, vocab] or None, next tokens [n])."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        n = toks.size
        logits = np.empty((n, self.vocab), dtype=np.float32) if want_logits else None
        nxt = np.empty(n, dtype=np.int32)
        check(_lib.load().jq_decoder_forward(self._h, toks.ctypes.data, n, pos0, None if logits is None else logits.ctypes.data, nxt.ctypes.data, stream))
        return logits, nxt

    def enqueue(self, tokens, pos0, stream=None):
        """As forward, but only enqueues the work (no outputs, no wait)."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        check(_lib.load().jq_decoder_forward(self._h, toks.ctypes.data, toks.size, pos0, None, None, stream))

    def close(self):
        if self._h is not None:
            h, self._h = self._h, None
            check(_lib.load().jq_decoder_destroy(h))
        self._weights = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
