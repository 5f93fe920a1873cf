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
    """With ``group`` (a torch.distributed process group of more than one rank, one process per GPU) the decoder is
    split by output rows of every linear: each rank keeps rows [rank * n / world, (rank + 1) * n / world) of each weight,
    the ranks exchange activations through peer buffers (set up here, collectively), and every rank must make the same
    forward calls. Results are bitwise those of one GPU on the general kernels."""

    def __init__(self, layers, dim, heads, kv_heads, hidden, vocab, max_seq, eps=1e-5, rope_base=10000.0, device=0, group=None, sharded=False):
        self.layers, self.dim, self.vocab, self.max_seq, self.device = layers, dim, vocab, max_seq, device
        self._weights = []  # keeps the borrowed weights alive
        self.rank, self.world, self.group = 0, 1, group
        self._own, self._opened = None, []
        h = ctypes.c_void_p()
        L = _lib.load()
        check(L.jq_decoder_create(device, layers, dim, heads, kv_heads, hidden, vocab, max_seq, eps, rope_base, ctypes.byref(h)))
        self._h = h
        if sharded:
            self._set_up_shard(group)

    def _set_up_shard(self, group):
        import torch.distributed as dist
        L = _lib.load()
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world == 1:
            return
        nbytes = ctypes.c_int64()
        check(L.jq_decoder_peer_bytes(self._h, ctypes.byref(nbytes)))
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        check(L.jq_peer_alloc(self.device, nbytes.value, ctypes.byref(own), handle))
        self._own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        buffers = (ctypes.c_void_p * self.world)()
        for r, hb in enumerate(handles):
            if r == self.rank:
                buffers[r] = self._own
            else:
                p = ctypes.c_void_p()
                check(L.jq_peer_open(self.device, ctypes.create_string_buffer(hb, 64), ctypes.byref(p)))
                buffers[r] = p.value
                self._opened.append(p.value)
        check(L.jq_decoder_set_shard(self._h, self.rank, self.world, buffers))
        dist.barrier(group=group)

    def load(self, weights, local=False):
        """weights: name -> (type name, raw blocks, n, k) for linears, float32 arrays for norms and the embedding table.
        A sharded decoder uploads only its own rows of each linear; with ``local`` the tuples already hold just those
        rows (n = rows of this rank)."""
        L = _lib.load()
        for name, value in weights.items():
            parts = name.split(".")
            if isinstance(value, tuple):
                t, raw, n, k = value
                if self.world > 1 and not local:
                    per = n // self.world
                    w = Tensor.quantized(t, raw, n, k, device=self.device, rows=(self.rank * per, (self.rank + 1) * per))
                else:
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

    def forward(self, tokens, pos0, want_logits=True, stream=None, seq=0):
        """Runs up to 16 tokens of sequence `seq` starting at position pos0; returns (logits [n, vocab] or None, next tokens [n])."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        n = toks.size
        logits = np.empty((n, self.vocab), dtype=np.float32) if want_logits else None
        nxt = np.empty(n, dtype=np.int32)
        check(_lib.load().jq_decoder_forward_seq(self._h, seq, toks.ctypes.data, n, pos0, None if logits is None else logits.ctypes.data,
                                                 nxt.ctypes.data, stream))
        return logits, nxt

    def enqueue(self, tokens, pos0, stream=None, seq=0):
        """As forward, but only enqueues the work (no outputs, no wait)."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        check(_lib.load().jq_decoder_forward_seq(self._h, seq, toks.ctypes.data, toks.size, pos0, None, None, stream))

    def prompt(self, tokens, pos0, want_logits=True, stream=None, seq=0):
        """Runs a long run of tokens (up to 4096) of sequence `seq` starting at position pos0 in one pass over the weights, the
        linears on the tensor-core prefill kernel with bfloat16 operands; returns (logits [vocab] of the last token or None,
        the greedy token after it)."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.vocab, dtype=np.float32) if want_logits else None
        nxt = np.empty(1, dtype=np.int32)
        check(_lib.load().jq_decoder_prompt(self._h, seq, toks.ctypes.data, toks.size, pos0, None if logits is None else logits.ctypes.data,
                                            nxt.ctypes.data, stream))
        return logits, int(nxt[0])

    def set_sequences(self, sequences):
        """Key/value caches for `sequences` (1..16) independent sequences; cached positions are lost."""
        check(_lib.load().jq_decoder_set_sequences(self._h, sequences))

    def forward_batch(self, tokens, pos, want_logits=True, stream=None):
        """One token of each of the sequences 0 .. len(tokens) - 1, all at position `pos`, in one pass over the weights;
        returns (logits [n, vocab] or None, next tokens [n])."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        n = toks.size
        logits = np.empty((n, self.vocab), dtype=np.float32) if want_logits else None
        nxt = np.empty(n, dtype=np.int32)
        check(_lib.load().jq_decoder_forward_batch(self._h, toks.ctypes.data, n, pos, None if logits is None else logits.ctypes.data,
                                                   nxt.ctypes.data, stream))
        return logits, nxt

    def close(self, collective=True):
        """Collective for a sharded decoder: the ranks unmap each other's buffers before any is freed."""
        if self._h is not None:
            h, self._h = self._h, None
            L = _lib.load()
            check(L.jq_decoder_destroy(h))
            if self._own is not None:
                for p in self._opened:
                    L.jq_peer_close(p)
                self._opened = []
                if collective:
                    import torch.distributed as dist
                    dist.barrier(group=self.group)
                L.jq_peer_free(self._own)
                self._own = None
        self._weights = []

    def __del__(self):
        try:
            self.close(collective=False)  # no collective from the garbage collector
        except Exception:
            pass
