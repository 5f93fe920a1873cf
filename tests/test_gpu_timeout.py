"""A bounded device-side wait that runs out: the kernel returns, the status word says which rank was missing, the device stays usable.

The reference tests its abort path on the host (jitnn-core/src/test/java/.../dist/HostCollectiveAbortTest.java:29-54: a rank that
never joins makes the others' collective fail instead of hang). Here the same situation is made on one GPU without faulting or
hanging anything: two peer buffers are allocated on the same device as "rank 0" and "rank 1" of a world of two, and only rank 0
ever calls. Its exchange stores its slice into its own y and, as marked words, into the other buffer's staging area, then waits
for rank 1's words in its own staging area, which nothing writes: the wait gives up after its limit (option "peer_wait_us",
0.4 s by default), records 32 + 1 and the kernel returns.
After a timeout the ranks' exchange numbers on those buffers are out of step: the buffers are to be freed and allocated anew
(jq_peer_free / jq_peer_alloc), which is what the test does before it checks that the device still works.
"""
import ctypes
import time

import numpy as np
import pytest
import torch

import jitnn_b200
from jitnn_b200 import Gguf, Tensor, _lib, synth

pytestmark = pytest.mark.gpu


def alloc_pair(L, payload):
    bufs = []
    for _ in range(2):
        p, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        _lib.check(L.jq_peer_alloc(0, payload, ctypes.byref(p), handle))
        bufs.append(p.value)
    return bufs


def status(L):
    s = ctypes.c_int(-1)
    _lib.check(L.jq_device_status(0, ctypes.byref(s)))
    return s.value


def test_a_rank_that_never_publishes_makes_the_wait_give_up():
    L = jitnn_b200.load()
    assert status(L) == 0
    n_total, n_slice = 256, 128
    payload = 3 * 4 * 16 * n_total  # y [16, n_total] floats, then as many 8-byte staging words
    staging = 4 * 16 * n_total
    bufs = alloc_pair(L, payload)
    buffers = (ctypes.c_void_p * 2)(*bufs)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    # the plain gather: slice -> every rank's y, then the wait for the other rank
    piece = torch.randn(1, n_slice, device="cuda")
    t0 = time.time()
    _lib.check(L.jq_peer_gather(piece.data_ptr(), 1, n_slice, n_total, 0, buffers, 0, staging, 0, 2, stream))
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0  # bounded: it comes back
    assert status(L) == 32 + 1  # rank 1's slice did not arrive
    assert status(L) == 0  # reading clears the word
    # rank 0's own slice did land: in its own y as floats, in rank 1's staging area as words {value, exchange number 1}
    off = L.jq_peer_payload_offset()
    holder = type("M", (), {})()
    holder.__cuda_array_interface__ = {"shape": (1, n_total), "typestr": "<f4", "data": (bufs[0] + off, False), "version": 3}
    assert torch.equal(torch.as_tensor(holder, device="cuda")[:, :n_slice], piece)
    holder = type("M", (), {})()
    holder.__cuda_array_interface__ = {"shape": (1, n_total, 2), "typestr": "<u4", "data": (bufs[1] + off + staging, False), "version": 3}
    words = torch.as_tensor(holder, device="cuda").cpu().numpy()
    assert np.array_equal(words[0, :n_slice, 0], piece.cpu().numpy().view(np.uint32)[0]) and (words[0, :n_slice, 1] == 1).all()

    # the fused form: a Q4_K row shard whose GEMV stores into every rank's y and then waits
    n, k = 128, 1024
    raw = synth.random_valid_blocks("Q4_K", 2 * n, k, seed=5).numpy()
    shard = Tensor.quantized("Q4_K", raw, 2 * n, k, rows=(0, n))
    x = torch.randn(1, k, device="cuda")
    _lib.check(L.jq_linear_f32_peer(shard._handle(), x.data_ptr(), 1, None, 2 * n, 0, buffers, 0, staging, 0, 2, stream))
    torch.cuda.synchronize()
    assert status(L) == 32 + 1
    whole = Gguf.linear(x, Tensor.quantized("Q4_K", raw, 2 * n, k), None)
    holder = type("M", (), {})()
    holder.__cuda_array_interface__ = {"shape": (1, 2 * n), "typestr": "<f4", "data": (bufs[0] + off, False), "version": 3}
    assert torch.equal(torch.as_tensor(holder, device="cuda")[:, :n], whole[:, :n])  # this rank's rows are there, bitwise

    # recovery: fresh buffers; a world of one completes at once and the device is as usable as before
    for b in bufs:
        _lib.check(L.jq_peer_free(ctypes.c_void_p(b)))
    p, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    _lib.check(L.jq_peer_alloc(0, payload, ctypes.byref(p), handle))
    one = (ctypes.c_void_p * 1)(p.value)
    _lib.check(L.jq_peer_gather(piece.data_ptr(), 1, n_slice, n_slice, 0, one, 0, staging, 0, 1, stream))
    torch.cuda.synchronize()
    assert status(L) == 0
    _lib.check(L.jq_peer_free(p))
    y = Gguf.linear(x, shard, None)
    assert torch.isfinite(y).all()


def test_a_table_slot_is_never_reused_for_another_target():
    """A buffer's flag area has room for eight target tables; a ninth distinct target is refused instead of overwriting one that a
    captured graph may still point at."""
    L = jitnn_b200.load()
    payload = 4 * 4096
    staging = 2048
    p, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    _lib.check(L.jq_peer_alloc(0, payload, ctypes.byref(p), handle))
    one = (ctypes.c_void_p * 1)(p.value)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    raw = synth.random_valid_blocks("Q4_K", 16, 256, seed=1).numpy()
    w = Tensor.quantized("Q4_K", raw, 16, 256)
    x = torch.randn(1, 256, device="cuda")
    for i in range(8):  # eight distinct areas: eight tables
        assert L.jq_linear_f32_peer(w._handle(), x.data_ptr(), 1, None, 16, 0, one, 64 * i, staging, 0, 1, stream) == 0, _lib.last_error()
    assert L.jq_linear_f32_peer(w._handle(), x.data_ptr(), 1, None, 16, 0, one, 64 * 3, staging, 0, 1, stream) == 0  # found again
    assert L.jq_linear_f32_peer(w._handle(), x.data_ptr(), 1, None, 16, 0, one, 64 * 8, staging, 0, 1, stream) == _lib.JQ_ERR_INVALID
    assert "distinct" in _lib.last_error()
    torch.cuda.synchronize()
    assert status(L) == 0
    _lib.check(L.jq_peer_free(p))
