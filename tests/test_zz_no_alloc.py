"""The allocation-free Q4_K entry point gives what jq_linear_f32 gives.

jq_linear_q4k_f32_noalloc is for callers that must not cause a device allocation (all GPU memory already
handed to their own pools, or a decode loop that cannot sit through cudaMalloc's device-wide wait): its
intermediate buffer is a fixed array inside the library instead of buffers allocated on first use. This file
is collected last on purpose, so that a run stopping at the first failure has already run everything else;
it also passes on its own in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

from jitnn_b200 import Gguf, Tensor, _lib, synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3  # the bound the other GPU tests use for FP32-accumulating kernels


def call_noalloc(w, x, bias, y):
    L = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return L.jq_linear_q4k_f32_noalloc(w._handle(), x.data_ptr(), x.shape[0], None if bias is None else bias.data_ptr(), y.data_ptr(), stream)


@pytest.mark.parametrize("n,k", [(100, 1024), (4096, 4096), (1030, 11008)])
def test_matches_the_allocating_entry_point_twice_in_a_row(n, k):
    g = torch.Generator().manual_seed(n + k)
    raw = synth.quantize_q4_k(torch.randn(n, k, generator=g) * 0.02).numpy()
    w = Tensor.quantized("Q4_K", raw, n, k)
    bias = torch.randn(n, generator=g).cuda()
    # two calls in a row with different row counts and inputs: the second must not see anything of the first
    for m in (5, 1, 2, 3, 8):
        x = torch.randn(m, k, generator=g).cuda()
        expect = Gguf.linear(x, w, bias)
        y = torch.full((m, n), float("nan"), device="cuda")
        assert call_noalloc(w, x, bias, y) == 0, _lib.last_error()
        torch.cuda.synchronize()
        diff = float((y - expect).abs().max() / expect.abs().max())
        assert diff <= REL_TOL, diff
        assert torch.equal(y, expect)  # same kernels, same summation order


def test_no_device_memory_is_allocated():
    """After a first call (which may load the kernels' code), further calls on a stream the library has never seen leave the
    device's free memory where it was: the allocating entry point would have created scratch buffers for that stream."""
    n, k = 512, 2048
    w = Tensor.quantized("Q4_K", synth.random_valid_blocks("Q4_K", n, k, seed=1).numpy(), n, k)
    x = torch.randn(16, k, device="cuda")
    y = torch.empty(16, n, device="cuda")
    L = _lib.load()
    for m in (1, 2, 5, 8):  # one warm-up call per kernel variant
        assert L.jq_linear_q4k_f32_noalloc(w._handle(), x.data_ptr(), m, None, y.data_ptr(), None) == 0, _lib.last_error()
    torch.cuda.synchronize()
    fresh = torch.cuda.Stream()
    free_before = torch.cuda.mem_get_info()[0]
    for m in (1, 2, 5, 8):
        assert L.jq_linear_q4k_f32_noalloc(w._handle(), x.data_ptr(), m, None, y.data_ptr(), ctypes.c_void_p(fresh.cuda_stream)) == 0
    fresh.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before


def test_refuses_what_it_cannot_hold():
    L = _lib.load()
    raw = synth.random_valid_blocks("Q4_K", 8, 512, seed=3).numpy()
    w = Tensor.quantized("Q4_K", raw, 8, 512)
    x = torch.zeros(9, 512, device="cuda")
    y = torch.zeros(9, 8, device="cuda")
    assert call_noalloc(w, x, None, y) == _lib.JQ_ERR_INVALID and "1 to 8" in _lib.last_error()
    q8 = Tensor.quantized("Q8_0", synth.random_valid_blocks("Q8_0", 8, 512, seed=4).numpy(), 8, 512)
    assert call_noalloc(q8, x[:1], None, y[:1]) == _lib.JQ_ERR_UNSUPPORTED and "not Q4_K" in _lib.last_error()
    # k = 65536 with 8 rows needs 256 * 7008 bytes of image: more than the 1 MiB the library carries
    big = Tensor.quantized("Q4_K", np.zeros(65536 // 256 * 144, np.uint8), 1, 65536)
    xb = torch.zeros(8, 65536, device="cuda")
    assert call_noalloc(big, xb, None, y[:8, :1].contiguous()) == _lib.JQ_ERR_INVALID
    assert "built-in scratch holds" in _lib.last_error()
    assert L.jq_linear_q4k_f32_noalloc(None, x.data_ptr(), 1, None, y.data_ptr(), None) == _lib.JQ_ERR_INVALID
