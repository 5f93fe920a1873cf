"""The tensor-core prefill path (jq_linear_bf16, tcgen05) against the oracle.

Two references: (1) the same computation at the same operand precision, bf16(x) times bf16(dequantised W) summed in
double, which the kernel must match to FP32-accumulation accuracy; (2) the reference operator's own FP32 semantics
(oracle.linear), which it must match within the 1e-2 relative bound stated for BF16 tensor-core prefill.
"""
import numpy as np
import pytest
import torch

from conftest import LINEAR_TYPES
from jitnn_b200 import Gguf, Tensor, _lib, device_status, synth
from oracle import oracle

pytestmark = pytest.mark.gpu


def bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16)


def check(t, n, k, m, seed, weights="random"):
    g = torch.Generator().manual_seed(seed)
    if weights == "random":
        raw = synth.random_valid_blocks(t, n, k, seed=seed).numpy()
    else:
        wf = torch.randn(n, k, generator=g) * 0.02
        raw = oracle.quantize_q8_0(wf.numpy()) if t == "Q8_0" else synth.QUANTIZERS[t](wf).numpy()
    w = Tensor.quantized(t, raw, n, k)
    x = torch.randn(m, k, generator=g)
    xb = x.to(torch.bfloat16)
    bias = torch.randn(n, generator=g)
    y = Gguf.linearBf16(xb.cuda(), w, bias.cuda()).cpu().numpy()
    assert device_status(0) == 0
    wd = oracle.dequantize(t, raw).reshape(n, k)
    same_precision = (xb.double().numpy() @ bf16_round(wd).double().numpy().T + bias.double().numpy()).astype(np.float32)
    scale = np.abs(same_precision).max()
    assert np.abs(y - same_precision).max() <= 2e-4 * scale, (t, n, k, m, float(np.abs(y - same_precision).max() / scale))
    full = oracle.linear(t, raw, x.numpy(), bias.numpy(), threads=4)
    assert np.abs(y - full).max() <= 1e-2 * np.abs(full).max()
    return y, w, xb, bias


@pytest.mark.parametrize("t", LINEAR_TYPES)
def test_one_tile(t):
    check(t, 128, 256, 128, seed=1)


@pytest.mark.parametrize("t", LINEAR_TYPES)
def test_ragged_tiles_and_long_k(t):
    check(t, 200, 1280, 130, seed=2)


@pytest.mark.parametrize("t", ["Q4_K", "Q6_K"])
def test_benchmark_weights(t):
    check(t, 512, 4096, 512, seed=3, weights="synthetic")


@pytest.mark.parametrize("t,n,k", [("Q4_K", 4096, 4096), ("Q4_K", 11008, 4096), ("Q6_K", 4096, 11008), ("Q6_K", 32000, 4096)])
def test_benchmark_shapes_against_a_gpu_reference(t, n, k):
    """At the benchmark's sizes (M = 512) the kernel takes its other tile shapes: 256 tokens with k split in two for the
    4096-row weights, two feature tiles per CTA for 11008 rows. The CPU oracle would take minutes here, so the reference is
    the same product at the same operand precision in float64 on the GPU, from the library's bit-exact dequantiser."""
    m = 512
    g = torch.Generator(device="cuda").manual_seed(n + k)
    wf = torch.randn(n, k, generator=g, device="cuda") * 0.02
    raw = synth.QUANTIZERS[t](wf).cpu().numpy()
    del wf
    w = Tensor.quantized(t, raw, n, k)
    xb = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
    bias = torch.randn(n, generator=g, device="cuda")
    y = Gguf.linearBf16(xb, w, bias)
    assert device_status(0) == 0
    wd = torch.as_tensor(np.asarray(Gguf.dequantize(w))).cuda().to(torch.bfloat16).double()
    ref = xb.double() @ wd.T + bias.double()
    err = (torch.as_tensor(np.asarray(y.cpu())).cuda().double() - ref).abs().max().item()
    assert err <= 2e-4 * ref.abs().max().item(), (t, n, k, err / ref.abs().max().item())
    # twice the same call: the two halves of k add into y in either order with the same result
    assert torch.equal(Gguf.linearBf16(xb, w, bias), y)


def test_small_m_and_host_memory():
    y, w, xb, bias = check("Q4_K", 130, 512, 5, seed=4)
    host = Gguf.linearBf16(xb.view(torch.uint16).numpy(), w, bias.numpy())
    assert np.array_equal(host, y)


def test_f32_entry_uses_prefill_only_when_asked():
    L = _lib.load()
    raw = synth.random_valid_blocks("Q4_K", 256, 512, seed=5).numpy()
    w = Tensor.quantized("Q4_K", raw, 256, 512)
    x = torch.randn(160, 512, generator=torch.Generator().manual_seed(5))
    exact = oracle.linear("Q4_K", raw, x.numpy(), None, threads=4)
    y32 = Gguf.linear(x.cuda(), w, None).cpu().numpy()
    assert np.abs(y32 - exact).max() <= 2e-4 * np.abs(exact).max()
    try:
        assert L.jq_set_option(b"prefill_min_rows", 128) == 0
        ybf = Gguf.linear(x.cuda(), w, None).cpu().numpy()
        assert device_status(0) == 0
        direct = Gguf.linearBf16(x.to(torch.bfloat16).cuda(), w, None).cpu().numpy()
        assert np.array_equal(ybf, direct)
        assert np.abs(ybf - exact).max() <= 1e-2 * np.abs(exact).max()
        assert np.abs(ybf - exact).max() > 0  # really the bf16 path
    finally:
        L.jq_set_option(b"prefill_min_rows", 0)


def test_k_not_multiple_of_64_is_refused():
    raw = synth.random_valid_blocks("Q8_0", 4, 96, seed=6).numpy()
    w = Tensor.quantized("Q8_0", raw, 4, 96)
    with pytest.raises(ValueError, match="multiple of 64"):
        Gguf.linearBf16(torch.zeros(2, 96, dtype=torch.bfloat16, device="cuda"), w)
