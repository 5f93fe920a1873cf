"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the reference's vectors.

Mirrors the reference's own checks: GgufChecks.check (values, dequantize, linear for 1, 5 and 40
rows), the gguf_* golden cases, and OpsAccelTest.q8. Integer/byte work is compared bit for bit;
float products within the reference's own tolerances, which are tighter than the 1e-3 relative bound
asked of an FP32-accumulating kernel.
"""
import numpy as np
import pytest
import torch

from conftest import EXTRA_TYPES, GOLDEN_FORMATS, LINEAR_TYPES, close_like_reference, golden_close
from jitnn_b200 import DType, F, Gguf, Quant, Tensor, synth
from oracle import oracle

pytestmark = pytest.mark.gpu

CODE_TO_TYPE = {0: "Q4_0", 1: "Q4_1", 2: "Q4_K", 3: "Q5_K", 4: "Q6_K"}
REL_TOL = 1e-3  # FP32-accumulation bound: max |diff| / max |expect|


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def max_rel(expect, got):
    return float(np.abs(expect - got).max() / max(1e-30, np.abs(expect).max()))


# ---- dequantisation: bit-exact -----------------------------------------------------------------
@pytest.mark.parametrize("t", LINEAR_TYPES + EXTRA_TYPES)
def test_fixture_values_and_dequantize(fixture_gguf, t):
    w = Tensor.quantized(t, fixture_gguf["w." + t], 3, 512)
    expect = fixture_gguf["expect." + t].reshape(-1)
    assert np.array_equal(bits(w.toFloatArray()), bits(expect))
    d = Quant.dequantize(w) if t == "Q8_0" else Gguf.dequantize(w)
    assert np.array_equal(bits(d.reshape(-1)), bits(expect))
    out = torch.empty(3, 512, device="cuda")
    Gguf.dequantize(w, out)
    assert np.array_equal(bits(out.cpu().numpy().reshape(-1)), bits(expect))
    assert np.array_equal(w.blocks(), fixture_gguf["w." + t].reshape(-1))  # the upload is lossless
    w.release()


@pytest.mark.parametrize("fmt", GOLDEN_FORMATS)
def test_golden_dequantize(golden_cases, fmt):
    name = "gguf_dequant_" + fmt
    code, rows = golden_cases[name + ".attrs"]
    w = Tensor.quantized(CODE_TO_TYPE[int(code)], golden_cases[name + ".in0"], int(rows), 512)
    assert np.array_equal(bits(w.toFloatArray()), bits(golden_cases[name + ".out"].reshape(-1)))


@pytest.mark.parametrize("t", LINEAR_TYPES + EXTRA_TYPES)
@pytest.mark.parametrize("n,k", [(1, 256), (5, 768), (7, 11008)])
def test_dequantize_random_blocks_vs_oracle(t, n, k):
    raw = synth.random_valid_blocks(t, n, k, seed=n * 1000 + k).numpy()
    w = Tensor.quantized(t, raw, n, k)
    assert np.array_equal(bits(w.toFloatArray()), bits(oracle.dequantize(t, raw)))
    assert np.array_equal(w.blocks(), raw.reshape(-1))


# ---- linear: the reference's own vectors -----------------------------------------------------------
@pytest.mark.parametrize("rows", [1, 5, 40])
@pytest.mark.parametrize("fmt", GOLDEN_FORMATS)
def test_golden_linear(golden_cases, fmt, rows):
    name = "gguf_linear_%s_r%d" % (fmt, rows)
    code, n = golden_cases[name + ".attrs"]
    w = Tensor.quantized(CODE_TO_TYPE[int(code)], golden_cases[name + ".in1"], int(n), 512)
    y = Gguf.linear(golden_cases[name + ".in0"], w, golden_cases[name + ".in2"])
    assert y.shape == (rows, int(n))
    golden_close(golden_cases[name + ".out"], y, what=name)


@pytest.mark.parametrize("rows", [1, 5, 40])
@pytest.mark.parametrize("fmt", GOLDEN_FORMATS)
def test_golden_linear_input_gradient(golden_cases, fmt, rows):
    """The golden cases' gradient with respect to x for the loss sum(w * out): gx = w . dequant(W)."""
    name = "gguf_linear_%s_r%d" % (fmt, rows)
    code, n = golden_cases[name + ".attrs"]
    w = Tensor.quantized(CODE_TO_TYPE[int(code)], golden_cases[name + ".in1"], int(n), 512)
    gx = Gguf.linearBackward(golden_cases[name + ".w"], w)
    assert gx.shape == (rows, 512)
    golden_close(golden_cases[name + ".grad0"], gx, what=name + ".grad0")


@pytest.mark.parametrize("t", LINEAR_TYPES)
@pytest.mark.parametrize("n,k,m", [(300, 1024, 3), (4096, 4096, 8), (17, 256, 1), (11008, 4096, 5)])
def test_linear_backward_vs_oracle(t, n, k, m):
    """gx = g . dequant(W) against float64 over the oracle's dequantised weight, 1e-3 of the largest magnitude; device
    and host memory give the same bits."""
    import torch
    raw = synth.random_valid_blocks(t, n, k, seed=n + k + m).numpy()
    w = Tensor.quantized(t, raw, n, k)
    g = np.random.default_rng(n + m).standard_normal((m, n)).astype(np.float32)
    ref = g.astype(np.float64) @ oracle.dequantize(t, raw).reshape(n, k).astype(np.float64)
    gx = Gguf.linearBackward(g, w)
    assert np.abs(gx - ref).max() <= 1e-3 * np.abs(ref).max()
    gx_dev = Gguf.linearBackward(torch.from_numpy(g).cuda(), w).cpu().numpy()
    assert np.array_equal(bits(gx), bits(gx_dev))


def test_linear_backward_edges():
    raw = synth.random_valid_blocks("Q4_K", 8, 256, seed=1).numpy()
    w = Tensor.quantized("Q4_K", raw, 8, 256)
    assert Gguf.linearBackward(np.zeros((0, 8), np.float32), w).shape == (0, 256)
    with pytest.raises(ValueError, match="gradient"):
        Gguf.linearBackward(np.zeros((2, 9), np.float32), w)
    empty = Tensor.quantized("Q4_K", np.zeros(0, np.uint8), 0, 256)
    assert np.array_equal(Gguf.linearBackward(np.zeros((2, 0), np.float32), empty), np.zeros((2, 256), np.float32))


@pytest.mark.parametrize("t", LINEAR_TYPES)
def test_fixture_linear_like_gguf_checks(fixture_gguf, t):
    rng = np.random.default_rng(LINEAR_TYPES.index(t))
    w = Tensor.quantized(t, fixture_gguf["w." + t], 3, 512)
    expect = fixture_gguf["expect." + t].astype(np.float64)
    bias = np.array([0.25, -0.5, 1.0], dtype=np.float32)
    for rows in (1, 5, 40):
        x = (rng.random((rows, 512), dtype=np.float32) * 2 - 1).astype(np.float32)
        ref = (bias.astype(np.float64) + x.astype(np.float64) @ expect.T).astype(np.float32)
        close_like_reference(ref, Gguf.linear(x, w, bias), "%s linear, %d rows (host)" % (t, rows))
        yd = Gguf.linear(torch.from_numpy(x).cuda(), w, torch.from_numpy(bias).cuda())
        close_like_reference(ref, yd.cpu().numpy(), "%s linear, %d rows (device)" % (t, rows))


# ---- linear against the oracle on seeded inputs -------------------------------------------------------
@pytest.mark.parametrize("t", LINEAR_TYPES)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 7, 8, 13, 16, 17, 33])
def test_linear_rows_sweep_vs_oracle(t, m):
    n, k = 37, 1024
    raw = synth.random_valid_blocks(t, n, k, seed=m).numpy()
    rng = np.random.default_rng(100 + m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    w = Tensor.quantized(t, raw, n, k)
    expect = oracle.linear(t, raw, x, bias)
    got = Gguf.linear(x, w, bias)
    assert max_rel(expect, got) <= REL_TOL
    close_like_reference(expect, got, "%s m=%d" % (t, m))


@pytest.mark.parametrize("t", LINEAR_TYPES)
@pytest.mark.parametrize("n,k", [(1, 256), (3, 512), (23, 2816), (64, 11008), (130, 4096)])
def test_linear_shapes_vs_oracle(t, n, k):
    """Odd row counts and block counts: K = 11008 is 43 super-blocks per row, 2816 is 11."""
    raw = synth.random_valid_blocks(t, n, k, seed=n + k).numpy()
    rng = np.random.default_rng(n * 7 + k)
    w = Tensor.quantized(t, raw, n, k)
    for m in (1, 8):
        x = rng.standard_normal((m, k)).astype(np.float32)
        expect = oracle.linear(t, raw, x, None, threads=4)
        got = Gguf.linear(x, w, None)
        assert max_rel(expect, got) <= REL_TOL, (t, n, k, m)
        close_like_reference(expect, got, "%s [%d,%d] m=%d" % (t, n, k, m))


@pytest.mark.parametrize("t", ["Q4_K", "Q6_K", "Q8_0"])
def test_linear_synthetic_weights_vs_oracle(t):
    """Weights ~ N(0, 0.02) through the synthetic quantiser, activations ~ N(0, 1): the benchmark's inputs."""
    n, k = 256, 4096
    g = torch.Generator().manual_seed(11)
    wf = torch.randn(n, k, generator=g) * 0.02
    raw = oracle.quantize_q8_0(wf.numpy()) if t == "Q8_0" else synth.QUANTIZERS[t](wf).numpy()
    w = Tensor.quantized(t, raw, n, k)
    x = torch.randn(8, k, generator=g).numpy()
    for m in (1, 8):
        expect = oracle.linear(t, raw, x[:m], None, threads=4)
        assert max_rel(expect, Gguf.linear(x[:m], w, None)) <= REL_TOL


def test_leading_axes_are_flattened_and_restored():
    raw = synth.random_valid_blocks("Q4_K", 20, 512, seed=5).numpy()
    w = Tensor.quantized("Q4_K", raw, 20, 512)
    x = np.random.default_rng(44).uniform(-1, 1, (2, 3, 512)).astype(np.float32)
    y = Gguf.linear(x, w, None)
    assert y.shape == (2, 3, 20)
    close_like_reference(oracle.linear("Q4_K", raw, x.reshape(6, 512)), y.reshape(6, 20))


# ---- Q8_0 operators (OpsAccelTest.q8 of the reference) -------------------------------------------------
def test_q8_quantise_bit_exact_and_linear():
    rng = np.random.default_rng(41)
    x = rng.uniform(-1, 1, (6, 256)).astype(np.float32)
    wf = rng.uniform(-0.5, 0.5, (300, 256)).astype(np.float32)
    wf[7, 64:96] = 0
    blocks = Quant.quantizeQ8Blocks(wf)
    assert np.array_equal(blocks, oracle.quantize_q8_0(wf))
    dev_blocks = Quant.quantizeQ8Blocks(torch.from_numpy(wf).cuda())
    assert np.array_equal(dev_blocks.cpu().numpy(), blocks)
    qw = F.quantizeQ8(wf)
    back = F.dequantize(qw)
    assert np.abs(back - wf).max() <= 0.5 / 127 + 1e-6
    bias = rng.uniform(-1, 1, 300).astype(np.float32)
    expect = oracle.linear("Q8_0", blocks, x, bias)
    got = F.linearQ8(x, qw, bias)
    assert np.allclose(got, expect, rtol=1e-5, atol=1e-5)
    xb = rng.uniform(-1, 1, (2, 3, 256)).astype(np.float32)
    assert np.allclose(F.linearQ8(xb, qw, None).reshape(6, 300), oracle.linear("Q8_0", blocks, xb.reshape(6, 256)), rtol=1e-5, atol=1e-5)
    exact = x.astype(np.float64) @ wf.astype(np.float64).T
    quantised = F.linearQ8(x, qw, None)
    assert np.sqrt(((exact - quantised) ** 2).sum() / (exact ** 2).sum()) < 0.01


# ---- sharding by output rows: bitwise equal to the whole weight ------------------------------------------
@pytest.mark.parametrize("t", LINEAR_TYPES)
def test_row_shards_concatenate_bitwise(t):
    n, k = 48, 1024
    raw = synth.random_valid_blocks(t, n, k, seed=9).numpy()
    x = np.random.default_rng(9).standard_normal((3, k)).astype(np.float32)
    whole = Gguf.linear(x, Tensor.quantized(t, raw, n, k), None)
    for shards in (2, 4, 8):
        parts = []
        for g in range(shards):
            ws = Tensor.quantized(t, raw, n, k, rows=(g * n // shards, (g + 1) * n // shards))
            assert ws.shape() == (n // shards, k)
            parts.append(Gguf.linear(x, ws, None))
        assert np.array_equal(bits(np.concatenate(parts, axis=1)), bits(whole))


# ---- error behaviour -------------------------------------------------------------------------------------
def test_misuse_raises_like_the_reference():
    raw = synth.random_valid_blocks("Q4_K", 4, 512, seed=1).numpy()
    w = Tensor.quantized("Q4_K", raw, 4, 512)
    with pytest.raises(ValueError, match=r"Q4_K linear: input \[2, 256\] and weight \[4, 512\]"):
        Gguf.linear(np.zeros((2, 256), np.float32), w)
    with pytest.raises(ValueError, match="FP32"):
        Gguf.linear(np.zeros((2, 512), np.float64), w)
    with pytest.raises(ValueError, match="Q8_0 linear"):
        Quant.linear(np.zeros((2, 512), np.float32), w)
    q2 = Tensor.quantized("Q2_K", synth.random_valid_blocks("Q2_K", 2, 256, seed=2).numpy(), 2, 256)
    with pytest.raises(ValueError, match="dequantise-only"):
        Gguf.linear(np.zeros((1, 256), np.float32), q2)
    assert Gguf.linear(np.zeros((0, 512), np.float32), w).shape == (0, 4)
    w.release()
    with pytest.raises(RuntimeError, match="released"):
        Gguf.linear(np.zeros((1, 512), np.float32), w)


def test_full_size_linearity_property():
    """At a benchmark shape, where the oracle would take minutes: W(a x1 + b x2) = a W x1 + b W x2,
    and a one-hot activation reads back one dequantised column exactly."""
    n, k = 4096, 4096
    g = torch.Generator().manual_seed(3)
    raw = synth.quantize_q4_k((torch.randn(n, k, generator=g) * 0.02).cuda()).cpu().numpy()
    w = Tensor.quantized("Q4_K", raw, n, k)
    x = torch.randn(2, k, generator=g).numpy()
    y = Gguf.linear(x, w, None)
    combo = (0.5 * x[0] - 2.0 * x[1]).astype(np.float32)[None]
    assert max_rel(0.5 * y[0] - 2.0 * y[1], Gguf.linear(combo, w, None)[0]) < 1e-5
    onehot = np.zeros((1, k), np.float32)
    onehot[0, 1234] = 1.0
    col = Gguf.dequantize(w)[:, 1234]
    assert np.array_equal(bits(Gguf.linear(onehot, w, None)[0]), bits(col))
    sample = oracle.linear("Q4_K", raw[:64], x, None, threads=4)
    assert max_rel(sample, y[:, :64]) <= REL_TOL


def test_full_size_q8_round_trip_and_gradient_properties():
    """Size-independent properties at BASELINE configs[0]'s shape (4096 x 4096, Q8_0): quantise -> dequantise -> quantise
    gives the same blocks (every non-zero block has a value of magnitude 127, so its scale survives the round trip);
    the input gradient is linear in g, and a one-hot g reads back one dequantised row exactly."""
    n, k = 4096, 4096
    g = torch.Generator().manual_seed(17)
    wf = (torch.randn(n, k, generator=g) * 0.02).cuda()
    blocks = Quant.quantizeQ8Blocks(wf)
    w = Tensor.quantized("Q8_0", blocks.cpu().numpy(), n, k)
    back = torch.empty(n, k, device="cuda")
    Quant.dequantize(w, back)
    assert torch.equal(Quant.quantizeQ8Blocks(back), blocks)
    assert float((back - wf).abs().max()) <= float(wf.abs().max()) / 127 * 0.5 + 1e-7
    g2 = torch.randn(2, n, generator=g).cuda()
    gx = Gguf.linearBackward(g2, w)
    combo = (0.25 * g2[0] + 3.0 * g2[1])[None].contiguous()
    assert max_rel((0.25 * gx[0] + 3.0 * gx[1]).cpu().numpy(), Gguf.linearBackward(combo, w)[0].cpu().numpy()) < 1e-5
    onehot = torch.zeros(1, n, device="cuda")
    onehot[0, 321] = 1.0
    assert torch.equal(Gguf.linearBackward(onehot, w)[0], back[321])


def test_page_locked_host_buffers_are_used_in_place():
    """jq_linear_f32 with page-locked host x, bias and y (kernels read and write them across PCIe, no staging copies) gives
    bit for bit what the same call gives with pageable buffers; a large output still goes through a copy."""
    import ctypes
    from jitnn_b200 import _lib
    L = _lib.load()
    for t, n, k, m in [("Q4_K", 1024, 1024, 1), ("Q6_K", 640, 512, 3), ("Q8_0", 256, 512, 2), ("Q4_K", 16400, 256, 8)]:
        raw = synth.random_valid_blocks(t, n, k, seed=n + m).numpy()
        w = Tensor.quantized(t, raw, n, k)
        g = torch.Generator().manual_seed(n)
        x, bias = torch.randn(m, k, generator=g), torch.randn(n, generator=g)
        pageable = Gguf.linear(x.numpy(), w, bias.numpy())
        xp, bp, yp = x.pin_memory(), bias.pin_memory(), torch.empty(m, n).pin_memory()
        _lib.check(L.jq_linear_f32(w._handle(), xp.data_ptr(), m, bp.data_ptr(), yp.data_ptr(), _lib.JQ_MEM_HOST, None))
        assert np.array_equal(bits(yp.numpy()), bits(pageable)), (t, n, k, m)
