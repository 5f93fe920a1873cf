"""Quantisers that turn float32 weights into valid GGUF blocks, for synthetic benchmarks and tests.

The reference only ever *consumes* K-quant blocks (its fixtures are random bytes); it has no
Q4_K/Q5_K/Q6_K/Q4_0/Q4_1 quantiser to match. These are simple min/max quantisers of this project's
own design, written with torch tensor ops so they run on the CPU or on a GPU: parity is defined
downstream of the blocks, so any quantiser that emits valid blocks is admissible.

Every function takes a float32 tensor [N, K] and returns a uint8 tensor [N, K/QK*B] of raw blocks
in GGUF's byte layout.
"""
import torch


def _half_bytes(v):
    """float32 [...,] -> uint8 [..., 2] holding the little-endian fp16 of v."""
    return v.to(torch.float16).contiguous().view(torch.uint8).reshape(*v.shape, 2)


def _half_round(v):
    return v.to(torch.float16).to(torch.float32)


def quantize_q4_0(w):
    n, k = w.shape
    b = w.reshape(n, k // 32, 32).float()
    d = _half_round(b.abs().amax(dim=-1) / 7.0)
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.clamp(torch.round(b * inv[..., None]) + 8, 0, 15).to(torch.uint8)
    packed = q[..., :16] | (q[..., 16:] << 4)
    return torch.cat([_half_bytes(d), packed], dim=-1).reshape(n, -1)


def quantize_q4_1(w):
    n, k = w.shape
    b = w.reshape(n, k // 32, 32).float()
    lo = _half_round(b.amin(dim=-1))
    d = _half_round((b.amax(dim=-1) - lo) / 15.0)
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.clamp(torch.round((b - lo[..., None]) * inv[..., None]), 0, 15).to(torch.uint8)
    packed = q[..., :16] | (q[..., 16:] << 4)
    return torch.cat([_half_bytes(d), _half_bytes(lo), packed], dim=-1).reshape(n, -1)


def _pack_k_scales(sc, mn):
    """8 six-bit scales and 8 six-bit mins -> the 12 bytes of Q4_K/Q5_K (see GgufKernels.scaleMin)."""
    sc = sc.to(torch.uint8)
    mn = mn.to(torch.uint8)
    out = torch.empty(*sc.shape[:-1], 12, dtype=torch.uint8, device=sc.device)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 15) | ((mn[..., 4:8] & 15) << 4)
    return out


def _k_scales(b, levels):
    """b [..., 8, 32] -> fp16-rounded d, dmin and integer sub-block scales/mins for `levels` steps."""
    lo = torch.clamp(b.amin(dim=-1), max=0.0)
    offset = -lo
    step = (b.amax(dim=-1) + offset) / float(levels)
    d = _half_round(step.amax(dim=-1) / 63.0)
    dmin = _half_round(offset.amax(dim=-1) / 63.0)
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    inv_m = torch.where(dmin > 0, 1.0 / dmin, torch.zeros_like(dmin))
    sc = torch.clamp(torch.round(step * inv_d[..., None]), 0, 63)
    mn = torch.clamp(torch.round(offset * inv_m[..., None]), 0, 63)
    eff = d[..., None] * sc
    inv = torch.where(eff > 0, 1.0 / eff, torch.zeros_like(eff))
    q = torch.clamp(torch.round((b + (dmin[..., None] * mn)[..., None]) * inv[..., None]), 0, levels)
    return d, dmin, sc, mn, q.to(torch.uint8)


def quantize_q4_k(w):
    n, k = w.shape
    b = w.reshape(n, k // 256, 8, 32).float()
    d, dmin, sc, mn, q = _k_scales(b, 15)
    q = q.reshape(n, k // 256, 4, 2, 32)
    qs = (q[..., 0, :] | (q[..., 1, :] << 4)).reshape(n, k // 256, 128)
    return torch.cat([_half_bytes(d), _half_bytes(dmin), _pack_k_scales(sc, mn), qs], dim=-1).reshape(n, -1)


def quantize_q5_k(w):
    n, k = w.shape
    b = w.reshape(n, k // 256, 8, 32).float()
    d, dmin, sc, mn, q = _k_scales(b, 31)
    low = (q & 15).reshape(n, k // 256, 4, 2, 32)
    qs = (low[..., 0, :] | (low[..., 1, :] << 4)).reshape(n, k // 256, 128)
    bits = (q >> 4).to(torch.int32)  # [n, blocks, 8, 32]
    shifts = torch.arange(8, device=w.device, dtype=torch.int32).reshape(1, 1, 8, 1)
    qh = (bits << shifts).sum(dim=2).to(torch.uint8)
    return torch.cat([_half_bytes(d), _half_bytes(dmin), _pack_k_scales(sc, mn), qh, qs], dim=-1).reshape(n, -1)


def quantize_q6_k(w):
    n, k = w.shape
    nb = k // 256
    b = w.reshape(n, nb, 16, 16).float()
    amax = b.abs().amax(dim=-1)
    step = amax / 31.0
    d = _half_round(step.amax(dim=-1) / 127.0)
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    sc = torch.clamp(torch.round(step * inv_d[..., None]), 0, 127)
    eff = d[..., None] * sc
    inv = torch.where(eff > 0, 1.0 / eff, torch.zeros_like(eff))
    q = (torch.clamp(torch.round(b * inv[..., None]), -32, 31) + 32).to(torch.uint8).reshape(n, nb, 2, 4, 32)
    low = q & 15
    high = q >> 4
    # element e = 128 h + 32 kk + l: ql[64 h + l + 32 (kk % 2)] nibble (kk / 2), qh[32 h + l] bits 2 kk
    ql = torch.cat([low[:, :, :, 0] | (low[:, :, :, 2] << 4), low[:, :, :, 1] | (low[:, :, :, 3] << 4)], dim=-1).reshape(n, nb, 128)
    qh = (high[:, :, :, 0] | (high[:, :, :, 1] << 2) | (high[:, :, :, 2] << 4) | (high[:, :, :, 3] << 6)).reshape(n, nb, 64)
    scales = sc.to(torch.int8).view(torch.uint8)
    return torch.cat([ql, qh, scales, _half_bytes(d)], dim=-1).reshape(n, -1)


QUANTIZERS = {"Q4_0": quantize_q4_0, "Q4_1": quantize_q4_1, "Q4_K": quantize_q4_k, "Q5_K": quantize_q5_k, "Q6_K": quantize_q6_k}


def random_valid_blocks(dtype_name, n, k, seed, device="cpu"):
    """Uniformly random bytes with the fp16 fields forced into U(0.002, 0.03): the adversarial blocks
    the reference's own fixtures use (scripts/gguf/gguf_fixture.py:44-49 of the reference)."""
    geo = {"Q8_0": (32, 34, [0]), "Q4_0": (32, 18, [0]), "Q4_1": (32, 20, [0, 2]), "Q4_K": (256, 144, [0, 2]),
           "Q5_K": (256, 176, [0, 2]), "Q6_K": (256, 210, [208]), "Q5_0": (32, 22, [0]), "Q5_1": (32, 24, [0, 2]),
           "Q2_K": (256, 84, [80, 82]), "Q3_K": (256, 110, [108])}[dtype_name]
    qk, nb, offs = geo
    g = torch.Generator(device="cpu").manual_seed(seed)
    raw = torch.randint(0, 256, (n * k // qk, nb), generator=g, dtype=torch.uint8)
    for off in offs:
        v = torch.rand(raw.shape[0], generator=g) * 0.028 + 0.002
        raw[:, off:off + 2] = _half_bytes(v)
    return raw.reshape(n, k // qk * nb).to(device)
