"""Extracts the reference's own test vectors for the quantised-linear path into small .npz files.

Run once in a container that has the reference tree (the GPU machine does not):

    python tests/golden/make_golden.py <path of the reference checkout>

Sources (paths inside the reference project):
  * jitnn-gguf/src/test/resources/gguf/fixture.gguf          -> gguf_fixture.npz
    tensors ``w.<T>`` (raw blocks, [3, 512]) and ``expect.<T>`` (float32) for the block formats,
    written by the reference's scripts/gguf/gguf_fixture.py with llama.cpp's ``gguf`` package.
  * jitnn-core/src/test/resources/golden/{manifest.txt,data.bin} -> golden_gguf_cases.npz
    the 15 ``gguf_linear_*`` and 5 ``gguf_dequant_*`` cases written by scripts/pytorch/goldens.py
    (manifest format: ``case <name> <op> <attrs>`` lines, then ``<name> <role> <f32|i32> <offset>
    <dims...>`` lines addressing little-endian arrays in data.bin).
  * the same two files -> golden_decoder_ops.npz: the cases of the operators the decoder is made of
    (rms_norm*, rope_heads, sdpa_bthd_causal, silu*, swiglu, embedding*, argmax), inputs and expected
    outputs only (the gradients are left out), which pin the decoder oracle operator by operator.
  * jitnn-gguf/src/test/resources/gguf/fixture.gguf is also copied as it is (106 400 bytes): the reader tests
    parse the reference's own file, not only files from this project's writer.
The parser for the GGUF file is written here (header, metadata skip, tensor table) so that the
extraction does not depend on any package.
"""
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BLOCK = {2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 10: (256, 84), 11: (256, 110),
         12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292)}
NAMES = {2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K"}
SCALAR = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}


def read_gguf_tensors(path):
    data = open(path, "rb").read()
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from("<" + fmt, data, pos)
        pos += struct.calcsize("<" + fmt)
        return v[0]

    def string():
        nonlocal pos
        n = take("Q")
        s = data[pos:pos + n].decode("utf-8")
        pos += n
        return s

    def value(t):
        if t in SCALAR:
            return take(SCALAR[t])
        if t == 8:
            return string()
        if t == 9:
            sub = take("I")
            return [value(sub) for _ in range(take("Q"))]
        raise ValueError("metadata type %d" % t)

    assert take("I") == 0x46554747
    assert take("I") in (2, 3)
    n_tensors, n_kv = take("Q"), take("Q")
    meta = {}
    for _ in range(n_kv):
        key = string()
        meta[key] = value(take("I"))
    infos = []
    for _ in range(n_tensors):
        name = string()
        nd = take("I")
        dims = [take("Q") for _ in range(nd)]
        infos.append((name, dims[::-1], take("I"), take("Q")))
    align = meta.get("general.alignment", 32)
    base = (pos + align - 1) // align * align
    out = {}
    for name, dims, typ, off in infos:
        numel = int(np.prod(dims))
        if typ == 0:
            out[name] = np.frombuffer(data, dtype="<f4", count=numel, offset=base + off).reshape(dims).copy()
        elif typ in BLOCK and typ in NAMES:
            qk, nb = BLOCK[typ]
            out[name] = np.frombuffer(data, dtype=np.uint8, count=numel // qk * nb, offset=base + off).reshape(dims[0], -1).copy()
    return out


DECODER_CASES = ("rms_norm", "rms_norm_3d", "rms_norm_long", "rms_norm_rows", "rope_heads", "sdpa_bthd_causal", "silu", "silu_tails", "swiglu",
                 "embedding", "embedding_padding", "embedding_wide", "argmax")


def read_golden_cases(root, decoder_ops=False):
    res = os.path.join(root, "jitnn-core/src/test/resources/golden")
    blob = open(os.path.join(res, "data.bin"), "rb").read()
    cases, arrays = {}, {}
    for line in open(os.path.join(res, "manifest.txt")):
        p = line.split()
        if not p:
            continue
        if p[0] == "case":
            if (p[1] in DECODER_CASES) if decoder_ops else (p[2] in ("gguf_linear", "gguf_dequant")):
                cases[p[1]] = (p[2], [float(a) for a in p[3:]])
        elif p[0] in cases:
            name, role, kind, off = p[0], p[1], p[2], int(p[3])
            if decoder_ops and (role.startswith("grad") or role == "w"):
                continue
            dims = [int(d) for d in p[4:]]
            a = np.frombuffer(blob, dtype="<f4" if kind == "f32" else "<i4", count=int(np.prod(dims)), offset=off).reshape(dims)
            if kind == "i32" and not decoder_ops:
                assert a.min() >= 0 and a.max() <= 255
                a = a.astype(np.uint8)
            arrays["%s.%s" % (name, role)] = a.copy()
    for name, (op, attrs) in cases.items():
        arrays["%s.attrs" % name] = np.array(attrs, dtype=np.float64 if decoder_ops else np.int32)
    return arrays


def main(root):
    tensors = read_gguf_tensors(os.path.join(root, "jitnn-gguf/src/test/resources/gguf/fixture.gguf"))
    keep = {}
    for t in NAMES.values():
        keep["w." + t] = tensors["w." + t]
        keep["expect." + t] = tensors["expect." + t]
        assert keep["expect." + t].shape == (3, 512)
    np.savez_compressed(os.path.join(HERE, "gguf_fixture.npz"), **keep)
    cases = read_golden_cases(root)
    np.savez_compressed(os.path.join(HERE, "golden_gguf_cases.npz"), **cases)
    ops = read_golden_cases(root, decoder_ops=True)
    assert all(name + ".out" in ops for name in DECODER_CASES)
    np.savez_compressed(os.path.join(HERE, "golden_decoder_ops.npz"), **ops)
    with open(os.path.join(root, "jitnn-gguf/src/test/resources/gguf/fixture.gguf"), "rb") as src, open(os.path.join(HERE, "fixture.gguf"), "wb") as dst:
        dst.write(src.read())
    print("fixture tensors:", len(keep), "golden arrays:", len(cases), "decoder operator arrays:", len(ops))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
