"""The GGUF reader (jq_gguf_*, C++ inside the library) on files made by tests/gguf_writer.py: the tensor table and
metadata come back as written, tensor bytes are the reference fixture's blocks, and the hostile inputs of the
reference's GgufFileTest (:115-155) are refused with an error instead of a read outside the file."""
import os
import struct

import numpy as np
import pytest

import gguf_writer
from conftest import GOLDEN
from jitnn_b200 import gguf

# the reference fixture's tensors (w.<T> raw blocks, expect.<T> float32), extracted to npz by tests/golden/make_golden.py
FIXTURE = os.path.join(GOLDEN, "gguf_fixture.npz")
TYPE_IDS = {"Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14}


def make_file(path, alignment=32):
    fx = np.load(FIXTURE)
    tensors = [("w." + t, (3, 512), tid, fx["w." + t].tobytes()) for t, tid in TYPE_IDS.items() if "w." + t in fx]
    tensors.append(("expect.Q4_K", (3, 512), 0, fx["expect.Q4_K"].astype("<f4").tobytes()))
    tensors.append(("odd.type", (4,), 999, b""))
    meta = [("general.architecture", "str", "llama"), ("llama.block_count", "u32", 2), ("llama.rope.freq_base", "f32", 10000.0),
            ("tokenizer.ggml.tokens", "arr", ("str", ["a", "bc", "def"])), ("x.nested", "arr", ("arr", [("i32", [1, 2]), ("i32", [3])])),
            ("x.flag", "bool", 1), ("x.big", "u64", 2 ** 40 + 5)]
    gguf_writer.write(path, tensors, meta, alignment=alignment)
    return fx, tensors


@pytest.mark.parametrize("alignment", [32, 64])
def test_reads_back_what_was_written(tmp_path, alignment):
    p = tmp_path / "m.gguf"
    fx, tensors = make_file(p, alignment)
    with gguf.GgufFile(p) as f:
        assert (f.version, f.alignment) == (3, alignment)
        assert f.data_offset % alignment == 0
        assert list(f.tensors) == [t[0] for t in tensors]
        for name, shape, tid, data in tensors[:-1]:
            info = f.info(name)
            assert (info.shape, info.ggml_type, info.nbytes) == (tuple(shape), tid, len(data))
            assert info.offset % alignment == 0
            assert f.raw(name).tobytes() == data
        assert f.info("odd.type").nbytes == -1
        with pytest.raises(Exception, match="unknown"):
            f.raw("odd.type")
        with pytest.raises(ValueError, match="no tensor"):
            f.info("no.such.tensor")
        assert f.string("general.architecture") == "llama"
        assert f.number("llama.block_count") == 2 and f.number("x.flag") == 1 and f.number("x.big") == 2 ** 40 + 5
        assert f.number("llama.rope.freq_base") == 10000.0
        with pytest.raises(ValueError, match="not a number"):
            f.number("tokenizer.ggml.tokens")
        with pytest.raises(ValueError, match="no metadata key"):
            f.string("absent")


def crafted(dim, offset, metadata=b"", kv_count=0, version=3, ndims=1):
    """A header with one F32 tensor of the given innermost dimension and offset, then 64 bytes of data."""
    out = struct.pack("<IIQQ", 0x46554747, version, 1, kv_count) + metadata
    out += struct.pack("<Q", 1) + b"w" + struct.pack("<I", ndims) + struct.pack("<Q", dim & (2 ** 64 - 1)) * ndims + struct.pack("<IQ", 0, offset & (2 ** 64 - 1))
    return out + b"\0" * 96


def test_refuses_hostile_files(tmp_path):
    def refused(name, data, match):
        p = tmp_path / name
        p.write_bytes(data)
        with pytest.raises(ValueError, match=match):
            gguf.GgufFile(p)

    refused("zeros.bin", bytes(64), "not a GGUF file")
    refused("short.bin", b"GGUF", "not a GGUF file")
    refused("v1.gguf", crafted(4, 0, version=1), "version 1 is not supported")
    good = tmp_path / "good.gguf"
    make_file(good)
    whole = good.read_bytes()
    refused("truncated.gguf", whole[:600], "truncated|outside the file")
    refused("cut_in_table.gguf", whole[:200], "truncated")
    refused("dim.gguf", crafted(-1, 0), "dimension")                          # 2^64 - 1
    refused("offset.gguf", crafted(4, 2 ** 63 - 32), "offset|outside")        # overflows past the data start
    refused("outside.gguf", crafted(1 << 20, 0), "outside the file")
    refused("unaligned.gguf", crafted(4, 8), "not aligned")
    refused("overflow.gguf", crafted(2 ** 62, 0, ndims=2), "overflows")       # 2^124 elements
    refused("count.gguf", struct.pack("<IIQQ", 0x46554747, 3, 2 ** 60, 0) + bytes(64), "exceeds the file")
    deep = struct.pack("<Q", 4) + b"deep" + struct.pack("<I", 9)
    for _ in range(200):                                                      # arrays nested 200 deep
        deep += struct.pack("<IQ", 9, 1)
    deep += struct.pack("<IQ", 4, 0)
    refused("deep.gguf", crafted(4, 0, deep, 1), "nested deeper")
    bad_align = struct.pack("<Q", 17) + b"general.alignment" + struct.pack("<II", 4, 24)
    refused("align.gguf", crafted(4, 0, bad_align, 1), "not a power of two")
    bad_type = struct.pack("<Q", 1) + b"k" + struct.pack("<I", 77)
    refused("vtype.gguf", crafted(4, 0, bad_type, 1), "value type 77")
    huge_string = struct.pack("<Q", 1) + b"k" + struct.pack("<IQ", 8, 2 ** 50)
    refused("string.gguf", crafted(4, 0, huge_string, 1), "exceeds the file")
    with pytest.raises(ValueError, match="cannot be opened"):
        gguf.GgufFile(tmp_path / "absent.gguf")


@pytest.mark.gpu
def test_weights_upload_from_the_mapping(tmp_path):
    import torch
    from jitnn_b200 import Gguf
    p = tmp_path / "m.gguf"
    fx, _ = make_file(p)
    with gguf.GgufFile(p) as f:
        for t in ("Q4_K", "Q6_K", "Q8_0"):
            w = f.weight("w." + t)
            assert w.shape() == (3, 512)
            got = Gguf.dequantize(w)
            assert np.array_equal(np.asarray(got).view(np.uint32), fx["expect." + t].astype(np.float32).reshape(3, 512).view(np.uint32))
            shard = f.weight("w." + t, rows=(1, 3))
            assert np.array_equal(np.asarray(Gguf.dequantize(shard)), np.asarray(got)[1:3])
        with pytest.raises(ValueError, match="2-D tensor of a known type"):
            f.weight("odd.type")


# ---- the reference's own fixture file (jitnn-gguf/src/test/resources/gguf/fixture.gguf, copied by tests/golden/make_golden.py) ----
REFERENCE_FILE = os.path.join(GOLDEN, "fixture.gguf")


def meta_kind(f, key):
    import ctypes
    from jitnn_b200 import _lib
    vt, n, et = ctypes.c_int(), ctypes.c_int64(), ctypes.c_int()
    _lib.check(f._lib.jq_gguf_meta_find(f._h, key.encode(), ctypes.byref(vt), ctypes.byref(n), ctypes.byref(et)))
    return vt.value, n.value, et.value


def test_reference_fixture_header_and_metadata_of_every_type():
    """GgufFileTest.header and .metadataOfEveryType (GgufFileTest.java:41-86): version, alignment, the 13 value types."""
    with gguf.GgufFile(REFERENCE_FILE) as f:
        assert (f.version, f.alignment) == (3, 32)
        assert f.data_offset % 32 == 0
        assert len(f.tensors) == 30
        assert f.string("general.architecture") == "llama"
        assert f.number("test.u8") == 250 and f.number("test.i8") == -100
        assert f.number("test.u16") == 60000 and f.number("test.i16") == -30000
        assert f.number("test.u32") == 3_000_000_000 and f.number("test.i32") == -2_000_000_000
        assert f.number("test.f32") == 1.5 and f.number("test.bool") == 1
        assert f.string("test.string") == "héllo, wörld"
        assert f.number("test.u64") == (1 << 40) + 3 and f.number("test.i64") == -(1 << 40)
        assert f.number("test.f64") == 2.25
        assert f.number("llama.block_count") == 2
        # arrays: found with their element type and length (type ids of the GGUF specification: 4 u32, 5 i32, 6 f32, 7 bool, 8 string, 9 array, 12 f64)
        assert meta_kind(f, "test.ints") == (9, 3, 5) and meta_kind(f, "test.floats") == (9, 2, 6)
        assert meta_kind(f, "test.strings") == (9, 3, 8) and meta_kind(f, "test.bools") == (9, 2, 7)
        assert meta_kind(f, "test.nested") == (9, 2, 9) and meta_kind(f, "test.u32s") == (9, 2, 4) and meta_kind(f, "test.f64s") == (9, 2, 12)
        with pytest.raises(ValueError, match="no metadata key"):
            f.string("llama.missing")
        with pytest.raises(ValueError):
            f.string("test.u8")


def test_reference_fixture_tensor_table():
    """GgufFileTest.shapesInJitnnOrder and .typesWithoutJitnnCounterpart (:88-113): shapes outermost first, 1-D / 3-D / I32
    tensors, a block type this library has no kernels for."""
    fx = np.load(FIXTURE)
    with gguf.GgufFile(REFERENCE_FILE) as f:
        q = f.info("w.Q4_K")
        assert (q.shape, q.ggml_type, q.nbytes) == ((3, 512), 12, 3 * 512 // 256 * 144)
        assert f.info("axes.1d").shape == (5,) and f.info("axes.3d").shape == (2, 3, 4)
        assert np.array_equal(f.raw("axes.3d").view("<f4"), np.arange(24, dtype=np.float32))  # numpy's row-major order is jitNN's
        assert np.array_equal(f.raw("axes.1d").view("<f4"), np.arange(5, dtype=np.float32))
        ints = f.info("ints.I32")
        assert ints.ggml_type == 26 and list(f.raw("ints.I32").view("<i4")) == [1, -2, 3, 4, 5, -6]
        q8k = f.info("w.Q8_K")
        assert q8k.ggml_type == 15 and q8k.nbytes == 3 * 512 // 256 * 292 and f.raw("w.Q8_K").size == q8k.nbytes
        with pytest.raises(ValueError, match="no tensor"):
            f.info("no.such.tensor")
        for t in TYPE_IDS:  # the block tensors are byte for byte what make_golden.py extracted with its own parser
            assert f.raw("w." + t).tobytes() == fx["w." + t].tobytes()
            assert f.raw("expect." + t).tobytes() == fx["expect." + t].astype("<f4").tobytes()


@pytest.mark.gpu
def test_reference_fixture_uploads_and_dequantises_bit_exactly():
    """Every block tensor of the reference's file, uploaded straight from the mapping, dequantises to its expect.<T> bit for bit;
    the type without kernels is refused."""
    from jitnn_b200 import Gguf, Quant
    with gguf.GgufFile(REFERENCE_FILE) as f:
        for t in TYPE_IDS:
            w = f.weight("w." + t)
            got = w.toFloatArray()
            assert np.array_equal(got.view(np.uint32), f.raw("expect." + t).view(np.uint32)), t
            w.release()
        with pytest.raises(ValueError):
            f.weight("w.Q8_K")
