"""A minimal GGUF v3 writer for the tests (this project's own code, following the published container layout):
header, metadata key/values, tensor table with the innermost dimension first, data section on the alignment grid."""
import struct

import numpy as np

VALUE_TYPES = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "arr": 9, "u64": 10, "i64": 11, "f64": 12}
PACK = {"u8": "<B", "i8": "<b", "u16": "<H", "i16": "<h", "u32": "<I", "i32": "<i", "f32": "<f", "bool": "<B", "u64": "<Q", "i64": "<q", "f64": "<d"}


def _string(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _value(kind, v):
    if kind == "str":
        return _string(v)
    if kind == "arr":  # v = (element kind, list)
        ek, items = v
        return struct.pack("<IQ", VALUE_TYPES[ek], len(items)) + b"".join(_value(ek, i) for i in items)
    return struct.pack(PACK[kind], v)


def header(tensor_count, metadata, version=3):
    out = struct.pack("<IIQQ", 0x46554747, version, tensor_count, len(metadata))
    for key, kind, v in metadata:
        out += _string(key) + struct.pack("<I", VALUE_TYPES[kind]) + _value(kind, v)
    return out


def tensor_entry(name, shape, ggml_type, offset):
    out = _string(name) + struct.pack("<I", len(shape))
    for d in reversed(shape):
        out += struct.pack("<Q", d)
    return out + struct.pack("<IQ", ggml_type, offset)


def write(path, tensors, metadata=(), alignment=32, version=3):
    """tensors: list of (name, shape outermost first, ggml type id, bytes-like)."""
    meta = list(metadata)
    if alignment != 32:
        meta.append(("general.alignment", "u32", alignment))
    head = header(len(tensors), meta, version)
    offsets, pos = [], 0
    for _, _, _, data in tensors:
        offsets.append(pos)
        pos += (len(bytes(data)) + alignment - 1) // alignment * alignment
    for (name, shape, t, _), off in zip(tensors, offsets):
        head += tensor_entry(name, shape, t, off)
    pad = (-len(head)) % alignment
    body = b""
    for (_, _, _, data), off in zip(tensors, offsets):
        raw = bytes(np.asarray(data).tobytes() if not isinstance(data, (bytes, bytearray)) else data)
        body += raw + b"\0" * ((-len(raw)) % alignment)
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad + body)
    return len(head) + pad
