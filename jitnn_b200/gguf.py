"""GGUF files: the mirror of the reference's ``GgufFile`` (jitnn-gguf/.../GgufFile.java:100-175,329-418) over the
library's reader (``jq_gguf_*``): open, list tensors and metadata, view a tensor's bytes, upload a weight.

Parsing, bounds checks and the upload are C++ inside the library; this module only forwards. A malformed file raises
``ValueError`` with the library's message (the reference throws ``IOException``).
"""
import ctypes

import numpy as np

from . import _lib


class TensorInfo:
    def __init__(self, index, name, ggml_type, shape, offset, nbytes):
        self.index, self.name, self.ggml_type, self.shape, self.offset, self.nbytes = index, name, ggml_type, shape, offset, nbytes

    def __repr__(self):
        return "TensorInfo(%r, type %d, shape %s, offset %d, %d bytes)" % (self.name, self.ggml_type, self.shape, self.offset, self.nbytes)


class GgufFile:
    def __init__(self, path):
        self._lib = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(self._lib.jq_gguf_open(str(path).encode(), ctypes.byref(h)))
        self._h = h
        ver, al, off, nt, nm = ctypes.c_int(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        _lib.check(self._lib.jq_gguf_info(h, ctypes.byref(ver), ctypes.byref(al), ctypes.byref(off), ctypes.byref(nt), ctypes.byref(nm)))
        self.version, self.alignment, self.data_offset, self.metadata_count = ver.value, al.value, off.value, nm.value
        self.tensors = {}
        for i in range(nt.value):
            name, t, nd = ctypes.c_char_p(), ctypes.c_int(), ctypes.c_int()
            dims, o, nb = (ctypes.c_int64 * 8)(), ctypes.c_int64(), ctypes.c_int64()
            _lib.check(self._lib.jq_gguf_tensor(h, i, ctypes.byref(name), ctypes.byref(t), ctypes.byref(nd), dims, ctypes.byref(o), ctypes.byref(nb)))
            info = TensorInfo(i, name.value.decode(), t.value, tuple(dims[d] for d in range(nd.value)), o.value, nb.value)
            self.tensors[info.name] = info

    def _live(self):
        if self._h is None:
            raise RuntimeError("the GGUF file is closed")
        return self._h

    def info(self, name):
        if name not in self.tensors:
            raise ValueError("no tensor %s" % name)
        return self.tensors[name]

    def raw(self, name):
        """The tensor's bytes as a numpy uint8 array (a copy of the mapped bytes)."""
        t = self.info(name)
        p = ctypes.c_void_p()
        _lib.check(self._lib.jq_gguf_tensor_data(self._live(), t.index, ctypes.byref(p)))
        return np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctypes.c_uint8)), shape=(t.nbytes,)).copy()

    def number(self, key):
        """A numeric or boolean metadata value (ints come back as int, floats as float)."""
        v, i, vt = ctypes.c_double(), ctypes.c_int64(), ctypes.c_int()
        _lib.check(self._lib.jq_gguf_meta_find(self._live(), key.encode(), ctypes.byref(vt), None, None))
        _lib.check(self._lib.jq_gguf_meta_number(self._live(), key.encode(), ctypes.byref(v), ctypes.byref(i)))
        return v.value if vt.value in (6, 12) else i.value

    def string(self, key):
        p, n = ctypes.c_void_p(), ctypes.c_int64()
        _lib.check(self._lib.jq_gguf_meta_string(self._live(), key.encode(), ctypes.byref(p), ctypes.byref(n)))
        return ctypes.string_at(p, n.value).decode()

    def weight(self, name, device=0, rows=None):
        """The 2-D quantised tensor `name` (or its rows [rows[0], rows[1])) uploaded to `device`: a ``Tensor``."""
        from .ops import DType, Tensor
        t = self.info(name)
        h = ctypes.c_void_p()
        lo, hi = (0, -1) if rows is None else rows
        _lib.check(self._lib.jq_gguf_upload(self._live(), t.index, device, lo, hi, ctypes.byref(h)))
        n = t.shape[0] if rows is None else hi - lo
        return Tensor(h, DType(t.ggml_type), (n, t.shape[1]))

    def close(self):
        if self._h is not None:
            self._lib.jq_gguf_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
