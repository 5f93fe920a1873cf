"""Host-side mirror of the reference's operator interface for the quantised linear path.

Names and argument meaning follow the reference's Java API so that tests read like its own:

* ``DType``                  ai.beestream.jitnn.DType (block geometry, DType.java:75-98)
* ``Tensor.quantized``       Tensor.quantized(DType, byte[], dims...) (Tensor.java:249-278)
* ``Gguf.linear/dequantize`` ops/Gguf.java:68-98
* ``Quant.linear/dequantize/quantizeQ8`` ops/Quant.java:40-80
* ``F.linearQ8/quantizeQ8/dequantize``   F.java:1048-1051

Activations and results are either numpy arrays (host memory: the library copies in and out) or
torch CUDA tensors (device memory: the call is enqueued on torch's current stream). All compute
happens in ``libjitnn_b200.so``; nothing here falls back to the CPU.
"""
import ctypes
import enum

import numpy as np

from . import _lib
from ._lib import JQ_MEM_DEVICE, JQ_MEM_HOST, check


class DType(enum.Enum):
    """Block formats by ggml type id (jitnn-gguf GgmlType.java:27-51)."""
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14

    def blockValues(self):
        return 32 if self in (DType.Q8_0, DType.Q4_0, DType.Q4_1, DType.Q5_0, DType.Q5_1) else 256

    def blockBytes(self):
        return {DType.Q8_0: 34, DType.Q4_0: 18, DType.Q4_1: 20, DType.Q4_K: 144, DType.Q5_K: 176, DType.Q6_K: 210,
                DType.Q5_0: 22, DType.Q5_1: 24, DType.Q2_K: 84, DType.Q3_K: 110}[self]

    def isBlockQuantized(self):
        return True


def _dtype(t):
    if isinstance(t, DType):
        return t
    if isinstance(t, str):
        return DType[t]
    return DType(int(t))


def _is_torch(x):
    return type(x).__module__.startswith("torch")


class Tensor:
    """A persistent quantised weight on one GPU (the handle behind ``jq_weight``)."""

    def __init__(self, handle, dtype, dims):
        self._h = handle
        self._dtype = dtype
        self._dims = tuple(dims)

    @staticmethod
    def quantized(dtype, blocks, *dims, device=0, rows=None):
        """Uploads raw GGUF blocks of a weight of shape ``dims`` ([N, K]).

        ``rows=(begin, end)`` uploads only those output rows (one GPU's shard of a row-split
        linear); the tensor then has shape [end - begin, K].
        """
        dtype = _dtype(dtype)
        if len(dims) == 1 and isinstance(dims[0], (tuple, list)):
            dims = tuple(dims[0])
        if len(dims) != 2:
            raise ValueError("%s weight of shape %s: the linear path needs a rank-2 weight" % (dtype.name, list(dims)))
        raw = np.ascontiguousarray(np.frombuffer(blocks, dtype=np.uint8) if isinstance(blocks, (bytes, bytearray, memoryview))
                                   else np.asarray(blocks, dtype=np.uint8)).reshape(-1)
        n, k = int(dims[0]), int(dims[1])
        out = ctypes.c_void_p()
        L = _lib.load()
        if rows is None:
            check(L.jq_weight_upload(device, dtype.value, raw.ctypes.data, raw.size, n, k, _lib.JQ_LAYOUT_AUTO, ctypes.byref(out)))
            shape = (n, k)
        else:
            check(L.jq_weight_upload_rows(device, dtype.value, raw.ctypes.data, raw.size, n, k, int(rows[0]), int(rows[1]),
                                          _lib.JQ_LAYOUT_AUTO, ctypes.byref(out)))
            shape = (int(rows[1]) - int(rows[0]), k)
        return Tensor(out, dtype, shape)

    def _handle(self):
        if self._h is None:
            raise RuntimeError("tensor was released")  # IllegalStateException in the reference
        return self._h

    def dtype(self):
        return self._dtype

    def shape(self):
        return self._dims

    def dim(self, i):
        return self._dims[i]

    def rank(self):
        return len(self._dims)

    def numel(self):
        return self._dims[0] * self._dims[1]

    def device(self):
        info = (ctypes.c_int64 * 8)()
        check(_lib.load().jq_weight_info(self._handle(), info))
        return int(info[4])

    def deviceBytes(self):
        info = (ctypes.c_int64 * 8)()
        check(_lib.load().jq_weight_info(self._handle(), info))
        return int(info[5])

    def toFloatArray(self):
        """Dequantised values as a flat float32 numpy array (Tensor.toFloatArray, Tensor.java:539-555)."""
        return Gguf.dequantize(self).reshape(-1)

    def blocks(self):
        """The original GGUF block bytes, read back from the device."""
        nbytes = self.numel() // self._dtype.blockValues() * self._dtype.blockBytes()
        out = np.empty(nbytes, dtype=np.uint8)
        check(_lib.load().jq_weight_download(self._handle(), out.ctypes.data, nbytes))
        return out

    def release(self):
        if self._h is not None:
            h, self._h = self._h, None
            check(_lib.load().jq_weight_free(h))

    close = release

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def _stream_of(t):
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _linear(x, w, bias, who):
    L = _lib.load()
    if not isinstance(w, Tensor):
        raise ValueError("%s: weight is not a quantised tensor" % who)
    n, k = w.shape()
    if _is_torch(x):
        import torch
        if x.dtype != torch.float32:
            raise ValueError("needs an FP32 tensor, got %s" % x.dtype)  # Checks.f32
        if x.dim() == 0 or x.shape[-1] != k:
            raise ValueError("%s linear: input %s and weight %s" % (w.dtype().name, list(x.shape), list(w.shape())))
        if not x.is_cuda or x.device.index != w.device():
            raise ValueError("%s linear: input on %s, weight on cuda:%d" % (w.dtype().name, x.device, w.device()))
        xc = x.contiguous()
        m = xc.numel() // k if k else 0
        y = torch.empty(list(x.shape[:-1]) + [n], dtype=torch.float32, device=x.device)
        b = None
        if bias is not None:
            b = bias.contiguous()
            if b.dtype != torch.float32 or b.numel() != n or b.device != x.device:
                raise ValueError("%s linear: bias %s for %d outputs" % (w.dtype().name, list(bias.shape), n))
        with torch.cuda.device(x.device):
            check(L.jq_linear_f32(w._handle(), xc.data_ptr(), m, None if b is None else b.data_ptr(), y.data_ptr(), JQ_MEM_DEVICE, _stream_of(x)))
        return y
    x = np.asarray(x)
    if x.dtype != np.float32:
        raise ValueError("needs an FP32 tensor, got %s" % x.dtype)
    if x.ndim == 0 or x.shape[-1] != k:
        raise ValueError("%s linear: input %s and weight %s" % (w.dtype().name, list(x.shape), list(w.shape())))
    xc = np.ascontiguousarray(x)
    m = xc.size // k if k else 0
    y = np.empty(x.shape[:-1] + (n,), dtype=np.float32)
    b = None
    if bias is not None:
        b = np.ascontiguousarray(bias, dtype=np.float32)
        if b.size != n:
            raise ValueError("%s linear: bias %s for %d outputs" % (w.dtype().name, list(b.shape), n))
    check(L.jq_linear_f32(w._handle(), xc.ctypes.data, m, None if b is None else b.ctypes.data, y.ctypes.data, JQ_MEM_HOST, None))
    return y


def _linear_backward(g, w):
    L = _lib.load()
    if not isinstance(w, Tensor):
        raise ValueError("linear backward: weight is not a quantised tensor")
    n, k = w.shape()
    if _is_torch(g):
        import torch
        if g.dtype != torch.float32:
            raise ValueError("needs an FP32 tensor, got %s" % g.dtype)
        if g.dim() == 0 or g.shape[-1] != n:
            raise ValueError("%s linear backward: gradient %s and weight %s" % (w.dtype().name, list(g.shape), list(w.shape())))
        if not g.is_cuda or g.device.index != w.device():
            raise ValueError("%s linear backward: gradient on %s, weight on cuda:%d" % (w.dtype().name, g.device, w.device()))
        gc = g.contiguous()
        m = gc.numel() // n if n else int(np.prod(g.shape[:-1]))
        gx = torch.empty(list(g.shape[:-1]) + [k], dtype=torch.float32, device=g.device)
        with torch.cuda.device(g.device):
            check(L.jq_linear_backward_f32(w._handle(), gc.data_ptr(), m, gx.data_ptr(), JQ_MEM_DEVICE, _stream_of(g)))
        return gx
    g = np.asarray(g)
    if g.dtype != np.float32:
        raise ValueError("needs an FP32 tensor, got %s" % g.dtype)
    if g.ndim == 0 or g.shape[-1] != n:
        raise ValueError("%s linear backward: gradient %s and weight %s" % (w.dtype().name, list(g.shape), list(w.shape())))
    gc = np.ascontiguousarray(g)
    m = gc.size // n if n else int(np.prod(g.shape[:-1]))
    gx = np.empty(g.shape[:-1] + (k,), dtype=np.float32)
    check(L.jq_linear_backward_f32(w._handle(), gc.ctypes.data, m, gx.ctypes.data, JQ_MEM_HOST, None))
    return gx


def _dequantize(w, out=None):
    L = _lib.load()
    n, k = w.shape()
    if out is not None and _is_torch(out):
        check(L.jq_dequantize(w._handle(), out.data_ptr(), JQ_MEM_DEVICE, _stream_of(out)))
        return out
    y = np.empty((n, k), dtype=np.float32)
    check(L.jq_dequantize(w._handle(), y.ctypes.data, JQ_MEM_HOST, None))
    return y


class Gguf:
    """ops/Gguf.java of the reference: linear layers and dequantisation for GGUF block formats."""

    @staticmethod
    def linear(x, w, bias=None):
        """y = x W^T + b, W [N, K] in a GGUF format, x FP32 [..., K]; b may be None."""
        return _linear(x, w, bias, "Gguf.linear")

    @staticmethod
    def dequantize(w, out=None):
        return _dequantize(w, out)

    @staticmethod
    def linearBackward(g, w):
        """The input gradient of linear: gx [..., K] = g [..., N] . dequant(W) (ops/Gguf.java:208-212; the weight gets
        no gradient, the bias gradient is the column sum of g)."""
        return _linear_backward(g, w)

    @staticmethod
    def linearBf16(x, w, bias=None):
        """Prefill form: x bfloat16 [..., K] (a torch CUDA tensor, or a numpy uint16 array of bfloat16 bit patterns),
        y float32 [..., N]; dequantised weights rounded to bfloat16, tensor-core product, FP32 accumulation."""
        L = _lib.load()
        if not isinstance(w, Tensor):
            raise ValueError("Gguf.linearBf16: weight is not a quantised tensor")
        n, k = w.shape()
        if _is_torch(x):
            import torch
            if x.dtype != torch.bfloat16:
                raise ValueError("needs a BF16 tensor, got %s" % x.dtype)
            if x.dim() == 0 or x.shape[-1] != k:
                raise ValueError("%s linear: input %s and weight %s" % (w.dtype().name, list(x.shape), list(w.shape())))
            xc = x.contiguous()
            m = xc.numel() // k if k else 0
            y = torch.empty(list(x.shape[:-1]) + [n], dtype=torch.float32, device=x.device)
            b = None if bias is None else bias.contiguous()
            with torch.cuda.device(x.device):
                check(L.jq_linear_bf16(w._handle(), xc.data_ptr(), m, None if b is None else b.data_ptr(), y.data_ptr(), JQ_MEM_DEVICE, _stream_of(x)))
            return y
        x = np.asarray(x)
        if x.dtype != np.uint16:
            raise ValueError("needs bfloat16 bit patterns as uint16, got %s" % x.dtype)
        if x.ndim == 0 or x.shape[-1] != k:
            raise ValueError("%s linear: input %s and weight %s" % (w.dtype().name, list(x.shape), list(w.shape())))
        xc = np.ascontiguousarray(x)
        m = xc.size // k if k else 0
        y = np.empty(x.shape[:-1] + (n,), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        check(L.jq_linear_bf16(w._handle(), xc.ctypes.data, m, None if b is None else b.ctypes.data, y.ctypes.data, JQ_MEM_HOST, None))
        return y


def device_status(device=0):
    """Waits for the device and returns (then clears) the status word of the library's kernels: 0 when no bounded
    device-side wait ever gave up."""
    st = ctypes.c_int(-1)
    check(_lib.load().jq_device_status(device, ctypes.byref(st)))
    return st.value


class Quant:
    """ops/Quant.java of the reference: the Q8_0 operators."""

    @staticmethod
    def linear(x, w, bias=None):
        if not isinstance(w, Tensor) or w.dtype() != DType.Q8_0:
            raise ValueError("Q8_0 linear: weight %s" % (w.dtype().name if isinstance(w, Tensor) else type(w)))
        return _linear(x, w, bias, "Quant.linear")

    @staticmethod
    def linearBackward(g, w):
        """gx = g . dequant(W) for a Q8_0 weight (ops/Quant.java:191-197)."""
        if not isinstance(w, Tensor) or w.dtype() != DType.Q8_0:
            raise ValueError("Q8_0 linear backward: weight %s" % (w.dtype().name if isinstance(w, Tensor) else type(w)))
        return _linear_backward(g, w)

    @staticmethod
    def dequantize(q, out=None):
        if q.dtype() != DType.Q8_0:
            raise ValueError("dequantize needs a Q8_0 tensor, got %s" % q.dtype().name)
        return _dequantize(q, out)

    @staticmethod
    def quantizeQ8Blocks(x, device=0):
        """FP32 values (last axis a multiple of 32) to raw Q8_0 block bytes (numpy uint8)."""
        L = _lib.load()
        if _is_torch(x):
            import torch
            if x.dtype != torch.float32:
                raise ValueError("needs an FP32 tensor, got %s" % x.dtype)
            if x.shape[-1] % 32 != 0:
                raise ValueError("Q8_0 needs a last axis that is a multiple of 32, got %s" % list(x.shape))
            xc = x.contiguous()
            out = torch.empty(xc.numel() // 32 * 34, dtype=torch.uint8, device=x.device)
            with torch.cuda.device(x.device):
                check(L.jq_quantize_q8_0(x.device.index, xc.data_ptr(), xc.numel(), out.data_ptr(), JQ_MEM_DEVICE, _stream_of(x)))
            return out
        x = np.asarray(x)
        if x.dtype != np.float32:
            raise ValueError("needs an FP32 tensor, got %s" % x.dtype)
        if x.ndim == 0 or x.shape[-1] % 32 != 0:
            raise ValueError("Q8_0 needs a last axis that is a multiple of 32, got %s" % list(x.shape))
        xc = np.ascontiguousarray(x)
        out = np.empty(xc.size // 32 * 34, dtype=np.uint8)
        check(L.jq_quantize_q8_0(device, xc.ctypes.data, xc.size, out.ctypes.data, JQ_MEM_HOST, None))
        return out

    @staticmethod
    def quantizeQ8(x, device=0):
        """x [N, K] FP32 to a Q8_0 weight tensor on ``device``."""
        blocks = Quant.quantizeQ8Blocks(x, device)
        if _is_torch(blocks):
            blocks = blocks.cpu().numpy()
        shape = tuple(x.shape)
        if len(shape) != 2:
            shape = (int(np.prod(shape[:-1])), shape[-1])
        return Tensor.quantized(DType.Q8_0, blocks, *shape, device=device)


class F:
    """The functional aliases of F.java:1048-1051."""
    linearQ8 = staticmethod(Quant.linear)
    quantizeQ8 = staticmethod(Quant.quantizeQ8)
    dequantize = staticmethod(Quant.dequantize)
