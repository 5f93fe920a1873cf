"""ctypes binding of ``libjitnn_b200.so`` (the C ABI declared in ``include/jitnn_b200.h``).

The library is the product: there is no Python or CPU fallback. ``load()`` raises if the shared
object has not been built (``python -m jitnn_b200.build``).
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libjitnn_b200.so")

JQ_OK = 0
JQ_ERR_INVALID, JQ_ERR_OOM, JQ_ERR_CUDA, JQ_ERR_NCCL, JQ_ERR_TIMEOUT, JQ_ERR_UNSUPPORTED = -1, -2, -3, -4, -5, -6
JQ_MEM_HOST, JQ_MEM_DEVICE = 0, 1
JQ_LAYOUT_AUTO = 0

c_i64, c_int, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "jq_version": (c_int, []),
    "jq_last_error": (ctypes.c_char_p, []),
    "jq_block_values": (c_int, [c_int]),
    "jq_block_bytes": (c_int, [c_int]),
    "jq_device_count": (c_int, [ctypes.POINTER(c_int)]),
    "jq_weight_upload": (c_int, [c_int, c_int, vp, c_i64, c_i64, c_i64, c_int, ctypes.POINTER(vp)]),
    "jq_weight_upload_rows": (c_int, [c_int, c_int, vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, ctypes.POINTER(vp)]),
    "jq_weight_free": (c_int, [vp]),
    "jq_weight_info": (c_int, [vp, ctypes.POINTER(c_i64)]),
    "jq_weight_download": (c_int, [vp, vp, c_i64]),
    "jq_dequantize": (c_int, [vp, vp, c_int, vp]),
    "jq_linear_f32": (c_int, [vp, vp, c_i64, vp, vp, c_int, vp]),
    "jq_linear_backward_f32": (c_int, [vp, vp, c_i64, vp, c_int, vp]),
    "jq_linear_bf16": (c_int, [vp, vp, c_i64, vp, vp, c_int, vp]),
    "jq_linear_q4k_f32_noalloc": (c_int, [vp, vp, c_i64, vp, vp, vp]),
    "jq_device_status": (c_int, [c_int, ctypes.POINTER(c_int)]),
    "jq_peer_alloc": (c_int, [c_int, c_i64, ctypes.POINTER(vp), vp]),
    "jq_peer_open": (c_int, [c_int, vp, ctypes.POINTER(vp)]),
    "jq_peer_close": (c_int, [vp]),
    "jq_peer_free": (c_int, [vp]),
    "jq_peer_payload_offset": (c_i64, []),
    "jq_peer_gather": (c_int, [vp, c_i64, c_i64, c_i64, c_i64, ctypes.POINTER(vp), c_i64, c_i64, c_int, c_int, vp]),
    "jq_linear_f32_peer": (c_int, [vp, vp, c_i64, vp, c_i64, c_i64, ctypes.POINTER(vp), c_i64, c_i64, c_int, c_int, vp]),
    "jq_quantize_q8_0": (c_int, [c_int, vp, c_i64, vp, c_int, vp]),
    "jq_decoder_create": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, ctypes.c_float, ctypes.c_float, ctypes.POINTER(vp)]),
    "jq_decoder_destroy": (c_int, [vp]),
    "jq_decoder_set_linear": (c_int, [vp, c_int, c_int, vp]),
    "jq_decoder_set_norm": (c_int, [vp, c_int, c_int, vp]),
    "jq_decoder_set_embedding": (c_int, [vp, vp]),
    "jq_decoder_forward": (c_int, [vp, vp, c_int, c_int, vp, vp, vp]),
    "jq_decoder_set_sequences": (c_int, [vp, c_int]),
    "jq_decoder_forward_seq": (c_int, [vp, c_int, vp, c_int, c_int, vp, vp, vp]),
    "jq_decoder_forward_batch": (c_int, [vp, vp, c_int, c_int, vp, vp, vp]),
    "jq_decoder_prompt": (c_int, [vp, c_int, vp, c_int, c_int, vp, vp, vp]),
    "jq_decoder_peer_bytes": (c_int, [vp, ctypes.POINTER(ctypes.c_int64)]),
    "jq_decoder_set_shard": (c_int, [vp, c_int, c_int, vp]),
    "jq_set_option": (c_int, [ctypes.c_char_p, c_i64]),
    "jq_get_option": (c_int, [ctypes.c_char_p, ctypes.POINTER(c_i64)]),
    "jq_gguf_open": (c_int, [ctypes.c_char_p, ctypes.POINTER(vp)]),
    "jq_gguf_close": (c_int, [vp]),
    "jq_gguf_info": (c_int, [vp, ctypes.POINTER(c_int), ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), ctypes.POINTER(c_i64)]),
    "jq_gguf_tensor": (c_int, [vp, c_i64, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_i64),
                               ctypes.POINTER(c_i64), ctypes.POINTER(c_i64)]),
    "jq_gguf_find_tensor": (c_int, [vp, ctypes.c_char_p, ctypes.POINTER(c_i64)]),
    "jq_gguf_tensor_data": (c_int, [vp, c_i64, ctypes.POINTER(vp)]),
    "jq_gguf_meta_find": (c_int, [vp, ctypes.c_char_p, ctypes.POINTER(c_int), ctypes.POINTER(c_i64), ctypes.POINTER(c_int)]),
    "jq_gguf_meta_number": (c_int, [vp, ctypes.c_char_p, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(c_i64)]),
    "jq_gguf_meta_string": (c_int, [vp, ctypes.c_char_p, ctypes.POINTER(vp), ctypes.POINTER(c_i64)]),
    "jq_gguf_upload": (c_int, [vp, c_i64, c_int, c_i64, c_i64, ctypes.POINTER(vp)]),
    "jq_host_alloc": (c_int, [ctypes.POINTER(vp), c_i64]),
    "jq_host_free": (c_int, [vp]),
    "jq_launch_count": (c_i64, []),
}

_lib = None


class JitnnError(RuntimeError):
    """A runtime failure inside the library (the reference wraps these in JitnnException)."""


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libjitnn_b200.so is not built: run `python -m jitnn_b200.build` (needs nvcc); there is no fallback path")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error():
    return load().jq_last_error().decode("utf-8", "replace")


def check(rc):
    """Maps a status code to the exception the reference's Java API would throw."""
    if rc == JQ_OK:
        return
    msg = last_error()
    if rc in (JQ_ERR_INVALID, JQ_ERR_UNSUPPORTED):
        raise ValueError(msg)  # IllegalArgumentException
    if rc == JQ_ERR_OOM:
        raise MemoryError(msg)
    if rc == JQ_ERR_TIMEOUT:
        raise TimeoutError(msg)
    raise JitnnError(msg)
