"""ctypes binding of libkvq_b200.so (C ABI declared in include/kvq_b200.h).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# KVQ_B200_LIB points at another build of the same library (e.g. an installed copy); default: the in-tree build
LIB_PATH = os.environ.get("KVQ_B200_LIB") or os.path.join(os.path.dirname(_HERE), "lib", "libkvq_b200.so")

_c_i64, _c_int, _c_ptr = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p

# name -> (restype, argtypes); mirrors include/kvq_b200.h
SIGNATURES = {
    "kvq_version": (_c_int, []),
    "kvq_last_error": (ctypes.c_char_p, []),
    "kvq_quant_cache": (_c_int, [_c_ptr] * 8 + [_c_i64, _c_int, _c_int, _c_int] + [_c_i64] * 10 + [_c_int, _c_int, _c_ptr]),
    "kvq_quant_q": (_c_int, [_c_ptr] * 4 + [_c_i64, _c_int, _c_int, _c_int, _c_int, _c_i64, _c_i64, _c_int, _c_ptr]),
    "kvq_decode_workspace_size": (ctypes.c_size_t, [_c_int, _c_int]),
    "kvq_int8_decode_attention": (_c_int, [_c_ptr] * 9 + [ctypes.c_double] + [_c_int] * 5 + [_c_i64] * 12 +
                                  [_c_int] * 4 + [_c_ptr, ctypes.c_size_t, _c_ptr]),
    "kvq_int8_decode_attention_qgroup": (_c_int, [_c_ptr] * 9 + [ctypes.c_double] + [_c_int] * 5 + [_c_i64] * 12 +
                                         [_c_int] * 5 + [_c_ptr, ctypes.c_size_t, _c_ptr]),
    "kvq_static_workspace_bytes": (ctypes.c_size_t, []),
    "kvq_int8_decode_attention_noalloc": (_c_int, [_c_ptr] * 9 + [ctypes.c_double] + [_c_int] * 5 + [_c_i64] * 12 +
                                          [_c_int] * 4 + [_c_ptr]),
    "kvq_decode_status": (_c_int, [_c_ptr, ctypes.POINTER(_c_int), _c_ptr]),
    "kvq_debug_kernel_events": (_c_int, [_c_ptr, _c_ptr]),
    "kvq_debug_decode_split": (_c_int, [_c_ptr, _c_ptr] + [_c_int] * 8 + [_c_ptr, _c_ptr]),
    "kvq_prefill_workspace_size": (ctypes.c_size_t, [_c_int]),
    "kvq_int8_prefill_attention": (_c_int, [_c_ptr] * 9 + [ctypes.c_double, _c_int, _c_i64] + [_c_int] * 4 + [_c_i64] * 12 +
                                   [_c_int] * 3 + [_c_ptr, ctypes.c_size_t, _c_ptr]),
    "kvq_calib_stats": (_c_int, [_c_ptr] * 3 + [_c_i64, _c_int, _c_int] + [_c_i64] * 4 + [_c_ptr] * 9 + [_c_ptr]),
    "kvq_peer_allgather": (_c_int, [_c_ptr, ctypes.c_size_t, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr]),
    "kvq_pages_to_wire": (_c_int, [_c_ptr] * 4 + [_c_i64, _c_int, _c_int, _c_int] + [_c_i64] * 6 + [_c_ptr]),
    "kvq_wire_to_pages": (_c_int, [_c_ptr] * 4 + [_c_i64, _c_int, _c_int, _c_int] + [_c_i64] * 6 + [_c_ptr]),
    "kvq_dequant_pages": (_c_int, [_c_ptr] * 9 + [_c_i64, _c_int, _c_int, _c_int] + [_c_i64] * 7 + [_c_int, _c_int, _c_ptr]),
}

_LIB = None


def lib():
    """The loaded library; built by `python int8-kvcache_b200/build.py`."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"kvq_b200: native library not found at {LIB_PATH}; run int8-kvcache_b200/build.py "
                               "(there is no non-CUDA fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _LIB = handle
    return _LIB


def check(code):
    """Turn a non-zero status into the RuntimeError the reference's TORCH_CHECKs would raise."""
    if code != 0:
        raise RuntimeError("kvq_b200: " + lib().kvq_last_error().decode())
