"""ctypes access to the C++ host helpers (``ollama_b200/native/*.cpp`` -> ``libb200host.so``): GGML block codecs, BPE merges.

The library is optional on a machine without a compiler: every caller keeps a pure-Python path and asks
:func:`lib` first (None = not available).
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_NATIVE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "native")
_PATH = os.path.join(_NATIVE, "libb200host.so")
_lock = threading.Lock()
_lib = None
_tried = False


def lib():
    """The loaded library, built on first use when missing or older than its sources; None when that is not possible."""
    global _lib, _tried
    if _lib is not None or _tried:
        return _lib
    with _lock:
        if _lib is not None or _tried:
            return _lib
        _tried = True
        if os.environ.get("B200_NO_NATIVE"):
            return None
        try:
            from ..kernels.build import build_host
            build_host()
            L = C.CDLL(_PATH)
            L.b2h_codec_supported.argtypes = [C.c_int, C.c_int]
            L.b2h_dequantize.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
            L.b2h_quantize.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
            _lib = L
        except (OSError, RuntimeError, AttributeError):
            _lib = None
    return _lib


def codec_supported(t: int, encode: bool) -> bool:
    L = lib()
    return bool(L is not None and L.b2h_codec_supported(int(t), 1 if encode else 0))
