"""ctypes binding of libsage_b200.so (declared in include/sage_b200.h).

The reference binds its kernels the same way -- extern "C" symbols reached through ctypes with raw
pointers on torch's current stream, so that no torch C++ ABI is involved
(sageattention/sk1_backend/sk1_loader.py:1-23,160-298 of the reference).  There is no fallback: if
the library is missing or cannot be loaded every entry point raises.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsage_b200.so")

SAGE_F16, SAGE_BF16 = 0, 1
SAGE_QK_INT8, SAGE_QK_E4M3 = 0, 1
SAGE_QK_NO_FAST_PATH = 0x100
SAGE_E_ARG, SAGE_E_UNSUPPORTED, SAGE_E_CUDA, SAGE_E_WORKSPACE = -1, -2, -3, -4

_I64 = ctypes.c_int64
_P = ctypes.c_void_p
_S3 = ctypes.POINTER(ctypes.c_int64)

#: name -> (restype, argtypes); the complete export list of the header.
SIGNATURES = {
    "sage_version": (ctypes.c_int, []),
    "sage_last_error": (ctypes.c_char_p, []),
    "sage_pad_len": (_I64, [_I64]),
    "sage_prologue_ctrl_bytes": (ctypes.c_size_t, [_I64, _I64, _I64]),
    "sage_prologue": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                     _I64, _I64, _I64, _I64, _S3, _S3, _S3,
                                     ctypes.c_int, ctypes.c_int, ctypes.c_int, _P]),
    "sage_prologue_static_ctrl_capacity": (ctypes.c_size_t, []),
    "sage_prologue_static_ctrl": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                                 _I64, _I64, _I64, _I64, _S3, _S3, _S3,
                                                 ctypes.c_int, ctypes.c_int, ctypes.c_int, _P, _P]),
    "sage_attn_fwd": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P,
                                     _I64, _I64, _I64, _I64, _S3,
                                     ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int, _P, _P]),
    "sage_prologue_ex": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                        _I64, _I64, _I64, _I64, _I64, _I64, _I64, _S3, _S3, _S3,
                                        ctypes.c_int, ctypes.c_int, ctypes.c_int, _P]),
    "sage_attn_fwd_ex": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                        _I64, _I64, _I64, _I64, _I64, _I64, _I64, _S3,
                                        ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int, _P, _P]),
    "sage_workspace_bytes_ex": (ctypes.c_size_t, [_I64, _I64, _I64, _I64, _I64]),
    "sage_workspace_layout_ex": (ctypes.c_int, [_I64, _I64, _I64, _I64, _I64, ctypes.POINTER(ctypes.c_size_t)]),
    "sage_attention_ex": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, ctypes.c_size_t, _I64, _I64, _I64, _I64, _I64, _I64,
                                         _S3, _S3, _S3, _S3, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_int, ctypes.c_float, _P]),
    "sage_attention_varlen": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, ctypes.c_size_t,
                                             _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64,
                                             _S3, _S3, _S3, _S3, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                             ctypes.c_int, ctypes.c_float, _P]),
    "sage_status_mirror": (ctypes.c_int, [_P, _P, ctypes.c_int, _P]),
    "sage_debug_tiles_per_cta": (None, [ctypes.c_int]),
    "sage_debug_skip_threshold": (None, [ctypes.c_float]),
    "sage_attention_tiles_per_cta": (ctypes.c_int, [_I64, _I64, _I64, ctypes.c_int, ctypes.c_int]),
    "sage_workspace_bytes": (ctypes.c_size_t, [_I64, _I64, _I64]),
    "sage_workspace_layout": (ctypes.c_int, [_I64, _I64, _I64, ctypes.POINTER(ctypes.c_size_t)]),
    "sage_attention": (ctypes.c_int, [_P, _P, _P, _P, _P, ctypes.c_size_t, _I64, _I64, _I64,
                                      _S3, _S3, _S3, _S3, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_float, _P]),
}

_lock = threading.Lock()
_lib = None


class SageNativeError(RuntimeError):
    """The CUDA library is missing, failed to load, or returned an error code."""


def load():
    """Load the library once (thread-safe) and declare every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise SageNativeError(
                    "libsage_b200.so is not built (expected at %s). Build it with "
                    "`python sageattention-rdna4_b200/build.py`; there is no fallback path." % LIB_PATH)
            try:
                lib = ctypes.CDLL(LIB_PATH)
            except OSError as exc:
                raise SageNativeError("cannot load %s: %s" % (LIB_PATH, exc)) from exc
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = res, args
            _lib = lib
    return _lib


def strides3(batch: int, head: int, row: int):
    return (ctypes.c_int64 * 3)(int(batch), int(head), int(row))


def strides2(token: int, head: int):
    return (ctypes.c_int64 * 2)(int(token), int(head))


def check(rc: int, what: str):
    """Turn a negative return code into the exception class the Python API documents."""
    if rc == 0:
        return
    msg = load().sage_last_error().decode("utf-8", "replace")
    text = "%s failed (%d): %s" % (what, rc, msg)
    if rc == SAGE_E_ARG:
        raise ValueError(text)
    if rc == SAGE_E_UNSUPPORTED:
        raise NotImplementedError(text)
    raise SageNativeError(text)
