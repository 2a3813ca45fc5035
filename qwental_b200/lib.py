"""ctypes binding of libqw_gpu_cuda.so -- the C ABI declared in include/qw_gpu.h, qw_gpu_ext.h, qw_engine.h.

There is no CPU fallback: if the library is missing or no CUDA device opens, the calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "libqw_gpu_cuda.so")


class QwBuf(C.Structure):
    _fields_ = [("handle", C.c_void_p), ("ptr", C.c_void_p), ("size", C.c_size_t)]


_lib = None


def load() -> C.CDLL:
    """Load the library (built by `python -m qwental_b200.build`); raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError("libqw_gpu_cuda.so is not built: run `python -m qwental_b200.build` (needs nvcc)")
    L = C.CDLL(LIB_PATH)
    vp, sz, u, d, b, cp = C.c_void_p, C.c_size_t, C.c_uint, C.c_double, C.c_bool, C.c_char_p
    P = C.POINTER
    sig = {
        "qw_gpu_open": (vp, []), "qw_gpu_close": (None, [vp]), "qw_gpu_name": (cp, [vp]),
        "qw_gpu_max_working_set": (sz, [vp]),
        "qw_gpu_compile": (b, [vp, cp, sz, cp, sz]), "qw_kernel_get": (vp, [vp, cp]),
        "qw_kernel_max_threads": (u, [vp]), "qw_kernel_simd_width": (u, [vp]),
        "qw_buf_new": (b, [vp, sz, P(QwBuf)]), "qw_buf_free": (None, [P(QwBuf)]),
        "qw_pool_push": (vp, []), "qw_pool_pop": (None, [vp]), "qw_buf_wrap": (b, [vp, vp, sz, P(QwBuf)]),
        "qw_batch_begin": (vp, [vp, b]), "qw_batch_kernel": (None, [vp, vp]),
        "qw_batch_buf": (None, [vp, u, P(QwBuf), sz]), "qw_batch_bytes": (None, [vp, u, vp, sz]),
        "qw_batch_threadgroup_mem": (None, [vp, u, sz]),
        "qw_batch_dispatch": (None, [vp, u, u, u, u, u, u]), "qw_batch_barrier": (None, [vp]),
        "qw_batch_flush": (None, [vp]), "qw_batch_end": (d, [vp]), "qw_batch_submit": (None, [vp]),
        "qw_batch_wait": (d, [vp]), "qw_batch_poll": (b, [vp]), "qw_gpu_set_stream": (None, [vp, C.c_int]),
        "qw_profile_enable": (None, [vp, b]), "qw_profile_count": (C.c_int, [vp]),
        "qw_profile_get": (cp, [vp, C.c_int, P(d)]),
        "qw_gpu_empty_commit_latency": (d, [vp, vp, C.c_int]), "qw_power_desc": (None, [cp, sz]),
        "qw_on_battery": (b, []), "qw_now": (d, []),
        # qw_gpu_ext.h
        "qw_buf_new_kind": (b, [vp, sz, C.c_int, P(QwBuf)]),
        "qw_buf_upload": (b, [vp, P(QwBuf), sz, vp, sz]), "qw_buf_download": (b, [vp, P(QwBuf), sz, vp, sz]),
        "qw_buf_zero": (b, [vp, P(QwBuf), sz, sz]), "qw_buf_device_ptr": (vp, [P(QwBuf)]),
        "qw_gpu_stream_handle": (vp, [vp, C.c_int]), "qw_gpu_last_error": (cp, [vp]),
        "qw_gpu_launch_count": (C.c_ulonglong, [vp]), "qw_gpu_set_graphs": (None, [vp, b]),
        "qw_gpu_family_count": (C.c_int, []), "qw_gpu_family_name": (cp, [C.c_int]),
    }
    for name, (res, args) in sig.items():
        f = getattr(L, name)
        f.restype, f.argtypes = res, args
    _lib = L
    return L


GPU_H_SYMBOLS = [
    "qw_gpu_open", "qw_gpu_close", "qw_gpu_name", "qw_gpu_max_working_set", "qw_gpu_compile", "qw_kernel_get",
    "qw_kernel_max_threads", "qw_kernel_simd_width", "qw_buf_new", "qw_buf_free", "qw_pool_push", "qw_pool_pop",
    "qw_buf_wrap", "qw_batch_begin", "qw_batch_kernel", "qw_batch_buf", "qw_batch_bytes", "qw_batch_threadgroup_mem",
    "qw_batch_dispatch", "qw_batch_barrier", "qw_batch_flush", "qw_batch_end", "qw_batch_submit", "qw_batch_wait",
    "qw_batch_poll", "qw_gpu_set_stream", "qw_profile_enable", "qw_profile_count", "qw_profile_get",
    "qw_gpu_empty_commit_latency", "qw_power_desc", "qw_on_battery", "qw_now",
]
