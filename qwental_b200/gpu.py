"""Thin Python face of the device interface (include/qw_gpu.h): the same calls the reference's host makes
through src/gpu.h -- compile a prelude, get kernels by name, bind buffers/bytes by index, dispatch, wait.
Used by the tests and the benchmark; all work happens in libqw_gpu_cuda.so.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as _lib
from .lib import QwBuf

SHARED, DEVICE, HOSTIO = 0, 1, 2


class GpuError(RuntimeError):
    pass


class Buf:
    def __init__(self, gpu: "Gpu", size: int, kind: int = DEVICE):
        self.gpu, self.b = gpu, QwBuf()
        if not gpu.L.qw_buf_new_kind(gpu.g, size, kind, C.byref(self.b)):
            raise GpuError("qw_buf_new_kind(%d bytes) failed: %s" % (size, gpu.last_error()))
        self.size, self.kind = size, kind

    def upload(self, arr: np.ndarray, offset: int = 0) -> "Buf":
        a = np.ascontiguousarray(arr)
        if not self.gpu.L.qw_buf_upload(self.gpu.g, C.byref(self.b), offset, a.ctypes.data, a.nbytes):
            raise GpuError("upload failed: " + self.gpu.last_error())
        return self

    def download(self, dtype, count: int, offset: int = 0) -> np.ndarray:
        out = np.empty(count, dtype)
        if not self.gpu.L.qw_buf_download(self.gpu.g, C.byref(self.b), offset, out.ctypes.data, out.nbytes):
            raise GpuError("download failed: " + self.gpu.last_error())
        return out

    def zero(self):
        if not self.gpu.L.qw_buf_zero(self.gpu.g, C.byref(self.b), 0, self.size):
            raise GpuError("zero failed: " + self.gpu.last_error())
        return self

    @property
    def dev_ptr(self) -> int:
        return int(self.gpu.L.qw_buf_device_ptr(C.byref(self.b)) or 0)

    def free(self):
        if self.b.handle:
            self.gpu.L.qw_buf_free(C.byref(self.b))

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Batch:
    def __init__(self, gpu: "Gpu"):
        self.gpu, self.L = gpu, gpu.L
        self.b = self.L.qw_batch_begin(gpu.g, False)
        self._keep = []

    def kernel(self, k):
        self.L.qw_batch_kernel(self.b, k)
        return self

    def buf(self, index: int, buf: Buf, offset: int = 0):
        self.L.qw_batch_buf(self.b, index, C.byref(buf.b), offset)
        return self

    def bytes(self, index: int, data):
        raw = data.tobytes() if isinstance(data, np.ndarray) else bytes(data)
        cb = C.create_string_buffer(raw, len(raw))
        self._keep.append(cb)
        self.L.qw_batch_bytes(self.b, index, C.cast(cb, C.c_void_p), len(raw))
        return self

    def dispatch(self, grid, block):
        g = tuple(grid) + (1,) * (3 - len(grid))
        t = tuple(block) + (1,) * (3 - len(block))
        self.L.qw_batch_dispatch(self.b, *g, *t)
        return self

    def end(self) -> float:
        secs = self.L.qw_batch_end(self.b)
        self.b = None
        if secs < 0:
            raise GpuError("batch failed: " + self.gpu.last_error())
        return secs


class Gpu:
    def __init__(self):
        self.L = _lib.load()
        self.g = self.L.qw_gpu_open()
        if not self.g:
            raise GpuError("qw_gpu_open failed: no CUDA device (this library has no CPU path)")

    def name(self) -> str:
        return self.L.qw_gpu_name(self.g).decode()

    def last_error(self) -> str:
        return self.L.qw_gpu_last_error(self.g).decode()

    def compile(self, family: str, name: str | None = None, **defs) -> C.c_void_p:
        """Register a precompiled family under `name` with integer defines; returns the kernel handle."""
        src = "#define QW_KERNEL %s\n#define QW_NAME %s\n" % (family, name or family)
        src += "".join("#define %s %d\n" % (k, int(v)) for k, v in defs.items())
        src += "// body: precompiled sm_100a kernel\n"
        err = C.create_string_buffer(512)
        raw = src.encode()
        if not self.L.qw_gpu_compile(self.g, raw, len(raw), err, 512):
            raise GpuError("qw_gpu_compile: " + err.value.decode())
        k = self.L.qw_kernel_get(self.g, (name or family).encode())
        if not k:
            raise GpuError("qw_kernel_get(%s) returned NULL" % (name or family))
        return k

    def buf(self, size: int, kind: int = DEVICE) -> Buf:
        return Buf(self, size, kind)

    def buf_from(self, arr: np.ndarray, kind: int = DEVICE) -> Buf:
        a = np.ascontiguousarray(arr)
        return Buf(self, max(a.nbytes, 16), kind).upload(a)

    def batch(self) -> Batch:
        return Batch(self)

    def launches(self) -> int:
        return int(self.L.qw_gpu_launch_count(self.g))

    def close(self):
        if self.g:
            self.L.qw_gpu_close(self.g)
            self.g = None
