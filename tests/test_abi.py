"""CPU-only checks of the C-ABI library: it loads, exports every symbol include/*.h declares, and refuses to
open without a CUDA device (no CPU fallback)."""
import os
import re

import pytest

from qwental_b200 import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(qw_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    L = lib.load()
    decl = declared_symbols()
    assert set(lib.GPU_H_SYMBOLS) <= decl
    missing = [n for n in sorted(decl) if not hasattr(L, n)]
    assert not missing, missing


def test_reference_device_api_is_complete():
    # the 33 functions of the reference's src/gpu.h:18-83
    assert len(lib.GPU_H_SYMBOLS) == 33


def test_kernel_families_registered():
    L = lib.load()
    fams = {L.qw_gpu_family_name(i).decode() for i in range(L.qw_gpu_family_count())}
    assert {"dq_test", "qmv_gg", "qmv_mma"} <= fams


def test_open_fails_without_device_and_nothing_falls_back():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    L = lib.load()
    assert not L.qw_gpu_open()
    from qwental_b200.gpu import Gpu, GpuError
    with pytest.raises(GpuError):
        Gpu()
