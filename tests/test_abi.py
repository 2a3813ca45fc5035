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
    assert {"dq_test", "qmv_gg", "qmv_mma", "moe_route", "moe_gu", "moe_dn", "moe_ffn", "iq3x_pack", "iq3x_dq_test", "add_rmsnorm", "qsa_prep",
            "qsa_attn", "qsa_merge", "dn_epi", "gdn_fstep", "k_topk", "stream_probe", "umma_test", "umma_bench"} <= fams


def test_open_fails_without_device_and_nothing_falls_back():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    L = lib.load()
    assert not L.qw_gpu_open()
    from qwental_b200.gpu import Gpu, GpuError
    with pytest.raises(GpuError):
        Gpu()


def describe(src: str):
    import ctypes as C
    L = lib.load()
    L.qw_gpu_prelude_describe.restype = C.c_bool
    L.qw_gpu_prelude_describe.argtypes = [C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t]
    out = C.create_string_buffer(512)
    raw = src.encode()
    ok = L.qw_gpu_prelude_describe(raw, len(raw), out, 512)
    return ok, out.value.decode()


def test_compile_prelude_parsing_matches_the_reference_hosts_habits():
    # the form this repository's hosts use
    ok, d = describe("#define QW_KERNEL qmv_mma\n#define QW_NAME lm_head\n#define GF 8\n#define KD 2048 // K\n#define YT_F32 1\nkernel void ...")
    assert ok and d.split()[:2] == ["qmv_mma", "lm_head"] and {"GF=8", "KD=2048", "YT_F32=1"} <= set(d.split())
    # the reference's own prelude style (src/engine.c:705-716): shape defines, the output type, and the entry renamed
    ok, d = describe("// injected by the host\n#define GF 21\n#define KD 4096\n#define RB 1760\n#define NB 8\n#define YT float\n"
                     "#define qmv_gg qmv_gg_o_proj\n#include <metal_stdlib>\nusing namespace metal;\n#define IGNORED 5\n")
    assert ok and d.split()[:2] == ["qmv_gg", "qmv_gg_o_proj"]
    assert {"GF=21", "KD=4096", "RB=1760", "NB=8", "YT_F32=1"} <= set(d.split()) and "IGNORED=5" not in d
    # errors: no family, unknown family, bad entry name
    assert describe("#define KD 2048\n")[0] is False
    ok, msg = describe("#define QW_KERNEL no_such_kernel\n")
    assert not ok and "unknown kernel family" in msg
    assert describe("#define QW_KERNEL qmv_gg\n#define QW_NAME 9bad\n")[0] is False
    # a flag define without a value reads as 1; hex values parse
    ok, d = describe("#define QW_KERNEL moe_cmb\n#define RESID\n#define D 0x800\n")
    assert ok and {"RESID=1", "D=2048"} <= set(d.split())
