"""Python face of the engine C ABI (include/qw_engine.h): the batched decode step `qw_engine_par_step` and its
slot management, mirroring the reference's src/engine.h:77-127.  All work happens in libqw_gpu_cuda.so."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import lib as _lib
from .gpu import Gpu, GpuError


class ModelCfg(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden", "layers", "attn_every", "vocab", "experts", "topk", "expert_inter", "qh", "kvh", "hd", "hk", "hv",
                                        "max_slots", "max_ctx", "kv_pages", "ep_rank", "ep_size", "fma")] + [("seed", C.c_ulonglong)]


class StepBytes(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("moe", "dense", "lm_head", "kv", "gdn_state", "other", "total")] + \
               [("unique_experts_sum", C.c_int), ("ctx_tokens", C.c_longlong), ("moe_iq3s", C.c_double)]


def _bind(L):
    vp, ip, i32p = C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int32)
    sig = {
        "qw_model_cfg_default": (None, [C.POINTER(ModelCfg)]),
        "qw_engine_open_synth": (vp, [vp, C.POINTER(ModelCfg)]), "qw_engine_close": (None, [vp]),
        "qw_engine_error": (C.c_char_p, [vp]), "qw_engine_gpu": (vp, [vp]),
        "qw_engine_par_slots": (C.c_int, [vp]), "qw_engine_par_pick": (C.c_int, [vp, i32p, C.c_int, C.c_ulonglong]),
        "qw_engine_par_seed": (C.c_int, [vp, C.c_int, C.c_int, C.c_ulonglong]),
        "qw_engine_par_step": (C.POINTER(C.c_float), [vp, ip, i32p, C.c_int, C.POINTER(C.c_double)]),
        "qw_engine_par_step_greedy": (i32p, [vp, ip, i32p, C.c_int, C.POINTER(C.c_double)]),
        "qw_engine_par_decode_greedy": (C.c_int, [vp, ip, i32p, C.c_int, C.c_int, i32p, C.POINTER(C.c_double)]),
        "qw_engine_par_finish": (None, [vp, C.c_int, i32p, C.c_int]), "qw_engine_par_cost": (C.c_double, [vp, C.c_int]),
        "qw_engine_par_mem": (C.c_size_t, [vp]), "qw_engine_par_pos": (C.c_int, [vp, C.c_int]),
        "qw_engine_last_step_bytes": (None, [vp, C.POINTER(StepBytes)]),
        "qw_engine_tap": (C.c_size_t, [vp, C.c_char_p, C.c_int, vp, C.c_size_t]),
        "qw_ep_unique_id": (C.c_int, [vp]), "qw_engine_ep_init": (C.c_int, [vp, vp]),
        "qw_engine_par_prefill": (C.c_void_p, [vp, C.c_int, vp, C.c_int, vp]),
        "qw_engine_sample_v": (C.c_int32, [vp, C.c_int, vp, vp]), "qw_engine_sample": (C.c_int32, [vp, vp, vp]),
        "qw_engine_sample_set_vocab": (None, [C.c_int]), "qw_engine_set_moe_probe": (C.c_int, [vp, C.c_int]),
        "qw_engine_par_step_sample": (C.c_int, [vp, vp, vp, C.c_int, vp, vp, vp, vp]),
        "qw_engine_ep_export": (C.c_int, [vp, vp]), "qw_engine_ep_connect": (C.c_int, [vp, vp, C.c_int]),
    }
    for name, (res, args) in sig.items():
        f = getattr(L, name)
        f.restype, f.argtypes = res, args


def default_cfg(**over) -> ModelCfg:
    L = _lib.load()
    _bind(L)
    c = ModelCfg()
    L.qw_model_cfg_default(C.byref(c))
    for k, v in over.items():
        setattr(c, k, v)
    return c


def tiny_cfg(**over) -> ModelCfg:
    """A small model of the same architecture for parity tests (the oracle finishes in seconds)."""
    base = dict(hidden=256, layers=4, attn_every=4, vocab=512, experts=32, topk=4, expert_inter=256, qh=8, kvh=1, hd=256, hk=4, hv=8,
                max_slots=8, max_ctx=2048, kv_pages=0, seed=1)
    base.update(over)
    return default_cfg(**base)


SAMPLE_DT = np.dtype([("temperature", np.float32), ("top_k", np.int32), ("top_p", np.float32)])


def sample(logits: np.ndarray, temperature: float, top_k: int, top_p: float, rng: np.ndarray) -> int:
    """qw_engine_sample_v through the C ABI (host only: works without a GPU); rng = uint64 array of one element."""
    L = _lib.load()
    _bind(L)
    lg = np.ascontiguousarray(logits, np.float32)
    g = np.zeros(1, SAMPLE_DT)
    g[0] = (temperature, top_k, top_p)
    return int(L.qw_engine_sample_v(lg.ctypes.data, lg.size, g.ctypes.data, rng.ctypes.data))


def wide_cfg(**over) -> ModelCfg:
    """Few layers and experts but the full-size layer shapes (hidden 2048, 16/2 attention heads, 16/32 GDN heads), so the
    engine picks the same kernel variants as for the benchmark model (fused projection epilogues included)."""
    base = dict(hidden=2048, layers=4, attn_every=4, vocab=512, experts=32, topk=4, expert_inter=512, qh=16, kvh=2, hd=256, hk=16, hv=32,
                max_slots=8, max_ctx=2048, kv_pages=0, seed=2)
    base.update(over)
    return default_cfg(**base)


class Engine:
    def __init__(self, gpu: Gpu, cfg: ModelCfg):
        self.L = gpu.L
        _bind(self.L)
        self.gpu, self.cfg = gpu, cfg
        self.e = self.L.qw_engine_open_synth(gpu.g, C.byref(cfg))
        if not self.e:
            raise GpuError("qw_engine_open_synth: " + self.L.qw_engine_error(None).decode())

    def error(self) -> str:
        return self.L.qw_engine_error(self.e).decode()

    def seed_slot(self, sid: int, ctx_len: int, seed: int):
        if self.L.qw_engine_par_seed(self.e, sid, ctx_len, seed) != 0:
            raise GpuError("par_seed: " + self.error())

    def pick(self, busy: int = 0) -> int:
        return self.L.qw_engine_par_pick(self.e, None, 0, busy)

    def pos(self, sid: int) -> int:
        return self.L.qw_engine_par_pos(self.e, sid)

    def finish(self, sid: int):
        self.L.qw_engine_par_finish(self.e, sid, None, 0)

    @staticmethod
    def _rows(sids, toks):
        s = np.ascontiguousarray(sids, np.int32)
        t = np.ascontiguousarray(toks, np.int32)
        assert s.shape == t.shape and s.ndim == 1
        return s, t

    def step(self, sids, toks):
        """One decode step: fp32 logits [B][vocab] (copied out of the engine's host buffer) and device ms."""
        s, t = self._rows(sids, toks)
        ms = C.c_double()
        p = self.L.qw_engine_par_step(self.e, s.ctypes.data_as(C.POINTER(C.c_int)), t.ctypes.data_as(C.POINTER(C.c_int32)), len(s), C.byref(ms))
        if not p:
            raise GpuError("par_step: " + self.error())
        return np.ctypeslib.as_array(p, shape=(len(s), self.cfg.vocab)).copy(), ms.value

    def step_greedy(self, sids, toks):
        s, t = self._rows(sids, toks)
        ms = C.c_double()
        p = self.L.qw_engine_par_step_greedy(self.e, s.ctypes.data_as(C.POINTER(C.c_int)), t.ctypes.data_as(C.POINTER(C.c_int32)), len(s), C.byref(ms))
        if not p:
            raise GpuError("par_step_greedy: " + self.error())
        return np.ctypeslib.as_array(p, shape=(len(s),)).copy(), ms.value

    def decode_greedy(self, sids, toks, nsteps: int):
        s, t = self._rows(sids, toks)
        out = np.empty((nsteps, len(s)), np.int32)
        ms = C.c_double()
        r = self.L.qw_engine_par_decode_greedy(self.e, s.ctypes.data_as(C.POINTER(C.c_int)), t.ctypes.data_as(C.POINTER(C.c_int32)), len(s), nsteps,
                                               out.ctypes.data_as(C.POINTER(C.c_int32)), C.byref(ms))
        if r != nsteps:
            raise GpuError("par_decode_greedy: " + self.error())
        return out, ms.value

    def set_moe_probe(self, on: bool) -> bool:
        """Measurement aid: run the copy-only twin of the fused expert FFN kernel in its place (see qw_engine.h)."""
        return self.L.qw_engine_set_moe_probe(self.e, int(on)) == 0

    def cost(self, B: int) -> float:
        return self.L.qw_engine_par_cost(self.e, B)

    def mem(self) -> int:
        return int(self.L.qw_engine_par_mem(self.e))

    def step_bytes(self) -> StepBytes:
        b = StepBytes()
        self.L.qw_engine_last_step_bytes(self.e, C.byref(b))
        return b

    def tap(self, name: str, index: int, dtype) -> np.ndarray:
        n = self.L.qw_engine_tap(self.e, name.encode(), index, None, 0)
        if n == 0:
            raise GpuError("tap(%s, %d): nothing to read" % (name, index))
        out = np.empty(n // np.dtype(dtype).itemsize, dtype)
        got = self.L.qw_engine_tap(self.e, name.encode(), index, out.ctypes.data, out.nbytes)
        if got != n:
            raise GpuError("tap(%s, %d) failed" % (name, index))
        return out

    def prefill(self, sid: int, prompt) -> np.ndarray:
        """Feeds a prompt into an empty slot (token by token through the decode step); returns the last position's logits."""
        p = np.ascontiguousarray(prompt, np.int32)
        ptr = self.L.qw_engine_par_prefill(self.e, sid, p.ctypes.data, len(p), None)
        if not ptr:
            raise GpuError("prefill: " + self.error())
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(self.cfg.vocab,)).copy()

    def step_sample(self, sids, toks, params, rng):
        """One decode step with sampling: params = [(temperature, top_k, top_p)] per row, rng = uint64 state per row
        (advanced in place for rows that draw).  Returns (ids int32 [B], gpu_ms)."""
        B = len(sids)
        s, t = np.ascontiguousarray(sids, np.int32), np.ascontiguousarray(toks, np.int32)
        g = np.zeros(B, SAMPLE_DT)
        for i, (T, k, p) in enumerate(params):
            g[i] = (T, k, p)
        out = np.empty(B, np.int32)
        ms = C.c_double()
        if self.L.qw_engine_par_step_sample(self.e, s.ctypes.data, t.ctypes.data, B, g.ctypes.data, rng.ctypes.data, out.ctypes.data, C.addressof(ms)) != B:
            raise GpuError("step_sample: " + self.error())
        return out, ms.value

    def ep_init(self, id128: bytes):
        buf = C.create_string_buffer(id128, 128)
        if self.L.qw_engine_ep_init(self.e, C.cast(buf, C.c_void_p)) != 0:
            raise GpuError("ep_init: " + self.error())

    def ep_export(self) -> bytes:
        """Fused exchange, step 1: this rank's 64-byte buffer handle (gather them in rank order)."""
        buf = C.create_string_buffer(64)
        if self.L.qw_engine_ep_export(self.e, C.cast(buf, C.c_void_p)) != 0:
            raise GpuError("ep_export: " + self.error())
        return buf.raw

    def ep_connect(self, handles):
        """Fused exchange, step 2: map every rank's buffer (handles: list of ep_size 64-byte strings)."""
        raw = b"".join(handles)
        buf = C.create_string_buffer(raw, len(raw))
        if self.L.qw_engine_ep_connect(self.e, C.cast(buf, C.c_void_p), len(handles)) != 0:
            raise GpuError("ep_connect: " + self.error())

    def close(self):
        if self.e:
            self.L.qw_engine_close(self.e)
            self.e = None


def ep_unique_id() -> bytes:
    L = _lib.load()
    _bind(L)
    buf = C.create_string_buffer(128)
    if L.qw_ep_unique_id(C.cast(buf, C.c_void_p)) != 0:
        raise GpuError("qw_ep_unique_id failed (NCCL not loadable)")
    return buf.raw
