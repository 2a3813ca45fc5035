"""CPU oracle for the batched decode step -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import this module.
The product (qwental_b200) never imports it and has no CPU fallback.

Two layers:
  * ctypes bindings of oracle/_build/libqw_oracle.so (oracle/qw_oracle.c): bit-exact block decode,
    canonical-order fp32 matvec / router, FP64 matvec, top-k;
  * numpy FP64 layer references restated from the reference's Python checkers and bench CPU checks:
      MoE layer        tools/moe_ref.py:60,72-82 and bench/moe_decode.c:133-177
      decode attention bench/qsa.c:181-200 + output gate kernels/qsa_dec.metal:643-644
      GDN step         bench/gdn_decode.c:74-85 and tools/dn_ref.py:63-80 (norms, decay, gated RMSNorm,
                       fp16 rounding points)
Parity pin: see tests/test_oracle_pins.py -- block decode against gguf.quants 0.19.0 on golden blocks and the
reference's src/ggml_dq.c compiled into oracle/_ref (Q8_0); the three FP64 layer references against the reference's own
CPU double-precision checks (bench/gdn_decode.c:74-84, bench/qsa.c:184-201, bench/moe_decode.c:133-177) compiled into
oracle/_ref/liblayer_ref.so by oracle/gen_layer_ref.py, live where the reference tree is present and through the
committed vectors tests/golden/layer_ref_golden.npz everywhere.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "libqw_oracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libggml_dq_ref.so")
REF_DQCPU = os.path.join(HERE, "_ref", "dqcpu")
REF_LAYERS = os.path.join(HERE, "_ref", "liblayer_ref.so")  # the reference's CPU layer checks (oracle/gen_layer_ref.py)

IQ3_S, Q8_0 = 21, 8
_u8p, _u16p, _f32p, _f64p, _i32p = (C.POINTER(t) for t in (C.c_uint8, C.c_uint16, C.c_float, C.c_double, C.c_int32))


def build(force: bool = False) -> None:
    """Compile the oracle (and oracle/_ref when the reference tree is present)."""
    if force or not os.path.exists(LIB):
        subprocess.run(["make", "-C", HERE], check=True, capture_output=True)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = C.CDLL(LIB)
        _lib.orc_row_bytes.restype = C.c_long
    return _lib


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def row_bytes(qtype: int, K: int) -> int:
    return {IQ3_S: K // 256 * 110, Q8_0: K // 32 * 34}[qtype]


def dq_rows(qtype: int, W: np.ndarray, K: int) -> np.ndarray:
    """Decode rows of ggml blocks (uint8 [N][row_bytes]) to fp32 [N][K], bit-exact."""
    W = np.ascontiguousarray(W, dtype=np.uint8).reshape(-1, row_bytes(qtype, K))
    out = np.empty((W.shape[0], K), np.float32)
    rc = lib().orc_dq_rows(qtype, _p(W, _u8p), W.shape[0], K, _p(out, _f32p))
    assert rc == 0
    return out


def qmv_canon(qtype: int, W: np.ndarray, K: int, x16: np.ndarray) -> np.ndarray:
    """Canonical-order fp32 matvec: x16 fp16 [B][K] -> fp32 [B][N] (bit-exact target of the FMA kernels)."""
    W = np.ascontiguousarray(W, dtype=np.uint8).reshape(-1, row_bytes(qtype, K))
    x16 = np.ascontiguousarray(x16, dtype=np.float16).reshape(-1, K)
    N, B = W.shape[0], x16.shape[0]
    y = np.empty((B, N), np.float32)
    rc = lib().orc_qmv_canon(qtype, _p(W, _u8p), N, K, _p(x16.view(np.uint16), _u16p), B, K, _p(y, _f32p), N)
    assert rc == 0
    return y


def qmv_f64(qtype: int, W: np.ndarray, K: int, x16: np.ndarray) -> np.ndarray:
    W = np.ascontiguousarray(W, dtype=np.uint8).reshape(-1, row_bytes(qtype, K))
    x16 = np.ascontiguousarray(x16, dtype=np.float16).reshape(-1, K)
    N, B = W.shape[0], x16.shape[0]
    y = np.empty((B, N), np.float64)
    rc = lib().orc_qmv_f64(qtype, _p(W, _u8p), N, K, _p(x16.view(np.uint16), _u16p), B, K, _p(y, _f64p), N)
    assert rc == 0
    return y


def qmv_cpu(qtype: int, W: np.ndarray, K: int, xf: np.ndarray, nthreads: int = 0):
    """The timed CPU baseline: decode each row to fp32, fp32 dot per token.  Returns (y, threads used)."""
    W = np.ascontiguousarray(W, dtype=np.uint8).reshape(-1, row_bytes(qtype, K))
    xf = np.ascontiguousarray(xf, dtype=np.float32).reshape(-1, K)
    N, B = W.shape[0], xf.shape[0]
    y = np.empty((B, N), np.float32)
    used = lib().orc_qmv_cpu(qtype, _p(W, _u8p), N, K, _p(xf, _f32p), B, _p(y, _f32p), nthreads)
    assert used > 0
    return y, used


def router_canon(Wr16: np.ndarray, x16: np.ndarray) -> np.ndarray:
    """fp16 router rows [E][D] x fp16 tokens [B][D] -> fp32 logits [B][E] in the canonical order."""
    Wr16 = np.ascontiguousarray(Wr16, dtype=np.float16)
    x16 = np.ascontiguousarray(x16, dtype=np.float16)
    E, D = Wr16.shape
    B = x16.shape[0]
    lg = np.empty((B, E), np.float32)
    lib().orc_router_canon(_p(Wr16.view(np.uint16), _u16p), E, D, _p(x16.view(np.uint16), _u16p), B, _p(lg, _f32p), E)
    return lg


def topk(logits: np.ndarray, k: int):
    """Per token: ids (ties -> lowest id) and softmax weights over the picked logits."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    B, E = logits.shape
    ids = np.empty((B, k), np.int32)
    w = np.empty((B, k), np.float32)
    for t in range(B):
        lib().orc_topk(_p(logits[t], _f32p), E, k, _p(ids[t], _i32p), _p(w[t], _f32p))
    return ids, w


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ----------------------------------------------------------------------------------------------- reference build
def ref_dq_q8_0_rows(W: np.ndarray, K: int) -> np.ndarray:
    """Q8_0 rows decoded by the reference's own src/ggml_dq.c (qw_ggml_dq_row), compiled into oracle/_ref."""
    r = C.CDLL(REF_LIB)
    r.qw_ggml_dq_row.restype = C.c_bool
    W = np.ascontiguousarray(W, dtype=np.uint8).reshape(-1, row_bytes(Q8_0, K))
    out = np.empty((W.shape[0], K), np.float32)
    for i in range(W.shape[0]):
        ok = r.qw_ggml_dq_row(8, _p(W[i], _u8p), _p(out[i], _f32p), K)
        assert ok
    return out


# ----------------------------------------------------------------------------------------------- FP64 layer references
def silu(v):
    return v / (1.0 + np.exp(-v))


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def h16(a):
    """Round through fp16 (the reference's rounding points, tools/dn_ref.py:58)."""
    return np.asarray(a).astype(np.float16).astype(np.float64)


def moe_ref(x16, Wr16, wsg16, gate, up, down, sh_gate, sh_up, sh_down, D, I, topk_n=10, ids=None, ref_arith=False):
    """FP64 MoE layer (tools/moe_ref.py:60,72-82).  gate/up: raw IQ3_S [E][I][rb(D)], down: [E][D][rb(I)];
    shared expert the same shapes without the E axis.  `ids` (optional [B][topk]) overrides the FP64
    selection so the output can be compared for the experts a device actually chose.
    ref_arith=True reproduces the arithmetic of the reference's C check (bench/moe_decode.c:133-177) instead of
    pure FP64: expert products weight * activation are formed in fp32 before they are summed in double, and H is
    rounded to fp16 (:170) -- the mode tests/test_oracle_pins.py holds against that code.
    Returns (out [B][D] float64, ids64 [B][topk], gap [B] = 10th minus 11th FP64 logit)."""
    x = np.asarray(x16, np.float16).astype(np.float64)
    Wr = np.asarray(Wr16, np.float16).astype(np.float64)
    B = x.shape[0]
    lg = x @ Wr.T
    ids64 = np.argsort(-lg, axis=1, kind="stable")[:, :topk_n]
    srt = -np.sort(-lg, axis=1)
    gap = srt[:, topk_n - 1] - srt[:, topk_n]
    use = ids64 if ids is None else np.asarray(ids)

    def mv(M, v):
        if not ref_arith:
            return M.astype(np.float64) @ v
        return (M.astype(np.float32) * np.asarray(v, np.float32)[None, :]).astype(np.float64).sum(1)

    def expert(G, U, Dn, xt):
        h = silu(mv(G, xt)) * mv(U, xt)
        if ref_arith:
            h = h.astype(np.float32).astype(np.float16).astype(np.float32)
        return mv(Dn, h)

    SG, SU, SD = dq_rows(IQ3_S, sh_gate, D), dq_rows(IQ3_S, sh_up, D), dq_rows(IQ3_S, sh_down, I)
    out = np.zeros((B, D))
    cache = {}
    for t in range(B):
        l = lg[t, use[t]]
        w = np.exp(l - l[0] if ref_arith else l - l.max())
        w /= w.sum()
        for e, we in zip(use[t], w):
            e = int(e)
            if e not in cache:
                cache[e] = (dq_rows(IQ3_S, gate[e], D), dq_rows(IQ3_S, up[e], D), dq_rows(IQ3_S, down[e], I))
            G, U, Dn = cache[e]
            out[t] += we * expert(G, U, Dn, x[t])
        sgl = float(np.asarray(wsg16, np.float16).astype(np.float64) @ x[t])
        out[t] += sigmoid(sgl) * expert(SG, SU, SD, x[t])
    return out, ids64, gap


def attn_ref(q16, K16, V16, gate16):
    """FP64 decode attention of one slot (bench/qsa.c:181-200) with the output gate of
    kernels/qsa_dec.metal:643-644.  q16 [QH][HD], K16/V16 [L][KVH][HD], gate16 [QH][HD] (pre-sigmoid).
    Returns y [QH][HD] float64 = fp16(o) * sigmoid(gate)."""
    g = np.asarray(gate16, np.float16).astype(np.float64)
    return h16(attn_core_ref(q16, K16, V16)) * sigmoid(g)


def rope_ref(v, pos, rd=64, theta=1e7):
    """Partial RoPE on the first rd dims, pairs (i, i + rd/2) (kernels/qsa_dec.metal:40-60)."""
    v = np.array(v, np.float64)
    i = np.arange(rd // 2)
    f = theta ** (-2.0 * i / rd) * pos
    c, s = np.cos(f), np.sin(f)
    a, b = v[..., :rd // 2].copy(), v[..., rd // 2:rd].copy()
    v[..., :rd // 2] = a * c - b * s
    v[..., rd // 2:rd] = b * c + a * s
    return v


def rmsnorm_ref(x, w, eps=1e-6):
    x = np.asarray(x, np.float64)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * np.asarray(w, np.float64)


def gdn_core_ref(S, qn, kn, v, la, beta, hk_of):
    """The recurrence alone (bench/gdn_decode.c:74-84) on already normalised q / k [HK][DK]: S [HV][DK][DV] is decayed,
    mem = S^T k, delta = beta (v - mem), S += k delta^T, o = S^T q.  Returns (S_new, o [HV][DV]) in float64."""
    S = np.array(S, np.float64)
    kk, qq = np.asarray(kn, np.float64)[hk_of], np.asarray(qn, np.float64)[hk_of]
    S *= np.exp(np.asarray(la, np.float64))[:, None, None]
    mem = np.einsum("hkd,hk->hd", S, kk)
    d = np.asarray(beta, np.float64)[:, None] * (np.asarray(v, np.float64) - mem)
    S += kk[:, :, None] * d[:, None, :]
    return S, np.einsum("hkd,hk->hd", S, qq)


def gdn_step_ref(S, q16, k16, v16, la, beta, z16, nw, hk_of, eps=1e-6):
    """FP64 Gated DeltaNet step of one slot (bench/gdn_decode.c:74-85, tools/dn_ref.py:63-80).
    S [HV][DK][DV] (updated copy returned), q16/k16 [HK][DK] raw conv outputs (normalised here: q also
    times DK^-1/2, both rounded to fp16 as dn_ref.py:63-64), v16 [HV][DV], la/beta [HV],
    z16 [HV][DV], nw [DV].  Returns (S_new, o16 [HV][DV] (fp16-rounded), y [HV][DV] gated RMSNorm)."""
    q = np.asarray(q16, np.float16).astype(np.float64)
    k = np.asarray(k16, np.float16).astype(np.float64)
    v = np.asarray(v16, np.float16).astype(np.float64)
    DK = q.shape[-1]
    qn = h16(q / np.sqrt((q * q).mean(-1, keepdims=True) + eps) / DK)
    kn = h16(k / np.sqrt((k * k).mean(-1, keepdims=True) + eps) / np.sqrt(DK))
    S, o = gdn_core_ref(S, qn, kn, v, la, beta, hk_of)
    o = h16(o)
    r = 1.0 / np.sqrt((o * o).mean(-1, keepdims=True) + eps)
    y = o * r * np.asarray(nw, np.float64) * sigmoid(np.asarray(z16, np.float16).astype(np.float64))
    return S, o, y


def attn_core_ref(q16, K16, V16):
    """softmax(q . K / sqrt(HD)) . V per head in float64, before the fp16 rounding and the gate (bench/qsa.c:184-201)."""
    q = np.asarray(q16, np.float16).astype(np.float64)
    K = np.asarray(K16, np.float16).astype(np.float64)
    V = np.asarray(V16, np.float16).astype(np.float64)
    QH, HD = q.shape
    KVH = K.shape[1]
    o = np.empty((QH, HD))
    for h in range(QH):
        kv = h // (QH // KVH)
        s = K[:, kv, :] @ q[h] / np.sqrt(HD)
        p = np.exp(s - s.max())
        o[h] = (p / p.sum()) @ V[:, kv, :]
    return o


# ---- the reference's own CPU checks of these layers, compiled from its bench sources into oracle/_ref/liblayer_ref.so
def _layer_ref():
    r = C.CDLL(REF_LAYERS)
    return r


def ref_gdn_core(S, qn16, kn16, v16, la, beta):
    """bench/gdn_decode.c:74-84 on fp16 q / k / v: (S_new, o) in float64; v-head h reads k-head h // (HV / HK)."""
    S0 = np.array(S, np.float64)
    HV, DK, DV = S0.shape
    qn16, kn16, v16 = (np.ascontiguousarray(a, np.float16) for a in (qn16, kn16, v16))
    pa, pb = np.ascontiguousarray(la, np.float32), np.ascontiguousarray(beta, np.float32)
    out = np.zeros((HV, DV))
    _layer_ref().ref_gdn_core(HV, qn16.shape[0], DK, DV, _p(pa, _f32p), _p(pb, _f32p), _p(qn16.view(np.uint16), _u16p),
                              _p(kn16.view(np.uint16), _u16p), _p(v16.view(np.uint16), _u16p), _p(S0, _f64p), _p(out, _f64p))
    return S0, out


def ref_attn_core(q16, K16, V16):
    """bench/qsa.c:184-201 for 16 query heads, 2 kv heads, head dim 256: o [16][256] float64."""
    q16, K16, V16 = (np.ascontiguousarray(a, np.float16) for a in (q16, K16, V16))
    assert q16.shape == (16, 256) and K16.shape[1:] == (2, 256)
    out = np.zeros((16, 256))
    _layer_ref().ref_attn_core(K16.shape[0], _p(q16.view(np.uint16), _u16p), _p(K16.view(np.uint16), _u16p), _p(V16.view(np.uint16), _u16p),
                               _p(out, _f64p))
    return out


def ref_moe_check(x16, wsg16, Wr, G, U, Dn, SG, SU, SD):
    """bench/moe_decode.c:133-177 for one token at E 32, TOPK 4, D 256, I 256; all matrices dequantised fp32
    (Wr [E][D], G/U [E*I][D], Dn [E*D][I], shared SG/SU [I][D], SD [D][I]).  Returns (ids [4], out [256] float64)."""
    f = lambda a: np.ascontiguousarray(a, np.float32)
    x16, wsg16 = np.ascontiguousarray(x16, np.float16), np.ascontiguousarray(wsg16, np.float16)
    Wr, G, U, Dn, SG, SU, SD = map(f, (Wr, G, U, Dn, SG, SU, SD))
    assert Wr.shape == (32, 256) and G.shape == (32 * 256, 256) and Dn.shape == (32 * 256, 256)
    ids, out, gpu = np.zeros(4, np.int32), np.zeros(256), np.zeros(4, np.uint32)
    _layer_ref().ref_moe_check(_p(x16.view(np.uint16), _u16p), _p(wsg16.view(np.uint16), _u16p), _p(Wr, _f32p), _p(G, _f32p), _p(U, _f32p),
                               _p(Dn, _f32p), _p(SG, _f32p), _p(SU, _f32p), _p(SD, _f32p), gpu.ctypes.data_as(C.POINTER(C.c_uint32)),
                               _p(ids, _i32p), _p(out, _f64p))
    return ids, out


# ---- sampling: make_dist + dist_draw + splitmix64 of the reference host (src/engine.c:6085-6143, 9410-9418), with its
# float / double mix kept (p is float, the running sums are double; expf is the C library's)
_libm = C.CDLL("libm.so.6")
_libm.expf.restype = C.c_float
_libm.expf.argtypes = [C.c_float]
_M64 = (1 << 64) - 1


def splitmix64(state: int):
    state = (state + 0x9E3779B97F4A7C15) & _M64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return state, z ^ (z >> 31)


def sample_ref(logits: np.ndarray, temperature: float, top_k: int, top_p: float, rng_state: int):
    """Returns (token, new rng state) as qw_engine_sample would (src/engine.c:9410-9418)."""
    lg = np.asarray(logits, np.float32)
    if temperature <= 0:
        return int(np.argmax(lg)), rng_state  # first maximum, as argmax_cpu (src/engine.c:6144-6148)
    k = top_k if 0 < top_k < 256 else 256
    order = np.lexsort((np.arange(lg.size), -lg.astype(np.float64)))[:k]  # value descending, ties by id ascending
    n = len(order)
    f32 = np.float32
    T, mx = f32(temperature), lg[order[0]]
    p = [f32(_libm.expf(f32(f32(lg[i] - mx) / T))) for i in order]
    total = 0.0
    for v in p:
        total += float(v)
    c, keep = 0.0, n
    for i in range(n):
        p[i] = f32(float(p[i]) / total)
        c += float(p[i])
        if 0 < top_p < 1 and c >= float(f32(top_p)):
            keep = i + 1
            break
    s2 = 0.0
    for i in range(keep):
        s2 += float(p[i])
    for i in range(keep):
        p[i] = f32(float(p[i]) / s2)
    tot = 0.0
    for i in range(keep):
        tot += float(p[i])
    if tot <= 0:
        return int(order[0]), rng_state
    rng_state, z = splitmix64(rng_state)
    u = float(z >> 11) * (1.0 / 9007199254740992.0) * tot
    for i in range(keep):
        u -= float(p[i])
        if u <= 0:
            return int(order[i]), rng_state
    return int(order[keep - 1]), rng_state
