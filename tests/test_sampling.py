"""Sampling (the caller's side of the decode step): the host sampler behind the C ABI against the Python restatement of
the reference's make_dist / dist_draw (CPU test), the device candidate selection against a stable sort, and the sampled
step against the same sampler applied to the step's full logits (GPU tests)."""
import numpy as np
import pytest

from oracle import oracle as orc

CASES = [(0.0, 0, 1.0), (0.8, 40, 0.95), (1.0, 0, 1.0), (1.3, 300, 0.5), (0.7, 1, 1.0), (0.05, 256, 0.9), (2.0, 7, 0.999)]


def _logits(rng, V, ties=True):
    lg = (rng.standard_normal(V) * 3).astype(np.float32)
    if ties:  # equal values at the top and at a cut boundary
        top = np.argsort(-lg)[:6]
        lg[top[1]] = lg[top[0]]
        lg[top[5]] = lg[top[4]]
        lg[rng.integers(0, V, 50)] = lg[top[3]]
    return lg


def test_host_sampler_matches_reference_restatement():
    from qwental_b200.engine import sample
    rng = np.random.default_rng(11)
    for V in (512, 5000, 151936):
        lg = _logits(rng, V)
        for T, k, p in CASES:
            state = np.array([rng.integers(0, 2**63)], np.uint64)
            want_state = int(state[0])
            for _ in range(4):  # a few consecutive draws from the same stream
                want, want_state = orc.sample_ref(lg, T, k, p, want_state)
                got = sample(lg, T, k, p, state)
                assert got == want and int(state[0]) == want_state, (V, T, k, p)


def test_host_sampler_matches_the_reference_code():
    """qw_engine_sample of this library against the reference's own qw_engine_sample, compiled from its source lines into
    oracle/_ref/libsample_ref.so by oracle/Makefile (skipped where that file was not built)."""
    import ctypes as C
    import os
    from qwental_b200.engine import sample
    so = os.path.join(os.path.dirname(orc.__file__), "_ref", "libsample_ref.so")
    if not os.path.exists(so):
        pytest.skip("oracle/_ref/libsample_ref.so not built (reference tree absent)")

    class QwGen(C.Structure):  # src/engine.h:39-52
        _fields_ = [("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("seed", C.c_ulonglong), ("max_tokens", C.c_int),
                    ("stop", C.c_void_p), ("nstop", C.c_int), ("spec", C.c_bool), ("persist", C.c_void_p), ("npersist", C.c_int),
                    ("yield_", C.c_void_p), ("pf_yield", C.c_void_p)]
    ref = C.CDLL(so)
    ref.qw_engine_sample.restype = C.c_int32
    ref.qw_engine_sample.argtypes = [C.c_void_p, C.POINTER(QwGen), C.POINTER(C.c_ulonglong)]
    rng = np.random.default_rng(3)
    for V in (512, 151936):
        C.c_int.in_dll(ref, "ref_vocab").value = V
        lg = _logits(rng, V)
        for T, k, p in CASES:
            mine = np.array([rng.integers(0, 2**63)], np.uint64)
            theirs = C.c_ulonglong(int(mine[0]))
            g = QwGen(temperature=T, top_k=k, top_p=p)
            for _ in range(6):
                want = ref.qw_engine_sample(lg.ctypes.data, C.byref(g), C.byref(theirs))
                got = sample(lg, T, k, p, mine)
                assert got == want and int(mine[0]) == theirs.value, (V, T, k, p)
            # the entry point with the reference's own signature, given the very same qw_gen bytes
            from qwental_b200 import lib
            L = lib.load()
            L.qw_engine_sample.restype = C.c_int32
            L.qw_engine_sample.argtypes = [C.c_void_p, C.POINTER(QwGen), C.POINTER(C.c_ulonglong)]
            L.qw_engine_sample_set_vocab(V)
            a, b = C.c_ulonglong(12345), C.c_ulonglong(12345)
            for _ in range(3):
                assert L.qw_engine_sample(lg.ctypes.data, C.byref(g), C.byref(a)) == ref.qw_engine_sample(lg.ctypes.data, C.byref(g), C.byref(b))
                assert a.value == b.value


def test_host_sampler_matches_reference_golden_vectors():
    """The committed vectors were drawn by the reference's own sampler (tests/golden/gen_sample_golden.py)."""
    import os
    from qwental_b200.engine import sample
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "sample_golden.npz"))
    for pi, (T, k, p) in enumerate(g["params"]):
        for r in range(g["logits"].shape[0]):
            st = np.array([g["seeds"][pi, r]], np.uint64)
            for d in range(g["toks"].shape[2]):
                tok = sample(g["logits"][r], float(T), int(k), float(p), st)
                assert tok == g["toks"][pi, r, d] and st[0] == g["states"][pi, r, d], (pi, r, d)


def test_sampler_follows_the_distribution():
    from qwental_b200.engine import sample
    lg = np.log(np.array([0.5, 0.25, 0.125, 0.125], np.float32))
    state = np.array([12345], np.uint64)
    n = 20000
    cnt = np.bincount([sample(lg, 1.0, 0, 1.0, state) for _ in range(n)], minlength=4) / n
    assert np.abs(cnt - np.array([0.5, 0.25, 0.125, 0.125])).max() < 0.015
    cnt = np.bincount([sample(lg, 1.0, 0, 0.6, state) for _ in range(n)], minlength=4) / n  # nucleus keeps the first two
    assert cnt[2] == 0 and cnt[3] == 0 and abs(cnt[0] - 2 / 3) < 0.015


@pytest.mark.gpu
@pytest.mark.parametrize("V,B,k", [(151936, 5, 256), (151936, 2, 40), (512, 3, 256), (300, 2, 256), (70000, 64, 17)])
def test_candidate_kernel_equals_stable_sort(V, B, k):
    from qwental_b200.gpu import Gpu
    gpu = Gpu()
    try:
        rng = np.random.default_rng(V + B)
        lg = np.stack([_logits(rng, V) for _ in range(B)])
        lg[0, : min(V, 400)] = 1e9  # more equal maxima than candidates: the lowest ids win
        lb, ids, vals = gpu.buf_from(lg), gpu.buf(B * 256 * 4), gpu.buf(B * 256 * 4)
        kk = gpu.compile("k_topk", "k_topk_t")
        gpu.batch().kernel(kk).buf(0, lb).buf(1, ids).buf(2, vals).bytes(3, np.array([B, V, k], np.uint32)).dispatch((B,), (1024,)).end()
        gi, gv = ids.download(np.int32, B * 256).reshape(B, 256), vals.download(np.float32, B * 256).reshape(B, 256)
        n = min(k, V)
        for r in range(B):
            order = np.lexsort((np.arange(V), -lg[r].astype(np.float64)))[:n]
            assert np.array_equal(gi[r, :n], order), r
            assert np.array_equal(gv[r, :n].view(np.uint32), lg[r][order].view(np.uint32))
            assert (gi[r, n:] == -1).all()
    finally:
        gpu.close()


@pytest.mark.gpu
def test_sampled_step_equals_sampler_on_full_logits():
    from qwental_b200.engine import Engine, tiny_cfg
    from qwental_b200.gpu import Gpu
    gpu = Gpu()
    eng = Engine(gpu, tiny_cfg())
    try:
        ctx = {0: 300, 3: 5, 5: 777, 6: 255}
        sids, toks = [0, 3, 5, 6], [7, 100, 511, 0]
        params = [(0.0, 0, 1.0), (0.8, 40, 0.95), (1.0, 0, 1.0), (1.5, 300, 0.3)]
        for rep in range(3):
            for s, n in ctx.items():
                eng.seed_slot(s, n, 1000 + s)
            logits, _ = eng.step(sids, toks)
            for s, n in ctx.items():
                eng.seed_slot(s, n, 1000 + s)
            state = np.array([101 + rep, 202, 303 + rep, 404], np.uint64)
            want = [orc.sample_ref(logits[i], *params[i], int(state[i])) for i in range(4)]
            ids, ms = eng.step_sample(sids, toks, params, state)
            assert ms > 0
            assert list(ids) == [w[0] for w in want]
            assert [int(x) for x in state] == [w[1] for w in want]
    finally:
        eng.close()
        gpu.close()


def test_reference_signature_entry_point_equals_the_explicit_one():
    """qw_engine_sample(logits, const qw_gen *, rng) -- the reference's signature (src/engine.h:125) -- reads the first
    three fields of qw_gen and the vocabulary set for the process; it must draw what qw_engine_sample_v draws."""
    import ctypes as C
    from qwental_b200 import lib
    from qwental_b200.engine import sample

    class QwGen(C.Structure):  # src/engine.h:39-52
        _fields_ = [("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("seed", C.c_ulonglong), ("max_tokens", C.c_int),
                    ("stop", C.c_void_p), ("nstop", C.c_int), ("spec", C.c_bool), ("persist", C.c_void_p), ("npersist", C.c_int),
                    ("yield_", C.c_void_p), ("pf_yield", C.c_void_p)]
    L = lib.load()
    L.qw_engine_sample.restype = C.c_int32
    L.qw_engine_sample.argtypes = [C.c_void_p, C.POINTER(QwGen), C.POINTER(C.c_ulonglong)]
    rng = np.random.default_rng(11)
    V = 4096
    lg = _logits(rng, V)
    L.qw_engine_sample_set_vocab(0)
    assert L.qw_engine_sample(lg.ctypes.data, C.byref(QwGen(temperature=1.0)), C.byref(C.c_ulonglong(1))) == -1  # no vocabulary known yet
    L.qw_engine_sample_set_vocab(V)
    for T, k, p in CASES:
        st = np.array([rng.integers(0, 2**63)], np.uint64)
        theirs = C.c_ulonglong(int(st[0]))
        g = QwGen(temperature=T, top_k=k, top_p=p, seed=99, max_tokens=7)
        for _ in range(4):
            assert L.qw_engine_sample(lg.ctypes.data, C.byref(g), C.byref(theirs)) == sample(lg, T, k, p, st)
            assert theirs.value == int(st[0])
