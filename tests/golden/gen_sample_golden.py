#!/usr/bin/env python3
"""Golden vectors for the host sampler, produced by the reference's own code.

oracle/Makefile compiles the reference's sampler (src/engine.c:6086-6148, 9410-9418) from the reference tree into
oracle/_ref/libsample_ref.so.  This script feeds it seeded logit rows (with ties at the top and at the cut) under several
temperature / top-k / top-p settings and records the tokens it draws and the RNG state it leaves, so that the test can check
this library's qw_engine_sample where the reference tree (and with it oracle/_ref) is absent.

    make -C oracle && python tests/golden/gen_sample_golden.py      # writes tests/golden/sample_golden.npz
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "..", "..", "oracle", "_ref", "libsample_ref.so")


class QwGen(C.Structure):  # src/engine.h:39-52
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("seed", C.c_ulonglong), ("max_tokens", C.c_int),
                ("stop", C.c_void_p), ("nstop", C.c_int), ("spec", C.c_bool), ("persist", C.c_void_p), ("npersist", C.c_int),
                ("yield_", C.c_void_p), ("pf_yield", C.c_void_p)]


def main():
    ref = C.CDLL(SO)
    ref.qw_engine_sample.restype = C.c_int32
    ref.qw_engine_sample.argtypes = [C.c_void_p, C.POINTER(QwGen), C.POINTER(C.c_ulonglong)]
    rng = np.random.default_rng(2024)
    V, rows, draws = 1024, 6, 8
    C.c_int.in_dll(ref, "ref_vocab").value = V
    logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    for r in range(rows):
        top = np.argsort(-logits[r])[:8]
        logits[r, top[1]] = logits[r, top[0]]
        logits[r, top[6]] = logits[r, top[5]]
        logits[r, rng.integers(0, V, 30)] = logits[r, top[3]]
    params = np.array([(0.0, 0, 1.0), (0.8, 40, 0.95), (1.0, 0, 1.0), (1.3, 300, 0.5), (0.7, 1, 1.0), (0.05, 256, 0.9), (2.0, 7, 0.999)], np.float32)
    seeds = rng.integers(1, 2**62, size=(len(params), rows)).astype(np.uint64)
    toks = np.zeros((len(params), rows, draws), np.int32)
    states = np.zeros((len(params), rows, draws), np.uint64)
    for pi, (T, k, p) in enumerate(params):
        g = QwGen(temperature=float(T), top_k=int(k), top_p=float(p))
        for r in range(rows):
            st = C.c_ulonglong(int(seeds[pi, r]))
            for d in range(draws):
                toks[pi, r, d] = ref.qw_engine_sample(logits[r].ctypes.data, C.byref(g), C.byref(st))
                states[pi, r, d] = st.value
    np.savez_compressed(os.path.join(HERE, "sample_golden.npz"), logits=logits, params=params, seeds=seeds, toks=toks, states=states)
    print("wrote sample_golden.npz:", toks.shape, "draws")


if __name__ == "__main__":
    main()
