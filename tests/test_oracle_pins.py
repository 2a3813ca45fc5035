"""Pins the CPU oracle before anything is compared against it (CPU only).

Golden vectors (tests/golden/dq_golden.npz, made by tests/golden/gen_golden.py) hold the outputs of
gguf.quants.dequantize -- the arithmetic the reference's tools/dqtest.py:33-38 checks its kernels against --
and of the reference's own src/ggml_dq.c (through tools/dqcpu.c) for Q8_0.
"""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from qwental_b200 import synth


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_iq3s_decode_bit_exact_vs_gguf(golden):
    got = orc.dq_rows(orc.IQ3_S, golden["iq3s_raw"], 2048)
    assert np.array_equal(bits(got), bits(golden["iq3s_ref"]))


def test_iq3s_edge_blocks_bit_exact_vs_gguf(golden):
    got = orc.dq_rows(orc.IQ3_S, golden["edge_raw"], 256)
    assert np.array_equal(bits(got), bits(golden["edge_ref"]))


def test_q8_0_decode_bit_exact_vs_gguf_and_reference_c(golden):
    got = orc.dq_rows(orc.Q8_0, golden["q8_raw"], 2048)
    assert np.array_equal(bits(got), bits(golden["q8_ref"]))
    assert "q8_refc" in golden.files, "fixture lacks the reference's ggml_dq.c output"
    assert np.array_equal(bits(got), bits(golden["q8_refc"]))


@pytest.mark.skipif(not os.path.exists(orc.REF_LIB), reason="oracle/_ref not built (reference tree absent)")
def test_q8_0_decode_vs_live_reference_library():
    rng = np.random.default_rng(5)
    W = synth.q8_0_rows(rng, 7, 1024)
    assert np.array_equal(bits(orc.dq_rows(orc.Q8_0, W, 1024)), bits(orc.ref_dq_q8_0_rows(W, 1024)))


def test_live_gguf_agrees_when_installed():
    quants = pytest.importorskip("gguf.quants")
    from gguf import GGMLQuantizationType as Q
    rng = np.random.default_rng(11)
    W = synth.iq3s_rows(rng, 9, 4096)
    ref = quants.dequantize(W, Q.IQ3_S).reshape(9, 4096).astype(np.float32)
    assert np.array_equal(bits(orc.dq_rows(orc.IQ3_S, W, 4096)), bits(ref))


@pytest.mark.parametrize("qtype,K", [(21, 2048), (21, 512), (8, 2048), (8, 64)])
def test_canonical_matvec_close_to_fp64(qtype, K):
    rng = np.random.default_rng(3)
    W = synth.quant_rows(rng, qtype, 24, K)
    x = synth.acts_fp16(rng, 3, K)
    yc = orc.qmv_canon(qtype, W, K, x)
    y64 = orc.qmv_f64(qtype, W, K, x)
    assert np.abs(yc - y64).max() <= 1e-5 * np.abs(y64).max() + 1e-6
    # batched rows are bit-identical to each row alone (the oracle's own order does not depend on B)
    for b in range(3):
        assert np.array_equal(bits(orc.qmv_canon(qtype, W, K, x[b:b + 1])[0]), bits(yc[b]))


def test_cpu_baseline_matvec_matches_fp64():
    rng = np.random.default_rng(4)
    W = synth.iq3s_rows(rng, 40, 2048)
    x = synth.acts_fp16(rng, 2, 2048)
    y, used = orc.qmv_cpu(21, W, 2048, x.astype(np.float32), 0)
    assert used >= 1
    y64 = orc.qmv_f64(21, W, 2048, x)
    assert np.abs(y - y64).max() <= 1e-4 * np.abs(y64).max()


def test_topk_ties_lowest_id_and_softmax_rank_order():
    lg = np.zeros((1, 16), np.float32)
    lg[0, [3, 7, 9]] = 2.0
    lg[0, 12] = 5.0
    ids, w = orc.topk(lg, 4)
    assert ids[0].tolist() == [12, 3, 7, 9]
    e = np.exp(np.float64(lg[0, ids[0]]) - 5.0)
    assert np.allclose(w[0], e / e.sum(), rtol=1e-6)


def test_router_canon_close_to_fp64():
    rng = np.random.default_rng(6)
    Wr = (rng.standard_normal((32, 2048)) * 0.02).astype(np.float16)
    x = synth.acts_fp16(rng, 4, 2048)
    lg = orc.router_canon(Wr, x)
    ref = x.astype(np.float64) @ Wr.astype(np.float64).T
    assert np.abs(lg - ref).max() < 1e-5


def test_counter_fill_blocks_have_valid_fields():
    W = synth.fill_quant_rows(1234, 21, 5, 2048, row0=3)
    d = W.reshape(5, 8, 110)[:, :, :2].copy().view(np.float16).astype(np.float64)
    assert d.min() >= 9.9e-4 and d.max() <= 2.0e-2 + 1e-4
    # rows are position-addressed: regenerating a sub-range gives the same bytes
    assert np.array_equal(W[2], synth.fill_quant_rows(1234, 21, 1, 2048, row0=5)[0])
    Q = synth.fill_quant_rows(99, 8, 4, 2048)
    q = Q.reshape(4, 64, 34)[:, :, 2:].view(np.int8)
    assert q.min() >= -127
