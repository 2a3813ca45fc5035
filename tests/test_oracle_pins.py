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


# ---- the floating-point layer references against the reference's own CPU checks
def _layer_cases():
    import importlib.util
    spec = importlib.util.spec_from_file_location("gen_layer_golden", os.path.join(os.path.dirname(__file__), "golden", "gen_layer_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _numpy_layer_outputs(d):
    g, a, m = d["gdn"], d["attn"], d["moe"]
    S1, o1 = orc.gdn_core_ref(g["S"], g["qn"].astype(np.float64), g["kn"].astype(np.float64), g["v"].astype(np.float64), g["la"], g["beta"], g["hk_of"])
    out, ids, _ = orc.moe_ref(m["x"], m["Wr"], m["wsg"], m["gate"], m["up"], m["down"], m["sg"], m["su"], m["sd"], m["D"], m["I"], m["T"], ref_arith=True)
    return dict(gdn_o=o1, gdn_S_sample=S1.reshape(-1)[::97], attn_o=orc.attn_core_ref(a["q"], a["K"], a["V"]), moe_ids=ids, moe_out=out)


def _close(got, want, tol=1e-12):
    return np.abs(np.asarray(got, np.float64) - want).max() <= tol * np.abs(want).max()


def test_fp_layer_references_match_reference_golden_vectors():
    """gdn_core_ref, attn_core_ref and moe_ref (the references every GPU parity test compares against) reproduce, to 1e-12
    relative, what the reference's own CPU checks computed on the same seeded inputs (tests/golden/layer_ref_golden.npz,
    written by tests/golden/gen_layer_golden.py from bench/gdn_decode.c:74-84, bench/qsa.c:184-201,
    bench/moe_decode.c:133-177)."""
    want = np.load(os.path.join(os.path.dirname(__file__), "golden", "layer_ref_golden.npz"))
    got = _numpy_layer_outputs(_layer_cases().layer_inputs())
    assert np.array_equal(got["moe_ids"], want["moe_ids"])
    for k in ("gdn_o", "gdn_S_sample", "attn_o", "moe_out"):
        assert _close(got[k], want[k]), k


@pytest.mark.skipif(not os.path.exists(orc.REF_LAYERS), reason="oracle/_ref/liblayer_ref.so not built (reference tree absent)")
def test_fp_layer_references_match_live_reference_code():
    mod = _layer_cases()
    d = mod.layer_inputs()
    want, got = mod.reference_outputs(d), _numpy_layer_outputs(d)
    assert np.array_equal(got["moe_ids"], want["moe_ids"])
    for k in ("gdn_o", "gdn_S_sample", "attn_o", "moe_out"):
        assert _close(got[k], want[k]), k
    # other shapes than the committed ones: the benchmark's 32 / 16 heads, a longer context
    rng = np.random.default_rng(77)
    HV, HK, DK, DV = 32, 16, 128, 128
    q, k = rng.standard_normal((HK, DK)), rng.standard_normal((HK, DK))
    qn = (q / np.linalg.norm(q, axis=1, keepdims=True) / np.sqrt(DK)).astype(np.float16)
    kn = (k / np.linalg.norm(k, axis=1, keepdims=True)).astype(np.float16)
    S = (rng.standard_normal((HV, DK, DV)) * 0.1).astype(np.float32).astype(np.float64)
    v = rng.standard_normal((HV, DV)).astype(np.float16)
    la, be = np.log(0.9 + 0.1 * rng.random(HV)).astype(np.float32), (0.1 + 0.8 * rng.random(HV)).astype(np.float32)
    S1, o1 = orc.ref_gdn_core(S, qn, kn, v, la, be)
    S2, o2 = orc.gdn_core_ref(S, qn.astype(np.float64), kn.astype(np.float64), v.astype(np.float64), la, be, np.arange(HV) // (HV // HK))
    assert _close(S2, S1) and _close(o2, o1)
    L = 2500
    qq, K, V = (rng.standard_normal(s).astype(np.float16) for s in ((16, 256), (L, 2, 256), (L, 2, 256)))
    assert _close(orc.attn_core_ref(qq, K, V), orc.ref_attn_core(qq, K, V))
