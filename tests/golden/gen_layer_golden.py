#!/usr/bin/env python3
"""Writes tests/golden/layer_ref_golden.npz: outputs of the reference's own CPU checks of the three floating-point
layers (bench/gdn_decode.c:74-84, bench/qsa.c:184-201, bench/moe_decode.c:133-177, compiled into
oracle/_ref/liblayer_ref.so by oracle/gen_layer_ref.py) on seeded inputs.  tests/test_oracle_pins.py rebuilds the same
inputs from the seeds (layer_inputs below) and holds the numpy references of oracle/oracle.py to these outputs, so the
pin also works where the reference tree is absent.

    python tests/golden/gen_layer_golden.py        (needs oracle/_ref/liblayer_ref.so, i.e. the reference tree)
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def layer_inputs():
    """Seeded inputs of the three checks (shared by this script and the test)."""
    from oracle import oracle as orc
    from qwental_b200 import synth
    rng = np.random.default_rng(20240)
    d = {}
    HV, HK, DK, DV = 4, 2, 128, 128
    q, k = rng.standard_normal((HK, DK)), rng.standard_normal((HK, DK))
    d["gdn"] = dict(S=(rng.standard_normal((HV, DK, DV)) * 0.1).astype(np.float32).astype(np.float64),
                    qn=(q / np.linalg.norm(q, axis=1, keepdims=True) / np.sqrt(DK)).astype(np.float16),
                    kn=(k / np.linalg.norm(k, axis=1, keepdims=True)).astype(np.float16),
                    v=rng.standard_normal((HV, DV)).astype(np.float16),
                    la=np.log(0.9 + 0.1 * rng.random(HV)).astype(np.float32), beta=(0.1 + 0.8 * rng.random(HV)).astype(np.float32),
                    hk_of=np.arange(HV) // (HV // HK))
    L = 300
    d["attn"] = dict(q=rng.standard_normal((16, 256)).astype(np.float16), K=rng.standard_normal((L, 2, 256)).astype(np.float16),
                     V=rng.standard_normal((L, 2, 256)).astype(np.float16))
    E, D, I, T = 32, 256, 256, 4
    m = dict(E=E, D=D, I=I, T=T, Wr=(rng.standard_normal((E, D)) * 0.02).astype(np.float16), wsg=(rng.standard_normal(D) * 0.02).astype(np.float16),
             gate=synth.iq3s_rows(rng, E * I, D, 1 / 8).reshape(E, I, -1), up=synth.iq3s_rows(rng, E * I, D, 1 / 8).reshape(E, I, -1),
             down=synth.iq3s_rows(rng, E * D, I, 1 / 8).reshape(E, D, -1), sg=synth.iq3s_rows(rng, I, D, 1 / 8), su=synth.iq3s_rows(rng, I, D, 1 / 8),
             sd=synth.iq3s_rows(rng, D, I, 1 / 8), x=synth.acts_fp16(rng, 3, D))
    d["moe"] = m
    return d


def reference_outputs(d):
    from oracle import oracle as orc
    g, a, m = d["gdn"], d["attn"], d["moe"]
    S1, o1 = orc.ref_gdn_core(g["S"], g["qn"], g["kn"], g["v"], g["la"], g["beta"])
    att = orc.ref_attn_core(a["q"], a["K"], a["V"])
    dq = lambda W, K: orc.dq_rows(21, W.reshape(-1, W.shape[-1]), K)
    mats = (m["Wr"].astype(np.float32), dq(m["gate"], m["D"]), dq(m["up"], m["D"]), dq(m["down"], m["I"]), dq(m["sg"], m["D"]), dq(m["su"], m["D"]),
            dq(m["sd"], m["I"]))
    ids, outs = zip(*(orc.ref_moe_check(m["x"][t], m["wsg"], *mats) for t in range(m["x"].shape[0])))
    return dict(gdn_o=o1, gdn_S_sample=S1.reshape(-1)[::97].copy(), attn_o=att, moe_ids=np.stack(ids), moe_out=np.stack(outs))


if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "layer_ref_golden.npz")
    np.savez_compressed(out, **reference_outputs(layer_inputs()))
    print("wrote", out, os.path.getsize(out), "bytes")
