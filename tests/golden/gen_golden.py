#!/usr/bin/env python3
"""Generate tests/golden/dq_golden.npz -- run in a container that has the `gguf` package and the
reference tree (the GPU box has neither requirement: it only reads the committed .npz).

Contents:
  iq3s_raw  uint8 [16][880]    seeded random IQ3_S rows, K = 2048 (generator: qwental_b200.synth)
  iq3s_ref  float32 [16][2048] gguf.quants.dequantize(iq3s_raw, IQ3_S)  -- the arithmetic the reference's
                               tools/dqtest.py:33-38 holds its IQ3_S kernels to
  q8_raw    uint8 [16][2176]   seeded random Q8_0 rows, K = 2048
  q8_ref    float32 [16][2048] gguf.quants.dequantize(q8_raw, Q8_0)
  q8_refc   float32 [16][2048] the reference's own src/ggml_dq.c through tools/dqcpu.c (oracle/_ref/dqcpu),
                               present only if that binary was built
  edge_raw / edge_ref          IQ3_S rows with extreme fields (all-zero, all-0xFF, max scale, every qh/sign bit)
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from gguf import quants, GGMLQuantizationType as Q  # noqa: E402
from qwental_b200 import synth  # noqa: E402

K = 2048
rng = np.random.default_rng(0)
iq3s_raw = synth.iq3s_rows(rng, 16, K)
q8_raw = synth.q8_0_rows(rng, 16, K)
iq3s_ref = quants.dequantize(iq3s_raw, Q.IQ3_S).reshape(16, K).astype(np.float32)
q8_ref = quants.dequantize(q8_raw, Q.Q8_0).reshape(16, K).astype(np.float32)

edge = np.zeros((6, 1, 110), np.uint8)
one = np.array([1.0], np.float16).view(np.uint8)
edge[1, 0, :] = 0xFF
edge[1, 0, 0:2] = one
edge[2, 0, 0:2] = np.array([65504.0], np.float16).view(np.uint8)
edge[2, 0, 106:110] = 0xFF
edge[2, 0, 2:66] = np.arange(64, dtype=np.uint8) * 4
edge[3, 0, 0:2] = one
edge[3, 0, 2:66] = np.arange(64, dtype=np.uint8)
edge[3, 0, 66:74] = 0xFF
edge[4, 0, 0:2] = one
edge[4, 0, 2:66] = 255 - np.arange(64, dtype=np.uint8)
edge[4, 0, 74:106] = np.arange(32, dtype=np.uint8) * 8 + 1
edge[5, 0, 0:2] = np.array([6e-8], np.float16).view(np.uint8)  # subnormal scale
edge[5, 0, 2:110] = rng.integers(0, 256, 108, dtype=np.uint8)
edge_raw = edge.reshape(6, 110)
edge_ref = quants.dequantize(edge_raw, Q.IQ3_S).reshape(6, 256).astype(np.float32)

out = dict(iq3s_raw=iq3s_raw, iq3s_ref=iq3s_ref, q8_raw=q8_raw, q8_ref=q8_ref, edge_raw=edge_raw, edge_ref=edge_ref)
dqcpu = os.path.join(ROOT, "oracle", "_ref", "dqcpu")
if os.path.exists(dqcpu):
    with tempfile.TemporaryDirectory() as td:
        q8_raw.tofile(td + "/in")
        subprocess.run([dqcpu, "8", str(K), "16", td + "/in", td + "/out"], check=True)
        out["q8_refc"] = np.fromfile(td + "/out", np.float32).reshape(16, K)
np.savez_compressed(os.path.join(ROOT, "tests", "golden", "dq_golden.npz"), **out)
print({k: v.shape for k, v in out.items()})
