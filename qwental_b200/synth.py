"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark configs.

They stand in for the real model file (which is not distributed) and for the reference's server-level
benchmark requests.  Block layouts follow the GGML formats the reference decodes:
IQ3_S super-block of 256 weights in 110 bytes (kernels/moe_iq.metal:102-118: d fp16 @0, qs[64] @2,
qh[8] @66, signs[32] @74, scales[4] @106) and Q8_0 block of 32 weights in 34 bytes (src/ggml_dq.c:34-37).
"""
from __future__ import annotations

import numpy as np

IQ3_S, Q8_0 = 21, 8


def row_bytes(qtype: int, K: int) -> int:
    if qtype == IQ3_S:
        assert K % 256 == 0
        return K // 256 * 110
    if qtype == Q8_0:
        assert K % 32 == 0
        return K // 32 * 34
    raise ValueError("unsupported ggml type %d" % qtype)


def _scales_fp16(rng, n, d_scale=1.0):
    """d as fp16 drawn uniform in [1e-3, 2e-2], optionally times a power-of-two d_scale.

    A stack of random matrices at the stated range overflows fp16 after two contractions (a SwiGLU expert's
    output has rms ~1.5e5), so the layer- and model-level configs scale d per tensor to keep every block
    output O(1); the single-matvec configs use d_scale = 1."""
    return (rng.uniform(1e-3, 2e-2, size=n) * d_scale).astype(np.float16)


def d_scale_for(K: int) -> float:
    """Power of two that brings the output rms of a random IQ3_S [N][K] matvec on unit-rms input near 1."""
    return {256: 2.0 ** -5, 512: 2.0 ** -5, 2048: 2.0 ** -6, 4096: 2.0 ** -7}.get(K, 2.0 ** -6)


def iq3s_rows(rng: np.random.Generator, nrows: int, K: int, d_scale: float = 1.0) -> np.ndarray:
    """uint8 [nrows][K/256*110]: every byte uniform in [0,255] except the fp16 scale d (times d_scale)."""
    nb = K // 256
    blk = rng.integers(0, 256, size=(nrows, nb, 110), dtype=np.uint8)
    blk[:, :, 0:2] = _scales_fp16(rng, nrows * nb, d_scale).view(np.uint8).reshape(nrows, nb, 2)
    return blk.reshape(nrows, nb * 110)


def q8_0_rows(rng: np.random.Generator, nrows: int, K: int, d_scale: float = 1.0) -> np.ndarray:
    """uint8 [nrows][K/32*34]: fp16 scale d as above, int8 uniform in [-127, 127]."""
    nb = K // 32
    blk = np.empty((nrows, nb, 34), np.uint8)
    blk[:, :, 2:] = rng.integers(-127, 128, size=(nrows, nb, 32), dtype=np.int8).view(np.uint8)
    blk[:, :, 0:2] = _scales_fp16(rng, nrows * nb, d_scale).view(np.uint8).reshape(nrows, nb, 2)
    return blk.reshape(nrows, nb * 34)


def quant_rows(rng, qtype: int, nrows: int, K: int) -> np.ndarray:
    return iq3s_rows(rng, nrows, K) if qtype == IQ3_S else q8_0_rows(rng, nrows, K)


def acts_fp16(rng: np.random.Generator, B: int, K: int) -> np.ndarray:
    return rng.standard_normal((B, K)).astype(np.float16)


def ragged_contexts(rng: np.random.Generator, nslots: int, lo: int = 1024, hi: int = 49152) -> np.ndarray:
    """Per-slot context lengths, log-uniform in [lo, hi]."""
    return np.round(np.exp(rng.uniform(np.log(lo), np.log(hi), size=nslots))).astype(np.int64)


# --------------------------------------------------------------------------- counter-based fill (full model)
# The full-size model (tens of GB of random blocks) is filled on the device by the `synth_fill` kernel; the
# same function in numpy lets a test or the CPU baseline regenerate any tensor.  byte i of a tensor with
# seed s is the low byte of mix64(s * 0x9E3779B97F4A7C15 + i).
_M1, _M2 = np.uint64(0xBF58476D1CE4E5B9), np.uint64(0x94D049BB133111EB)


def mix64(z: np.ndarray) -> np.ndarray:
    z = z.astype(np.uint64)
    with np.errstate(over="ignore"):
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def tensor_seed(master: int, layer: int, name: str) -> int:
    h = np.uint64(master & 0xFFFFFFFFFFFFFFFF)
    with np.errstate(over="ignore"):
        for ch in ("%d/%s" % (layer, name)).encode():
            h = mix64(np.array([h ^ np.uint64(ch)], np.uint64))[0]
    return int(h)


def hash_u64(seed: int, idx: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return mix64(np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15) + idx.astype(np.uint64))


def fill_scale_bits(seed: int, blk_idx: np.ndarray, d_scale: float = 1.0) -> np.ndarray:
    """fp16 bit pattern of d for block blk_idx: (1e-3 + u * 1.9e-2) * d_scale, u = 24-bit uniform, rounded to fp16."""
    u = (hash_u64(seed ^ 0x5CA1E, blk_idx) >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    d = ((np.float32(1e-3) + u * np.float32(1.9e-2)).astype(np.float32) * np.float32(d_scale)).astype(np.float32)
    return d.astype(np.float16).view(np.uint16)


def fill_quant_rows(seed: int, qtype: int, nrows: int, K: int, row0: int = 0, d_scale: float = 1.0) -> np.ndarray:
    """Rows row0 .. row0+nrows-1 of the tensor the device `synth_fill` kernel writes for (seed, qtype, K)."""
    rb = row_bytes(qtype, K)
    bb = 110 if qtype == IQ3_S else 34
    i = np.arange(row0 * rb, (row0 + nrows) * rb, dtype=np.uint64)
    by = (hash_u64(seed, i) & np.uint64(0xFF)).astype(np.uint8)
    if qtype == Q8_0:
        by = np.where(by == 0x80, np.uint8(0x81), by)  # keep int8 in [-127, 127]
    blk = i // np.uint64(bb)
    off = (i % np.uint64(bb)).astype(np.int64)
    sb = fill_scale_bits(seed, blk, d_scale)
    by = np.where(off == 0, (sb & 0xFF).astype(np.uint8), by)
    by = np.where(off == 1, (sb >> 8).astype(np.uint8), by)
    return by.reshape(nrows, rb)


def fill_fp16_normal(seed: int, n: int, std: float, i0: int = 0) -> np.ndarray:
    """fp16 values ~ N(0, std) by Box-Muller on two 24-bit uniforms (same arithmetic as the device fill)."""
    i = np.arange(i0, i0 + n, dtype=np.uint64)
    h = hash_u64(seed, i)
    u1 = ((h >> np.uint64(40)).astype(np.float32) + np.float32(1.0)) * np.float32(1.0 / 16777216.0)
    u2 = ((h >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    r = np.sqrt(np.float32(-2.0) * np.log(u1)).astype(np.float32)
    v = (r * np.cos(np.float32(6.283185307179586) * u2).astype(np.float32) * np.float32(std)).astype(np.float32)
    return v.astype(np.float16)
