"""GPU parity of the MoE decode layer (benchmark config 2), through the C ABI.

Router logits and the chosen expert ids must be bit-exact against the CPU oracle's canonical-order router and
top-k; the layer output must be within the reference's own tolerance (max error / max |ref| < 1e-2,
bench/moe_decode.c:181-182 -- we hold 2e-3) of the FP64 layer (tools/moe_ref.py:72-82) and agree on top-1;
each token's output must be bit-identical whether it runs alone or in a batch."""
import numpy as np
import pytest

from oracle import oracle as orc
from qwental_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    from qwental_b200.gpu import Gpu
    g = Gpu()
    yield g
    g.close()


def make_layer(gpu, E, D, I, topk, seed, shared=True, e_lo=0, e_hi=None, ffn="auto"):
    from qwental_b200.layers import MoeLayer
    rng = np.random.default_rng(seed)
    h = {}
    h["Wr"] = (rng.standard_normal((E, D)) * 0.02).astype(np.float16)
    h["wsg"] = (rng.standard_normal(D) * 0.02).astype(np.float16)
    # block scales d are the stated range times a power of two per tensor so that the layer output stays O(1):
    # at the unscaled range a SwiGLU expert's output has rms ~1.5e5 and the fp16 layer output would be inf
    sD, sI = synth.d_scale_for(D), synth.d_scale_for(I)
    h["gate"] = synth.iq3s_rows(rng, E * I, D, sD).reshape(E, I, -1)
    h["up"] = synth.iq3s_rows(rng, E * I, D, sD).reshape(E, I, -1)
    h["down"] = synth.iq3s_rows(rng, E * D, I, sI).reshape(E, D, -1)
    h["sg"] = synth.iq3s_rows(rng, I, D, sD)
    h["su"] = synth.iq3s_rows(rng, I, D, sD)
    h["sd"] = synth.iq3s_rows(rng, D, I, sI)
    b = {k: gpu.buf_from(v) for k, v in h.items()}
    layer = MoeLayer(gpu, E, D, I, topk, b["Wr"], b["wsg"], b["gate"], b["up"], b["down"],
                     b["sg"] if shared else None, b["su"] if shared else None, b["sd"] if shared else None, e_lo, e_hi, ffn)
    return layer, h, b


def run_layer(gpu, layer, x, fused_route=False):
    nb = x.shape[0]
    xb, ob = gpu.buf_from(x), gpu.buf(nb * layer.D * 2).zero()
    bt = gpu.batch()
    layer.encode(bt, xb, ob, nb, fused_route=fused_route)
    bt.end()
    return ob.download(np.float16, nb * layer.D).reshape(nb, layer.D)


@pytest.mark.parametrize("ffn", ["iq3x", "fused", "split"])
@pytest.mark.parametrize("E,B", [(64, 16), (64, 1), (64, 64), (512, 16)])
def test_moe_layer_parity(gpu, E, B, ffn):
    """ffn = "iq3x": gate/up + down in one launch with H in shared memory, on expert weights re-coded once into the kernel's
    own layout (what the engine runs at these shapes); "fused": the same kernel on the raw IQ3_S blocks; "split": the
    two-launch family that serves every other shape."""
    D, I, topk = 2048, 512, 10
    layer, h, _ = make_layer(gpu, E, D, I, topk, seed=10 + E, ffn=ffn)
    x = synth.acts_fp16(np.random.default_rng(B), B, D)
    out = run_layer(gpu, layer, x)

    # 1. router logits bit-exact (canonical order), shared-gate row included
    lg = layer.read_logits(B)
    ref_lg = orc.router_canon(np.concatenate([h["Wr"], h["wsg"][None]]), x)
    assert np.array_equal(lg.view(np.uint32), ref_lg.view(np.uint32))
    # 2. expert ids bit-exact; weights to 1e-6; grouping consistent
    U, ids, w, ue, off, ent = layer.read_sel(B)
    ref_ids, ref_w = orc.topk(ref_lg[:, :E], topk)
    assert np.array_equal(ids, ref_ids)
    assert np.allclose(w[:, :topk], ref_w, rtol=2e-6, atol=1e-7)
    assert np.allclose(w[:, topk], 1 / (1 + np.exp(-ref_lg[:, E].astype(np.float64))), rtol=2e-6)
    uniq = np.unique(ref_ids)
    assert U == len(uniq) and np.array_equal(ue, uniq) and off[-1] == B * topk
    pairs = sorted((int(e >> 8), int(e & 255)) for e in ent)
    assert pairs == sorted((t, k) for t in range(B) for k in range(topk))
    for u in range(U):
        for e in ent[off[u]:off[u + 1]]:
            assert ref_ids[e >> 8, e & 255] == ue[u]
    # 3. layer output vs the FP64 layer on the same experts
    ref, ids64, gap = orc.moe_ref(x, h["Wr"], h["wsg"], h["gate"], h["up"], h["down"], h["sg"], h["su"], h["sd"], D, I, topk, ids=ids)
    err = np.abs(out.astype(np.float64) - ref).max() / np.abs(ref).max()
    assert err < 2e-3, err
    assert np.array_equal(out.astype(np.float64).argmax(1), ref.argmax(1))
    # the FP64 router picks the same set wherever its 10th/11th gap exceeds the fp32 error bound
    for t in range(B):
        if gap[t] > 1e-5:
            assert set(ids64[t]) == set(ids[t])


@pytest.mark.parametrize("ffn", ["iq3x", "fused", "split"])
def test_moe_batched_equals_alone(gpu, ffn):
    D, I, topk, E, B = 2048, 512, 10, 64, 24
    layer, h, _ = make_layer(gpu, E, D, I, topk, seed=3, ffn=ffn)
    x = synth.acts_fp16(np.random.default_rng(9), B, D)
    out = run_layer(gpu, layer, x)
    for t in (0, 7, 23):
        alone = run_layer(gpu, layer, x[t:t + 1])
        assert np.array_equal(alone[0].view(np.uint16), out[t].view(np.uint16))
    # identical tokens in one batch give identical rows (more than 8 tokens on one expert -> several column tiles)
    xs = np.repeat(x[:1], 20, axis=0)
    outs = run_layer(gpu, layer, xs)
    assert all(np.array_equal(outs[i].view(np.uint16), out[0].view(np.uint16)) for i in range(20))


@pytest.mark.parametrize("ffn", ["iq3x", "fused", "split"])
def test_moe_expert_range_partitions_the_work(gpu, ffn):
    """Expert-parallel building block: with experts restricted to [lo, hi) each part writes only its own
    (token, rank) rows; the union over a partition equals the full layer's rows bit for bit."""
    D, I, topk, E, B = 2048, 512, 10, 64, 16
    full, h, b = make_layer(gpu, E, D, I, topk, seed=5, ffn=ffn)
    x = synth.acts_fp16(np.random.default_rng(2), B, D)
    run_layer(gpu, full, x)
    pg_full = full.Pg.download(np.float32, B * (topk + 1) * D).reshape(B, topk + 1, D)
    _, ids, _, _, _, _ = full.read_sel(B)
    from qwental_b200.layers import MoeLayer
    acc = np.zeros_like(pg_full)
    for lo, hi in ((0, 32), (32, 64)):
        part = MoeLayer(gpu, E, D, I, topk, b["Wr"], b["wsg"], b["gate"], b["up"], b["down"], b["sg"], b["su"], b["sd"], lo, hi, ffn)
        run_layer(gpu, part, x)
        pg = part.Pg.download(np.float32, B * (topk + 1) * D).reshape(B, topk + 1, D)
        mine = (ids >= lo) & (ids < hi)
        assert np.all(pg[:, :topk][~mine] == 0)
        acc[:, :topk] += pg[:, :topk]
        acc[:, topk] = pg[:, topk]
    assert np.array_equal(acc.view(np.uint32), pg_full.view(np.uint32))


@pytest.mark.parametrize("B", [1, 16, 64])
def test_fused_router_select_equals_two_launches(gpu, B):
    """moe_route (router + selection in one launch, last block selects) gives the same logits, selection record and
    layer output, bit for bit, as moe_router followed by moe_select -- also when launched repeatedly (the hand-over
    counter must be left at zero)."""
    D, I, topk, E = 2048, 512, 10, 64
    layer, h, _ = make_layer(gpu, E, D, I, topk, seed=21)
    x = synth.acts_fp16(np.random.default_rng(B + 5), B, D)
    out = run_layer(gpu, layer, x)
    lg, sel = layer.read_logits(B).copy(), layer.sel.download(np.uint8, layer.sel.size).copy()
    for _ in range(3):
        layer.sel.zero()
        layer.logits.zero()
        out2 = run_layer(gpu, layer, x, fused_route=True)
        assert np.array_equal(layer.read_logits(B).view(np.uint32), lg.view(np.uint32))
        got = layer.sel.download(np.uint8, layer.sel.size)
        U, ids, w, ue, off, ent = layer.read_sel(B)
        n = 16 + 64 * 16 * 4 + 64 * 17 * 4
        ref_ids = sel[16:16 + 64 * 16 * 4].view(np.int32).reshape(64, 16)[:B, :topk]
        assert np.array_equal(ids, ref_ids)
        assert np.array_equal(got[n:n + 4 * U], sel[n:n + 4 * U]) and got[:4].view(np.uint32)[0] == sel[:4].view(np.uint32)[0]
        assert np.array_equal(out2.view(np.uint16), out.view(np.uint16))


def test_selection_with_equal_logits_takes_lowest_ids(gpu):
    """Ties in the router: equal logits resolve to the lower expert id (as the reference's stable selection,
    kernels/moe_gg.metal:118-189).  Token 0 is all zeros (every logit equal: 512 candidates, the general path of the
    selection); in the other tokens some router rows are duplicated, so winners and the cut-off come in equal pairs
    (the fast path with a few candidates more than top-k)."""
    D, I, topk, E = 2048, 512, 10, 512
    layer, h, b = make_layer(gpu, E, D, I, topk, seed=33)
    Wr = h["Wr"].copy()
    rng = np.random.default_rng(8)
    for _ in range(60):  # duplicated rows -> exactly equal logits for every token
        a, c = rng.integers(0, E, 2)
        Wr[c] = Wr[a]
    b["Wr"].upload(Wr)
    x = synth.acts_fp16(rng, 6, D)
    x[0] = 0
    for fused in (False, True):
        layer.sel.zero()
        run_layer(gpu, layer, x, fused_route=fused)
        lg = layer.read_logits(6)
        ref_lg = orc.router_canon(np.concatenate([Wr, h["wsg"][None]]), x)
        assert np.array_equal(lg.view(np.uint32), ref_lg.view(np.uint32))
        U, ids, w, ue, off, ent = layer.read_sel(6)
        ref_ids, ref_w = orc.topk(ref_lg[:, :E], topk)
        assert np.array_equal(ids[:6, :topk], ref_ids), fused
        assert list(ids[0, :topk]) == list(range(topk))
        assert np.abs(w[:6, :topk] - ref_w).max() < 1e-6


def test_iq3x_recoding_is_lossless(gpu):
    """iq3x_pack followed by the IQ3X decoder gives, bit for bit, what the CPU oracle decodes from the original IQ3_S blocks
    (the oracle itself is pinned against gguf and the reference's decoder): the re-coding keeps every weight's exact value.
    Edge blocks included: all-zero and all-one fields, largest scales, every sign pattern."""
    from qwental_b200.layers import u32
    rng = np.random.default_rng(77)
    rows, K = 256, 1024
    W = synth.iq3s_rows(rng, rows, K, 1.0).copy()
    blk = W.reshape(rows, K // 256, 110)
    blk[0, 0, 2:110] = 0          # every index 0, no signs, scale 0
    blk[1, 0, 2:110] = 255        # every index 511, all signs, scale 15
    blk[2, 1, 74:106] = 0xAA      # alternating signs
    blk[3, 2, 66:74] = 0x55       # alternating codebook high bits
    src = gpu.buf_from(W)
    dst = gpu.buf((rows // 128) * (K // 512) * 128 * 272)
    y = gpu.buf(rows * K * 4)
    bt = gpu.batch()
    bt.kernel(gpu.compile("iq3x_pack", "iq3x_pack")).buf(0, src).buf(2, dst).bytes(3, u32(1, 1, K, rows)).dispatch((1,), (256,))
    bt.kernel(gpu.compile("iq3x_dq_test", "iq3x_dq_test")).buf(0, dst).buf(1, y).bytes(2, u32(rows, K)).dispatch((1,), (128,))
    bt.end()
    got = y.download(np.float32, rows * K).reshape(rows, K)
    ref = orc.dq_rows(orc.IQ3_S, W, K)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
