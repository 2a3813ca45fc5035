"""GPU parity of the ragged paged-KV decode attention and of the Gated DeltaNet step (benchmark config 3),
through the C ABI.  Tolerances are the reference's own: attention < 2e-3 absolute (bench/qsa.c:203-206), GDN output
< 1e-3 (bench/gdn_decode.c:86); its state bound of 1e-5 holds there because both sides get the same normalised k,
here the fp16 rounding of the normalised k may differ by one ulp (5e-4 relative) between device and oracle, which
moves a state element by up to |k| * 5e-4 * |delta| ~ 5e-5, so the state bound is 1e-4; a slot's result must be
bit-identical alone and in a batch."""
import numpy as np
import pytest

from oracle import oracle as orc
from qwental_b200 import synth

pytestmark = pytest.mark.gpu
QH, KVH, HD = 16, 2, 256


@pytest.fixture(scope="module")
def gpu():
    from qwental_b200.gpu import Gpu
    g = Gpu()
    yield g
    g.close()


def attn_setup(gpu, lens, seed, nlayers=2, layer=1, family="qsa_attn"):
    """Slots with the given context lengths (tokens already cached); pages handed out in a shuffled order."""
    from qwental_b200.layers import AttnCore
    rng = np.random.default_rng(seed)
    B = len(lens)
    max_pages = max((int(l) + 1 + 255) // 256 for l in lens) + 1
    n_pages = sum((int(l) + 1 + 255) // 256 for l in lens) + 3
    core = AttnCore(gpu, QH, KVH, HD, max_slots=B + 2, max_pages=max_pages, n_pages=n_pages, nlayers=nlayers, attn_family=family)
    order = rng.permutation(n_pages)
    pool = np.zeros((n_pages, nlayers, 2, KVH, 256, HD), np.float16)
    ptab = np.zeros((B + 2, max_pages), np.int32)
    sids = rng.permutation(B + 2)[:B].astype(np.int32)
    Ks, Vs, nxt = [], [], 0
    for i, L in enumerate(lens):
        L = int(L)
        npg = (L + 1 + 255) // 256
        K = rng.standard_normal((npg * 256, KVH, HD)).astype(np.float16)
        V = rng.standard_normal((npg * 256, KVH, HD)).astype(np.float16)
        for p in range(npg):
            pg = order[nxt]
            nxt += 1
            ptab[sids[i], p] = pg
            pool[pg, layer, 0] = K[p * 256:(p + 1) * 256].transpose(1, 0, 2)
            pool[pg, layer, 1] = V[p * 256:(p + 1) * 256].transpose(1, 0, 2)
        Ks.append(K)
        Vs.append(V)
    core.pool.upload(pool)
    core.ptab.upload(ptab)
    stride = QH * 2 * HD + 2 * KVH * HD
    qkv = rng.standard_normal((B, stride)).astype(np.float16)
    qn = (1 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    return core, dict(qkv=qkv, qn=qn, kn=kn, sids=sids, pos=np.asarray(lens, np.int32), K=Ks, V=Vs, stride=stride, layer=layer, max_pages=max_pages)


def attn_run(gpu, core, d, rows):
    rows = list(rows)
    nb = len(rows)
    qkv, pos, sids = gpu.buf_from(d["qkv"][rows]), gpu.buf_from(d["pos"][rows]), gpu.buf_from(d["sids"][rows])
    qn, kn, y = gpu.buf_from(d["qn"]), gpu.buf_from(d["kn"]), gpu.buf(nb * QH * HD * 2).zero()
    mc = max((int(d["pos"][r]) + 1 + 255) // 256 for r in rows)
    bt = gpu.batch()
    core.encode(bt, qkv, qn, kn, pos, sids, y, nb, d["layer"], d["stride"], mc)
    bt.end()
    return y.download(np.float16, nb * QH * HD).reshape(nb, QH, HD)


def attn_oracle(d, r):
    L = int(d["pos"][r])
    row = d["qkv"][r].astype(np.float64)
    q = np.stack([row[h * 2 * HD:h * 2 * HD + HD] for h in range(QH)])
    gate = np.stack([d["qkv"][r][h * 2 * HD + HD:(h + 1) * 2 * HD] for h in range(QH)])
    k = row[QH * 2 * HD:QH * 2 * HD + KVH * HD].reshape(KVH, HD)
    v = d["qkv"][r][QH * 2 * HD + KVH * HD:].reshape(KVH, HD)
    qn = orc.rope_ref(orc.rmsnorm_ref(q, d["qn"]), L).astype(np.float16)
    kk = orc.rope_ref(orc.rmsnorm_ref(k, d["kn"]), L).astype(np.float16)
    K = d["K"][r][:L + 1].copy()
    V = d["V"][r][:L + 1].copy()
    K[L], V[L] = kk, v
    return orc.attn_ref(qn, K, V, gate), kk


@pytest.mark.parametrize("family", ["qsa_attn", "qsa_attn_simt"])
@pytest.mark.parametrize("lens", [[0, 1, 3, 15, 16, 17, 63, 64, 65, 255, 256, 257, 1500, 2049], [1024, 3001, 8195, 20000, 48000]])
def test_attention_parity_ragged(gpu, lens, family):
    core, d = attn_setup(gpu, lens, seed=len(lens), family=family)
    y = attn_run(gpu, core, d, range(len(lens)))
    for r in range(len(lens)):
        ref, kk = attn_oracle(d, r)
        assert np.abs(y[r].astype(np.float64) - ref).max() < 2e-3, (r, lens[r])
    # the new key/value were appended at position L of the slot's page
    pool = core.pool.download(np.float16, core.pool.size // 2).reshape(-1, 2, 2, KVH, 256, HD)
    ptab = core.ptab.download(np.int32, core.ptab.size // 4).reshape(-1, d["max_pages"])
    for r, L in enumerate(lens):
        pg = ptab[d["sids"][r], L // 256]
        _, kk = attn_oracle(d, r)
        assert np.abs(pool[pg, 1, 0, :, L % 256].astype(np.float64) - kk.astype(np.float64)).max() < 2e-3
        v = d["qkv"][r][QH * 2 * HD + KVH * HD:].reshape(KVH, HD)
        assert np.array_equal(pool[pg, 1, 1, :, L % 256], v)


def test_attention_batched_equals_alone(gpu):
    lens = [700, 5000, 31, 12000, 256]
    core, d = attn_setup(gpu, lens, seed=77)
    y = attn_run(gpu, core, d, range(len(lens)))
    for r in (0, 1, 3):
        ya = attn_run(gpu, core, d, [r])
        assert np.array_equal(ya[0].view(np.uint16), y[r].view(np.uint16))
    yp = attn_run(gpu, core, d, [3, 0, 4])
    assert np.array_equal(yp[0].view(np.uint16), y[3].view(np.uint16)) and np.array_equal(yp[2].view(np.uint16), y[4].view(np.uint16))


def gdn_setup(gpu, B, seed, HK=16, HV=32):
    from qwental_b200.layers import GdnCore
    rng = np.random.default_rng(seed)
    core = GdnCore(gpu, HK, HV, max_slots=B + 1, nlayers=2)
    C = core.C
    stride = C + HV * 128 + 2 * HV
    d = dict(HK=HK, HV=HV, C=C, stride=stride, layer=1)
    d["proj"] = rng.standard_normal((B, stride)).astype(np.float16)
    d["S"] = (rng.standard_normal((B + 1, 2, HV, 128, 128)) * 0.1).astype(np.float32)
    d["conv"] = rng.standard_normal((B + 1, 2, 3, C)).astype(np.float32)
    d["cw"] = (rng.standard_normal((C, 4)) * 0.5).astype(np.float32)
    d["A"] = -np.exp(rng.standard_normal(HV) * 0.3).astype(np.float32)
    d["dt"] = (rng.standard_normal(HV) * 0.5).astype(np.float32)
    d["nw"] = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    d["sids"] = rng.permutation(B + 1)[:B].astype(np.int32)
    return core, d


def gdn_run(gpu, core, d, rows):
    rows = list(rows)
    nb = len(rows)
    core.S.upload(d["S"])
    core.conv.upload(d["conv"])
    proj, sids = gpu.buf_from(d["proj"][rows]), gpu.buf_from(d["sids"][rows])
    cw, A, dt, nw = (gpu.buf_from(d[k]) for k in ("cw", "A", "dt", "nw"))
    gy = gpu.buf(nb * d["HV"] * 128 * 2).zero()
    bt = gpu.batch()
    core.encode(bt, proj, d["stride"], cw, A, dt, nw, sids, gy, nb, d["layer"])
    bt.end()
    S = core.S.download(np.float32, d["S"].size).reshape(d["S"].shape)
    conv = core.conv.download(np.float32, d["conv"].size).reshape(d["conv"].shape)
    o = core.o.download(np.float16, nb * d["HV"] * 128).reshape(nb, d["HV"], 128)
    return gy.download(np.float16, nb * d["HV"] * 128).reshape(nb, d["HV"], 128), o, S, conv


def gdn_oracle(d, r):
    HK, HV, C = d["HK"], d["HV"], d["C"]
    sid, lay = d["sids"][r], d["layer"]
    pf = d["proj"][r].astype(np.float64)
    cs = d["conv"][sid, lay].astype(np.float64)
    cw = d["cw"].astype(np.float64)
    yv = cw[:, 0] * cs[0] + cw[:, 1] * cs[1] + cw[:, 2] * cs[2] + cw[:, 3] * pf[:C]
    cv = orc.silu(yv).astype(np.float16)
    conv_new = np.stack([cs[1], cs[2], pf[:C]])
    z = d["proj"][r][C:C + HV * 128].reshape(HV, 128)
    xa = pf[C + HV * 128:C + HV * 128 + HV] + d["dt"]
    la = d["A"].astype(np.float64) * np.where(xa > 20, xa, np.log1p(np.exp(np.minimum(xa, 20))))
    be = orc.sigmoid(pf[C + HV * 128 + HV:C + HV * 128 + 2 * HV])
    q, k, v = cv[:HK * 128].reshape(HK, 128), cv[HK * 128:2 * HK * 128].reshape(HK, 128), cv[2 * HK * 128:].reshape(HV, 128)
    S, o16, y = orc.gdn_step_ref(d["S"][sid, lay], q, k, v, la, be, z, d["nw"], np.arange(HV) % HK)
    return y, o16, S, conv_new


def test_gdn_step_parity(gpu):
    B = 16
    core, d = gdn_setup(gpu, B, seed=4)
    gy, o, S, conv = gdn_run(gpu, core, d, range(B))
    for r in range(B):
        y, o16, Sref, cref = gdn_oracle(d, r)
        sid = d["sids"][r]
        assert np.abs(o[r].astype(np.float64) - o16).max() < 1e-3 * max(1.0, np.abs(o16).max())
        assert np.abs(S[sid, 1].astype(np.float64) - Sref).max() < 1e-4 * max(1.0, np.abs(Sref).max())
        assert np.abs(gy[r].astype(np.float64) - y).max() < 4e-3 * max(1.0, np.abs(y).max())
        assert np.array_equal(conv[sid, 1], cref.astype(np.float32))
    # the other layer's state and the unused slot are untouched
    assert np.array_equal(S[:, 0], d["S"][:, 0]) and np.array_equal(conv[:, 0], d["conv"][:, 0])
    spare = [s for s in range(B + 1) if s not in set(d["sids"])][0]
    assert np.array_equal(S[spare], d["S"][spare])


def test_gdn_batched_equals_alone(gpu):
    B = 6
    core, d = gdn_setup(gpu, B, seed=8)
    gy, o, S, conv = gdn_run(gpu, core, d, range(B))
    for r in (0, 5):
        gya, oa, Sa, ca = gdn_run(gpu, core, d, [r])
        sid = d["sids"][r]
        assert np.array_equal(gya[0].view(np.uint16), gy[r].view(np.uint16))
        assert np.array_equal(Sa[sid, 1].view(np.uint32), S[sid, 1].view(np.uint32))
