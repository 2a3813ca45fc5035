"""FP64 reference of one full decode step (all layers) -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Chains the per-layer references of oracle.py the way the reference's step chains its layers
(src/engine.c:8886-9021, with the plain residual + RMSNorm that stands in for the hyper-connection mix):
embedding, then per layer [RMSNorm -> gated attention | Gated DeltaNet -> residual -> RMSNorm -> MoE -> residual],
final RMSNorm, lm_head.  fp16 rounding is applied where the device stores fp16 (block inputs and outputs,
projections, q/k/v, conv output), as tools/dn_ref.py:58-66 does with its h16().

The model's tensors are passed in as numpy arrays read back from the device (Engine.tap), so the comparison
does not depend on reproducing the device's random fill.
"""
from __future__ import annotations

import numpy as np

from . import oracle as orc

PAGE = 256


def f16(a):
    return np.asarray(a).astype(np.float16)


class RefModel:
    def __init__(self, cfg, eng):
        """cfg: ModelCfg; eng: qwental_b200.engine.Engine to read the tensors from."""
        self.c = c = cfg
        self.D, self.L, self.V, self.E, self.I, self.TOPK = c.hidden, c.layers, c.vocab, c.experts, c.expert_inter, c.topk
        self.QH, self.KVH, self.HD, self.HK, self.HV = c.qh, c.kvh, c.hd, c.hk, c.hv
        self.C = 2 * c.hk * 128 + c.hv * 128
        D, I, E = self.D, self.I, self.E
        self.emb = eng.tap("emb", 0, np.float16).reshape(self.V, D)
        self.lm = eng.tap("lm_head", 0, np.uint8)
        self.fnorm = eng.tap("final_norm", 0, np.float32)
        self.layers = []
        na = ng = 0
        for l in range(self.L):
            attn = (l % c.attn_every) == c.attn_every - 1
            sm = eng.tap("small", l, np.float32)
            W = dict(attn=attn, w_in=eng.tap("w_in", l, np.uint8), w_out=eng.tap("w_out", l, np.uint8), n1=sm[:D], n2=sm[D:2 * D])
            o = 2 * D
            if attn:
                W.update(qn=sm[o:o + 256], kn=sm[o + 256:o + 512], idx=na)
                na += 1
            else:
                C = self.C
                W.update(cw=sm[o:o + 4 * C].reshape(C, 4), A=sm[o + 4 * C:o + 4 * C + self.HV], dt=sm[o + 4 * C + self.HV:o + 4 * C + 2 * self.HV],
                         nw=sm[o + 4 * C + 2 * self.HV:o + 4 * C + 2 * self.HV + 128], idx=ng)
                ng += 1
            r = eng.tap("router", l, np.float16).reshape(E + 1, D)
            rbD, rbI = D // 256 * 110, I // 256 * 110
            W.update(Wr=r[:E], wsg=r[E], exg=eng.tap("exg", l, np.uint8).reshape(E, I, rbD), exu=eng.tap("exu", l, np.uint8).reshape(E, I, rbD),
                     exd=eng.tap("exd", l, np.uint8).reshape(E, D, rbI), shg=eng.tap("shg", l, np.uint8).reshape(I, rbD),
                     shu=eng.tap("shu", l, np.uint8).reshape(I, rbD), shd=eng.tap("shd", l, np.uint8).reshape(D, rbI))
            self.layers.append(W)
        self.n_attn, self.n_gdn = na, ng

    def read_slot(self, eng, sid):
        """Host copy of a slot's state: KV [n_attn][2][KVH][pos][HD] fp16, S, conv."""
        pos = eng.pos(sid)
        pages = eng.tap("pages", sid, np.int32)
        na = max(1, self.n_attn)
        kv = np.zeros((na, 2, self.KVH, len(pages) * PAGE, self.HD), np.float16)
        for i, p in enumerate(pages):
            pg = eng.tap("kvpage", int(p), np.float16).reshape(na, 2, self.KVH, PAGE, self.HD)
            kv[:, :, :, i * PAGE:(i + 1) * PAGE] = pg
        ng = max(1, self.n_gdn)
        S = eng.tap("sstate", sid, np.float32).reshape(ng, self.HV, 128, 128).astype(np.float64)
        cs = eng.tap("cstate", sid, np.float32).reshape(ng, 3, self.C).astype(np.float64)
        return dict(pos=pos, kv=kv, S=S, conv=cs)

    def step(self, st, tok, ids_by_layer=None):
        """Advance one slot (state dict from read_slot, updated in place) by one token.
        Returns (logits float64 [V], h float64 [D], chosen expert ids per layer)."""
        D, HD, QH, KVH, HK, HV, C = self.D, self.HD, self.QH, self.KVH, self.HK, self.HV, self.C
        pos = st["pos"]
        h = self.emb[tok].astype(np.float64)
        pending = None
        chosen = []
        for l, W in enumerate(self.layers):
            if pending is not None:
                h = h + pending
            x = f16(orc.rmsnorm_ref(h, W["n1"]))
            if W["attn"]:
                proj = f16(orc.qmv_f64(21, W["w_in"], D, x[None])[0])
                pf = proj.astype(np.float64)
                q = np.stack([pf[hh * 2 * HD: hh * 2 * HD + HD] for hh in range(QH)])
                gate = np.stack([proj[hh * 2 * HD + HD: (hh + 1) * 2 * HD] for hh in range(QH)])
                k = pf[QH * 2 * HD: QH * 2 * HD + KVH * HD].reshape(KVH, HD)
                v = proj[QH * 2 * HD + KVH * HD: QH * 2 * HD + 2 * KVH * HD].reshape(KVH, HD)
                qn = f16(orc.rope_ref(orc.rmsnorm_ref(q, W["qn"]), pos))
                kn = f16(orc.rope_ref(orc.rmsnorm_ref(k, W["kn"]), pos))
                kv = st["kv"]
                kv[W["idx"], 0, :, pos] = kn
                kv[W["idx"], 1, :, pos] = v
                K = kv[W["idx"], 0, :, :pos + 1].transpose(1, 0, 2)
                V = kv[W["idx"], 1, :, :pos + 1].transpose(1, 0, 2)
                y = f16(orc.attn_ref(qn, K, V, gate)).reshape(-1)
                o = f16(orc.qmv_f64(21, W["w_out"], QH * HD, y[None])[0])
            else:
                proj = f16(orc.qmv_f64(21, W["w_in"], D, x[None])[0])
                pf = proj.astype(np.float64)
                cs = st["conv"][W["idx"]]
                cw = W["cw"].astype(np.float64)
                yv = cw[:, 0] * cs[0] + cw[:, 1] * cs[1] + cw[:, 2] * cs[2] + cw[:, 3] * pf[:C]
                cv = f16(orc.silu(yv))
                cs[0], cs[1], cs[2] = cs[1].copy(), cs[2].copy(), pf[:C].copy()
                z = proj[C:C + HV * 128].reshape(HV, 128)
                xa = pf[C + HV * 128: C + HV * 128 + HV] + W["dt"].astype(np.float64)
                la = W["A"].astype(np.float64) * np.where(xa > 20, xa, np.log1p(np.exp(np.minimum(xa, 20))))
                be = orc.sigmoid(pf[C + HV * 128 + HV: C + HV * 128 + 2 * HV])
                qv = cv[:HK * 128].reshape(HK, 128)
                kk = cv[HK * 128:2 * HK * 128].reshape(HK, 128)
                vv = cv[2 * HK * 128:].reshape(HV, 128)
                S, o16, yy = orc.gdn_step_ref(st["S"][W["idx"]], qv, kk, vv, la, be, z, W["nw"], np.arange(HV) % HK)
                st["S"][W["idx"]] = S
                gy = f16(yy).reshape(-1)
                o = f16(orc.qmv_f64(21, W["w_out"], HV * 128, gy[None])[0])
            h = h + o.astype(np.float64)
            x = f16(orc.rmsnorm_ref(h, W["n2"]))
            lg = orc.router_canon(np.concatenate([W["Wr"], W["wsg"][None]]), x[None])
            ids, _ = orc.topk(lg[:, :self.E], self.TOPK)
            if ids_by_layer is not None:
                ids = np.asarray(ids_by_layer[l])[None]
            chosen.append(ids[0].copy())
            out, _, _ = orc.moe_ref(x[None], W["Wr"], W["wsg"], W["exg"], W["exu"], W["exd"], W["shg"], W["shu"], W["shd"], D, self.I, self.TOPK, ids=ids)
            pending = f16(out[0]).astype(np.float64)
        h = h + pending
        x = f16(orc.rmsnorm_ref(h, self.fnorm))
        logits = orc.qmv_f64(8, self.lm, D, x[None])[0]
        st["pos"] = pos + 1
        return logits, h, chosen
