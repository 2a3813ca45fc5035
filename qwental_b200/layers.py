"""Python mirror of the engine's per-layer call sites: each function encodes the dispatches of one block into a
batch, through the device interface only (kernel by name, buffers and bytes by index, grid in thread blocks) --
the way the reference's src/engine.c encodes them (gg_moe at src/engine.c:568-646, qmv_gg at :689-724,
qsa_layer at :5619-5805, the GDN layer at :8968-9008).  Used by the parity tests and the per-config benchmarks;
the C++ engine (csrc/engine.cpp) encodes the same sequences.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as _lib
from .gpu import DEVICE, Batch, Buf, Gpu

MOE_MAXB = 64


def moe_sel_bytes() -> int:
    L = _lib.load()
    L.qw_moe_sel_bytes.restype = C.c_size_t
    return int(L.qw_moe_sel_bytes())


def u32(*v) -> np.ndarray:
    return np.array(v, np.uint32)


class Qmv:
    """One quantized matrix [N][K] and its matvec kernel (family qmv_mma or qmv_gg)."""

    def __init__(self, gpu: Gpu, W: Buf, qtype: int, N: int, K: int, f32_out: bool = False, family: str = "qmv_mma", woff: int = 0):
        self.gpu, self.W, self.N, self.K, self.f32, self.woff = gpu, W, N, K, f32_out, woff
        self.k = gpu.compile(family, "%s_g%d_k%d_%s" % (family, qtype, K, "f" if f32_out else "h"), GF=qtype, KD=K, NB=64,
                             YT_F32=int(f32_out))

    def encode(self, b: Batch, x: Buf, y: Buf, nb: int, xstride: int | None = None, ystride: int | None = None, xoff: int = 0, yoff: int = 0):
        args = u32(self.N, xstride or self.K, ystride or self.N, nb)
        b.kernel(self.k).buf(0, self.W, self.woff).buf(3, x, xoff).buf(4, y, yoff).bytes(5, args).dispatch(((self.N + 7) // 8,), (256,))


IQ3X_STAGE = 128 * 272


def iq3x_pack(gpu: Gpu, Wg: Buf, Wu: Buf, Wd: Buf, experts: int, D: int, I: int):
    """Re-codes the IQ3_S matrices of `experts` experts (gate / up [experts][I][D/256*110], down [experts][D][I/256*110]) into
    the stage-ordered IQ3X form the fused expert-FFN kernel streams; returns (gate+up buffer, down buffer)."""
    k = gpu.compile("iq3x_pack", "iq3x_pack")
    gu = gpu.buf(experts * (I // 64) * (D // 512) * IQ3X_STAGE)
    dn = gpu.buf(experts * (D // 128) * (I // 512) * IQ3X_STAGE)
    b = gpu.batch()
    b.kernel(k).buf(0, Wg).buf(1, Wu).buf(2, gu).bytes(3, u32(0, experts, I, D)).dispatch((1,), (256,))
    b.kernel(k).buf(0, Wd).buf(2, dn).bytes(3, u32(1, experts, I, D)).dispatch((1,), (256,))
    b.end()
    return gu, dn


class MoeLayer:
    """Router + top-k/grouping + gathered expert FFN + shared expert + combine for up to 64 tokens."""

    def __init__(self, gpu: Gpu, E: int, D: int, I: int, topk: int, Wr: Buf, Wsg: Buf, Wg: Buf, Wu: Buf, Wd: Buf,
                 Sg: Buf | None, Su: Buf | None, Sd: Buf | None, e_lo: int = 0, e_hi: int | None = None, ffn: str = "auto"):
        self.gpu, self.E, self.D, self.I, self.topk = gpu, E, D, I, topk
        # expert FFN: "fused" = gate/up + down in one launch (moe_ffn; D a multiple of 2048, I = 512), "split" = moe_gu then
        # moe_dn; "auto" takes the fused kernel where its shapes allow, as the engine does
        # "iq3x" = the fused kernel on expert weights re-coded once by iq3x_pack (lossless; 136 instead of 110 bytes per 256 weights)
        assert ffn in ("auto", "fused", "split", "iq3x")
        self.iq3x = ffn == "iq3x"
        self.fused_ffn = ffn in ("fused", "iq3x") or (ffn == "auto" and D == 2048 and I == 512)
        self.Wr, self.Wsg, self.Wg, self.Wu, self.Wd, self.Sg, self.Su, self.Sd = Wr, Wsg, Wg, Wu, Wd, Sg, Su, Sd
        self.e_lo, self.e_hi = e_lo, E if e_hi is None else e_hi
        tag = "_e%d_d%d_i%d_k%d" % (E, D, I, topk)
        tag += "_s%d" % int(Sg is not None)
        d = dict(E=E, D=D, I=I, TOPK=topk, SHARED=int(Sg is not None))
        self.k_router = gpu.compile("moe_router", "moe_router" + tag, **d)
        self.k_select = gpu.compile("moe_select", "moe_select" + tag, **d)
        self.k_route = gpu.compile("moe_route", "moe_route" + tag, **d)
        self.route_cnt = gpu.buf(256).zero()
        self.k_gu = gpu.compile("moe_gu", "moe_gu" + tag, **d)
        self.k_dn = gpu.compile("moe_dn", "moe_dn" + tag, **d)
        self.k_ffn = gpu.compile("moe_ffn", "moe_ffn" + tag + ("_x" if self.iq3x else ""), IQ3X=int(self.iq3x), **d) if self.fused_ffn else None
        if self.iq3x:
            self.Xgu, self.Xd = iq3x_pack(gpu, Wg, Wu, Wd, E, D, I)
            self.XSgu, self.XSd = iq3x_pack(gpu, Sg, Su, Sd, 1, D, I) if Sg is not None else (None, None)
        self.k_cmb = gpu.compile("moe_cmb", "moe_cmb" + tag, RESID=0, **d)
        self.k_cmb_res = gpu.compile("moe_cmb", "moe_cmb_res" + tag, RESID=1, **d)
        self.logits = gpu.buf(MOE_MAXB * (E + 1) * 4)
        self.sel = gpu.buf(moe_sel_bytes()).zero()
        self.Hhi = gpu.buf(MOE_MAXB * (topk + 1) * I * 2).zero()
        self.Hlo = gpu.buf(MOE_MAXB * (topk + 1) * I * 2).zero()
        self.Pg = gpu.buf(MOE_MAXB * (topk + 1) * D * 4).zero()
        # moe_ffn's scratch (csrc/moe_sel.h): 8 KB of counters, then H of up to 640 items
        self.ffn_scr = gpu.buf(8192 + 640 * 16 * I * 2).zero() if self.fused_ffn else None

    def encode(self, b: Batch, x: Buf, out: Buf, nb: int, resid: Buf | None = None, fused_route: bool = False):
        E, D, I = self.E, self.D, self.I
        if fused_route:  # router + selection in one launch (what the engine uses)
            b.kernel(self.k_route).buf(0, self.Wr).buf(1, self.Wsg).buf(2, x).buf(3, self.logits).buf(4, self.route_cnt).buf(5, self.sel) \
                .bytes(14, u32(nb, self.e_lo, self.e_hi)).dispatch(((E + 1 + 7) // 8,), (1024,))
            return self._encode_ffn(b, x, out, nb, resid)
        b.kernel(self.k_router).buf(0, self.Wr).buf(1, self.Wsg).buf(2, x).buf(3, self.logits).bytes(14, u32(nb)) \
            .dispatch(((E + 1 + 7) // 8,), (256,))
        b.kernel(self.k_select).buf(0, self.logits).buf(1, self.sel).bytes(2, u32(nb, self.e_lo, self.e_hi)).dispatch((1,), (1024,))
        self._encode_ffn(b, x, out, nb, resid)

    def _encode_ffn(self, b: Batch, x: Buf, out: Buf, nb: int, resid: Buf | None):
        D, I = self.D, self.I
        if self.iq3x:
            b.kernel(self.k_ffn).buf(0, self.Xgu)
            if self.Sg is not None:
                b.buf(2, self.XSgu).buf(7, self.XSd)
            b.buf(4, x).buf(5, self.sel).buf(6, self.Xd).buf(8, self.ffn_scr).buf(9, self.Pg).dispatch((I // 16, nb * self.topk + 1), (256,))
        elif self.fused_ffn:
            b.kernel(self.k_ffn).buf(0, self.Wg).buf(1, self.Wu)
            if self.Sg is not None:
                b.buf(2, self.Sg).buf(3, self.Su).buf(7, self.Sd)
            b.buf(4, x).buf(5, self.sel).buf(6, self.Wd).buf(8, self.ffn_scr).buf(9, self.Pg).dispatch((I // 16, nb * self.topk + 1), (256,))
        else:
            b.kernel(self.k_gu).buf(0, self.Wg).buf(1, self.Wu)
            if self.Sg is not None:
                b.buf(2, self.Sg).buf(3, self.Su)
            b.buf(4, x).buf(5, self.sel).buf(6, self.Hhi).buf(7, self.Hlo).dispatch((I // 16, nb * self.topk + 1), (256,))
            b.kernel(self.k_dn).buf(0, self.Wd)
            if self.Sd is not None:
                b.buf(2, self.Sd)
            b.buf(5, self.sel).buf(6, self.Hhi).buf(7, self.Hlo).buf(9, self.Pg).dispatch((D // 64, nb * self.topk + 1), (256,))
        b.kernel(self.k_cmb if resid is None else self.k_cmb_res).buf(3, self.sel).buf(4, out).buf(9, self.Pg).bytes(8, u32(nb))
        if resid is not None:
            b.buf(5, resid)
        b.dispatch((D // 256, nb), (256,))

    # ---- read-backs for the parity tests
    def read_logits(self, nb: int) -> np.ndarray:
        return self.logits.download(np.float32, nb * (self.E + 1)).reshape(nb, self.E + 1)

    def read_sel(self, nb: int):
        raw = self.sel.download(np.uint8, moe_sel_bytes())
        U = int(raw[:4].view(np.uint32)[0])
        o = 16
        ids = raw[o:o + 64 * 16 * 4].view(np.int32).reshape(64, 16)[:nb, :self.topk].copy()
        o += 64 * 16 * 4
        w = raw[o:o + 64 * 17 * 4].view(np.float32).reshape(64, 17)[:nb, :self.topk + 1].copy()
        o += 64 * 17 * 4
        ue = raw[o:o + 1024 * 4].view(np.uint32)[:U].copy()
        o += 1024 * 4
        off = raw[o:o + 1025 * 4].view(np.uint32)[:U + 1].copy()
        o += 1025 * 4
        ent = raw[o:o + 1024 * 2].view(np.uint16)[:int(off[-1]) if U else 0].copy()
        return U, ids, w, ue, off, ent


class AttnCore:
    """qsa_prep + qsa_attn + qsa_merge over a paged KV pool (one attention layer's slice of the pages)."""

    def __init__(self, gpu: Gpu, QH: int, KVH: int, HD: int, max_slots: int, max_pages: int, n_pages: int, nlayers: int = 1,
                 attn_family: str = "qsa_attn"):
        self.gpu, self.QH, self.KVH, self.HD, self.max_pages, self.nlayers = gpu, QH, KVH, HD, max_pages, nlayers
        d = dict(QH=QH, KVH=KVH, HD=HD)
        self.k_prep = gpu.compile("qsa_prep", "qsa_prep_t", **d)
        self.k_attn = gpu.compile(attn_family, attn_family + "_t", **d)
        self.attn_threads = 256 if attn_family == "qsa_attn_simt" else 128
        self.k_merge = gpu.compile("qsa_merge", "qsa_merge_t", **d)
        self.page_halves = nlayers * 2 * KVH * 256 * HD
        self.pool = gpu.buf(n_pages * self.page_halves * 2).zero()
        self.ptab = gpu.buf(max_slots * max_pages * 4).zero()
        self.part = gpu.buf(MOE_MAXB * max_pages * QH * (HD + 2) * 4)
        self.q = gpu.buf(MOE_MAXB * QH * HD * 2)

    def args(self, nb: int, layer: int, qkv_stride: int, max_chunks: int) -> np.ndarray:
        return u32(nb, layer, self.nlayers, qkv_stride, self.max_pages, max_chunks, 0, 0)

    def encode(self, b: Batch, qkv: Buf, qn: Buf, kn: Buf, pos: Buf, sids: Buf, y: Buf, nb: int, layer: int, qkv_stride: int, max_chunks: int):
        a = self.args(nb, layer, qkv_stride, max_chunks)
        b.kernel(self.k_prep).buf(0, qkv).buf(1, qn).buf(2, kn).buf(3, self.q).buf(4, self.pool).buf(5, self.ptab).buf(6, pos).buf(7, sids) \
            .bytes(8, a).dispatch((self.QH + self.KVH, nb), (256,))
        b.kernel(self.k_attn).buf(0, self.q).buf(1, self.pool).buf(2, self.ptab).buf(3, pos).buf(4, sids).buf(5, self.part).bytes(6, a) \
            .dispatch((max_chunks, self.KVH, nb), (self.attn_threads,))
        b.kernel(self.k_merge).buf(0, self.part).buf(1, qkv).buf(2, y).buf(3, pos).bytes(4, a).dispatch((self.QH, nb), (256,))


class GdnCore:
    """dn_epi (conv + SiLU, decay, beta) + gdn_fstep (recurrence + gated RMSNorm) for nb slots."""

    def __init__(self, gpu: Gpu, HK: int, HV: int, max_slots: int, nlayers: int = 1, o_out: bool = True):
        self.gpu, self.HK, self.HV, self.nlayers = gpu, HK, HV, nlayers
        self.C = 2 * HK * 128 + HV * 128
        d = dict(HK=HK, HV=HV, DK=128, DV=128, GDN_TILED=1)
        self.k_epi = gpu.compile("dn_epi", "dn_epi_t", **d)
        self.k_gdn = gpu.compile("gdn_fstep", "gdn_fstep_t", O_OUT=int(o_out), **d)
        self.S = gpu.buf(max_slots * nlayers * HV * 128 * 128 * 4)
        self.conv = gpu.buf(max_slots * nlayers * 3 * self.C * 4)
        self.cv = gpu.buf(MOE_MAXB * self.C * 2)
        self.la = gpu.buf(MOE_MAXB * HV * 4)
        self.be = gpu.buf(MOE_MAXB * HV * 4)
        self.o = gpu.buf(MOE_MAXB * HV * 128 * 2)

    def encode(self, b: Batch, proj: Buf, proj_stride: int, cw: Buf, A: Buf, dt: Buf, nw: Buf, sids: Buf, gy: Buf, nb: int, layer: int):
        C, HV = self.C, self.HV
        b.kernel(self.k_epi).buf(0, proj).buf(1, cw).buf(2, self.conv).buf(3, A).buf(4, dt).buf(5, self.cv).buf(6, self.la).buf(7, self.be) \
            .buf(8, sids).bytes(9, u32(nb, layer, self.nlayers, proj_stride)).dispatch(((C + 2 * HV + 255) // 256, nb), (256,))
        b.kernel(self.k_gdn).buf(0, self.cv).buf(1, self.la).buf(2, self.be).buf(3, self.S).buf(4, proj, C * 2).buf(5, nw).buf(6, gy) \
            .buf(7, sids).bytes(8, u32(nb, layer, self.nlayers, proj_stride)).buf(9, self.o).dispatch((HV, nb), (512,))
