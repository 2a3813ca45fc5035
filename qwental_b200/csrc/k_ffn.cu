// MoE expert FFN in one launch: gate/up, SiLU * up and the down projection of every (expert, pass of 8 tokens) item.
// Replaces the reference's moe_gu_gg + moe_dn_gg pair (kernels/moe_gg.metal:600-652; host src/engine.c:568-646) for the
// benchmark shapes (D = 2048, I = 512); the two-launch family in k_moe.cu stays for every other shape.
//
// Work.  An item is one pass (up to 8 token columns) of one distinct expert, or of the shared expert.  A decode step of 16
// slots touches about a hundred items -- fewer than there are SMs, and far fewer when the experts are spread over ranks --
// so an item is cut into pieces: GT gate/up pieces (64 intermediate indices each, all of K = D) and DT down pieces (128
// output rows each, all of K = I).  Persistent blocks (one per SM for IQ3_S, two for IQ3X) take an even, contiguous share of
// the gate/up piece list, then an even share of the down piece list.  H = silu(gate x) * (up x) travels from the blocks that ran an item's
// gate/up pieces to the blocks that run its down pieces through a small global buffer (it stays in L2) and a per-item
// counter: a block only ever waits for H after it has finished all of its own gate/up pieces, so every wait is on blocks
// that are running and never wait themselves.  The arithmetic of a piece does not depend on which block runs it.
//
// A block is 16 consumer warps + 1 producer warp around a ring of weight stages:
//   gate/up   stage = 64 gate rows + 64 up rows of the expert x 512 K values.  IQ3_S: two 2-D tiled TMA boxes of 64 rows x
//             240 bytes (two 110-byte super-blocks plus what 16-byte alignment of the box start costs); rows land 240
//             bytes apart, so the eight rows a warp instruction touches fall into eight different groups of four banks.
//             IQ3X: one contiguous 34 KB run.
//   down      stage = 128 rows of the down matrix over all of K = 512 (contiguous: one 1-D bulk copy).
// and a ring of eight activation rows (the tokens of an item's columns for its gate/up pieces, the two planes of its H for the down
// pieces): an item takes as many rows as it has columns, so the next item's rows are usually copied while this one's are read;
// filled by the producer with bulk copies.  Consumer warp w = (row group r = w % 8, K half kh = w / 8) owns 16 MMA rows of
// the stage and one of the stage's two super-blocks; the accumulators live across the stages of a piece, and the two K
// halves of a row group meet once per piece through shared memory (always low half + high half: the order never depends on
// the batch).  In a gate/up piece MMA row g is gate row 8r + g and row g + 8 is the up row of the same intermediate
// index, so a lane holds both factors of H and no exchange between row groups exists.  B operands (the tokens, then H
// as fp16 high + low planes) come from padded shared-memory rows by one 16-byte load per sub-block; lanes whose column is
// absent load nothing.  Every wait is bounded (about two seconds); a warp that gives up records ST_MBAR_TIMEOUT and keeps
// walking the same control flow without waiting again, so no barrier is ever left short of a participant.
#include "iq3x.cuh"
#include "moe_sel.h"
#include "qmv_core.cuh"
#include "qw_kern.h"
#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>

using namespace qw;

namespace {

constexpr int FFN_CW = 16;                       // consumer warps
constexpr int FFN_THREADS = (FFN_CW + 1) * 32;   // + the producer warp
constexpr int FFN_MAXITEMS = MOE_FFN_MAXITEMS;   // see moe_sel.h: the scratch buffer
constexpr int FFN_SYNC_BYTES = MOE_FFN_SYNC_BYTES;
constexpr int FFN_PITCH = 240;                   // IQ3_S: bytes between staged gate/up rows
constexpr int FFN_D = 2048, FFN_I = 512;         // the shapes this kernel is built for (the launcher refuses others)
constexpr int FFN_MAXG = 520;                    // groups kept in shared memory: E <= 512 experts (+ end markers)
constexpr int FFN_RECS = 8;                      // items a block's gate/up share (and its down share) can touch
// Shared-memory plan per weight format.  FMT 0 = the raw IQ3_S blocks: 64 KB codebook, three 30 KB stages, one block per SM.
// FMT 1 = IQ3X (iq3x.cuh): no codebook and 56 registers per thread, so two blocks share an SM (two 34 KB stages each):
// while the warps of one wait -- for a stage, for their partner's partial sums, for a fixed-latency result -- the other's issue.
template <int FMT>
struct FfnCfg {
    static constexpr int PER_SM = FMT ? 2 : 1;
    static constexpr int STG = FMT ? 2 : 3;
    static constexpr int SLOT = FMT ? IQ3X_STAGE : 128 * FFN_PITCH;   // 30720 also holds an IQ3_S down tile of 128 x 220 bytes
    static constexpr int TAB = FMT ? 256 : 65536;                      // IQ3_S: the codebook; IQ3X: the multiply-add constants of the 16 scale values
    static constexpr int OFF_TAB = 128;
    static constexpr int OFF_PRE = OFF_TAB + TAB;                      // uint32 pre[FFN_MAXG] of the selection record, then 2 x FFN_RECS item records of 32 bytes
    static constexpr int OFF_REC = OFF_PRE + FFN_MAXG * 4;
    static constexpr int OFF_RED = OFF_REC + 2 * FFN_RECS * 32 + 32;   // [2][8 row groups][32 lanes] float4
    static constexpr int OFF_XS = (OFF_RED + 2 * 8 * 32 * 16 + 127) / 128 * 128;  // the activation slots, then the stages
};

struct FfnP {
    const uint8_t *Wd, *Sd;   // routed down [E][D][rbI], shared expert's down [D][rbI] (nullptr: no shared expert)
    const uint8_t *Wg, *Sg;   // IQ3X: routed / shared gate + up stages (IQ3_S copies go through the tensor maps)
    const __half *x;          // tokens fp16 [nb][D]
    float *Pg;                // [nb][topk+1][D]
    const moe_sel *ms;
    const QwTables *tab;
    unsigned *status;
    uint32_t ebase;
    unsigned *sync;           // [0 .. FFN_MAXITEMS) per-item counters of finished gate/up warps, [FFN_MAXITEMS] finished blocks; all zero between launches
    __half *H;                // [FFN_MAXITEMS][2][8][I]
    float *PgR[8];            // expert-parallel exchange: Pg of every rank (see moe_dn in k_moe.cu)
    EpPeers ep;
};

__device__ __forceinline__ void tma_box_2d(uint32_t dst, const CUtensorMap *tm, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(tm),
                 "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_s(uint32_t dst, const void *src, uint32_t bytes, uint64_t *bar) {  // 1-D bulk copy to a shared-space address
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bar_sync_n(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

struct __align__(16) FfnItem {
    uint32_t e0, c0, ncols, erow;  // first entry of the group, first column of the pass, columns, expert's row in the weight buffers
    uint32_t shared, pad[3];
};
// item number w -> (group, pass): routed groups first (pre[] = passes before each group, in shared memory), then the shared
// expert's passes.  The group's entries and expert come from the selection record in global memory.
__device__ __forceinline__ FfnItem ffn_item(const uint32_t *pre, const moe_sel *ms, uint32_t U, uint32_t nb, uint32_t ebase, uint32_t w) {
    FfnItem it{};
    const uint32_t routed = pre[U];
    uint32_t cnt;
    if (w >= routed) {
        it.shared = 1;
        it.e0 = 0;
        cnt = nb;
        it.c0 = (w - routed) * 8;
        it.erow = 0;
    } else {
        uint32_t lo = 0, hi = U;  // largest u with pre[u] <= w
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (pre[mid] <= w) lo = mid;
            else hi = mid;
        }
        it.shared = 0;
        it.e0 = ms->off[lo];
        cnt = ms->off[lo + 1] - it.e0;
        it.c0 = (w - pre[lo]) * 8;
        it.erow = ms->ue[lo] - ebase;
    }
    it.ncols = cnt - it.c0 < 8 ? cnt - it.c0 : 8;
    return it;
}
// column col of the item -> (token, rank)
__device__ __forceinline__ void ffn_entry(const moe_sel *ms, const FfnItem &it, uint32_t topk, uint32_t col, uint32_t &tok, uint32_t &rank) {
    if (it.shared) {
        tok = it.c0 + col;
        rank = topk;
    } else {
        const uint32_t en = ms->ent[it.e0 + it.c0 + col];
        tok = en >> 8;
        rank = en & 255;
    }
}

// ---- decode of this kernel.  The codebook sits in shared memory as its raw 4 bytes per entry in 32 interleaved copies (64 KB:
// lane l reads copy l, so a warp's 32 lookups hit 32 different banks in one wavefront).  A byte b becomes the fp16 subnormal
// with bit pattern 0x00bb = b * 2^-24 -- exact, and the tensor core multiplies subnormals like any other value -- so one byte
// permute builds two weights from two table bytes and two sign bytes (0x80 / 0x00 in the halves' upper bytes); the factor
// 2^24 is folded into the block scale d, a power of two that changes no rounding.  The four sign bytes of a codebook word come
// from the sign byte of the sub-block by one multiply (four non-overlapping shifted copies) and one AND.
struct RowHdr {
    float d, d2;        // block scale * 2^24 and twice it: sub-block scale = d + d2 * s
    uint32_t qa0, qa1;  // bytes = this thread's codebook high bit for word 0 of sub-blocks 0..3 / 4..7 (0 or 1)
    uint32_t qb0, qb1;  // the same for word 1
    uint32_t sclo, schi;  // the 4-bit scales of sub-blocks 0,2,4,6 / 1,3,5,7, one per byte
};
__device__ __forceinline__ RowHdr row_hdr(uint32_t blk, int t) {
    RowHdr h;
    h.d = h2f((uint16_t)lds_u16<0>(blk)) * 16777216.0f;
    h.d2 = h.d + h.d;
    const uint32_t q0 = (lds_u16<66>(blk) | (lds_u16<68>(blk) << 16)) >> (2 * t);
    const uint32_t q1 = (lds_u16<70>(blk) | (lds_u16<72>(blk) << 16)) >> (2 * t);
    h.qa0 = q0 & 0x01010101u;
    h.qb0 = (q0 >> 1) & 0x01010101u;
    h.qa1 = q1 & 0x01010101u;
    h.qb1 = (q1 >> 1) & 0x01010101u;
    const uint32_t sc = lds_u16<106>(blk) | (lds_u16<108>(blk) << 16);
    h.sclo = sc & 0x0f0f0f0fu;
    h.schi = (sc >> 4) & 0x0f0f0f0fu;
    return h;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
// 16-byte load of a B fragment into registers that keep their value (zero) in lanes whose column is absent
template <int OFF>
__device__ __forceinline__ void lds_v4_if(uint4 &v, uint32_t a, uint32_t have) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\t@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%6];\n\t}"
                 : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
                 : "r"(a), "r"(have), "n"(OFF));
}
// this thread's 8 weights of sub-block IB of one row as four packed pairs; returns the sub-block scale d * (1 + 2 s) * 2^24
template <int IB>
__device__ __forceinline__ float row_sub(uint32_t blk_t, uint32_t blk_s, const RowHdr &h, uint32_t tabl, uint32_t (&w)[4]) {
    constexpr uint32_t k = IB & 3;
    constexpr uint32_t selA = (3u << 12) | (2u << 8) | ((4 + k) << 4) | 0, selB = (3u << 12) | (2u << 8) | ((4 + k) << 4) | 1;
    const uint32_t qs = lds_u16<2 + 8 * IB>(blk_t);
    const uint32_t sg = lds_u8<74 + 4 * IB>(blk_s);
    const uint32_t v0 = lds_u32(tabl + __byte_perm(qs, IB < 4 ? h.qa0 : h.qa1, selA) * 128);
    const uint32_t v1 = lds_u32(tabl + __byte_perm(qs, IB < 4 ? h.qb0 : h.qb1, selB) * 128);
    // sign bit j of the low / high nibble -> bit 7 of byte 3 - j
    const uint32_t s0 = (sg * 0x80402010u) & 0x80808080u, s1 = (sg * 0x08040201u) & 0x80808080u;
    w[0] = __byte_perm(v0, s0, 0x6170);
    w[1] = __byte_perm(v0, s0, 0x4352);
    w[2] = __byte_perm(v1, s1, 0x6170);
    w[3] = __byte_perm(v1, s1, 0x4352);
    const uint32_t n = __byte_perm(IB & 1 ? h.schi : h.sclo, 0, 0x4440 | (IB >> 1));
    return fmaf(h.d2, (float)n, h.d);
}
// one sub-block of rows g (at u0) and g + 8 (at u1): PLANES = 1 for fp16 tokens, 2 for H as fp16 high + low
template <int IB, int PLANES>
__device__ __forceinline__ void ffn_sub(uint32_t u0, uint32_t u1, int t, const RowHdr &h0, const RowHdr &h1, uint32_t tabl, const ZeroRegs &zr, uint32_t bh,
                                        uint32_t bl, uint32_t have, uint4 &xv, uint4 &xl, float (&acc)[4]) {
    lds_v4_if<IB * 64>(xv, bh, have);
    if (PLANES == 2) lds_v4_if<IB * 64>(xl, bl, have);
    uint32_t wa[4], wb[4];
    const float dba = row_sub<IB>(u0 + 2 * t, u0 + t, h0, tabl, wa);
    const float dbb = row_sub<IB>(u1 + 2 * t, u1 + t, h1, tabl, wb);
    const uint32_t a0[4] = {wa[0], wb[0], wa[1], wb[1]};
    const uint32_t a1[4] = {wa[2], wb[2], wa[3], wb[3]};
    float p[4];
    mma_f16(p, a0, xv.x, xv.y, zr.z);
    mma_f16(p, a1, xv.z, xv.w, p);
    if (PLANES == 2) {
        mma_f16(p, a0, xl.x, xl.y, p);
        mma_f16(p, a1, xl.z, xl.w, p);
    }
    acc[0] = fmaf(dba, p[0], acc[0]);
    acc[1] = fmaf(dba, p[1], acc[1]);
    acc[2] = fmaf(dbb, p[2], acc[2]);
    acc[3] = fmaf(dbb, p[3], acc[3]);
}
template <int PLANES>
__device__ __forceinline__ void ffn_unit(uint32_t u0, uint32_t u1, int t, uint32_t tabl, const ZeroRegs &zr, uint32_t bh, uint32_t bl, uint32_t have,
                                         float (&acc)[4]) {
    const RowHdr h0 = row_hdr(u0, t), h1 = row_hdr(u1, t);
    uint4 xv = make_uint4(0, 0, 0, 0), xl = make_uint4(0, 0, 0, 0);
    ffn_sub<0, PLANES>(u0, u1, t, h0, h1, tabl, zr, bh, bl, have, xv, xl, acc);
    ffn_sub<1, PLANES>(u0, u1, t, h0, h1, tabl, zr, bh, bl, have, xv, xl, acc);
    ffn_sub<2, PLANES>(u0, u1, t, h0, h1, tabl, zr, bh, bl, have, xv, xl, acc);
    ffn_sub<3, PLANES>(u0, u1, t, h0, h1, tabl, zr, bh, bl, have, xv, xl, acc);
    ffn_sub<4, PLANES>(u0, u1, t, h0, h1, tabl, zr, bh, bl, have, xv, xl, acc);
    ffn_sub<5, PLANES>(u0, u1, t, h0, h1, tabl, zr, bh, bl, have, xv, xl, acc);
    ffn_sub<6, PLANES>(u0, u1, t, h0, h1, tabl, zr, bh, bl, have, xv, xl, acc);
    ffn_sub<7, PLANES>(u0, u1, t, h0, h1, tabl, zr, bh, bl, have, xv, xl, acc);
}

// ---- IQ3X units (iq3x.cuh): rec = shared address of the row record, kh = which super-block of the pair.
// The sub-block's integer scale S = 1 + 2 s is folded into the weights: w * S is an integer below 2048, exact in fp16, and
// comes out of the same multiply-add that removes the exponent bias -- its two constants (S, -1040 S) and (S / 16, -80 S)
// are looked up per (row, sub-block) in a 16-entry table -- so the MMAs accumulate over the whole super-block and the block
// scale d is applied once per 256 weights.
struct XHdr {
    float d;
    uint32_t sc;  // the eight 4-bit scales, sub-block ib in bits 4 ib .. 4 ib + 3
};
__device__ __forceinline__ XHdr x_hdr(uint32_t rec, int kh) {
    XHdr h;
    h.d = h2f((uint16_t)lds_u16<256>(rec + 2 * kh));
    asm volatile("ld.shared.u32 %0, [%1+260];" : "=r"(h.sc) : "r"(rec + 4 * kh));
    return h;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds_u32_off(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
    return v;
}
// the lane word's eight codes times S as four packed fp16 pairs; c = the table entry of the sub-block's scale
__device__ __forceinline__ void iq3x_word_s(uint32_t q, const uint4 &c, uint32_t (&w)[4]) {
    const uint32_t r = __funnelshift_r(q, q, 8);
    const uint32_t h0 = lop3_and_or(q, 0x001E001Eu, 0x64016401u), h1 = lop3_and_or(q, 0x01E001E0u, 0x64106410u);
    const uint32_t h2 = lop3_and_or(r, 0x001E001Eu, 0x64016401u), h3 = lop3_and_or(r, 0x01E001E0u, 0x64106410u);
    const __half2 m0 = *(const __half2 *)&c.x, a0 = *(const __half2 *)&c.y, m1 = *(const __half2 *)&c.z, a1 = *(const __half2 *)&c.w;
    const __half2 v0 = __hfma2(*(const __half2 *)&h0, m0, a0), v1 = __hfma2(*(const __half2 *)&h1, m1, a1);
    const __half2 v2 = __hfma2(*(const __half2 *)&h2, m0, a0), v3 = __hfma2(*(const __half2 *)&h3, m1, a1);
    w[0] = *(const uint32_t *)&v0;
    w[1] = *(const uint32_t *)&v1;
    w[2] = *(const uint32_t *)&v2;
    w[3] = *(const uint32_t *)&v3;
}
// Software-pipelined over the sub-blocks: the MMAs of sub-block i are issued, then the loads and the decode of sub-block
// i + 1 -- the MMA results are not waited for.  (The predicated B loads keep zeros in lanes whose column is absent.)
struct XDec {
    uint32_t a0[4], a1[4];  // A fragments of the sub-block's two MMAs
};
template <int IB, int PLANES>
__device__ __forceinline__ void x_load(uint32_t c0, uint32_t c1, uint32_t bh, uint32_t bl, uint32_t have, uint32_t (&q)[2], uint4 &xv, uint4 &xl) {
    lds_v4_if<IB * 64>(xv, bh, have);
    if (PLANES == 2) lds_v4_if<IB * 64>(xl, bl, have);
    q[0] = lds_u32_off<IB * 16>(c0);
    q[1] = lds_u32_off<IB * 16>(c1);
}
template <int IB>
__device__ __forceinline__ void x_decode(const uint32_t (&q)[2], const XHdr &h0, const XHdr &h1, uint32_t stab, XDec &d) {
    uint32_t wa[4], wb[4];
    const uint32_t s0 = IB == 0 ? (h0.sc << 4) & 0xF0u : (h0.sc >> (4 * IB - 4)) & 0xF0u, s1 = IB == 0 ? (h1.sc << 4) & 0xF0u : (h1.sc >> (4 * IB - 4)) & 0xF0u;
    iq3x_word_s(q[0], lds_v4(stab + s0), wa);
    iq3x_word_s(q[1], lds_v4(stab + s1), wb);
    d.a0[0] = wa[0]; d.a0[1] = wb[0]; d.a0[2] = wa[1]; d.a0[3] = wb[1];
    d.a1[0] = wa[2]; d.a1[1] = wb[2]; d.a1[2] = wa[3]; d.a1[3] = wb[3];
}
template <int PLANES, bool FIRST>
__device__ __forceinline__ void x_mma(const XDec &d, const uint4 &xv, const uint4 &xl, const ZeroRegs &zr, float (&p)[4]) {
    if (FIRST) mma_f16(p, d.a0, xv.x, xv.y, zr.z);
    else mma_f16(p, d.a0, xv.x, xv.y, p);
    mma_f16(p, d.a1, xv.z, xv.w, p);
    if (PLANES == 2) {
        mma_f16(p, d.a0, xl.x, xl.y, p);
        mma_f16(p, d.a1, xl.z, xl.w, p);
    }
}
// rec0 / rec1: row records of MMA rows g and g + 8
template <int PLANES>
__device__ __forceinline__ void x_unit(uint32_t rec0, uint32_t rec1, int kh, int t, uint32_t stab, const ZeroRegs &zr, uint32_t bh, uint32_t bl, uint32_t have,
                                       float (&acc)[4]) {
    const uint32_t c0 = rec0 + kh * 128 + t * 4, c1 = rec1 + kh * 128 + t * 4;
    uint32_t q[2];
    uint4 xv = make_uint4(0, 0, 0, 0), xl = make_uint4(0, 0, 0, 0);
    XDec dec;
    float p[4];
    x_load<0, PLANES>(c0, c1, bh, bl, have, q, xv, xl);
    const XHdr h0 = x_hdr(rec0, kh), h1 = x_hdr(rec1, kh);
    x_decode<0>(q, h0, h1, stab, dec);
#define X_STEP(IB)                                           \
    x_mma<PLANES, IB == 0>(dec, xv, xl, zr, p);              \
    x_load<IB + 1, PLANES>(c0, c1, bh, bl, have, q, xv, xl); \
    x_decode<IB + 1>(q, h0, h1, stab, dec);
    X_STEP(0)
    X_STEP(1)
    X_STEP(2)
    X_STEP(3)
    X_STEP(4)
    X_STEP(5)
    X_STEP(6)
#undef X_STEP
    x_mma<PLANES, false>(dec, xv, xl, zr, p);
    acc[0] = fmaf(h0.d, p[0], acc[0]); acc[1] = fmaf(h0.d, p[1], acc[1]); acc[2] = fmaf(h1.d, p[2], acc[2]); acc[3] = fmaf(h1.d, p[3], acc[3]);
}

// PROBE = true is the copy-only twin used to measure what the staging pipeline alone can deliver: the same pieces, the same
// TMA boxes and bulk copies through the same ring, but the consumers only read every staged byte once (16-byte loads) and
// compute nothing -- the role of the reference's pure-read probes (bench/moe_bw.c:1-3, bench/qmv.c:357-382).
// (17 warps put five on one scheduler, whose 16 K registers then allow 96 per thread)
template <bool PROBE, int FMT>
__global__ void __launch_bounds__(FFN_THREADS, FfnCfg<FMT>::PER_SM) moe_ffn_k(const __grid_constant__ CUtensorMap mG, const __grid_constant__ CUtensorMap mU,
                                                           const __grid_constant__ CUtensorMap mSG, const __grid_constant__ CUtensorMap mSU, const FfnP p) {
    using C = FfnCfg<FMT>;
    constexpr int FFN_STG = C::STG, FFN_SLOT = C::SLOT;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = (uint64_t *)smem;
    uint64_t *full = bars, *empty = bars + FFN_STG, *tab_bar = bars + 2 * FFN_STG, *actfull = tab_bar + 1, *actfree = actfull + 2;
    uint32_t *pre = (uint32_t *)(smem + C::OFF_PRE);
    FfnItem *recs = (FfnItem *)(smem + C::OFF_REC);
    float4 *red = (float4 *)(smem + C::OFF_RED);
    constexpr uint32_t D = FFN_D, I = FFN_I, rbI = I / 256 * 110;
    constexpr uint32_t xpitch = D * 2 + 64, hpitch = I * 2 + 64, act_slot = 8 * xpitch;  // a slot holds 8 token rows or 16 H rows
    static_assert(act_slot >= 16 * hpitch, "activation slot");
    uint8_t *act0 = smem + C::OFF_XS, *stage0 = act0 + act_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    constexpr uint32_t KP = D / 512, GT = I / 64, DT = D / 128, KU = I / 256;

    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < FFN_STG; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], FFN_CW);
        }
        mbar_init(tab_bar, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(&actfull[s], 1);
            mbar_init(&actfree[s], FFN_CW);
        }
        mbar_init_fence();
        if (FMT == 0) {
            mbar_expect_tx(tab_bar, C::TAB);
            bulk_g2s(smem + C::OFF_TAB, p.tab->grid_u32x32, C::TAB, tab_bar);
        }
    }
    if (FMT == 1 && tid < 16) {  // constants of the decode multiply-adds for scale field s = tid: (S, -1040 S, S / 16, -80 S) as fp16 pairs, S = 1 + 2 s
        const float S = (float)(1 + 2 * tid);
        const __half2 m0 = __float2half2_rn(S), a0 = __float2half2_rn(-1040.0f * S), m1 = __float2half2_rn(S * 0.0625f), a1 = __float2half2_rn(-80.0f * S);
        *(uint4 *)(smem + C::OFF_TAB + 16 * tid) = make_uint4(*(const uint32_t *)&m0, *(const uint32_t *)&a0, *(const uint32_t *)&m1, *(const uint32_t *)&a1);
    }
    pdl_wait();  // the selection record, the tokens and Pg belong to earlier kernels
    const moe_sel *ms = p.ms;
    // passes before every group: independent loads, so the table is in shared memory after one latency
    for (uint32_t i = tid; i < FFN_MAXG; i += FFN_THREADS) pre[i] = ms->pre[i];
    const uint32_t U = ms->U, nb = ms->nb, topk = ms->topk;
    __syncthreads();
    uint32_t items = pre[U] + (p.Sd ? (nb + 7) / 8 : 0);
    if (items > FFN_MAXITEMS) {  // cannot happen with E <= 512 and 64 tokens; never index past the flags
        if (tid == 0) set_status(p.status, ST_BAD_ARG | 5);
        items = 0;
    }
    const uint32_t slot0 = smem_u32(stage0);
    // this block's pieces: gate/up tiles [a_lo, a_hi) of the items x GT list, then down tiles [b_lo, b_hi) of the items x DT list
    const uint32_t G = gridDim.x, bx_ = blockIdx.x;
    uint32_t a_lo = (uint32_t)((uint64_t)bx_ * items * GT / G), a_hi = (uint32_t)((uint64_t)(bx_ + 1) * items * GT / G);
    uint32_t b_lo = (uint32_t)((uint64_t)bx_ * items * DT / G), b_hi = (uint32_t)((uint64_t)(bx_ + 1) * items * DT / G);
    // the few items those shares touch, looked up once (thread k: item k of the gate/up share, thread FFN_RECS + k: of the down share)
    const uint32_t wa0 = a_lo / GT, wb0 = b_lo / DT;
    if ((a_hi > a_lo && (a_hi - 1) / GT - wa0 >= FFN_RECS) || (b_hi > b_lo && (b_hi - 1) / DT - wb0 >= FFN_RECS)) {  // a grid far smaller than the device's
        if (tid == 0) set_status(p.status, ST_BAD_ARG | 6);
        a_hi = a_lo;
        b_hi = b_lo;
    }
    if (tid < 2 * FFN_RECS) {
        const uint32_t k = tid % FFN_RECS, w = (tid < FFN_RECS ? wa0 : wb0) + k;
        const bool need = tid < FFN_RECS ? (a_hi > a_lo && w <= (a_hi - 1) / GT) : (b_hi > b_lo && w <= (b_hi - 1) / DT);
        if (need) recs[tid] = ffn_item(pre, ms, U, nb, p.ebase, w);
    }
    __syncthreads();
    const FfnItem *rec_a = recs - wa0, *rec_b = recs + FFN_RECS - wb0;  // rec_a[w], rec_b[w]

    if (warp == FFN_CW) {
        // ---- producer: one lane walks the block's pieces and keeps the ring full
        if (lane == 0) {
            bool ok = true;
            uint32_t j = 0, k = 0;
            auto slot_for = [&](uint32_t bytes) {  // waits until stage j % STG is free, arms its barrier; returns its address
                const uint32_t s = j % FFN_STG;
                if (j >= FFN_STG && ok && !mbar_wait(&empty[s], (j / FFN_STG - 1) & 1)) {
                    ok = false;
                    set_status(p.status, ST_MBAR_TIMEOUT | 6);
                }
                fence_proxy_async();  // the consumers' reads of the stage are ordered before the copy engine's writes
                mbar_expect_tx(&full[s], bytes);
                return slot0 + s * FFN_SLOT;
            };
            // The activation slot is a ring of eight rows (tokens of an item, or the two planes of its H): item k takes the next
            // ncols rows, so the rows of the next item are usually on their way while the consumers still read this one's.  Two
            // barrier pairs alternate by item; item k - 2 must have been released, item k - 1 too when the rows would overlap or
            // the layout changes (fresh).  Returns the first row's index.
            uint32_t rowbase = 0, prev_n = 8;
            auto act_for = [&](uint32_t ncols, uint32_t bytes, bool fresh) {
                const uint32_t s = k & 1, n = k >> 1;
                if (n >= 1 && ok && !mbar_wait(&actfree[s], (n - 1) & 1)) {
                    ok = false;
                    set_status(p.status, ST_MBAR_TIMEOUT | 7);
                }
                if (k >= 1 && (fresh || prev_n + ncols > 8) && ok && !mbar_wait(&actfree[(k - 1) & 1], ((k - 1) >> 1) & 1)) {
                    ok = false;
                    set_status(p.status, ST_MBAR_TIMEOUT | 7);
                }
                if (fresh) rowbase = 0;
                fence_proxy_async();
                mbar_expect_tx(&actfull[s], bytes);
                const uint32_t r0 = rowbase;
                rowbase = (rowbase + ncols) & 7;
                prev_n = ncols;
                return r0;
            };
            struct Src {
                const CUtensorMap *tg, *tu;
                const uint8_t *wg, *wu, *wd;
                uint32_t erow;
            };
            auto src_of = [&](const FfnItem &it) {
                Src c;
                c.erow = it.erow;
                c.tg = it.shared ? &mSG : &mG;
                c.tu = it.shared ? &mSU : &mU;
                if (FMT == 0) {
                    c.wg = c.wu = nullptr;  // the copies go through the tensor maps
                    c.wd = it.shared ? p.Sd : p.Wd + (size_t)c.erow * D * rbI;
                } else {  // IQ3X: stage-ordered records, gate and up interleaved in one buffer
                    c.wg = c.wu = (it.shared ? p.Sg : p.Wg) + (size_t)c.erow * GT * KP * IQ3X_STAGE;
                    c.wd = (it.shared ? p.Sd : p.Wd) + (size_t)c.erow * DT * (I / 512) * IQ3X_STAGE;
                }
                return c;
            };
            Src sc{};
            uint32_t cur = 0xffffffffu;
            for (uint32_t a = a_lo; a < a_hi; a++) {
                const uint32_t w = a / GT, gt = a - w * GT;
                const bool sw = w != cur;
                FfnItem it{};
                if (sw) {
                    cur = w;
                    it = rec_a[w];
                    sc = src_of(it);
                }
                for (uint32_t kp = 0; kp < KP; kp++, j++) {
                    const uint32_t dst = slot_for(FMT ? IQ3X_STAGE : 2 * 64 * FFN_PITCH);
                    if (FMT == 1) {  // one contiguous stage
                        bulk_s(dst, sc.wg + ((size_t)gt * KP + kp) * IQ3X_STAGE, IQ3X_STAGE, &full[j % FFN_STG]);
                    } else {
                        const int xc = (int)((220 * kp) & ~15u), yr = (int)(sc.erow * I + gt * 64);
                        tma_box_2d(dst, sc.tg, xc, yr, &full[j % FFN_STG]);
                        tma_box_2d(dst + 64 * FFN_PITCH, sc.tu, xc, yr, &full[j % FFN_STG]);
                    }
                    if (sw && kp == 0) {  // the tokens of a new item's columns, requested after its first weights (the longer wait)
                        const uint32_t r0 = act_for(it.ncols, it.ncols * D * 2, false);
                        for (uint32_t c = 0; c < it.ncols; c++) {
                            uint32_t tok, rank;
                            ffn_entry(ms, it, topk, c, tok, rank);
                            bulk_g2s(act0 + ((r0 + c) & 7) * xpitch, p.x + (size_t)tok * D, D * 2, &actfull[k & 1]);
                        }
                        k++;
                    }
                }
            }
            cur = 0xffffffffu;
            bool first_dn = true;  // the H rows have another pitch than the tokens: the ring starts over, once the last tokens are released
            for (uint32_t bi = b_lo; bi < b_hi; bi++, j++) {
                const uint32_t w = bi / DT, dt = bi - w * DT;
                const bool sw = w != cur;
                FfnItem it{};
                if (sw) {
                    cur = w;
                    it = rec_b[w];
                    sc = src_of(it);
                }
                const uint32_t bytes = FMT ? IQ3X_STAGE : 128 * rbI;
                const uint32_t dst = slot_for(bytes);
                bulk_s(dst, sc.wd + (size_t)dt * bytes, bytes, &full[j % FFN_STG]);
                if (sw) {  // H of a new item, after its first weights are on their way: written by the blocks that ran its gate/up
                           // pieces, complete when all GT x 8 warps have counted in
                    if (!PROBE && ok && ld_acquire_gpu(p.sync + w) < GT * 8) {
                        const uint64_t t0 = global_ns();
                        while (ld_acquire_gpu(p.sync + w) < GT * 8)
                            if (global_ns() - t0 > 2000000000ull) {
                                ok = false;
                                set_status(p.status, ST_MBAR_TIMEOUT | 11);
                                break;
                            }
                    }
                    asm volatile("fence.proxy.async.global;" ::: "memory");  // the H rows were written by ordinary stores; the copy engine reads them
                    const uint32_t r0 = act_for(it.ncols, 2 * it.ncols * I * 2, first_dn);
                    first_dn = false;
                    const __half *Hw = p.H + (size_t)w * 16 * I;
                    for (uint32_t c = 0; c < it.ncols; c++) {
                        const uint32_t rw = (r0 + c) & 7;
                        bulk_g2s(act0 + rw * hpitch, Hw + (size_t)c * I, I * 2, &actfull[k & 1]);
                        bulk_g2s(act0 + (8 + rw) * hpitch, Hw + (size_t)(8 + c) * I, I * 2, &actfull[k & 1]);
                    }
                    k++;
                }
            }
        }
    } else {
        // ---- consumers
        const int r = warp & 7, kh = warp >> 3;
        bool ok = FMT == 0 ? mbar_wait(tab_bar, 0) : true;
        if (!ok && lane == 0) set_status(p.status, ST_MBAR_TIMEOUT | 8);
        const uint32_t tabl = smem_u32(smem + C::OFF_TAB) + lane * 4;  // this lane's copy of the interleaved codebook
        const uint32_t stab = smem_u32(smem + C::OFF_TAB);             // IQ3X: the scale constants
        const ZeroRegs zr = zero_regs();
        uint32_t j = 0, k = 0, rc = 0;
        auto wait_full = [&]() {
            if (ok && !mbar_wait(&full[j % FFN_STG], (j / FFN_STG) & 1)) {
                ok = false;
                if (lane == 0) set_status(p.status, ST_MBAR_TIMEOUT | 9);
            }
            return slot0 + (j % FFN_STG) * FFN_SLOT;
        };
        auto release = [&]() {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[j % FFN_STG]);
            j++;
        };
        // activation slot of the next item: waits for its copy, returns its shared address
        // activation rows of the next item (see the producer's act_for): waits for their copy; returns the address of column g's row
        uint32_t rowbase = 0;
        auto act_wait = [&](uint32_t ncols, uint32_t pitch) {
            if (ok && !mbar_wait(&actfull[k & 1], (k >> 1) & 1)) {
                ok = false;
                if (lane == 0) set_status(p.status, ST_MBAR_TIMEOUT | 10);
            }
            const uint32_t a = smem_u32(act0) + ((rowbase + g) & 7) * pitch;
            rowbase = (rowbase + ncols) & 7;
            return a;
        };
        auto act_release = [&]() {  // this warp is done with the current item's rows
            __syncwarp();
            if (lane == 0) mbar_arrive(&actfree[k & 1]);
            k++;
        };
        auto probe_read = [&](uint32_t st, uint32_t bytes, uint32_t &sink) {
            for (uint32_t o = (warp * 32 + lane) * 16; o < bytes; o += FFN_CW * 32 * 16) {
                const uint4 v = lds_v4(st + o);
                sink ^= v.x ^ v.y ^ v.z ^ v.w;
            }
        };
        // the two K halves of a row group: the high half hands its partial sums over, the low half adds them to its own
        auto pair_sum = [&](float (&acc)[4]) {
            float4 *rd = red + ((rc & 1) * 8 + r) * 32 + lane;
            rc++;
            if (kh) *rd = make_float4(acc[0], acc[1], acc[2], acc[3]);
            bar_sync_n(1 + r, 64);
            if (!kh) {
                const float4 v = *rd;
                acc[0] += v.x;
                acc[1] += v.y;
                acc[2] += v.z;
                acc[3] += v.w;
            }
        };
        uint32_t sink = 0;
        // ---- gate/up pieces: tiles of 64 intermediate indices
        uint32_t cur = 0xffffffffu, have = 0, ncols = 0, xb0 = 0;
        for (uint32_t a = a_lo; a < a_hi; a++) {
            const uint32_t w = a / GT, gt = a - w * GT;
            if (w != cur) {
                if (cur != 0xffffffffu) act_release();
                cur = w;
                ncols = rec_a[w].ncols;
                have = (uint32_t)g < ncols ? 1u : 0u;
                xb0 = act_wait(ncols, xpitch) + t * 16;
            }
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (uint32_t kp = 0; kp < KP; kp++) {
                const uint32_t st = wait_full();
                const uint32_t bx = xb0 + (2 * kp + kh) * 512;
                if (PROBE) probe_read(st, FMT ? IQ3X_STAGE : 128 * FFN_PITCH, sink);
                else if (FMT == 1) {
                    const uint32_t rec0 = st + (8 * r + g) * IQ3X_REC;
                    x_unit<1>(rec0, rec0 + 64 * IQ3X_REC, kh, t, stab, zr, bx, bx, have, acc);
                } else {
                    const uint32_t u0 = st + (8 * r + g) * FFN_PITCH + ((220 * kp) & 15) + kh * 110, u1 = u0 + 64 * FFN_PITCH;
                    ffn_unit<1>(u0, u1, t, tabl, zr, bx, bx, have, acc);
                }
                release();
            }
            if (PROBE) continue;
            pair_sum(acc);
            if (!kh) {
                // acc[0], acc[1] = gate of index 64 gt + 8 r + g for columns 2t, 2t + 1; acc[2], acc[3] = up.  H travels to the
                // down pieces (run by whichever blocks hold them) through global memory as an fp16 high part plus an fp16
                // remainder (22 mantissa bits where the remainder is normal): [item][plane][column][I]
                const uint32_t idx = gt * 64 + 8 * r + g;
                __half *Hw = p.H + (size_t)w * 16 * I + idx;
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const float gs = acc[c], us = acc[2 + c];
                    float h = gs / (1.0f + expf(-gs)) * us;
                    h = fminf(fmaxf(h, -65504.0f), 65504.0f);
                    const __half hi = __float2half_rn(h);
                    const __half lo = __float2half_rn(h - __half2float(hi));
                    if ((uint32_t)(2 * t + c) < ncols) {
                        Hw[(size_t)(2 * t + c) * I] = hi;
                        Hw[(size_t)(8 + 2 * t + c) * I] = lo;
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    __threadfence();  // the warp's H values (cumulative over the warp barrier) before the count
                    atomicAdd(p.sync + w, 1u);
                }
            }
        }
        if (cur != 0xffffffffu) act_release();
        // ---- down pieces: tiles of 128 output rows; MMA row g is tile row 16 r + 2 g, row g + 8 the next one
        cur = 0xffffffffu;
        rowbase = 0;
        uint32_t hb0 = 0, oo[2] = {0xffffffffu, 0xffffffffu};  // element offsets of the output rows of columns 2t and 2t + 1
        for (uint32_t bi = b_lo; bi < b_hi; bi++) {
            const uint32_t w = bi / DT, dt = bi - w * DT;
            if (w != cur) {
                if (cur != 0xffffffffu) act_release();
                cur = w;
                const FfnItem it = rec_b[w];
                have = (uint32_t)g < it.ncols ? 1u : 0u;
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    oo[c] = 0xffffffffu;
                    if ((uint32_t)(2 * t + c) < it.ncols) {
                        uint32_t tok, rank;
                        ffn_entry(ms, it, topk, 2 * t + c, tok, rank);
                        oo[c] = (tok * (topk + 1) + rank) * D;
                    }
                }
                hb0 = act_wait(it.ncols, hpitch) + t * 16;
            }
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t st = wait_full();
            if (PROBE) {
                probe_read(st, FMT ? IQ3X_STAGE : 128 * rbI, sink);
                release();
                continue;
            }
            static_assert(KU == 2, "one super-block of K per K half");
            {
                const uint32_t ks = kh;
                const uint32_t bh = hb0 + ks * 512, bl = bh + 8 * hpitch;
                if (FMT == 1) {  // positions 16 r + g and 16 r + 8 + g hold output rows 16 r + 2 g and 16 r + 2 g + 1
                    const uint32_t rec0 = st + (16 * r + g) * IQ3X_REC;
                    x_unit<2>(rec0, rec0 + 8 * IQ3X_REC, kh, t, stab, zr, bh, bl, have, acc);
                } else {
                    const uint32_t u0 = st + (16 * r + 2 * g) * rbI + ks * 110, u1 = u0 + rbI;
                    ffn_unit<2>(u0, u1, t, tabl, zr, bh, bl, have, acc);
                }
            }
            release();
            pair_sum(acc);
            if (!kh) {
                // acc[0], acc[2] = rows 2g, 2g + 1 of column 2t; acc[1], acc[3] = the same rows of column 2t + 1
                const uint32_t row = dt * 128 + 16 * r + 2 * g;
                if (p.ep.nranks > 1) {
                    for (uint32_t q = 0; q < p.ep.nranks; q++) {
                        if (oo[0] != 0xffffffffu) *(float2 *)(p.PgR[q] + oo[0] + row) = make_float2(acc[0], acc[2]);
                        if (oo[1] != 0xffffffffu) *(float2 *)(p.PgR[q] + oo[1] + row) = make_float2(acc[1], acc[3]);
                    }
                } else {
                    if (oo[0] != 0xffffffffu) *(float2 *)(p.Pg + oo[0] + row) = make_float2(acc[0], acc[2]);
                    if (oo[1] != 0xffffffffu) *(float2 *)(p.Pg + oo[1] + row) = make_float2(acc[1], acc[3]);
                    // this warp's 16 rows of the tile are stored for every column: count it in on the columns' output rows (lanes
                    // t = 0 .. 3 of row g = 0 know two columns each), so that the combine + norm of a token can start when its rows are complete
                    __syncwarp();
                    if (g == 0) {
                        __threadfence();  // the warp's stores (cumulative over the warp barrier) before the counts
                        if (oo[0] != 0xffffffffu) atomicAdd(p.sync + MOE_FFN_ROWCNT + oo[0] / D, 1u);
                        if (oo[1] != 0xffffffffu) atomicAdd(p.sync + MOE_FFN_ROWCNT + oo[1] / D, 1u);
                    }
                }
            }
        }
        if (cur != 0xffffffffu) act_release();
        if (PROBE && sink == 0x9e3779b9u) p.Pg[0] = 0.f;  // keeps the loads observable; practically never taken
    }
    // the last block to finish clears the items' counters for the next launch (every block has read what it needed by then)
    __syncthreads();
    if (tid == 0 && !PROBE) {
        __threadfence();
        if (atomicAdd(p.sync + FFN_MAXITEMS, 1u) == gridDim.x - 1) {
            for (uint32_t i = 0; i < items; i++) p.sync[i] = 0;
            p.sync[FFN_MAXITEMS] = 0;
        }
    }
    if (p.ep.nranks > 1) ep_publish(p.ep);
}

// ---- tensor maps: an expert tensor [rows][pitch bytes] seen as a 2-D byte array, box = 240 bytes x 64 rows, no swizzle.
// cuTensorMapEncodeTiled is a driver entry point; it is looked up through the runtime so that the library has no link
// dependency on libcuda.
typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                    const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
bool ffn_encode_map(CUtensorMap *tm, const void *base, uint64_t pitch, uint64_t rows) {
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void *q = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &qr) != cudaSuccess || !q) return false;
        fn = (encode_tiled_fn)q;
    }
    const cuuint64_t gdim[2] = {pitch, rows};
    const cuuint64_t gstride[1] = {pitch};
    const cuuint32_t box[2] = {FFN_PITCH, 64}, estr[2] = {1, 1};
    return fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
const CUtensorMap *ffn_tensor_map(const void *base, uint64_t pitch, uint64_t rows) {
    static std::mutex mu;
    static std::map<std::tuple<const void *, uint64_t, uint64_t>, CUtensorMap> cache;
    std::lock_guard<std::mutex> lk(mu);
    const auto key = std::make_tuple(base, pitch, rows);
    auto itc = cache.find(key);
    if (itc != cache.end()) return &itc->second;
    CUtensorMap tm;
    if (!ffn_encode_map(&tm, base, pitch, rows)) return nullptr;
    return &(cache[key] = tm);
}

}  // namespace

// binds: 0 = routed gate, 1 = routed up [EL][I][rbD], 2 = shared gate, 3 = shared up (used unless SHARED is defined 0),
// 4 = x fp16 [nb][D], 5 = moe_sel, 6 = routed down [EL][D][rbI], 7 = shared down, 8 = scratch (MOE_FFN_SCRATCH_BYTES(I) of
// moe_sel.h, zeroed once by the owner, private to one stream), 9 = Pg fp32 [64][TOPK+1][D],
// 10 = id of the first expert held in the weight buffers (optional, default 0); with EPX = ranks also 11, 12, 16 + r,
// 24 + r as for moe_dn.  defines: E, D, I, TOPK, EL, SHARED, EPX.  The host's grid and block are ignored.
// With IQ3X defined 1 the weights are the re-coded form of iq3x.cuh (made by iq3x_pack): 0 = routed gate + up
// [EL][I/64][D/512] stages, 2 = the shared expert's, 6 = routed down [EL][D/128][I/512] stages, 7 = the shared expert's;
// binds 1 and 3 are not used.
static cudaError_t launch_moe_ffn(const QwLaunch &L) {
    FfnP p{};
    const uint32_t E = (uint32_t)L.def("E", 512), topk = (uint32_t)L.def("TOPK", 10);
    const bool x4 = L.def("IQ3X", 0) != 0;
    const uint32_t D = (uint32_t)L.def("D", 2048), I = (uint32_t)L.def("I", 512);
    QW_CHECK_ARG(D == FFN_D && I == FFN_I && topk < MOE_MAXK && E <= 512);
    const uint32_t rbD = D / 256 * 110, rbI = I / 256 * 110;
    const size_t act = (size_t)8 * (D * 2 + 64);  // an activation slot: 8 token rows, or 16 H rows
    const size_t smem = x4 ? FfnCfg<1>::OFF_XS + act + (size_t)FfnCfg<1>::STG * FfnCfg<1>::SLOT
                           : FfnCfg<0>::OFF_XS + act + (size_t)FfnCfg<0>::STG * FfnCfg<0>::SLOT;
    const int per_sm = x4 ? FfnCfg<1>::PER_SM : FfnCfg<0>::PER_SM;
    QW_CHECK_ARG((smem + 1024) * per_sm <= 227 * 1024 + 1024 && 128 * rbI <= FfnCfg<0>::SLOT && (128 * rbI) % 16 == 0);
    const bool shared = L.def("SHARED", 1) != 0;
    const uint32_t EL = (uint32_t)L.def("EL", E);
    p.ebase = L.has_bytes(10, 4) ? L.bytes<uint32_t>(10) : 0;
    QW_CHECK_ARG(EL >= 1 && p.ebase + EL <= E);
    const uint8_t *Wg = L.buf<uint8_t>(0), *Wu = x4 ? Wg : L.buf<uint8_t>(1), *Sg = shared ? L.buf<uint8_t>(2) : nullptr, *Su = !shared ? nullptr : x4 ? Sg : L.buf<uint8_t>(3);
    p.Wd = L.buf<uint8_t>(6);
    p.Wg = Wg;
    p.Sg = Sg;
    p.sync = L.buf<unsigned>(8);
    QW_CHECK_ARG(p.sync && ((uintptr_t)p.sync & 15) == 0 && L.avail(8) >= MOE_FFN_SCRATCH_BYTES(I));
    p.H = (__half *)((uint8_t *)p.sync + FFN_SYNC_BYTES);
    p.Sd = shared ? L.buf<uint8_t>(7) : nullptr;
    p.x = L.buf<__half>(4);
    p.ms = L.buf<moe_sel>(5);
    p.Pg = L.buf<float>(9);
    p.tab = (const QwTables *)L.tables;
    p.status = L.status;
    QW_CHECK_ARG(Wg && Wu && p.Wd && p.x && p.ms && p.Pg && L.avail(5) >= sizeof(moe_sel));
    QW_CHECK_ARG(!shared || (Sg && Su && p.Sd));
    if (x4) {
        const size_t gus = (size_t)(I / 64) * (D / 512) * IQ3X_STAGE, dns = (size_t)(D / 128) * (I / 512) * IQ3X_STAGE;
        QW_CHECK_ARG(L.avail(0) >= EL * gus && L.avail(6) >= EL * dns && (!shared || (L.avail(2) >= gus && L.avail(7) >= dns)));
    } else {
        const size_t wsz = (size_t)EL * I * rbD, ssz = (size_t)I * rbD;
        QW_CHECK_ARG(L.avail(0) >= wsz && L.avail(1) >= wsz && L.avail(6) >= wsz && (!shared || (L.avail(2) >= ssz && L.avail(3) >= ssz && L.avail(7) >= ssz)));
    }
    QW_CHECK_ARG((((uintptr_t)Wg | (uintptr_t)Wu | (uintptr_t)p.Wd | (uintptr_t)Sg | (uintptr_t)Su | (uintptr_t)p.Sd | (uintptr_t)p.x) & 15) == 0);
    QW_CHECK_ARG(L.avail(9) >= (size_t)MOE_MAXB * (topk + 1) * D * 4 && L.avail(4) >= (size_t)D * 2);
    p.ep = EpPeers{};
    p.ep.nranks = 1;
    if (L.def("EPX", 0) > 1) {
        p.ep.nranks = (uint32_t)L.def("EPX", 0);
        QW_CHECK_ARG(p.ep.nranks <= 8 && L.has_bytes(12, 4) && L.buf<unsigned>(11) && L.avail(11) >= 8);
        p.ep.rank = L.bytes<uint32_t>(12);
        QW_CHECK_ARG(p.ep.rank < p.ep.nranks);
        p.ep.seq = L.buf<unsigned>(11);
        p.ep.done = p.ep.seq + 1;
        for (uint32_t r = 0; r < p.ep.nranks; r++) {
            p.PgR[r] = L.buf<float>(16 + r);
            p.ep.flagR[r] = L.buf<unsigned>(24 + r);
            QW_CHECK_ARG(p.PgR[r] && p.ep.flagR[r] && L.avail(24 + r) >= p.ep.nranks * 4 && L.avail(16 + r) >= (size_t)MOE_MAXB * (topk + 1) * D * 4);
        }
    }
    static const CUtensorMap no_map{};  // IQ3X stages are contiguous: no tensor maps
    const CUtensorMap *mG = &no_map, *mU = &no_map, *mSG = &no_map, *mSU = &no_map;
    if (!x4) {
        mG = ffn_tensor_map(Wg, rbD, (uint64_t)EL * I);
        mU = ffn_tensor_map(Wu, rbD, (uint64_t)EL * I);
        mSG = shared ? ffn_tensor_map(Sg, rbD, I) : mG;
        mSU = shared ? ffn_tensor_map(Su, rbD, I) : mU;
        QW_CHECK_ARG(mG && mU && mSG && mSU);
    }
    const bool probe = L.def("PROBE", 0) != 0;  // PROBE defined 1: the copy-only twin (outputs are not written)
    auto kern = x4 ? (probe ? moe_ffn_k<true, 1> : moe_ffn_k<false, 1>) : (probe ? moe_ffn_k<true, 0> : moe_ffn_k<false, 0>);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int occ = 0;  // the blocks wait for one another's H: all of them must be resident together
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, FFN_THREADS, smem);
    if (e != cudaSuccess) return e;
    QW_CHECK_ARG(occ >= per_sm);
    qw_launch(kern, L.sm_count * per_sm, FFN_THREADS, smem, L.stream, *mG, *mU, *mSG, *mSU, p);
    return cudaGetLastError();
}
QW_FAMILY(moe_ffn, launch_moe_ffn, 512)
