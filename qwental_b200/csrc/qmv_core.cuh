// Shared core of the tensor-core quantized matvec kernels (dense qmv_mma, MoE gate/up and down).
//
// Work is cut into "units": 256 consecutive K values of 16 weight rows (one IQ3_S super-block per row, or eight
// Q8_0 blocks per row).  A warp owns a unit and walks its eight 32-value sub-blocks.  For each sub-block it
// builds the m16n8k16 A fragments straight from the raw block bytes in shared memory -- the weights' integer
// part (codebook value x sign for IQ3_S, the int8 for Q8_0) is exact in fp16/bf16 -- runs two MMAs per
// 8-token column tile against the activations, and applies the row's sub-block scale d*(1+2*scale) to the
// fp32 partial sums.  The dequantised weights never exist in memory.
//
// K is permuted inside each MMA so that a thread's four A values per MMA are one codebook word: thread
// (g = lane/4, t = lane%4) decodes weights 8t..8t+7 of the sub-block for rows g and g+8; k-slots
// (2t, 2t+1, 2t+8, 2t+9) of MMA 0 carry weights 8t..8t+3 and of MMA 1 weights 8t+4..8t+7; the B fragment of
// column g is the matching 16 bytes x[8t..8t+7].
//
// Every output column is a function of that column's activations only, with a fixed instruction sequence, so a
// token's result does not depend on how many other tokens are in the batch or which column it sits in.
#pragma once
#include "common.cuh"

namespace qw {

// IQ3_S codebook in shared memory as 4 fp16 (or bf16) values per entry; REP interleaved copies so that the 16
// lanes of a half-warp read different banks (REP = 16) or one compact copy (REP = 1).
template <int REP>
struct GridTab {
    const uint2 *tab;
    uint32_t c;
    __device__ __forceinline__ uint2 get(uint32_t e) const { return tab[e * REP + c]; }
};

// Decode this thread's 8 weights of sub-block ib of the IQ3_S super-block at blk (kernels/moe_iq.metal:102-118:
// qs @2, qh @66, signs @74, scales @106).  w[0..3] = packed pairs (w0,w1) (w2,w3) (w4,w5) (w6,w7) as signed
// integer-valued halves.  Returns the 4-bit scale field.
template <int REP>
__device__ __forceinline__ uint32_t iq3s_sub(const uint8_t *blk, int ib, int t, const GridTab<REP> &gt, uint32_t (&w)[4]) {
    const uint32_t qs = ldu16(blk + 2 + 8 * ib + 2 * t);
    const uint32_t qh = blk[66 + ib];
    const uint32_t sg = blk[74 + 4 * ib + t];
    const uint32_t sc = (blk[106 + (ib >> 1)] >> (4 * (ib & 1))) & 15;
    const uint32_t i0 = (qs & 255) | ((qh << (8 - 2 * t)) & 256);
    const uint32_t i1 = (qs >> 8) | ((qh << (7 - 2 * t)) & 256);
    const uint2 g0 = gt.get(i0), g1 = gt.get(i1);
    // sign bit 2j -> bit 15, sign bit 2j+1 -> bit 31 of pair j: one multiply spreads both, no carries
    w[0] = g0.x ^ ((sg * 0x40008000u) & 0x80008000u);
    w[1] = g0.y ^ ((sg * 0x10002000u) & 0x80008000u);
    w[2] = g1.x ^ ((sg * 0x04000800u) & 0x80008000u);
    w[3] = g1.y ^ ((sg * 0x01000200u) & 0x80008000u);
    return sc;
}

// Decode this thread's 8 int8 weights of the Q8_0 block at blk (src/ggml_dq.c:34-37: d @0, qs[32] @2) to
// integer-valued fp16 pairs: (q ^ 0x80) | 0x6400 is the half 1024 + (q + 128); subtracting 1152 is exact.
__device__ __forceinline__ void q8_sub(const uint8_t *blk, int t, uint32_t (&w)[4]) {
    const uint8_t *q = blk + 2 + 8 * t;
    const uint32_t lo = (ldu16(q) | ((uint32_t)ldu16(q + 2) << 16)) ^ 0x80808080u;
    const uint32_t hi = (ldu16(q + 4) | ((uint32_t)ldu16(q + 6) << 16)) ^ 0x80808080u;
    const uint32_t bias = 0x64806480u;
    const __half2 b2 = *(const __half2 *)&bias;
    uint32_t v[4] = {__byte_perm(lo, 0x64646464u, 0x4140), __byte_perm(lo, 0x64646464u, 0x4342), __byte_perm(hi, 0x64646464u, 0x4140),
                     __byte_perm(hi, 0x64646464u, 0x4342)};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const __half2 r = __hsub2(*(const __half2 *)&v[j], b2);
        w[j] = *(const uint32_t *)&r;
    }
}

// One unit (256 K values) for rows r0 (lanes' row g) and r1 (row g + 8): u0 / u1 point at the unit's bytes of
// those two rows in shared memory.  xcol[nt] (xlo[nt] for the low bf16 plane) is the activation row of column
// g + 8 nt in 16-byte units, nullptr for an absent column (it then contributes zeros); k8 = index of the unit's
// first 16-byte chunk.  The MMAs are warp-wide instructions: every lane of the warp must reach them, so a column
// tile is skipped only when it is absent for the whole warp (tile_on, a warp-uniform mask).
template <int NT>
__device__ __forceinline__ uint32_t tiles_on(const uint4 *const (&xcol)[NT]) {
    uint32_t m = 0;
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
        if (__any_sync(0xffffffffu, xcol[nt] != nullptr)) m |= 1u << nt;
    return m;
}

template <int GF, int NT, int REP, bool BF16>
__device__ __forceinline__ void unit_mma(const uint8_t *u0, const uint8_t *u1, const GridTab<REP> &gt, int t, const uint4 *const (&xcol)[NT],
                                         const uint4 *const (&xlo)[NT], uint32_t tile_on, int k8, float (&acc)[NT][4]) {
    float d0, d1;
    if (GF == 21) {
        d0 = h2f(ldu16(u0));
        d1 = h2f(ldu16(u1));
    }
#pragma unroll 2
    for (int ib = 0; ib < 8; ib++) {
        uint32_t wa[4], wb[4];
        float dba, dbb;
        if (GF == 21) {
            const uint32_t sa = iq3s_sub<REP>(u0, ib, t, gt, wa);
            const uint32_t sb = iq3s_sub<REP>(u1, ib, t, gt, wb);
            dba = __fmul_rn(d0, (float)(1 + 2 * (int)sa));
            dbb = __fmul_rn(d1, (float)(1 + 2 * (int)sb));
        } else {
            q8_sub(u0 + 34 * ib, t, wa);
            q8_sub(u1 + 34 * ib, t, wb);
            dba = h2f(ldu16(u0 + 34 * ib));
            dbb = h2f(ldu16(u1 + 34 * ib));
        }
        const uint32_t a0[4] = {wa[0], wb[0], wa[1], wb[1]};
        const uint32_t a1[4] = {wa[2], wb[2], wa[3], wb[3]};
        const int kk = k8 + 4 * ib + t;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            if (!(tile_on >> nt & 1)) continue;  // warp-uniform
            const uint4 zero = make_uint4(0, 0, 0, 0);
            const uint4 xv = xcol[nt] ? __ldcg(xcol[nt] + kk) : zero;
            float p[4] = {0.f, 0.f, 0.f, 0.f};
            if (BF16) {
                const uint4 xl = xcol[nt] ? __ldcg(xlo[nt] + kk) : zero;
                mma_bf16(p, a0, xv.x, xv.y, p);
                mma_bf16(p, a1, xv.z, xv.w, p);
                mma_bf16(p, a0, xl.x, xl.y, p);
                mma_bf16(p, a1, xl.z, xl.w, p);
            } else {
                mma_f16(p, a0, xv.x, xv.y, p);
                mma_f16(p, a1, xv.z, xv.w, p);
            }
            acc[nt][0] = fmaf(dba, p[0], acc[nt][0]);
            acc[nt][1] = fmaf(dba, p[1], acc[nt][1]);
            acc[nt][2] = fmaf(dbb, p[2], acc[nt][2]);
            acc[nt][3] = fmaf(dbb, p[3], acc[nt][3]);
        }
    }
}

// ---- variant for the MoE kernels: one 8-token column tile whose B fragments for the whole unit are already in
// registers (xf[ib], and xl[ib] for the low bf16 plane), per-unit header fields hoisted, sub-block loop fully
// unrolled so every shift and byte selector is an immediate, the two MMAs of a sub-block on independent
// accumulators.  Shared memory is addressed with 32-bit shared-space addresses and immediate offsets.
template <int OFF>
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
    uint32_t v;  // zero-extended into a 32-bit register
    asm volatile("ld.shared.u16 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
    return v;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}

__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}

struct Iq3sHdr {
    float d, d2;        // block scale and twice it: sub-block scale = d + d2 * s
    uint32_t qa0, qa1;  // bytes = this thread's codebook high bit for word 0 of sub-blocks 0..3 / 4..7 (0 or 1)
    uint32_t qb0, qb1;  // the same for word 1
    uint32_t sc;        // the eight 4-bit scales
};
// blk_t = shared address of the block + 2*t (the thread's qs pair); blk_s = shared address of the block + t (its sign byte)
__device__ __forceinline__ Iq3sHdr iq3s_hdr(uint32_t blk, int t) {
    Iq3sHdr h;
    h.d = h2f((uint16_t)lds_u16<0>(blk));
    h.d2 = h.d + h.d;
    const uint32_t q0 = (lds_u16<66>(blk) | (lds_u16<68>(blk) << 16)) >> (2 * t);
    const uint32_t q1 = (lds_u16<70>(blk) | (lds_u16<72>(blk) << 16)) >> (2 * t);
    h.qa0 = q0 & 0x01010101u;
    h.qb0 = (q0 >> 1) & 0x01010101u;
    h.qa1 = q1 & 0x01010101u;
    h.qb1 = (q1 >> 1) & 0x01010101u;
    h.sc = lds_u16<106>(blk) | (lds_u16<108>(blk) << 16);
    return h;
}
// Codebook index = qs byte | high bit << 8, assembled by one byte permute: byte 0 from qs, byte 1 = the 0/1 byte of
// the header word, bytes 2-3 = the upper bytes of the zero-extended 16-bit qs load (always zero).
template <int IB, int TS>  // TS = bytes between consecutive codebook entries (8 x copies)
__device__ __forceinline__ float iq3s_sub_h(uint32_t blk_t, uint32_t blk_s, const Iq3sHdr &h, uint32_t tabc, uint32_t (&w)[4]) {
    constexpr uint32_t k = IB & 3;
    constexpr uint32_t selA = (3u << 12) | (2u << 8) | ((4 + k) << 4) | 0;
    constexpr uint32_t selB = (3u << 12) | (2u << 8) | ((4 + k) << 4) | 1;
    const uint32_t qs = lds_u16<2 + 8 * IB>(blk_t);
    const uint32_t sg = lds_u8<74 + 4 * IB>(blk_s);
    const uint32_t i0 = __byte_perm(qs, IB < 4 ? h.qa0 : h.qa1, selA);
    const uint32_t i1 = __byte_perm(qs, IB < 4 ? h.qb0 : h.qb1, selB);
    const uint2 g0 = lds_v2(tabc + i0 * TS), g1 = lds_v2(tabc + i1 * TS);
    w[0] = g0.x ^ ((sg * 0x40008000u) & 0x80008000u);
    w[1] = g0.y ^ ((sg * 0x10002000u) & 0x80008000u);
    w[2] = g1.x ^ ((sg * 0x04000800u) & 0x80008000u);
    w[3] = g1.y ^ ((sg * 0x01000200u) & 0x80008000u);
    return fmaf(h.d2, (float)((h.sc >> (4 * IB)) & 15), h.d);
}

// Four registers that hold 0.0f and that the compiler cannot fold away: the C operand of each sub-block's first MMA
// (a literal zero would be re-materialised with moves in front of every MMA).
struct ZeroRegs {
    float z[4];
};
__device__ __forceinline__ ZeroRegs zero_regs() {
    ZeroRegs r;
    asm volatile("mov.f32 %0, 0f00000000;\n\tmov.f32 %1, 0f00000000;\n\tmov.f32 %2, 0f00000000;\n\tmov.f32 %3, 0f00000000;"
                 : "=f"(r.z[0]), "=f"(r.z[1]), "=f"(r.z[2]), "=f"(r.z[3]));
    return r;
}

template <bool BF16, int IB, int TS>
__device__ __forceinline__ void sub_mma1(uint32_t u0, uint32_t u1, int t, const Iq3sHdr &h0, const Iq3sHdr &h1, uint32_t tabc, const ZeroRegs &zr,
                                         const uint4 &xv, const uint4 &xl, float (&acc)[4]) {
    uint32_t wa[4], wb[4];
    const float dba = iq3s_sub_h<IB, TS>(u0 + 2 * t, u0 + t, h0, tabc, wa);
    const float dbb = iq3s_sub_h<IB, TS>(u1 + 2 * t, u1 + t, h1, tabc, wb);
    const uint32_t a0[4] = {wa[0], wb[0], wa[1], wb[1]};
    const uint32_t a1[4] = {wa[2], wb[2], wa[3], wb[3]};
    float p[4];
    if (BF16) {
        mma_bf16(p, a0, xv.x, xv.y, zr.z);
        mma_bf16(p, a1, xv.z, xv.w, p);
        mma_bf16(p, a0, xl.x, xl.y, p);
        mma_bf16(p, a1, xl.z, xl.w, p);
    } else {
        mma_f16(p, a0, xv.x, xv.y, zr.z);
        mma_f16(p, a1, xv.z, xv.w, p);
    }
    acc[0] = fmaf(dba, p[0], acc[0]);
    acc[1] = fmaf(dba, p[1], acc[1]);
    acc[2] = fmaf(dbb, p[2], acc[2]);
    acc[3] = fmaf(dbb, p[3], acc[3]);
}

// The same sub-block against an activation kept as two fp16 planes (value = high + low): four MMAs on one accumulator.
template <int IB, int TS>
__device__ __forceinline__ void sub_mma1_h2(uint32_t u0, uint32_t u1, int t, const Iq3sHdr &h0, const Iq3sHdr &h1, uint32_t tabc, const ZeroRegs &zr,
                                            const uint4 &xv, const uint4 &xl, float (&acc)[4]) {
    uint32_t wa[4], wb[4];
    const float dba = iq3s_sub_h<IB, TS>(u0 + 2 * t, u0 + t, h0, tabc, wa);
    const float dbb = iq3s_sub_h<IB, TS>(u1 + 2 * t, u1 + t, h1, tabc, wb);
    const uint32_t a0[4] = {wa[0], wb[0], wa[1], wb[1]};
    const uint32_t a1[4] = {wa[2], wb[2], wa[3], wb[3]};
    float p[4];
    mma_f16(p, a0, xv.x, xv.y, zr.z);
    mma_f16(p, a1, xv.z, xv.w, p);
    mma_f16(p, a0, xl.x, xl.y, p);
    mma_f16(p, a1, xl.z, xl.w, p);
    acc[0] = fmaf(dba, p[0], acc[0]);
    acc[1] = fmaf(dba, p[1], acc[1]);
    acc[2] = fmaf(dbb, p[2], acc[2]);
    acc[3] = fmaf(dbb, p[3], acc[3]);
}

// One IQ3_S unit (rows g and g+8 at shared addresses u0 / u1) against the cached B fragments of one column tile.
// d*(1+2s) is evaluated as fma(2d, s, d): both forms are exact products of a half-precision d and an odd integer
// below 32, so they give the same fp32 value.
template <bool BF16, int TS = 128>
__device__ __forceinline__ void unit_mma1(uint32_t u0, uint32_t u1, uint32_t tabc, int t, const ZeroRegs &zr, const uint4 (&xf)[8], const uint4 (&xl)[8],
                                          float (&acc)[4]) {
    const Iq3sHdr h0 = iq3s_hdr(u0, t), h1 = iq3s_hdr(u1, t);
    sub_mma1<BF16, 0, TS>(u0, u1, t, h0, h1, tabc, zr, xf[0], xl[0], acc);
    sub_mma1<BF16, 1, TS>(u0, u1, t, h0, h1, tabc, zr, xf[1], xl[1], acc);
    sub_mma1<BF16, 2, TS>(u0, u1, t, h0, h1, tabc, zr, xf[2], xl[2], acc);
    sub_mma1<BF16, 3, TS>(u0, u1, t, h0, h1, tabc, zr, xf[3], xl[3], acc);
    sub_mma1<BF16, 4, TS>(u0, u1, t, h0, h1, tabc, zr, xf[4], xl[4], acc);
    sub_mma1<BF16, 5, TS>(u0, u1, t, h0, h1, tabc, zr, xf[5], xl[5], acc);
    sub_mma1<BF16, 6, TS>(u0, u1, t, h0, h1, tabc, zr, xf[6], xl[6], acc);
    sub_mma1<BF16, 7, TS>(u0, u1, t, h0, h1, tabc, zr, xf[7], xl[7], acc);
}

// Two column tiles (16 tokens) against one decode of the unit (fp16 activations).
template <int IB, int TS>
__device__ __forceinline__ void sub_mma2(uint32_t u0, uint32_t u1, int t, const Iq3sHdr &h0, const Iq3sHdr &h1, uint32_t tabc, const ZeroRegs &zr,
                                         const uint4 &xa, const uint4 &xb, bool second, float (&acc)[2][4]) {
    uint32_t wa[4], wb[4];
    const float dba = iq3s_sub_h<IB, TS>(u0 + 2 * t, u0 + t, h0, tabc, wa);
    const float dbb = iq3s_sub_h<IB, TS>(u1 + 2 * t, u1 + t, h1, tabc, wb);
    const uint32_t a0[4] = {wa[0], wb[0], wa[1], wb[1]};
    const uint32_t a1[4] = {wa[2], wb[2], wa[3], wb[3]};
    float p[4];
    mma_f16(p, a0, xa.x, xa.y, zr.z);
    mma_f16(p, a1, xa.z, xa.w, p);
    acc[0][0] = fmaf(dba, p[0], acc[0][0]);
    acc[0][1] = fmaf(dba, p[1], acc[0][1]);
    acc[0][2] = fmaf(dbb, p[2], acc[0][2]);
    acc[0][3] = fmaf(dbb, p[3], acc[0][3]);
    if (second) {  // warp-uniform
        float r[4];
        mma_f16(r, a0, xb.x, xb.y, zr.z);
        mma_f16(r, a1, xb.z, xb.w, r);
        acc[1][0] = fmaf(dba, r[0], acc[1][0]);
        acc[1][1] = fmaf(dba, r[1], acc[1][1]);
        acc[1][2] = fmaf(dbb, r[2], acc[1][2]);
        acc[1][3] = fmaf(dbb, r[3], acc[1][3]);
    }
}
template <int TS>
__device__ __forceinline__ void unit_mma2(uint32_t u0, uint32_t u1, uint32_t tabc, int t, const ZeroRegs &zr, const uint4 (&xa)[8], const uint4 (&xb)[8],
                                          bool second, float (&acc)[2][4]) {
    const Iq3sHdr h0 = iq3s_hdr(u0, t), h1 = iq3s_hdr(u1, t);
    sub_mma2<0, TS>(u0, u1, t, h0, h1, tabc, zr, xa[0], xb[0], second, acc);
    sub_mma2<1, TS>(u0, u1, t, h0, h1, tabc, zr, xa[1], xb[1], second, acc);
    sub_mma2<2, TS>(u0, u1, t, h0, h1, tabc, zr, xa[2], xb[2], second, acc);
    sub_mma2<3, TS>(u0, u1, t, h0, h1, tabc, zr, xa[3], xb[3], second, acc);
    sub_mma2<4, TS>(u0, u1, t, h0, h1, tabc, zr, xa[4], xb[4], second, acc);
    sub_mma2<5, TS>(u0, u1, t, h0, h1, tabc, zr, xa[5], xb[5], second, acc);
    sub_mma2<6, TS>(u0, u1, t, h0, h1, tabc, zr, xa[6], xb[6], second, acc);
    sub_mma2<7, TS>(u0, u1, t, h0, h1, tabc, zr, xa[7], xb[7], second, acc);
}

// More than 16 tokens: the decoded A fragments of half a unit (four sub-blocks) stay in registers while the passes of 16 tokens
// run over them, so the unit is decoded once, not once per pass.  A column sees the same MMAs and the same scale products in the
// same sub-block order as in unit_mma2: results are bit-identical to the one-pass form.
struct UnitHalf {
    uint32_t a0[4][4], a1[4][4];  // A fragments of the two MMAs of sub-block i
    float da[4], db[4];           // sub-block scales of rows g and g + 8
};
template <int HF, int TS>
__device__ __forceinline__ void iq3s_decode_half(uint32_t u0, uint32_t u1, int t, const Iq3sHdr &h0, const Iq3sHdr &h1, uint32_t tabc, UnitHalf &A) {
    uint32_t wa[4], wb[4];
#define QW_HALF_SUB(I)                                                            \
    A.da[I] = iq3s_sub_h<4 * HF + I, TS>(u0 + 2 * t, u0 + t, h0, tabc, wa);       \
    A.db[I] = iq3s_sub_h<4 * HF + I, TS>(u1 + 2 * t, u1 + t, h1, tabc, wb);       \
    A.a0[I][0] = wa[0]; A.a0[I][1] = wb[0]; A.a0[I][2] = wa[1]; A.a0[I][3] = wb[1]; \
    A.a1[I][0] = wa[2]; A.a1[I][1] = wb[2]; A.a1[I][2] = wa[3]; A.a1[I][3] = wb[3];
    QW_HALF_SUB(0)
    QW_HALF_SUB(1)
    QW_HALF_SUB(2)
    QW_HALF_SUB(3)
#undef QW_HALF_SUB
}
// sub-block i of the half against the B fragments of two column tiles
__device__ __forceinline__ void half_mma(const UnitHalf &A, int i, const ZeroRegs &zr, const uint4 &xa, const uint4 &xb, bool second, float (&acc)[2][4]) {
    float p[4];
    mma_f16(p, A.a0[i], xa.x, xa.y, zr.z);
    mma_f16(p, A.a1[i], xa.z, xa.w, p);
    acc[0][0] = fmaf(A.da[i], p[0], acc[0][0]);
    acc[0][1] = fmaf(A.da[i], p[1], acc[0][1]);
    acc[0][2] = fmaf(A.db[i], p[2], acc[0][2]);
    acc[0][3] = fmaf(A.db[i], p[3], acc[0][3]);
    if (second) {  // warp-uniform
        float r[4];
        mma_f16(r, A.a0[i], xb.x, xb.y, zr.z);
        mma_f16(r, A.a1[i], xb.z, xb.w, r);
        acc[1][0] = fmaf(A.da[i], r[0], acc[1][0]);
        acc[1][1] = fmaf(A.da[i], r[1], acc[1][1]);
        acc[1][2] = fmaf(A.db[i], r[2], acc[1][2]);
        acc[1][3] = fmaf(A.db[i], r[3], acc[1][3]);
    }
}

// Q8_0 through the same shared-space path: unit = eight 34-byte blocks of a row (src/ggml_dq.c:34-37).  The thread's
// eight int8 values of block IB sit at byte 34*IB + 2 + 8t: 4-byte aligned for odd IB (two 32-bit loads), 2-byte aligned
// for even IB (four 16-bit loads).  (q ^ 0x80) | 0x6400 is the half 1024 + (q + 128); subtracting 1152 is exact.
template <int IB>
__device__ __forceinline__ float q8_sub_h(uint32_t row_t, uint32_t row, uint32_t (&w)[4]) {
    uint32_t lo, hi;
    if (IB & 1) {
        asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(lo) : "r"(row_t), "n"(34 * IB + 2));
        asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(hi) : "r"(row_t), "n"(34 * IB + 6));
    } else {
        lo = lds_u16<34 * IB + 2>(row_t) | (lds_u16<34 * IB + 4>(row_t) << 16);
        hi = lds_u16<34 * IB + 6>(row_t) | (lds_u16<34 * IB + 8>(row_t) << 16);
    }
    lo ^= 0x80808080u;
    hi ^= 0x80808080u;
    const uint32_t bias = 0x64806480u;
    const __half2 b2 = *(const __half2 *)&bias;
    const uint32_t v[4] = {__byte_perm(lo, 0x64646464u, 0x4140), __byte_perm(lo, 0x64646464u, 0x4342), __byte_perm(hi, 0x64646464u, 0x4140),
                           __byte_perm(hi, 0x64646464u, 0x4342)};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const __half2 r = __hsub2(*(const __half2 *)&v[j], b2);
        w[j] = *(const uint32_t *)&r;
    }
    return h2f((uint16_t)lds_u16<34 * IB>(row));
}
template <int IB>
__device__ __forceinline__ void sub_mma2_q8(uint32_t u0, uint32_t u1, int t, const ZeroRegs &zr, const uint4 &xa, const uint4 &xb, bool second,
                                            float (&acc)[2][4]) {
    uint32_t wa[4], wb[4];
    const float dba = q8_sub_h<IB>(u0 + 8 * t, u0, wa);
    const float dbb = q8_sub_h<IB>(u1 + 8 * t, u1, wb);
    const uint32_t a0[4] = {wa[0], wb[0], wa[1], wb[1]};
    const uint32_t a1[4] = {wa[2], wb[2], wa[3], wb[3]};
    float p[4];
    mma_f16(p, a0, xa.x, xa.y, zr.z);
    mma_f16(p, a1, xa.z, xa.w, p);
    acc[0][0] = fmaf(dba, p[0], acc[0][0]);
    acc[0][1] = fmaf(dba, p[1], acc[0][1]);
    acc[0][2] = fmaf(dbb, p[2], acc[0][2]);
    acc[0][3] = fmaf(dbb, p[3], acc[0][3]);
    if (second) {
        float r[4];
        mma_f16(r, a0, xb.x, xb.y, zr.z);
        mma_f16(r, a1, xb.z, xb.w, r);
        acc[1][0] = fmaf(dba, r[0], acc[1][0]);
        acc[1][1] = fmaf(dba, r[1], acc[1][1]);
        acc[1][2] = fmaf(dbb, r[2], acc[1][2]);
        acc[1][3] = fmaf(dbb, r[3], acc[1][3]);
    }
}
__device__ __forceinline__ void unit_mma2_q8(uint32_t u0, uint32_t u1, int t, const ZeroRegs &zr, const uint4 (&xa)[8], const uint4 (&xb)[8], bool second,
                                             float (&acc)[2][4]) {
    sub_mma2_q8<0>(u0, u1, t, zr, xa[0], xb[0], second, acc);
    sub_mma2_q8<1>(u0, u1, t, zr, xa[1], xb[1], second, acc);
    sub_mma2_q8<2>(u0, u1, t, zr, xa[2], xb[2], second, acc);
    sub_mma2_q8<3>(u0, u1, t, zr, xa[3], xb[3], second, acc);
    sub_mma2_q8<4>(u0, u1, t, zr, xa[4], xb[4], second, acc);
    sub_mma2_q8<5>(u0, u1, t, zr, xa[5], xb[5], second, acc);
    sub_mma2_q8<6>(u0, u1, t, zr, xa[6], xb[6], second, acc);
    sub_mma2_q8<7>(u0, u1, t, zr, xa[7], xb[7], second, acc);
}

// Q8_0 counterpart of iq3s_decode_half: blocks 4 HF .. 4 HF + 3 of the unit
template <int HF>
__device__ __forceinline__ void q8_decode_half(uint32_t u0, uint32_t u1, int t, UnitHalf &A) {
    uint32_t wa[4], wb[4];
#define QW_HALF_SUB(I)                                                            \
    A.da[I] = q8_sub_h<4 * HF + I>(u0 + 8 * t, u0, wa);                           \
    A.db[I] = q8_sub_h<4 * HF + I>(u1 + 8 * t, u1, wb);                           \
    A.a0[I][0] = wa[0]; A.a0[I][1] = wb[0]; A.a0[I][2] = wa[1]; A.a0[I][3] = wb[1]; \
    A.a1[I][0] = wa[2]; A.a1[I][1] = wb[2]; A.a1[I][2] = wa[3]; A.a1[I][3] = wb[3];
    QW_HALF_SUB(0)
    QW_HALF_SUB(1)
    QW_HALF_SUB(2)
    QW_HALF_SUB(3)
#undef QW_HALF_SUB
}

__host__ __device__ constexpr int unit_bytes(int GF) { return GF == 21 ? 110 : 272; }

}  // namespace qw
