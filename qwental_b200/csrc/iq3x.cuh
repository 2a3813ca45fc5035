// IQ3X: the expert weights of an IQ3_S model re-coded once, at load time, into the order and the bit layout the fused
// expert-FFN kernel consumes.  Lossless: every weight keeps its exact IQ3_S value d * (1 + 2 s) * (+-b), b in {1, 3, .., 15}
// (kernels/moe_iq.metal:102-118 in the reference); only the codebook lookup and the sign bits are resolved ahead of time, so
// that the step decodes a weight pair with one mask and one half-precision multiply-add instead of a shared-memory table
// lookup, an index assembly and a sign spread.  Cost: 136 bytes per 256 weights instead of 110 (4.25 bits per weight).
//
// A weight w = +-b is stored as the 4-bit code c = (w + 15) / 2.  A thread of the MMA layout (lane t of a row group, see
// qmv_core.cuh) owns the weights 8t .. 8t+7 of a 32-weight sub-block: one 32-bit word whose bit b(j) .. b(j)+3 (mod 32) hold
// the code of weight j, with b = 1, 17, 5, 21, 9, 25, 13, 29 for j = 0 .. 7 (the last code wraps around into bit 0).  The word
// and the word rotated right by 8, each masked with 0x001E001E / 0x01E001E0 and OR-ed with an fp16 exponent and a constant
// low bit (one three-input logic instruction), are fp16 pairs 1024 + (2c + 1) and 1024 + 16 (2c + 1); one multiply-add each
// gives the exact integers (w0, w1), (w2, w3), (w4, w5), (w6, w7) -- the four A registers of the sub-block's two MMAs.
//
// Row record (272 bytes = two super-blocks of one row; 272 = 16 mod 128, so the eight rows of a warp instruction fall
// into eight different groups of four shared-memory banks):
//     [0, 128)    codes of super-block A: sub-block ib at 16 ib, lane word t at + 4 t
//     [128, 256)  codes of super-block B
//     [256, 260)  d of A, d of B (fp16, as in the IQ3_S blocks)
//     [260, 268)  the four scale bytes of A, of B (two 4-bit scales per byte, as in the IQ3_S blocks)
//     [268, 272)  zero
// Stage = 128 row records (34 816 bytes), contiguous, in the order the kernel streams them:
//     gate/up of an expert   [tile gt of 64 intermediate indices][super-block pair kp][128 rows]: rows 0-63 = gate rows
//                            64 gt + r, rows 64-127 = the up rows of the same indices
//     down of an expert      [tile dt of 128 output rows][super-block pair kp][128 rows]: position 16 q + g holds output row
//                            128 dt + 16 q + 2 g, position 16 q + 8 + g holds row 128 dt + 16 q + 2 g + 1 (the two MMA rows of
//                            a lane are then neighbouring output rows: one 8-byte store)
#pragma once
#include "common.cuh"

namespace qw {

constexpr int IQ3X_REC = 272;                 // bytes of a row record
constexpr int IQ3X_STAGE = 128 * IQ3X_REC;    // bytes of a stage

// position of a weight of the lane word: weight j (0..7) -> bit offset of its code (the code of weight 7 wraps: bits 29, 30, 31, 0)
__host__ __device__ constexpr int iq3x_bit(int j) { return 1 + 16 * (j & 1) + 4 * (j >> 1); }
__host__ __device__ inline uint32_t iq3x_put(uint32_t c, int j) { return (c << iq3x_bit(j)) | (c >> (32 - iq3x_bit(j))); }  // rotate left

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {  // (a & b) | c in one instruction
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// the lane word's eight codes as four packed fp16 pairs of exact integers (w0,w1) (w2,w3) (w4,w5) (w6,w7)
__device__ __forceinline__ void iq3x_word(uint32_t q, uint32_t (&w)[4]) {
    const uint32_t r = __funnelshift_r(q, q, 8);  // rotate right by 8
    const uint32_t h0 = lop3_and_or(q, 0x001E001Eu, 0x64016401u), h1 = lop3_and_or(q, 0x01E001E0u, 0x64106410u);
    const uint32_t h2 = lop3_and_or(r, 0x001E001Eu, 0x64016401u), h3 = lop3_and_or(r, 0x01E001E0u, 0x64106410u);
    const __half2 m0 = __floats2half2_rn(1.0f, 1.0f), a0 = __floats2half2_rn(-1040.0f, -1040.0f);
    const __half2 m1 = __floats2half2_rn(0.0625f, 0.0625f), a1 = __floats2half2_rn(-80.0f, -80.0f);
    const __half2 v0 = __hfma2(*(const __half2 *)&h0, m0, a0), v1 = __hfma2(*(const __half2 *)&h1, m1, a1);
    const __half2 v2 = __hfma2(*(const __half2 *)&h2, m0, a0), v3 = __hfma2(*(const __half2 *)&h3, m1, a1);
    w[0] = *(const uint32_t *)&v0;
    w[1] = *(const uint32_t *)&v1;
    w[2] = *(const uint32_t *)&v2;
    w[3] = *(const uint32_t *)&v3;
}

}  // namespace qw
