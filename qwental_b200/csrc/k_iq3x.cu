// IQ3X (see iq3x.cuh): the one-time re-coding of IQ3_S expert matrices for the fused expert-FFN kernel, and a decoder of
// the re-coded form used by the parity tests.
//   iq3x_pack      IQ3_S rows -> stage-ordered IQ3X records (mode 0: gate + up of every expert, mode 1: down)
//   iq3x_dq_test   IQ3X (down order) -> fp32 rows, in the arithmetic of the IQ3_S decoder (db = d * (1 + 2 s); value = db * b,
//                  negated where the sign bit is set: kernels/moe_iq.metal:102-118), so that "pack, then decode" can be held
//                  bit for bit against the decode of the original blocks
#include "iq3x.cuh"
#include "qw_kern.h"

using namespace qw;

struct iq3x_pack_args {
    uint32_t mode, experts, I, D;  // mode 0: A = gate, B = up ([experts][I][D/256*110] each); mode 1: A = down [experts][D][I/256*110]
};

// One thread per (record, super-block of the pair).
__global__ void __launch_bounds__(256) iq3x_pack_k(const uint8_t *A, const uint8_t *B, uint8_t *dst, iq3x_pack_args a, const uint32_t *grid, uint64_t total) {
    pdl_sync();
    const uint64_t id = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (id >= total) return;
    const uint32_t kh = (uint32_t)(id & 1);
    const uint64_t rec = id >> 1;
    const uint32_t pos = (uint32_t)(rec % 128);
    const uint32_t K = a.mode == 0 ? a.D : a.I, KP = K / 512, T = a.mode == 0 ? a.I / 64 : a.D / 128;
    const uint64_t st = rec / 128;
    const uint32_t kp = (uint32_t)(st % KP), tile = (uint32_t)((st / KP) % T), e = (uint32_t)(st / KP / T);
    const uint32_t rb = K / 256 * 110, sb = 2 * kp + kh;
    const uint8_t *src;
    if (a.mode == 0) {
        const uint32_t row = tile * 64 + (pos & 63);
        src = (pos < 64 ? A : B) + ((size_t)e * a.I + row) * rb + (size_t)sb * 110;
    } else {
        const uint32_t q = pos >> 4, rem = pos & 15, row = tile * 128 + 16 * q + 2 * (rem & 7) + (rem >> 3);
        src = A + ((size_t)e * a.D + row) * rb + (size_t)sb * 110;
    }
    uint8_t *out = dst + rec * IQ3X_REC;
    uint32_t *codes = (uint32_t *)(out + kh * 128);
    for (int ib = 0; ib < 8; ib++) {
        const uint32_t qh = src[66 + ib];
        for (int t = 0; t < 4; t++) {
            const uint32_t g1 = grid[src[2 + 8 * ib + 2 * t] | ((qh << (8 - 2 * t)) & 256)];
            const uint32_t g2 = grid[src[2 + 8 * ib + 2 * t + 1] | ((qh << (7 - 2 * t)) & 256)];
            const uint32_t sg = src[74 + 4 * ib + t];
            uint32_t word = 0;
            for (int j = 0; j < 8; j++) {
                const uint32_t b = ((j < 4 ? g1 : g2) >> (8 * (j & 3))) & 255;  // 1, 3, .., 15
                const uint32_t c = (sg >> j) & 1 ? (15 - b) / 2 : (15 + b) / 2;
                word |= iq3x_put(c, j);
            }
            codes[ib * 4 + t] = word;
        }
    }
    out[256 + 2 * kh] = src[0];
    out[257 + 2 * kh] = src[1];
    for (int i = 0; i < 4; i++) out[260 + 4 * kh + i] = src[106 + i];
    if (kh == 0) *(uint32_t *)(out + 268) = 0;
}

// binds: 0 = A, 1 = B (mode 0 only), 2 = dst, 3 = iq3x_pack_args
static cudaError_t launch_iq3x_pack(const QwLaunch &L) {
    const iq3x_pack_args a = L.bytes<iq3x_pack_args>(3);
    QW_CHECK_ARG(L.has_bytes(3, 16) && a.mode <= 1 && a.experts >= 1 && a.I >= 64 && a.D >= 128);
    QW_CHECK_ARG(a.mode == 0 ? (a.D % 512 == 0 && a.I % 64 == 0) : (a.I % 512 == 0 && a.D % 128 == 0));
    const uint32_t K = a.mode == 0 ? a.D : a.I, N = a.mode == 0 ? a.I : a.D;
    const size_t src_bytes = (size_t)a.experts * N * (K / 256 * 110);
    const uint64_t stages = (uint64_t)a.experts * (a.mode == 0 ? a.I / 64 : a.D / 128) * (K / 512);
    QW_CHECK_ARG(L.buf<void>(0) && L.buf<void>(2) && L.avail(0) >= src_bytes && L.avail(2) >= stages * IQ3X_STAGE && ((uintptr_t)L.buf<void>(2) & 15) == 0);
    if (a.mode == 0) QW_CHECK_ARG(L.buf<void>(1) && L.avail(1) >= src_bytes);
    const uint64_t total = stages * 128 * 2;
    QW_CHECK_ARG((total + 255) / 256 < 0x7fffffffull);
    qw_launch(iq3x_pack_k, (unsigned)((total + 255) / 256), 256, 0, L.stream, L.buf<uint8_t>(0), a.mode == 0 ? L.buf<uint8_t>(1) : nullptr, L.buf<uint8_t>(2), a,
              ((const QwTables *)L.tables)->grid_u32, total);
    return cudaGetLastError();
}
QW_FAMILY(iq3x_pack, launch_iq3x_pack, 256)

// One thread per (output row, super-block): dst fp32 [rows][K] from the down order of one matrix.
__global__ void __launch_bounds__(128) iq3x_dq_test_k(const uint8_t *src, float *y, uint32_t rows, uint32_t K) {
    pdl_sync();
    const uint32_t id = blockIdx.x * 128 + threadIdx.x, nsb = K / 256;
    if (id >= rows * nsb) return;
    const uint32_t row = id / nsb, sb = id % nsb, kp = sb >> 1, kh = sb & 1;
    const uint32_t tile = row / 128, r = row % 128, q = r >> 4, g2 = r & 15, pos = 16 * q + (g2 >> 1) + 8 * (g2 & 1);
    const uint8_t *rec = src + (((size_t)tile * (K / 512) + kp) * 128 + pos) * IQ3X_REC;
    const float d = h2f(ldu16(rec + 256 + 2 * kh));
    for (int ib = 0; ib < 8; ib++) {
        const uint32_t s = (rec[260 + 4 * kh + (ib >> 1)] >> (4 * (ib & 1))) & 15;
        const float db = __fmul_rn(d, (float)(1 + 2 * (int)s));
        for (int t = 0; t < 4; t++) {
            uint32_t w[4];
            iq3x_word(*(const uint32_t *)(rec + kh * 128 + ib * 16 + t * 4), w);
            for (int j = 0; j < 8; j++) {
                const __half hv = __ushort_as_half((uint16_t)(w[j >> 1] >> (16 * (j & 1))));
                y[(size_t)row * K + sb * 256 + ib * 32 + 8 * t + j] = __fmul_rn(db, __half2float(hv));
            }
        }
    }
}

// binds: 0 = IQ3X (down order, one matrix), 1 = y fp32 [rows][K], 2 = {rows, K}
static cudaError_t launch_iq3x_dq_test(const QwLaunch &L) {
    struct { uint32_t rows, K; } a = L.bytes<decltype(a)>(2);
    QW_CHECK_ARG(L.has_bytes(2, 8) && a.rows % 128 == 0 && a.K % 512 == 0 && a.rows >= 128 && L.buf<void>(0) && L.buf<void>(1));
    QW_CHECK_ARG(L.avail(0) >= (size_t)(a.rows / 128) * (a.K / 512) * IQ3X_STAGE && L.avail(1) >= (size_t)a.rows * a.K * 4);
    const uint32_t n = a.rows * (a.K / 256);
    qw_launch(iq3x_dq_test_k, (n + 127) / 128, 128, 0, L.stream, L.buf<uint8_t>(0), L.buf<float>(1), a.rows, a.K);
    return cudaGetLastError();
}
QW_FAMILY(iq3x_dq_test, launch_iq3x_dq_test, 128)
