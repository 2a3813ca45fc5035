/* CPU oracle for the batched decode step -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may load this
 * library.  The CUDA library never calls into it and has no CPU fallback.
 *
 * Every function restates, in plain C, arithmetic that the reference defines only in Metal or Python:
 *   - IQ3_S block decode      kernels/moe_iq.metal:102-118 (dq32<21>), table kernels/iq_tables.metal:292
 *                             (the table text comes from the gguf package, see oracle/gen_tables.py)
 *   - Q8_0 block decode       src/ggml_dq.c:34-37 (dq_q8_0), kernels/moe_iq.metal:200-205 (dq32<8>)
 *   - quantized matvec        kernels/qmv_gg.metal:17-39 (lane-strided 32-value segments, fp32, lane reduce)
 *   - router + top-k          kernels/moe_gg.metal:16-41 (row dot), :118-160 (top-k, ties -> lowest id,
 *                             softmax over the picked logits summed in rank order)
 * Parity pin: orc_dq_row is checked bit-for-bit against gguf.quants.dequantize (the arithmetic the
 * reference's own tools/dqtest.py:33-38 checks its kernels against) and, for Q8_0, against the
 * reference's own src/ggml_dq.c compiled into oracle/_ref (tests/test_oracle_pins.py).
 *
 * "canon" functions use one fixed fp32 evaluation order, written with fmaf() and explicit adds so the
 * C compiler cannot reassociate; the FMA CUDA kernels implement the same order with __fmaf_rn/__fadd_rn
 * and must match bit for bit.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static const uint32_t iq3s_grid[512] = {
#include "_gen/iq3s_grid.inc"
};

static inline float h2f(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

int orc_block_values(int type) { return type == 21 ? 256 : type == 8 ? 32 : 0; }
int orc_block_bytes(int type) { return type == 21 ? 110 : type == 8 ? 34 : 0; }
long orc_row_bytes(int type, int K) { return (long)(K / orc_block_values(type)) * orc_block_bytes(type); }

/* one 32-value segment `sub` of a row (kernels/moe_iq.metal:102-118 for IQ3_S, :200-205 for Q8_0) */
static void dq32(int type, const uint8_t *row, int sub, float *y) {
    if (type == 8) {
        const uint8_t *b = row + (size_t)sub * 34;
        const float d = h2f(rd16(b));
        for (int l = 0; l < 32; l++) y[l] = d * (float)(int8_t)b[2 + l];
        return;
    }
    const uint8_t *b = row + (size_t)(sub / 8) * 110;
    const int ib = sub % 8;
    const float d = h2f(rd16(b));
    const uint8_t *qs = b + 2 + 8 * ib, *signs = b + 2 + 64 + 8 + 4 * ib;
    const unsigned qh = b[2 + 64 + ib];
    const float db = d * (float)(1 + 2 * ((b[2 + 64 + 8 + 32 + ib / 2] >> (4 * (ib % 2))) & 15));
    for (int l = 0; l < 4; l++) {
        const uint32_t g1 = iq3s_grid[qs[2 * l] | ((qh << (8 - 2 * l)) & 256)];
        const uint32_t g2 = iq3s_grid[qs[2 * l + 1] | ((qh << (7 - 2 * l)) & 256)];
        const unsigned s = signs[l];
        for (int j = 0; j < 4; j++) {
            const float a = db * (float)((g1 >> (8 * j)) & 255), c = db * (float)((g2 >> (8 * j)) & 255);
            y[8 * l + j] = (s >> j) & 1 ? -a : a;
            y[8 * l + 4 + j] = (s >> (j + 4)) & 1 ? -c : c;
        }
    }
}

int orc_dq_row(int type, const uint8_t *src, float *dst, int K) {
    if (type != 21 && type != 8) return -1;
    for (int s = 0; s < K / 32; s++) dq32(type, src, s, dst + 32 * s);
    return 0;
}

int orc_dq_rows(int type, const uint8_t *W, int N, int K, float *out) {
    if (type != 21 && type != 8) return -1;
    const long rb = orc_row_bytes(type, K);
    for (int r = 0; r < N; r++) orc_dq_row(type, W + (size_t)r * rb, out + (size_t)r * K, K);
    return 0;
}

/* lane reduce used by every canon function: xor butterfly 16, 8, 4, 2, 1, all lanes updated together */
static float lane_reduce(float *v) {
    for (int off = 16; off; off >>= 1) {
        float t[32];
        for (int l = 0; l < 32; l++) t[l] = v[l] + v[l ^ off];
        memcpy(v, t, sizeof t);
    }
    return v[0];
}

/* Canonical-order quantized matvec.  Lane l owns segments l, l+32, ...; a segment's 32 products are
 * chained with fmaf from zero, the segment sum is added to the lane accumulator, lanes are reduced by
 * lane_reduce().  x is fp16 [B][xstride]; y is fp32 [B][ystride]. */
int orc_qmv_canon(int type, const uint8_t *W, int N, int K, const uint16_t *x, int B, int xstride, float *y, int ystride) {
    if (type != 21 && type != 8) return -1;
    const long rb = orc_row_bytes(type, K);
    float *xf = malloc(sizeof(float) * (size_t)B * K);
    for (int b = 0; b < B; b++)
        for (int k = 0; k < K; k++) xf[(size_t)b * K + k] = h2f(x[(size_t)b * xstride + k]);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        float *w = malloc(sizeof(float) * (size_t)K);
        orc_dq_row(type, W + (size_t)n * rb, w, K);
        for (int b = 0; b < B; b++) {
            float acc[32];
            for (int l = 0; l < 32; l++) {
                acc[l] = 0.0f;
                for (int s = l; s < K / 32; s += 32) {
                    float p = 0.0f;
                    for (int i = 0; i < 32; i++) p = fmaf(w[32 * s + i], xf[(size_t)b * K + 32 * s + i], p);
                    acc[l] = acc[l] + p;
                }
            }
            y[(size_t)b * ystride + n] = lane_reduce(acc);
        }
        free(w);
    }
    free(xf);
    return 0;
}

/* FP64 matvec of the exactly-decoded weights (the tolerance reference, tools/ggmtest.py:44) */
int orc_qmv_f64(int type, const uint8_t *W, int N, int K, const uint16_t *x, int B, int xstride, double *y, int ystride) {
    if (type != 21 && type != 8) return -1;
    const long rb = orc_row_bytes(type, K);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        float *w = malloc(sizeof(float) * (size_t)K);
        orc_dq_row(type, W + (size_t)n * rb, w, K);
        for (int b = 0; b < B; b++) {
            double a = 0;
            for (int k = 0; k < K; k++) a += (double)w[k] * (double)h2f(x[(size_t)b * xstride + k]);
            y[(size_t)b * ystride + n] = a;
        }
        free(w);
    }
    return 0;
}

/* CPU baseline for the timed comparison: decode a row to fp32 (what tools/dqcpu.c:19 does per row), then
 * a plain fp32-accumulate dot per token.  nthreads <= 0 uses every core.  Returns the thread count used. */
int orc_qmv_cpu(int type, const uint8_t *W, int N, int K, const float *xf, int B, float *y, int nthreads) {
    if (type != 21 && type != 8) return -1;
    const long rb = orc_row_bytes(type, K);
    int used = 1;
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
    used = nthreads;
#pragma omp parallel for schedule(static) num_threads(nthreads)
#endif
    for (int n = 0; n < N; n++) {
        float w[8192];
        float *wp = K <= 8192 ? w : malloc(sizeof(float) * (size_t)K);
        orc_dq_row(type, W + (size_t)n * rb, wp, K);
        for (int b = 0; b < B; b++) {
            float a = 0;
            const float *xb = xf + (size_t)b * K;
            for (int k = 0; k < K; k++) a += wp[k] * xb[k];
            y[(size_t)b * N + n] = a;
        }
        if (wp != w) free(wp);
    }
    return used;
}

/* Canonical-order router: fp16 weights [E][D], fp16 x [B][D] -> fp32 logits [B][ldl].  Lane l owns the
 * 8-value chunks l, l+32, ...; one running fmaf chain per lane; lane_reduce().  (kernels/moe_gg.metal:16-41) */
void orc_router_canon(const uint16_t *Wr, int E, int D, const uint16_t *x, int B, float *logits, int ldl) {
#pragma omp parallel for schedule(static)
    for (int e = 0; e < E; e++)
        for (int b = 0; b < B; b++) {
            float acc[32];
            for (int l = 0; l < 32; l++) {
                float a = 0.0f;
                for (int c = l; c < D / 8; c += 32)
                    for (int i = 0; i < 8; i++) a = fmaf(h2f(Wr[(size_t)e * D + 8 * c + i]), h2f(x[(size_t)b * D + 8 * c + i]), a);
                acc[l] = a;
            }
            logits[(size_t)b * ldl + e] = lane_reduce(acc);
        }
}

/* top-k of one token: repeated arg-max, equal values -> lowest expert id (kernels/moe_gg.metal:118, :140-149);
 * weights = softmax over the picked logits, exp summed in rank order (:153-156). */
void orc_topk(const float *lg, int E, int topk, int32_t *ids, float *w) {
    char *used = calloc((size_t)E, 1);
    float pk[64];
    for (int k = 0; k < topk; k++) {
        int bi = -1;
        float best = -INFINITY;
        for (int e = 0; e < E; e++)
            if (!used[e] && (bi < 0 || lg[e] > best)) { best = lg[e]; bi = e; }
        used[bi] = 1;
        ids[k] = bi;
        pk[k] = best;
    }
    float sm = 0.0f, ex[64];
    for (int k = 0; k < topk; k++) { ex[k] = expf(pk[k] - pk[0]); sm = sm + ex[k]; }
    for (int k = 0; k < topk; k++) w[k] = ex[k] / sm;
    free(used);
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
