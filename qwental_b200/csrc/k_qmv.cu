// Dense batched quantized matvec for GGML IQ3_S (type 21) and Q8_0 (type 8) weights.
//
//   dq_test   decode rows to fp32                      -- role of dq_test, kernels/moe_iq.metal:208-217
//   qmv_gg    fp32 FMA matvec in one fixed order       -- role of qmv_gg,  kernels/qmv_gg.metal:17-39
//   qmv_mma   tensor-core matvec, raw blocks staged by bulk (TMA) copies, one weight pass for up to 64 tokens
//             -- replaces qmv / qmvb / qmv_gg / qmv_ggm for the batched step (src/engine.c:689-769, 5363-5423)
//
// Bind slots follow the reference's qmv_gg (kernels/qmv_gg.metal:18-19): 0 = W, 3 = x (fp16), 4 = y,
// 5 = {N, xstride, ystride, nb} (nb = number of tokens; 0 means the NB define).  Defines: GF (21 | 8),
// KD (K), NB (max tokens), YT_F32 (1: fp32 output, else fp16).
#include "qmv_core.cuh"
#include "qw_kern.h"

using namespace qw;

struct qmv_args {
    uint32_t N, xstride, ystride, nb;
};

// ------------------------------------------------------------------------------------------------ exact decode
// One 32-value segment in the oracle's order: db = d*(1+2*scale), value = +-(db * codebook byte).
template <int GF>
__device__ __forceinline__ void dq32(const uint8_t *row, int sub, float *y, const uint32_t *grid) {
    if (GF == 8) {
        const uint8_t *b = row + (size_t)sub * 34;
        const float d = h2f(ldu16(b));
#pragma unroll
        for (int l = 0; l < 32; l++) y[l] = __fmul_rn(d, (float)(int8_t)b[2 + l]);
        return;
    }
    const uint8_t *b = row + (size_t)(sub >> 3) * 110;
    const int ib = sub & 7;
    const float d = h2f(ldu16(b));
    const uint32_t qh = b[66 + ib];
    const float db = __fmul_rn(d, (float)(1 + 2 * ((b[106 + (ib >> 1)] >> (4 * (ib & 1))) & 15)));
#pragma unroll
    for (int l = 0; l < 4; l++) {
        const uint32_t g1 = __ldg(grid + (b[2 + 8 * ib + 2 * l] | ((qh << (8 - 2 * l)) & 256)));
        const uint32_t g2 = __ldg(grid + (b[2 + 8 * ib + 2 * l + 1] | ((qh << (7 - 2 * l)) & 256)));
        const uint32_t s = b[74 + 4 * ib + l];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float a = __fmul_rn(db, (float)((g1 >> (8 * j)) & 255)), c = __fmul_rn(db, (float)((g2 >> (8 * j)) & 255));
            y[8 * l + j] = (s >> j) & 1 ? -a : a;
            y[8 * l + 4 + j] = (s >> (j + 4)) & 1 ? -c : c;
        }
    }
}

// grid: rows x 32 threads; bytes(2) = {K, row bytes}
template <int GF>
__global__ void dq_test_k(const uint8_t *W, float *y, uint32_t K, uint32_t rb, const uint32_t *grid) {
    pdl_sync();
    const uint32_t r = blockIdx.x, lane = threadIdx.x;
    float v[32];
    for (uint32_t s = lane; s < K / 32; s += 32) {
        dq32<GF>(W + (size_t)r * rb, s, v, grid);
        for (int i = 0; i < 32; i++) y[(size_t)r * K + 32 * s + i] = v[i];
    }
}

static cudaError_t launch_dq_test(const QwLaunch &L) {
    const int gf = (int)L.def("DQ_TEST", L.def("GF", 21));
    struct { uint32_t K, rb; } a = L.bytes<decltype(a)>(2);
    QW_CHECK_ARG(L.buf<uint8_t>(0) && L.buf<float>(1) && a.K % 32 == 0 && L.tx == 32);
    QW_CHECK_ARG((gf == 21 && a.K % 256 == 0) || gf == 8);
    QW_CHECK_ARG(L.avail(0) >= (size_t)L.gx * a.rb && L.avail(1) >= (size_t)L.gx * a.K * 4);
    const uint32_t *grid = ((const QwTables *)L.tables)->grid_u32;
    if (gf == 21) qw_launch(dq_test_k<21>, L.gx, 32, 0, L.stream, L.buf<uint8_t>(0), L.buf<float>(1), a.K, a.rb, grid);
    else qw_launch(dq_test_k<8>, L.gx, 32, 0, L.stream, L.buf<uint8_t>(0), L.buf<float>(1), a.K, a.rb, grid);
    return cudaGetLastError();
}
QW_FAMILY(dq_test, launch_dq_test, 32)

// ------------------------------------------------------------------------------------------------ FMA matvec, canonical order
// One warp per row; lane owns segments lane, lane+32, ...; a segment's 32 products are chained with fma from
// zero and added to the lane accumulator; lanes are reduced by the xor butterfly.  Bit-exact against the CPU
// oracle.  Tokens are processed 8 at a time (the decoded segment is reused for the 8).
template <int GF, bool F32OUT>
__global__ void __launch_bounds__(256) qmv_gg_k(const uint8_t *W, const __half *x, void *y, qmv_args a, uint32_t K, uint32_t rb, const uint32_t *grid) {
    pdl_sync();
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= a.N) return;
    const uint8_t *wr = W + (size_t)row * rb;
    for (uint32_t b0 = 0; b0 < a.nb; b0 += 8) {
        float acc[8];
#pragma unroll
        for (int b = 0; b < 8; b++) acc[b] = 0.f;
        for (uint32_t s = lane; s < K / 32; s += 32) {
            float v[32];
            dq32<GF>(wr, s, v, grid);
#pragma unroll
            for (int b = 0; b < 8; b++) {
                if (b0 + b >= a.nb) continue;
                const uint4 *xp = (const uint4 *)(x + (size_t)(b0 + b) * a.xstride + 32 * s);
                float p = 0.f;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint4 q = __ldcg(xp + i);
                    const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float2 f = __half22float2(*(const __half2 *)&w4[j]);
                        p = __fmaf_rn(v[8 * i + 2 * j], f.x, p);
                        p = __fmaf_rn(v[8 * i + 2 * j + 1], f.y, p);
                    }
                }
                acc[b] = __fadd_rn(acc[b], p);
            }
        }
#pragma unroll
        for (int b = 0; b < 8; b++) {
            if (b0 + b >= a.nb) continue;
            const float t = warp_sum_canon(acc[b]);
            if (lane == 0) {
                if (F32OUT) ((float *)y)[(size_t)(b0 + b) * a.ystride + row] = t;
                else ((__half *)y)[(size_t)(b0 + b) * a.ystride + row] = __float2half_rn(t);
            }
        }
    }
}

static bool qmv_common_check(const QwLaunch &L, qmv_args &a, int &gf, uint32_t &K, uint32_t &rb, bool &f32) {
    gf = (int)L.def("GF", 21);
    K = (uint32_t)L.def("KD", 0);
    f32 = L.def("YT_F32", 0) != 0;
    a = L.bytes<qmv_args>(5);
    if (a.nb == 0) a.nb = (uint32_t)L.def("NB", 1);
    if (!(gf == 21 || gf == 8) || K == 0 || K % 256 != 0) return false;
    rb = gf == 21 ? K / 256 * 110 : K / 32 * 34;
    if (!L.buf<uint8_t>(0) || !L.buf<__half>(3) || !L.buf<void>(4) || !L.has_bytes(5, 12)) return false;
    if (a.nb == 0 || a.nb > 64 || a.N == 0 || a.xstride < K || a.xstride % 8 != 0 || a.ystride < a.N) return false;
    if (((uintptr_t)L.buf<__half>(3) & 15) != 0) return false;
    if (L.avail(0) < (size_t)a.N * rb) return false;
    if (L.avail(3) < ((size_t)(a.nb - 1) * a.xstride + K) * 2) return false;
    if (L.avail(4) < ((size_t)(a.nb - 1) * a.ystride + a.N) * (f32 ? 4 : 2)) return false;
    return true;
}

static cudaError_t launch_qmv_gg(const QwLaunch &L) {
    qmv_args a;
    int gf;
    uint32_t K, rb;
    bool f32;
    QW_CHECK_ARG(qmv_common_check(L, a, gf, K, rb, f32));
    QW_CHECK_ARG(L.tx == 256 && L.gx == (a.N + 7) / 8);
    const uint32_t *grid = ((const QwTables *)L.tables)->grid_u32;
    const uint8_t *W = L.buf<uint8_t>(0);
    const __half *x = L.buf<__half>(3);
    void *y = L.buf<void>(4);
#define GO(G, F) qw_launch(qmv_gg_k<G, F>, L.gx, 256, 0, L.stream, W, x, y, a, K, rb, grid)
    if (gf == 21) { if (f32) GO(21, true); else GO(21, false); }
    else { if (f32) GO(8, true); else GO(8, false); }
#undef GO
    return cudaGetLastError();
}
QW_FAMILY(qmv_gg, launch_qmv_gg, 256)

// ------------------------------------------------------------------------------------------------ tensor-core matvec
// Persistent blocks of 8 warps.  An item is a tile of 16*MT rows; the whole tile (full K, rows are contiguous)
// is brought into shared memory by one bulk copy per pipeline stage.  Warp w = (m-tile w / KS, K-slice w % KS)
// walks the units u = ks, ks + KS, ... of its 16 rows; the KS partial tiles of an m-tile are summed in slice
// order 0..KS-1 through shared memory, so the order never depends on the batch.
struct QmvMmaP {
    const uint8_t *W;
    const __half *x;
    void *y;
    const QwTables *tab;
    unsigned *status;
    uint32_t N, K, rb, xstride, ystride, nb, items;
    uint32_t rs;  // qmv_mma2: distance of the rows of a staged tile in shared memory (rb plus padding against bank conflicts)
    // qmv_mma2 with EPX defined: the fp16 output rows are stored into the buffer of every rank (peer memory) and the kernel
    // publishes afterwards -- the all-gather of a projection that every rank runs for its own slots only
    void *yR[8];
    EpPeers ep;  // ep.nranks <= 1: plain local output
};

constexpr int QMV_STAGES = 3;

template <int GF, int NT, int MT, bool F32OUT>
__global__ void __launch_bounds__(256) qmv_mma_k(const QmvMmaP p) {
    constexpr int KS = 8 / MT;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = (uint64_t *)smem;                         // QMV_STAGES full barriers
    uint2 *tab = (uint2 *)(smem + 64);                         // 512 x 8 B codebook (IQ3_S only)
    float4 *red = (float4 *)(smem + 64 + 4096);                // [8 warps][NT][32]
    uint8_t *stage0 = smem + 64 + 4096 + 8 * NT * 32 * 16;
    const uint32_t tile_bytes = 16 * MT * p.rb;
    const uint32_t stage_stride = (tile_bytes + 127) & ~127u;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int mt = warp / KS, ks = warp % KS;

    if (tid == 0) {
        for (int s = 0; s < QMV_STAGES; s++) mbar_init(&bars[s], 1);
        mbar_init_fence();
    }
    if (GF == 21)
        for (int e = tid; e < 512; e += 256) tab[e] = p.tab->grid_h4[e * 16];
    __syncthreads();

    const uint32_t first = blockIdx.x, step = gridDim.x;
    auto issue = [&](uint32_t j) {  // thread 0 only: item number j of this block into stage j % STAGES
        const uint32_t item = first + j * step;
        if (item >= p.items) return;
        const int s = j % QMV_STAGES;
        mbar_expect_tx(&bars[s], tile_bytes);
        bulk_g2s(stage0 + (size_t)s * stage_stride, p.W + (size_t)item * tile_bytes, tile_bytes, &bars[s]);
    };
    if (tid == 0)
        for (uint32_t j = 0; j < QMV_STAGES - 1; j++) issue(j);

    pdl_sync();  // the weight tiles above do not depend on earlier kernels; the activations and the output do
    // activation rows of this lane's columns
    const uint4 *xcol[NT], *xlo[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const uint32_t col = g + 8 * nt;
        xcol[nt] = col < p.nb ? (const uint4 *)(p.x + (size_t)col * p.xstride) : nullptr;
        xlo[nt] = nullptr;
    }
    const GridTab<1> gt{tab, 0};
    const uint32_t tile_on = tiles_on<NT>(xcol);
    const int units = p.K / 256;
    bool ok = true;

    for (uint32_t j = 0;; j++) {
        const uint32_t item = first + j * step;
        if (item >= p.items) break;
        if (tid == 0) issue(j + QMV_STAGES - 1);
        const int s = j % QMV_STAGES;
        if (!mbar_wait(&bars[s], (j / QMV_STAGES) & 1)) {
            ok = false;
            break;
        }
        const uint8_t *tile = stage0 + (size_t)s * stage_stride + (size_t)(16 * mt) * p.rb;
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        for (int u = ks; u < units; u += KS)
            unit_mma<GF, NT, 1, false>(tile + (size_t)g * p.rb + (size_t)u * unit_bytes(GF), tile + (size_t)(g + 8) * p.rb + (size_t)u * unit_bytes(GF),
                                       gt, t, xcol, xlo, tile_on, u * 32, acc);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) red[(warp * NT + nt) * 32 + lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
        __syncthreads();  // partial tiles visible; every warp is done reading stage s
        // reduce over the KS slices of each m-tile in slice order, then store
        for (int e = tid; e < MT * NT * 32 * 4; e += 256) {
            const int jj = e & 3, ln = (e >> 2) & 31, nt = (e >> 7) % NT, m = (e >> 7) / NT;
            float sum = 0.f;
#pragma unroll
            for (int k2 = 0; k2 < KS; k2++) sum += ((const float *)&red[((m * KS + k2) * NT + nt) * 32 + ln])[jj];
            const uint32_t row = item * 16 * MT + m * 16 + (ln >> 2) + 8 * (jj >> 1);
            const uint32_t col = nt * 8 + 2 * (ln & 3) + (jj & 1);
            if (col < p.nb && row < p.N) {
                if (F32OUT) ((float *)p.y)[(size_t)col * p.ystride + row] = sum;
                else ((__half *)p.y)[(size_t)col * p.ystride + row] = __float2half_rn(sum);
            }
        }
        __syncthreads();  // red may be overwritten, stage s may be refilled
    }
    if (!ok && lane == 0) set_status(p.status, ST_MBAR_TIMEOUT | 1);
}

template <int GF, int NT, int MT, bool F32OUT>
static cudaError_t qmv_mma_go(const QmvMmaP &p, int sm_count, cudaStream_t st) {
    const uint32_t tile_bytes = 16 * MT * p.rb;
    const size_t smem = 64 + 4096 + (size_t)8 * NT * 32 * 16 + (size_t)QMV_STAGES * ((tile_bytes + 127) & ~127u);
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    auto k = qmv_mma_k<GF, NT, MT, F32OUT>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int occ = 1;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k, 256, smem);
    if (e != cudaSuccess) return e;
    if (occ < 1) occ = 1;
    if (occ > 4) occ = 4;
    const uint32_t cap = (uint32_t)(sm_count * occ);
    const uint32_t grid = p.items < cap ? p.items : cap;
    qw_launch(k, grid, 256, smem, st, p);
    return cudaGetLastError();
}

template <int GF, int MT, bool F32OUT>
static cudaError_t qmv_mma_nt(const QmvMmaP &p, int sm, cudaStream_t st) {
    if (p.nb <= 8) return qmv_mma_go<GF, 1, MT, F32OUT>(p, sm, st);
    if (p.nb <= 16) return qmv_mma_go<GF, 2, MT, F32OUT>(p, sm, st);
    if (p.nb <= 32) return qmv_mma_go<GF, 4, MT, F32OUT>(p, sm, st);
    return qmv_mma_go<GF, 8, MT, F32OUT>(p, sm, st);
}

// ---- Variant used for the dense projections: a team of WARPS warps per 16-row tile, one warp per 256-K unit (8 warps
// at K = 2048, 16 at K = 4096); TEAMS teams share one block (and, for IQ3_S, one conflict-free 16-copy codebook of 64 KB
// that arrives by a bulk copy while the activations are loaded).  The activations' B fragments of up to 16 tokens stay
// in registers for the whole kernel.  More than 16 tokens run as passes of 16 over the staged tile: the MP form decodes half
// a unit into A fragments once and runs all passes over them, fetching the B fragments per pass.
template <int N>
__device__ __forceinline__ void team_bar(int id) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(N) : "memory");
}
template <int GF, int WARPS, int TEAMS, bool F32OUT, bool MP>
__global__ void __launch_bounds__(WARPS * TEAMS * 32, (WARPS * TEAMS == 8) ? 2 : 1) qmv_mma2_k(const QmvMmaP p) {
    constexpr int NT = 2, TS = 128, STG = GF == 8 ? 2 : QMV_STAGES, UB = GF == 21 ? 110 : 272, TABB = GF == 21 ? 65536 : 0;
    constexpr int TT = WARPS * 32;  // threads of a team
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = (uint64_t *)smem;  // [team][STG], then the table's
    uint2 *tab = (uint2 *)(smem + 128);
    const uint32_t tile_bytes = 16 * p.rb, stage_stride = (16 * p.rs + 127) & ~127u;
    const int tid = threadIdx.x, team = tid / TT, tt = tid % TT, warp = tt >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    float4 *red = (float4 *)(smem + 128 + TABB) + team * 2 * WARPS * NT * 32;  // [2][WARPS][NT][32] per team
    uint8_t *stage0 = smem + 128 + TABB + TEAMS * 2 * WARPS * NT * 32 * 16 + (size_t)team * STG * stage_stride;
    uint64_t *full = bars + team * STG;
    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < TEAMS * STG + 1; s++) mbar_init(&bars[s], 1);
        mbar_init_fence();
        if (GF == 21) {
            mbar_expect_tx(&bars[TEAMS * STG], TABB);
            bulk_g2s(tab, p.tab->grid_h4, TABB, &bars[TEAMS * STG]);
        }
    }
    __syncthreads();
    const uint32_t first = blockIdx.x * TEAMS + team, step = gridDim.x * TEAMS;
    auto issue = [&](uint32_t j) {
        const uint32_t item = first + j * step;
        if (item >= p.items) return;
        const int s = j % STG;
        mbar_expect_tx(&full[s], tile_bytes);
        if (p.rs == p.rb) bulk_g2s(stage0 + (size_t)s * stage_stride, p.W + (size_t)item * tile_bytes, tile_bytes, &full[s]);
        else  // one copy per row, so that the rows land rs bytes apart
            for (uint32_t r = 0; r < 16; r++)
                bulk_g2s(stage0 + (size_t)s * stage_stride + r * p.rs, p.W + (size_t)item * tile_bytes + (size_t)r * p.rb, p.rb, &full[s]);
    };
    if (tt == 0)
        for (uint32_t j = 0; j < STG - 1; j++) issue(j);
    const uint32_t tabc = smem_u32(tab) + (lane & 15) * 8;
    const ZeroRegs zr = zero_regs();
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint4 xf[NT][8];
    auto load_x = [&](uint32_t c0) {  // columns c0 + g and c0 + 8 + g of this warp's unit
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint32_t col = c0 + g + 8 * nt;
            const uint4 *xr = (const uint4 *)(p.x + (size_t)col * p.xstride) + warp * 32 + t;
#pragma unroll
            for (int ib = 0; ib < 8; ib++) xf[nt][ib] = col < p.nb ? __ldcg(xr + 4 * ib) : zero;
        }
    };
    pdl_wait();  // weight tiles and the codebook are static; the activations (and the output buffer) are not
    if (!MP) load_x(0);
    bool ok = GF == 21 ? mbar_wait(&bars[TEAMS * STG], 0) : true;
    const uint32_t passes = (p.nb + 15) / 16;
    uint32_t rb_i = 0;  // alternating reduce buffer
    for (uint32_t j = 0; ok; j++) {
        const uint32_t item = first + j * step;
        if (item >= p.items) break;
        if (tt == 0) issue(j + STG - 1);
        const int s = j % STG;
        if (!mbar_wait(&full[s], (j / STG) & 1)) {
            ok = false;
            break;
        }
        const uint32_t rows = smem_u32(stage0) + s * stage_stride + g * p.rs + warp * UB;
        if constexpr (MP) {
            // more than 16 tokens: decode half a unit once, run every pass of 16 tokens over it (bit-identical to the loop below)
            float accp[4][NT][4];
#pragma unroll
            for (int ps = 0; ps < 4; ps++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++) accp[ps][nt][0] = accp[ps][nt][1] = accp[ps][nt][2] = accp[ps][nt][3] = 0.f;
            auto run_half = [&](const UnitHalf &A, int hf) {
#pragma unroll
                for (int ps = 0; ps < 4; ps++) {
                    if ((uint32_t)ps >= passes) break;  // warp-uniform
                    const uint32_t ca = ps * 16 + g, cb = ca + 8;
                    const uint4 *xa = (const uint4 *)(p.x + (size_t)ca * p.xstride) + warp * 32 + t + 16 * hf;
                    const uint4 *xb = (const uint4 *)(p.x + (size_t)cb * p.xstride) + warp * 32 + t + 16 * hf;
                    uint4 va[4], vb[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        va[i] = ca < p.nb ? __ldcg(xa + 4 * i) : zero;
                        vb[i] = cb < p.nb ? __ldcg(xb + 4 * i) : zero;
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) half_mma(A, i, zr, va[i], vb[i], (uint32_t)ps * 16 + 8 < p.nb, accp[ps]);
                }
            };
            if constexpr (GF == 21) {
                const Iq3sHdr h0 = iq3s_hdr(rows, t), h1 = iq3s_hdr(rows + 8 * p.rs, t);
                UnitHalf A;
                iq3s_decode_half<0, TS>(rows, rows + 8 * p.rs, t, h0, h1, tabc, A);
                run_half(A, 0);
                iq3s_decode_half<1, TS>(rows, rows + 8 * p.rs, t, h0, h1, tabc, A);
                run_half(A, 1);
            } else {
                UnitHalf A;
                q8_decode_half<0>(rows, rows + 8 * p.rs, t, A);
                run_half(A, 0);
                q8_decode_half<1>(rows, rows + 8 * p.rs, t, A);
                run_half(A, 1);
            }
#pragma unroll
            for (int ps = 0; ps < 4; ps++) {
                if ((uint32_t)ps >= passes) break;
                float4 *rd = red + rb_i * WARPS * NT * 32;
                rb_i ^= 1;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) rd[(warp * NT + nt) * 32 + lane] = make_float4(accp[ps][nt][0], accp[ps][nt][1], accp[ps][nt][2], accp[ps][nt][3]);
                team_bar<TT>(team + 1);
                for (int e = tt; e < NT * 32 * 4; e += TT) {
                    const int jj = e & 3, ln = (e >> 2) & 31, nt = e >> 7;
                    float sum = 0.f;
#pragma unroll
                    for (int k2 = 0; k2 < WARPS; k2++) sum += ((const float *)&rd[(k2 * NT + nt) * 32 + ln])[jj];
                    const uint32_t row = item * 16 + (ln >> 2) + 8 * (jj >> 1), col = ps * 16 + nt * 8 + 2 * (ln & 3) + (jj & 1);
                    if (col < p.nb && row < p.N) {
                        if (F32OUT) ((float *)p.y)[(size_t)col * p.ystride + row] = sum;
                        else if (p.ep.nranks > 1) {
                            const __half hv = __float2half_rn(sum);
                            for (uint32_t r = 0; r < p.ep.nranks; r++) ((__half *)p.yR[r])[(size_t)col * p.ystride + row] = hv;
                        } else ((__half *)p.y)[(size_t)col * p.ystride + row] = __float2half_rn(sum);
                    }
                }
            }
        } else
        for (uint32_t ps = 0; ps < passes; ps++) {
            if (passes > 1) load_x(ps * 16);
            float acc[NT][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            if (GF == 21) unit_mma2<TS>(rows, rows + 8 * p.rs, tabc, t, zr, xf[0], xf[1], ps * 16 + 8 < p.nb, acc);
            else unit_mma2_q8(rows, rows + 8 * p.rs, t, zr, xf[0], xf[1], ps * 16 + 8 < p.nb, acc);
            float4 *rd = red + rb_i * WARPS * NT * 32;
            rb_i ^= 1;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) rd[(warp * NT + nt) * 32 + lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
            team_bar<TT>(team + 1);  // partial tiles visible; on the last pass every warp is also done with stage s
            for (int e = tt; e < NT * 32 * 4; e += TT) {
                const int jj = e & 3, ln = (e >> 2) & 31, nt = e >> 7;
                float sum = 0.f;
#pragma unroll
                for (int k2 = 0; k2 < WARPS; k2++) sum += ((const float *)&rd[(k2 * NT + nt) * 32 + ln])[jj];
                const uint32_t row = item * 16 + (ln >> 2) + 8 * (jj >> 1), col = ps * 16 + nt * 8 + 2 * (ln & 3) + (jj & 1);
                if (col < p.nb && row < p.N) {
                    if (F32OUT) ((float *)p.y)[(size_t)col * p.ystride + row] = sum;
                    else if (p.ep.nranks > 1) {
                        const __half hv = __float2half_rn(sum);
                        for (uint32_t r = 0; r < p.ep.nranks; r++) ((__half *)p.yR[r])[(size_t)col * p.ystride + row] = hv;
                    } else ((__half *)p.y)[(size_t)col * p.ystride + row] = __float2half_rn(sum);
                }
            }
        }
    }
    if (!ok && lane == 0) set_status(p.status, ST_MBAR_TIMEOUT | 5);
    if (!F32OUT && p.ep.nranks > 1) ep_publish(p.ep);
}

template <int GF, int WARPS, int TEAMS, bool F32OUT, bool MP = false>
static cudaError_t qmv_mma2_go(const QmvMmaP &p, int sm_count, cudaStream_t st) {
    // more than 16 tokens (at most 64): the form that decodes a unit once for all passes
    static const bool loop_passes = [] { const char *v = getenv("QW_QMV_PASSES"); return v && !strcmp(v, "loop"); }();  // for A/B timing
    if (!MP && p.nb > 16 && p.nb <= 64 && !loop_passes) return qmv_mma2_go<GF, WARPS, TEAMS, F32OUT, true>(p, sm_count, st);
    const size_t smem = 128 + (GF == 21 ? 65536 : 0) + (size_t)TEAMS * 2 * WARPS * 2 * 32 * 16 +
                        (size_t)TEAMS * (GF == 8 ? 2 : QMV_STAGES) * ((16 * p.rs + 127) & ~127u);
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    auto k = qmv_mma2_k<GF, WARPS, TEAMS, F32OUT, MP>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int occ = 1;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k, WARPS * TEAMS * 32, smem);
    if (e != cudaSuccess) return e;
    occ = occ < 1 ? 1 : occ > 4 ? 4 : occ;
    const uint32_t want = (p.items + TEAMS - 1) / TEAMS, cap = (uint32_t)(sm_count * occ), grid = want < cap ? want : cap;
    qw_launch(k, grid, WARPS * TEAMS * 32, smem, st, p);
    return cudaGetLastError();
}

// The grid and block given by the host are ignored (the kernels are persistent and size themselves).  Defines: GF (21 = IQ3_S,
// 8 = Q8_0), KD, YT_F32; EPX = ranks of a slot-sharded projection whose rows go to every rank (see below).
static cudaError_t launch_qmv_mma(const QwLaunch &L) {
    qmv_args a;
    int gf;
    uint32_t K, rb;
    bool f32;
    QW_CHECK_ARG(qmv_common_check(L, a, gf, K, rb, f32));
    QW_CHECK_ARG(L.tx == 256 || L.tx == 512);
    // rows per item: fixed by the matrix shape alone (never by the batch), so results do not depend on nb
    const int mt = 1;
    QW_CHECK_ARG(a.N % (16 * mt) == 0 && ((uintptr_t)L.buf<uint8_t>(0) & 15) == 0 && (16 * rb) % 16 == 0);
    QmvMmaP p{};
    p.W = L.buf<uint8_t>(0);
    p.x = L.buf<__half>(3);
    p.y = L.buf<void>(4);
    p.tab = (const QwTables *)L.tables;
    p.status = L.status;
    p.N = a.N; p.K = K; p.rb = rb; p.xstride = a.xstride; p.ystride = a.ystride; p.nb = a.nb;
    p.items = a.N / (16 * mt);
    // Rows of a staged tile: the eight rows a warp instruction touches must fall into different banks.  An IQ3_S lane
    // reads 2 bytes (row distance = 4, 12, 20 or 28 words mod 32), a Q8_0 lane 8 bytes (8 or 24 words mod 32: two rows
    // per bank group, the best a 32-byte-per-row access allows).  Padding is a multiple of 16 bytes (bulk-copy alignment).
    p.rs = rb;
    for (uint32_t pad = 0; pad < 128 && rb % 16 == 0; pad += 16) {
        const uint32_t wds = ((rb + pad) / 4) % 32;
        if (gf == 21 ? (wds % 8 == 4) : (wds % 16 == 8)) {
            p.rs = rb + pad;
            break;
        }
    }
    const uint32_t epx = (uint32_t)L.def("EPX", 0);
    if (epx > 1) {
        // binds 16 + r = y of rank r (row 0 = this rank's first row, as bind 4), 24 + r = flag array of rank r,
        // 11 = {seq, done} counters, 12 = {rank}; only for the fp16-output IQ3_S projections of the persistent kernel
        QW_CHECK_ARG(epx <= 8 && !f32 && gf == 21 && (K == 2048 || K == 4096) && L.has_bytes(12, 4) && L.buf<unsigned>(11) && L.avail(11) >= 8);
        p.ep.nranks = epx;
        p.ep.rank = L.bytes<uint32_t>(12);
        QW_CHECK_ARG(p.ep.rank < epx);
        p.ep.seq = L.buf<unsigned>(11);
        p.ep.done = p.ep.seq + 1;
        for (uint32_t r = 0; r < epx; r++) {
            p.yR[r] = L.buf<void>(16 + r);
            p.ep.flagR[r] = L.buf<unsigned>(24 + r);
            QW_CHECK_ARG(p.yR[r] && p.ep.flagR[r] && L.avail(24 + r) >= epx * 4 && L.avail(16 + r) >= ((size_t)(a.nb - 1) * a.ystride + a.N) * 2);
        }
    }
#define GO(G, M)                                                        \
    return f32 ? qmv_mma_nt<G, M, true>(p, L.sm_count, L.stream) : qmv_mma_nt<G, M, false>(p, L.sm_count, L.stream)
    if (gf == 21 && K == 2048) return f32 ? qmv_mma2_go<21, 8, 2, true>(p, L.sm_count, L.stream) : qmv_mma2_go<21, 8, 2, false>(p, L.sm_count, L.stream);
    if (gf == 21 && K == 4096) return f32 ? qmv_mma2_go<21, 16, 1, true>(p, L.sm_count, L.stream) : qmv_mma2_go<21, 16, 1, false>(p, L.sm_count, L.stream);
    if (gf == 8 && K == 2048) return f32 ? qmv_mma2_go<8, 8, 1, true>(p, L.sm_count, L.stream) : qmv_mma2_go<8, 8, 1, false>(p, L.sm_count, L.stream);
    if (gf == 21) GO(21, 1);
    else GO(8, 1);
#undef GO
}
QW_FAMILY(qmv_mma, launch_qmv_mma, 256)
