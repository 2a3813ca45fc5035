// MoE expert FFN in one launch: gate/up, SiLU * up and the down projection of every (expert, pass of 8 tokens) item,
// with H = silu(gate x) * (up x) kept in shared memory between the two halves.  Replaces the reference's moe_gu_gg +
// moe_dn_gg pair (kernels/moe_gg.metal:600-652; host src/engine.c:568-646) for the benchmark shapes (D a multiple of
// 2048 that fits, I = 512); the two-launch family in k_moe.cu stays for every other shape.
//
// Structure.  A work item is one pass (up to 8 token columns) of one distinct expert, or of the shared expert; items are
// dealt round-robin to persistent blocks (one per SM).  A block is 16 consumer warps + 1 producer warp around a ring of
// three 30 KB stages:
//   gate/up   stage = 64 gate rows + 64 up rows of the expert x 512 K values: two 2-D tiled TMA boxes of 64 rows x 240
//             bytes (two 110-byte super-blocks plus what 16-byte alignment of the box start costs).  Rows land 240 bytes
//             apart, so the eight rows a warp instruction touches fall into eight different groups of four banks.
//   down      stage = 128 rows of the down matrix over all of K = 512 (rows are contiguous: one 1-D bulk copy).
// Consumer warp w = (row group r = w % 8, K half kh = w / 8) owns 16 MMA rows of the stage and one of the stage's two
// super-blocks; the accumulators live across the stages of a tile, and the two K halves of a row group meet once per
// tile through shared memory (always low half + high half: the order never depends on the batch).  In the gate/up
// half MMA row g is gate row 8r + g and row g + 8 is the up row of the same intermediate index, so a lane holds both
// factors of H and no exchange between row groups exists.  B operands (the tokens, then H as fp16 high + low planes)
// come from padded shared-memory rows by one 16-byte load per sub-block; lanes whose column is absent load nothing.
// Every wait is bounded (about two seconds); a warp that gives up records ST_MBAR_TIMEOUT and keeps walking the same
// control flow without waiting again, so no barrier is ever left short of a participant.
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
constexpr int FFN_STG = 3;
constexpr int FFN_PITCH = 240;                   // bytes between staged gate/up rows
constexpr int FFN_SLOT = 128 * FFN_PITCH;        // 30720: also holds a down tile of 128 x 220 bytes
constexpr int FFN_TAB = 65536;
constexpr int FFN_OFF_TAB = 128;
constexpr int FFN_OFF_PRE = FFN_OFF_TAB + FFN_TAB;          // uint32 pre[MOE_MAXE + 2], padded to 4224 bytes
constexpr int FFN_OFF_RED = FFN_OFF_PRE + 4224;             // [2][8 row groups][32 lanes] float4
constexpr int FFN_OFF_XS = FFN_OFF_RED + 2 * 8 * 32 * 16;   // tokens of the pass, then H planes, then the stages

struct FfnP {
    const uint8_t *Wd, *Sd;   // routed down [E][D][rbI], shared expert's down [D][rbI] (nullptr: no shared expert)
    const __half *x;          // tokens fp16 [nb][D]
    float *Pg;                // [nb][topk+1][D]
    const moe_sel *ms;
    const QwTables *tab;
    unsigned *status;
    uint32_t D, I, rbD, rbI, ebase;
    float *PgR[8];            // expert-parallel exchange: Pg of every rank (see moe_dn in k_moe.cu)
    EpPeers ep;
};

__device__ __forceinline__ void tma_box_2d(uint32_t dst, const CUtensorMap *tm, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(tm),
                 "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bar_sync_n(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

struct FfnItem {
    uint32_t u, e0, cnt, c0, ncols;
    bool shared;
};
// item number w -> (group, pass): routed groups first (pre[] = passes before each group), then the shared expert's passes
__device__ __forceinline__ FfnItem ffn_item(const moe_sel *ms, const uint32_t *pre, uint32_t U, uint32_t nb, uint32_t w) {
    FfnItem it;
    const uint32_t routed = pre[U];
    if (w >= routed) {
        it.shared = true;
        it.u = U;
        it.e0 = 0;
        it.cnt = nb;
        it.c0 = (w - routed) * 8;
    } else {
        uint32_t lo = 0, hi = U;  // largest u with pre[u] <= w
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (pre[mid] <= w) lo = mid;
            else hi = mid;
        }
        it.shared = false;
        it.u = lo;
        it.e0 = ms->off[lo];
        it.cnt = ms->off[lo + 1] - it.e0;
        it.c0 = (w - pre[lo]) * 8;
    }
    it.ncols = it.cnt - it.c0 < 8 ? it.cnt - it.c0 : 8;
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

template <int IB>
__device__ __forceinline__ void ffn_sub_gu(uint32_t u0, uint32_t u1, int t, const Iq3sHdr &h0, const Iq3sHdr &h1, uint32_t tabc, const ZeroRegs &zr, uint32_t bx,
                                           bool have, float (&acc)[4]) {
    uint4 xv = make_uint4(0, 0, 0, 0);
    if (have) xv = lds_v4(bx + IB * 64);
    sub_mma1<false, IB, 128>(u0, u1, t, h0, h1, tabc, zr, xv, xv, acc);
}
template <int IB>
__device__ __forceinline__ void ffn_sub_dn(uint32_t u0, uint32_t u1, int t, const Iq3sHdr &h0, const Iq3sHdr &h1, uint32_t tabc, const ZeroRegs &zr, uint32_t bh,
                                           uint32_t bl, bool have, float (&acc)[4]) {
    uint4 xv = make_uint4(0, 0, 0, 0), xl = make_uint4(0, 0, 0, 0);
    if (have) {
        xv = lds_v4(bh + IB * 64);
        xl = lds_v4(bl + IB * 64);
    }
    sub_mma1_h2<IB, 128>(u0, u1, t, h0, h1, tabc, zr, xv, xl, acc);
}

// PROBE = true is the copy-only twin used to measure what the staging pipeline alone can deliver: the same items, the same
// TMA boxes and bulk copies through the same ring, but the consumers only read every staged byte once (16-byte loads) and
// compute nothing -- the role of the reference's pure-read probes (bench/moe_bw.c:1-3, bench/qmv.c:357-382).
template <bool PROBE>
__global__ void __launch_bounds__(FFN_THREADS, 1) moe_ffn_k(const __grid_constant__ CUtensorMap mG, const __grid_constant__ CUtensorMap mU,
                                                           const __grid_constant__ CUtensorMap mSG, const __grid_constant__ CUtensorMap mSU, const FfnP p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = (uint64_t *)smem;
    uint64_t *full = bars, *empty = bars + FFN_STG, *tab_bar = bars + 2 * FFN_STG, *xfull = tab_bar + 1, *xfree = tab_bar + 2;
    uint32_t *pre = (uint32_t *)(smem + FFN_OFF_PRE);
    float4 *red = (float4 *)(smem + FFN_OFF_RED);
    const uint32_t xpitch = p.D * 2 + 64, hpitch = p.I * 2 + 64;
    uint8_t *xs = smem + FFN_OFF_XS, *hs = xs + 8 * xpitch, *stage0 = hs + 16 * hpitch;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const uint32_t KP = p.D / 512, GT = p.I / 64, DT = p.D / 128, KU = p.I / 256;

    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < FFN_STG; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], FFN_CW);
        }
        mbar_init(tab_bar, 1);
        mbar_init(xfull, 1);
        mbar_init(xfree, FFN_CW);
        mbar_init_fence();
        mbar_expect_tx(tab_bar, FFN_TAB);
        bulk_g2s(smem + FFN_OFF_TAB, p.tab->grid_h4, FFN_TAB, tab_bar);
    }
    pdl_wait();  // the selection record, the tokens and Pg belong to earlier kernels
    const moe_sel *ms = p.ms;
    for (uint32_t i = tid; i <= MOE_MAXE + 1; i += FFN_THREADS) pre[i] = ms->pre[i];
    const uint32_t U = ms->U, nb = ms->nb, topk = ms->topk;
    __syncthreads();
    const uint32_t items = pre[U] + (p.Sd ? (nb + 7) / 8 : 0);
    const uint32_t slot0 = smem_u32(stage0);

    if (warp == FFN_CW) {
        // ---- producer: one lane walks the block's items and keeps the ring full
        if (lane == 0) {
            bool ok = true;
            uint32_t j = 0, n = 0;
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
            for (uint32_t w = blockIdx.x; w < items; w += gridDim.x, n++) {
                const FfnItem it = ffn_item(ms, pre, U, nb, w);
                if (n > 0 && ok && !mbar_wait(xfree, (n - 1) & 1)) {  // every consumer warp is done with the previous item's tokens
                    ok = false;
                    set_status(p.status, ST_MBAR_TIMEOUT | 7);
                }
                fence_proxy_async();
                mbar_expect_tx(xfull, it.ncols * p.D * 2);
                for (uint32_t c = 0; c < it.ncols; c++) {
                    uint32_t tok, rank;
                    ffn_entry(ms, it, topk, c, tok, rank);
                    bulk_g2s(xs + c * xpitch, p.x + (size_t)tok * p.D, p.D * 2, xfull);
                }
                const uint32_t erow = it.shared ? 0 : (ms->ue[it.u] - p.ebase);
                const CUtensorMap *tg = it.shared ? &mSG : &mG, *tu = it.shared ? &mSU : &mU;
                for (uint32_t gt = 0; gt < GT; gt++)
                    for (uint32_t kp = 0; kp < KP; kp++, j++) {
                        const uint32_t dst = slot_for(2 * 64 * FFN_PITCH);
                        const int xc = (int)((220 * kp) & ~15u), yr = (int)(erow * p.I + gt * 64);
                        tma_box_2d(dst, tg, xc, yr, &full[j % FFN_STG]);
                        tma_box_2d(dst + 64 * FFN_PITCH, tu, xc, yr, &full[j % FFN_STG]);
                    }
                const uint8_t *wd = it.shared ? p.Sd : p.Wd + (size_t)erow * p.D * p.rbI;
                for (uint32_t dt = 0; dt < DT; dt++, j++) {
                    const uint32_t dst = slot_for(128 * p.rbI);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                                 "l"(wd + (size_t)dt * 128 * p.rbI), "r"(128 * p.rbI), "r"(smem_u32(&full[j % FFN_STG]))
                                 : "memory");
                }
            }
        }
    } else {
        // ---- consumers
        const int r = warp & 7, kh = warp >> 3;
        bool ok = mbar_wait(tab_bar, 0);
        if (!ok && lane == 0) set_status(p.status, ST_MBAR_TIMEOUT | 8);
        const uint32_t tabc = smem_u32(smem + FFN_OFF_TAB) + (lane & 15) * 8;  // this lane's copy of the interleaved codebook
        const ZeroRegs zr = zero_regs();
        const uint32_t xb0 = smem_u32(xs) + g * xpitch + t * 16;
        const uint32_t hb0 = smem_u32(hs) + g * hpitch + t * 16;
        uint32_t j = 0, n = 0, rc = 0;
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
        for (uint32_t w = blockIdx.x; w < items; w += gridDim.x, n++) {
            const FfnItem it = ffn_item(ms, pre, U, nb, w);
            if (n > 0) bar_sync_n(9, FFN_CW * 32);  // nobody still reads the previous item's H rows
            const bool have = (uint32_t)g < it.ncols;
            uint32_t oo[2] = {0xffffffffu, 0xffffffffu};  // element offsets of the output rows of columns 2t and 2t + 1
#pragma unroll
            for (int c = 0; c < 2; c++)
                if ((uint32_t)(2 * t + c) < it.ncols) {
                    uint32_t tok, rank;
                    ffn_entry(ms, it, topk, 2 * t + c, tok, rank);
                    oo[c] = (tok * (topk + 1) + rank) * p.D;
                }
            if (ok && !mbar_wait(xfull, n & 1)) {
                ok = false;
                if (lane == 0) set_status(p.status, ST_MBAR_TIMEOUT | 10);
            }
            if (PROBE) {
                uint32_t sink = 0;
                for (uint32_t sidx = 0; sidx < GT * KP + DT; sidx++) {
                    const uint32_t st = wait_full(), bytes = sidx < GT * KP ? 128 * FFN_PITCH : 128 * p.rbI;
                    for (uint32_t o = (warp * 32 + lane) * 16; o < bytes; o += FFN_CW * 32 * 16) {
                        const uint4 v = lds_v4(st + o);
                        sink ^= v.x ^ v.y ^ v.z ^ v.w;
                    }
                    release();
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(xfree);
                if (sink == 0x9e3779b9u && oo[0] != 0xffffffffu) p.Pg[oo[0]] = 0.f;  // keeps the loads observable; practically never taken
                continue;
            }
            // ---- gate/up: tiles of 64 intermediate indices
            for (uint32_t gt = 0; gt < GT; gt++) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (uint32_t kp = 0; kp < KP; kp++) {
                    const uint32_t st = wait_full();
                    const uint32_t u0 = st + (8 * r + g) * FFN_PITCH + ((220 * kp) & 15) + kh * 110, u1 = u0 + 64 * FFN_PITCH;
                    const uint32_t bx = xb0 + (2 * kp + kh) * 512;
                    const Iq3sHdr h0 = iq3s_hdr(u0, t), h1 = iq3s_hdr(u1, t);
                    ffn_sub_gu<0>(u0, u1, t, h0, h1, tabc, zr, bx, have, acc);
                    ffn_sub_gu<1>(u0, u1, t, h0, h1, tabc, zr, bx, have, acc);
                    ffn_sub_gu<2>(u0, u1, t, h0, h1, tabc, zr, bx, have, acc);
                    ffn_sub_gu<3>(u0, u1, t, h0, h1, tabc, zr, bx, have, acc);
                    ffn_sub_gu<4>(u0, u1, t, h0, h1, tabc, zr, bx, have, acc);
                    ffn_sub_gu<5>(u0, u1, t, h0, h1, tabc, zr, bx, have, acc);
                    ffn_sub_gu<6>(u0, u1, t, h0, h1, tabc, zr, bx, have, acc);
                    ffn_sub_gu<7>(u0, u1, t, h0, h1, tabc, zr, bx, have, acc);
                    release();
                }
                pair_sum(acc);
                if (!kh) {
                    // acc[0], acc[1] = gate of index 64 gt + 8 r + g for columns 2t, 2t + 1; acc[2], acc[3] = up.  H travels to the
                    // down half as an fp16 high part plus an fp16 remainder (22 mantissa bits where the remainder is normal)
                    const uint32_t idx = gt * 64 + 8 * r + g;
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        const float gs = acc[c], us = acc[2 + c];
                        float h = gs / (1.0f + expf(-gs)) * us;
                        h = fminf(fmaxf(h, -65504.0f), 65504.0f);
                        const __half hi = __float2half_rn(h);
                        const __half lo = __float2half_rn(h - __half2float(hi));
                        uint8_t *hr = hs + (size_t)(2 * t + c) * hpitch + idx * 2;
                        *(__half *)hr = hi;
                        *(__half *)(hr + 8 * hpitch) = lo;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(xfree);
            bar_sync_n(9, FFN_CW * 32);  // H of the item is complete
            // ---- down: tiles of 128 output rows; MMA row g is tile row 16 r + 2 g, row g + 8 the next one
            for (uint32_t dt = 0; dt < DT; dt++) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                const uint32_t st = wait_full();
                for (uint32_t ks = kh; ks < KU; ks += 2) {
                    const uint32_t u0 = st + (16 * r + 2 * g) * p.rbI + ks * 110, u1 = u0 + p.rbI;
                    const uint32_t bh = hb0 + ks * 512, bl = bh + 8 * hpitch;
                    const Iq3sHdr h0 = iq3s_hdr(u0, t), h1 = iq3s_hdr(u1, t);
                    ffn_sub_dn<0>(u0, u1, t, h0, h1, tabc, zr, bh, bl, have, acc);
                    ffn_sub_dn<1>(u0, u1, t, h0, h1, tabc, zr, bh, bl, have, acc);
                    ffn_sub_dn<2>(u0, u1, t, h0, h1, tabc, zr, bh, bl, have, acc);
                    ffn_sub_dn<3>(u0, u1, t, h0, h1, tabc, zr, bh, bl, have, acc);
                    ffn_sub_dn<4>(u0, u1, t, h0, h1, tabc, zr, bh, bl, have, acc);
                    ffn_sub_dn<5>(u0, u1, t, h0, h1, tabc, zr, bh, bl, have, acc);
                    ffn_sub_dn<6>(u0, u1, t, h0, h1, tabc, zr, bh, bl, have, acc);
                    ffn_sub_dn<7>(u0, u1, t, h0, h1, tabc, zr, bh, bl, have, acc);
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
                    }
                }
            }
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
// 4 = x fp16 [nb][D], 5 = moe_sel, 6 = routed down [EL][D][rbI], 7 = shared down, 9 = Pg fp32 [64][TOPK+1][D],
// 10 = id of the first expert held in the weight buffers (optional, default 0); with EPX = ranks also 11, 12, 16 + r,
// 24 + r as for moe_dn.  defines: E, D, I, TOPK, EL, SHARED, EPX.  The host's grid and block are ignored.
static cudaError_t launch_moe_ffn(const QwLaunch &L) {
    FfnP p{};
    const uint32_t E = (uint32_t)L.def("E", 512), topk = (uint32_t)L.def("TOPK", 10);
    p.D = (uint32_t)L.def("D", 2048);
    p.I = (uint32_t)L.def("I", 512);
    QW_CHECK_ARG(p.D % 2048 == 0 && p.I == 512 && topk < MOE_MAXK);
    p.rbD = p.D / 256 * 110;
    p.rbI = p.I / 256 * 110;
    const size_t smem = FFN_OFF_XS + (size_t)8 * (p.D * 2 + 64) + (size_t)16 * (p.I * 2 + 64) + (size_t)FFN_STG * FFN_SLOT;
    QW_CHECK_ARG(smem <= 227 * 1024 && 128 * p.rbI <= FFN_SLOT && (128 * p.rbI) % 16 == 0);
    const bool shared = L.def("SHARED", 1) != 0;
    const uint32_t EL = (uint32_t)L.def("EL", E);
    p.ebase = L.has_bytes(10, 4) ? L.bytes<uint32_t>(10) : 0;
    QW_CHECK_ARG(EL >= 1 && p.ebase + EL <= E);
    const uint8_t *Wg = L.buf<uint8_t>(0), *Wu = L.buf<uint8_t>(1), *Sg = shared ? L.buf<uint8_t>(2) : nullptr, *Su = shared ? L.buf<uint8_t>(3) : nullptr;
    p.Wd = L.buf<uint8_t>(6);
    p.Sd = shared ? L.buf<uint8_t>(7) : nullptr;
    p.x = L.buf<__half>(4);
    p.ms = L.buf<moe_sel>(5);
    p.Pg = L.buf<float>(9);
    p.tab = (const QwTables *)L.tables;
    p.status = L.status;
    const size_t wsz = (size_t)EL * p.I * p.rbD, ssz = (size_t)p.I * p.rbD;
    QW_CHECK_ARG(Wg && Wu && p.Wd && p.x && p.ms && p.Pg && L.avail(0) >= wsz && L.avail(1) >= wsz && L.avail(6) >= wsz && L.avail(5) >= sizeof(moe_sel));
    QW_CHECK_ARG(!shared || (Sg && Su && p.Sd && L.avail(2) >= ssz && L.avail(3) >= ssz && L.avail(7) >= ssz));
    QW_CHECK_ARG((((uintptr_t)Wg | (uintptr_t)Wu | (uintptr_t)p.Wd | (uintptr_t)Sg | (uintptr_t)Su | (uintptr_t)p.Sd | (uintptr_t)p.x) & 15) == 0);
    QW_CHECK_ARG(L.avail(9) >= (size_t)MOE_MAXB * (topk + 1) * p.D * 4 && L.avail(4) >= (size_t)p.D * 2);
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
            QW_CHECK_ARG(p.PgR[r] && p.ep.flagR[r] && L.avail(24 + r) >= p.ep.nranks * 4 && L.avail(16 + r) >= (size_t)MOE_MAXB * (topk + 1) * p.D * 4);
        }
    }
    const CUtensorMap *mG = ffn_tensor_map(Wg, p.rbD, (uint64_t)EL * p.I), *mU = ffn_tensor_map(Wu, p.rbD, (uint64_t)EL * p.I);
    const CUtensorMap *mSG = shared ? ffn_tensor_map(Sg, p.rbD, p.I) : mG, *mSU = shared ? ffn_tensor_map(Su, p.rbD, p.I) : mU;
    QW_CHECK_ARG(mG && mU && mSG && mSU);
    auto kern = L.def("PROBE", 0) ? moe_ffn_k<true> : moe_ffn_k<false>;  // PROBE defined 1: the copy-only twin (outputs are not written)
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    qw_launch(kern, L.sm_count, FFN_THREADS, smem, L.stream, *mG, *mU, *mSG, *mSU, p);
    return cudaGetLastError();
}
QW_FAMILY(moe_ffn, launch_moe_ffn, 512)
