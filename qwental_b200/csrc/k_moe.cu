// MoE decode layer for up to 64 tokens (one per slot): router, top-k + grouping by expert, gathered SwiGLU
// expert FFN (gate/up then down) with the shared expert as one more group, rank-ordered weighted combine.
// Replaces the reference's moe_pre_gg / gg_select / moe_gu_gg / moe_dn_gg / moe_cmb_gg
// (kernels/moe_gg.metal:118-189, 534-663; host src/engine.c:568-646).  What is kept from the reference:
//   - router logits in fp32 with one fixed summation order (so the chosen experts are reproducible),
//   - top-k with equal logits -> lowest expert id; weights = softmax over the picked logits
//     with the exponentials summed in rank order; shared-expert gate = sigmoid of an extra router row,
//   - every distinct expert's weights are read and decoded once per step and applied to each token that chose
//     it; a token's arithmetic does not depend on which other tokens are in the batch,
//   - H = silu(gate x) * (up x) is kept at better than fp16 precision between the two halves (here as a
//     bf16 high + low pair, 16 mantissa bits; the reference keeps fp32, src/engine.c:157),
//   - combine in rank order, then the shared expert, one rounding to fp16 (kernels/moe_gg.metal:655-663).
// What is new: groups hold up to 64 tokens (the reference's gg_sel has 8-bit masks), the contraction runs on
// tensor cores from raw IQ3_S blocks staged by bulk (TMA) copies, and experts can be restricted to a range
// [e_lo, e_hi) for expert-parallel execution.
#include "qmv_core.cuh"
#include "qw_kern.h"

using namespace qw;

#include "moe_sel.h"

// ------------------------------------------------------------------------------------------------ router
// logits [nb][E+1] fp32; row E is the shared-expert gate.  One warp per row, lane owns the 8-value chunks
// lane, lane+32, ...: a single fma chain per lane, then the xor butterfly (bit-exact against the CPU oracle).
// binds: 0 = Wr fp16 [E][D], 1 = Wsg fp16 [D], 2 = x fp16 [nb][D], 3 = logits, 14 = nb.  grid ceil((E+1)/8) x 256
template <int D>
__global__ void __launch_bounds__(256) moe_router_k(const __half *Wr, const __half *Wsg, const __half *x, float *logits, uint32_t E, uint32_t nb) {
    constexpr int CH = D / 8 / 32;
    const uint32_t r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r > E) return;
    const uint4 *w = (const uint4 *)(r < E ? Wr + (size_t)r * D : Wsg);
    uint4 wr[CH];
#pragma unroll
    for (int c = 0; c < CH; c++) wr[c] = __ldg(w + lane + 32 * c);
    pdl_sync();  // the router row is static; the tokens are the previous kernel's output
    for (uint32_t t = 0; t < nb; t++) {
        const uint4 *xt = (const uint4 *)(x + (size_t)t * D);
        float acc = 0.f;
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const uint4 xv = __ldcg(xt + lane + 32 * c);
            const uint32_t a4[4] = {wr[c].x, wr[c].y, wr[c].z, wr[c].w}, b4[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 a = __half22float2(*(const __half2 *)&a4[j]), b = __half22float2(*(const __half2 *)&b4[j]);
                acc = __fmaf_rn(a.x, b.x, acc);
                acc = __fmaf_rn(a.y, b.y, acc);
            }
        }
        const float v = warp_sum_canon(acc);
        if (lane == 0) logits[(size_t)t * (E + 1) + r] = v;
    }
}

static cudaError_t launch_moe_router(const QwLaunch &L) {
    const uint32_t E = (uint32_t)L.def("E", 512), D = (uint32_t)L.def("D", 2048);
    const uint32_t nb = L.bytes<uint32_t>(14);
    QW_CHECK_ARG(L.buf<void>(0) && L.buf<void>(1) && L.buf<void>(2) && L.buf<void>(3) && nb >= 1 && nb <= MOE_MAXB);
    QW_CHECK_ARG(L.avail(0) >= (size_t)E * D * 2 && L.avail(1) >= (size_t)D * 2 && L.avail(2) >= (size_t)nb * D * 2 &&
                 L.avail(3) >= (size_t)nb * (E + 1) * 4);
    QW_CHECK_ARG(L.tx == 256 && L.gx == (E + 1 + 7) / 8);
    if (D == 2048) qw_launch(moe_router_k<2048>, L.gx, 256, 0, L.stream, L.buf<__half>(0), L.buf<__half>(1), L.buf<__half>(2), L.buf<float>(3), E, nb);
    else if (D == 256) qw_launch(moe_router_k<256>, L.gx, 256, 0, L.stream, L.buf<__half>(0), L.buf<__half>(1), L.buf<__half>(2), L.buf<float>(3), E, nb);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}
QW_FAMILY(moe_router, launch_moe_router, 256)

// ------------------------------------------------------------------------------------------------ select + group
// One block of 1024 threads.  binds: 0 = logits [nb][E+1], 1 = moe_sel, 2 = {nb, e_lo, e_hi}.
struct sel_args {
    uint32_t nb, e_lo, e_hi;
};

// Body of the selection for one block of NTH threads (NTH >= E: thread e owns expert e in the scans).  Logits are read with .cg loads: in the fused router + select
// kernel they were written by other blocks of the same launch.
template <int NTH>
__device__ __forceinline__ void moe_select_body(const float *logits, moe_sel *ms, uint32_t E, uint32_t topk, sel_args a) {
    __shared__ uint32_t mlo[MOE_MAXE], mhi[MOE_MAXE], pos[MOE_MAXE], grp[MOE_MAXE];  // token bit masks per expert
    __shared__ uint16_t sid[MOE_MAXB * MOE_MAXK];
    __shared__ uint32_t wsum[2][32];
    __shared__ uint64_t cand_s[NTH / 32][32 + MOE_MAXK];  // per warp: candidates of the fast top-k path, then the winners' keys
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t PER = E / 32;
    constexpr uint32_t NW = NTH / 32;
    for (uint32_t e = tid; e < MOE_MAXE; e += NTH) mlo[e] = mhi[e] = 0;
    // 1. top-k per token: one warp per token, lane owns experts lane, lane + 32, ... (coalesced reads).  Equal
    //    logits -> lowest expert id: within a lane the strict '>' keeps the lowest id, across lanes the smallest id
    //    among the lanes holding the maximum wins.
    for (uint32_t t = warp; t < a.nb; t += NW) {
        const float *lg = logits + (size_t)t * (E + 1);
        // Logits as order-preserving unsigned keys (a float's bits with the sign folded), so a maximum is one hardware
        // warp reduction.  Equal floats give equal keys (a logit is never -0: every dot product starts from +0).
        auto key_of = [&](uint32_t j) {
            const uint32_t u = __float_as_uint(__ldcg(lg + lane + 32 * j));
            return u ^ ((u >> 31) ? 0xffffffffu : 0x80000000u);
        };
        uint32_t pkey = 0;
        if (PER == 16) {
            uint32_t kv[16];
#pragma unroll
            for (uint32_t j = 0; j < 16; j++) kv[j] = key_of(j);
            // Fast path.  T = the topk-th largest of the 32 lane maxima: at least topk values are >= T, so the winners are
            // among the values >= T -- usually little more than topk of them.  If they fit one per lane, each lane takes
            // one candidate and finds its rank by counting the candidates that beat it (larger key, or equal key and
            // lower id); ranks are distinct because ids are.  Otherwise (many equal logits) the general path below runs.
            uint32_t lm = kv[0];
#pragma unroll
            for (uint32_t j = 1; j < 16; j++) lm = max(lm, kv[j]);
            uint32_t cur = lm, T = 0;
            for (uint32_t k = 0; k < topk; k++) {
                T = __reduce_max_sync(0xffffffffu, cur);
                const uint32_t who = __ffs(__ballot_sync(0xffffffffu, cur == T)) - 1;
                if (lane == who) cur = 0;  // (a real key is never 0: that would be the bit pattern of -NaN)
            }
            uint32_t cnt = 0;
#pragma unroll
            for (uint32_t j = 0; j < 16; j++) cnt += kv[j] >= T;
            uint32_t pre = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t n = __shfl_up_sync(0xffffffffu, pre, o);
                if (lane >= (uint32_t)o) pre += n;
            }
            const uint32_t total = __shfl_sync(0xffffffffu, pre, 31);
            if (total <= 32) {
                uint64_t *cs = cand_s[warp];
                uint32_t at = pre - cnt;
#pragma unroll
                for (uint32_t j = 0; j < 16; j++)
                    if (kv[j] >= T) cs[at++] = ((uint64_t)kv[j] << 32) | (0xffffffffu - (lane + 32 * j));
                __syncwarp();
                const uint64_t mine = lane < total ? cs[lane] : 0;
                uint32_t rank = 0;
                for (uint32_t j = 0; j < total; j++) rank += __shfl_sync(0xffffffffu, mine, j) > mine;
                if (lane < total && rank < topk) {
                    const uint32_t id = 0xffffffffu - (uint32_t)mine;
                    ms->ids[t][rank] = (int32_t)id;
                    sid[t * MOE_MAXK + rank] = (uint16_t)id;
                    cs[32 + rank] = mine >> 32;  // key of rank r, for the softmax below
                }
                __syncwarp();
                if (lane < topk) pkey = (uint32_t)cs[32 + lane];
                __syncwarp();
            } else {
            // General path: the lane sorts its 16 (key, ~id) pairs once
            uint64_t s[16];
#pragma unroll
            for (uint32_t j = 0; j < 16; j++) s[j] = ((uint64_t)kv[j] << 32) | (0xffffffffu - (lane + 32 * j));
#define CE(A, B)                          \
    {                                     \
        const uint64_t x_ = s[A], y_ = s[B]; \
        const bool sw_ = y_ > x_;         \
        s[A] = sw_ ? y_ : x_;             \
        s[B] = sw_ ? x_ : y_;             \
    }
            CE(0, 1) CE(2, 3) CE(4, 5) CE(6, 7) CE(8, 9) CE(10, 11) CE(12, 13) CE(14, 15) CE(0, 2) CE(1, 3) CE(4, 6) CE(5, 7) CE(8, 10) CE(9, 11) CE(12, 14) CE(13, 15) CE(1, 2) CE(5, 6) CE(9, 10) CE(13, 14) CE(0, 4) CE(1, 5) CE(2, 6) CE(3, 7) CE(8, 12) CE(9, 13) CE(10, 14) CE(11, 15) CE(2, 4) CE(3, 5) CE(10, 12) CE(11, 13) CE(1, 2) CE(3, 4) CE(5, 6) CE(9, 10) CE(11, 12) CE(13, 14) CE(0, 8) CE(1, 9) CE(2, 10) CE(3, 11) CE(4, 12) CE(5, 13) CE(6, 14) CE(7, 15) CE(4, 8) CE(5, 9) CE(6, 10) CE(7, 11) CE(2, 4) CE(3, 5) CE(6, 8) CE(7, 9) CE(10, 12) CE(11, 13) CE(1, 2) CE(3, 4) CE(5, 6) CE(7, 8) CE(9, 10) CE(11, 12) CE(13, 14)
#undef CE
            for (uint32_t k = 0; k < topk; k++) {
                const uint32_t hk = (uint32_t)(s[0] >> 32), hi_ = (uint32_t)s[0];
                const uint32_t m = __reduce_max_sync(0xffffffffu, hk);
                const uint32_t nid = __reduce_max_sync(0xffffffffu, hk == m ? hi_ : 0u);  // largest ~id = lowest id
                const uint32_t id = 0xffffffffu - nid;
                if (lane == 0) {
                    ms->ids[t][k] = (int32_t)id;
                    sid[t * MOE_MAXK + k] = (uint16_t)id;
                }
                if (lane == k) pkey = m;
                if (lane == (id & 31)) {  // pop the head
#pragma unroll
                    for (uint32_t j = 0; j < 15; j++) s[j] = s[j + 1];
                    s[15] = 0;
                }
            }
            }  // general path
        } else {
            uint32_t v[8];  // small expert counts (E <= 256): rescan the lane's few values every round
#pragma unroll
            for (uint32_t j = 0; j < 8; j++) v[j] = j < PER ? key_of(j) : 0u;
            for (uint32_t k = 0; k < topk; k++) {
                uint32_t b0 = v[0], j0 = 0;
#pragma unroll
                for (uint32_t j = 1; j < 8; j++)
                    if (j < PER && v[j] > b0) { b0 = v[j]; j0 = j; }
                const uint32_t m = __reduce_max_sync(0xffffffffu, b0);
                const uint32_t id = __reduce_min_sync(0xffffffffu, b0 == m ? lane + 32 * j0 : 0xffffffffu);
                if (lane == 0) {
                    ms->ids[t][k] = (int32_t)id;
                    sid[t * MOE_MAXK + k] = (uint16_t)id;
                }
                if (lane == k) pkey = m;
                const uint32_t bl = id & 31, bj = id >> 5;
#pragma unroll
                for (uint32_t j = 0; j < 8; j++) v[j] = (lane == bl && j == bj) ? 0u : v[j];  // below every real key
            }
        }
        const float pk = __uint_as_float(pkey ^ ((pkey >> 31) ? 0x80000000u : 0xffffffffu));
        const float mx = __shfl_sync(0xffffffffu, pk, 0), ex = expf(pk - mx);
        float sm = 0.f;
        for (uint32_t k = 0; k < topk; k++) sm = __fadd_rn(sm, __shfl_sync(0xffffffffu, ex, k));  // rank order
        if (lane < topk) ms->w[t][lane] = ex / sm;
        if (lane == topk) ms->w[t][topk] = 1.0f / (1.0f + expf(-__ldcg(lg + E)));
    }
    __syncthreads();
    // 2. group by expert.  mask[e] = tokens that chose e; an entry's place inside its group is the number of
    //    earlier tokens in the mask, so groups are filled in token order without any serial scan.
    const uint32_t nent = a.nb * topk;
    for (uint32_t i = tid; i < nent; i += NTH) {
        const uint32_t t = i / topk, e = sid[t * MOE_MAXK + (i - t * topk)];
        if (e >= a.e_lo && e < a.e_hi) atomicOr(t < 32 ? &mlo[e] : &mhi[e], 1u << (t & 31));
    }
    __syncthreads();
    {   // exclusive scans over experts (thread e = expert e): entries (low 16 bits of one word) and passes of 8 entries
        // (high 16 bits: what the gate/up and down kernels enumerate their work units by), and non-empty flags
        const uint32_t c0 = tid < E ? __popc(mlo[tid]) + __popc(mhi[tid]) : 0, f = c0 ? 1u : 0u, c = c0 | (((c0 + 7) / 8) << 16);
        uint32_t sc = c, sf = f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t tc = __shfl_up_sync(0xffffffffu, sc, o), tf = __shfl_up_sync(0xffffffffu, sf, o);
            if (lane >= (uint32_t)o) { sc += tc; sf += tf; }
        }
        if (lane == 31) { wsum[0][warp] = sc; wsum[1][warp] = sf; }
        __syncthreads();
        if (warp == 0) {
            uint32_t xc = lane < NW ? wsum[0][lane] : 0, xf = lane < NW ? wsum[1][lane] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t tc = __shfl_up_sync(0xffffffffu, xc, o), tf = __shfl_up_sync(0xffffffffu, xf, o);
                if (lane >= (uint32_t)o) { xc += tc; xf += tf; }
            }
            wsum[0][lane] = xc;
            wsum[1][lane] = xf;
        }
        __syncthreads();
        const uint32_t bc = warp ? wsum[0][warp - 1] : 0, bf = warp ? wsum[1][warp - 1] : 0;
        const uint32_t ex = bc + sc - c;  // exclusive prefix: entries | passes << 16
        pos[tid] = ex & 0xffffu;          // first entry of expert tid
        grp[tid] = bf + sf - f;           // group number of expert tid (if non-empty)
        if (c0) {
            ms->ue[bf + sf - f] = tid;
            ms->off[bf + sf - f] = ex & 0xffffu;
            ms->pre[bf + sf - f] = ex >> 16;
        }
        if (tid == NTH - 1) {
            ms->U = bf + sf;
            ms->nb = a.nb;
            ms->topk = topk;
            ms->off[bf + sf] = (bc + sc) & 0xffffu;
            ms->pre[bf + sf] = (bc + sc) >> 16;
        }
    }
    __syncthreads();
    for (uint32_t i = tid; i < nent; i += NTH) {
        const uint32_t t = i / topk, k = i - t * topk, e = sid[t * MOE_MAXK + k];
        if (e >= a.e_lo && e < a.e_hi) {
            const uint32_t before = t < 32 ? __popc(mlo[e] & ((1u << t) - 1)) : __popc(mlo[e]) + __popc(mhi[e] & ((1u << (t - 32)) - 1));
            ms->ent[pos[e] + before] = (uint16_t)((t << 8) | k);
        }
    }
}

__global__ void __launch_bounds__(1024) moe_select_k(const float *logits, moe_sel *ms, uint32_t E, uint32_t topk, sel_args a) {
    pdl_sync();
    moe_select_body<1024>(logits, ms, E, topk, a);
}

static cudaError_t launch_moe_select(const QwLaunch &L) {
    const uint32_t E = (uint32_t)L.def("E", 512), topk = (uint32_t)L.def("TOPK", 10);
    sel_args a = L.bytes<sel_args>(2);
    QW_CHECK_ARG(L.buf<void>(0) && L.buf<void>(1) && L.has_bytes(2, 12));
    QW_CHECK_ARG(E % 32 == 0 && (E == 512 || E <= 256) && topk >= 1 && topk < MOE_MAXK && topk <= E && a.nb >= 1 && a.nb <= MOE_MAXB);
    QW_CHECK_ARG(L.avail(0) >= (size_t)a.nb * (E + 1) * 4 && L.avail(1) >= sizeof(moe_sel));
    if (a.e_hi > E) a.e_hi = E;
    qw_launch(moe_select_k, 1, 1024, 0, L.stream, L.buf<float>(0), L.buf<moe_sel>(1), E, topk, a);
    return cudaGetLastError();
}
QW_FAMILY(moe_select, launch_moe_select, 1024)

// ------------------------------------------------------------------------------------------------ router + select in one launch
// The role of moe_pre_gg's hand-over (kernels/moe_gg.metal:574-589): the block that finishes the router last (device
// counter + fences) runs the selection.  Blocks of 512 threads: warp = (row blockIdx*4 + warp%4, token group warp/4); the
// row sits in registers and the tokens in shared memory, both converted to fp32 once.
// binds: 0 = Wr, 1 = Wsg, 2 = x, 3 = logits, 4 = counter (uint32, zero before the first launch; left zero), 5 = moe_sel,
// 14 = {nb, e_lo, e_hi}.  The launcher sets the grid itself: ceil((E+1)/4) blocks of 512 threads.
template <int D>
__global__ void __launch_bounds__(512) moe_route_k(const __half *Wr, const __half *Wsg, const __half *x, float *logits, unsigned *counter, moe_sel *ms,
                                                   uint32_t E, uint32_t topk, sel_args a) {
    constexpr int CH = D / 8 / 32;
    // the tokens of one pass as fp32, converted once per block: [16 tokens][CH][2][32 lanes] float4, so that a lane's
    // eight values of a chunk are two conflict-free 16-byte loads
    extern __shared__ __align__(16) uint8_t route_smem[];
    float4 *xs = (float4 *)route_smem;
    __shared__ bool last;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = blockIdx.x * 4 + (warp & 3), tg = warp >> 2;
    pdl_launch();
    float wf[CH * 8];
    if (r <= E) {
        const uint4 *w = (const uint4 *)(r < E ? Wr + (size_t)r * D : Wsg);
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const uint4 v = __ldg(w + lane + 32 * c);
            const uint32_t a4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(*(const __half2 *)&a4[j]);
                wf[8 * c + 2 * j] = f.x;
                wf[8 * c + 2 * j + 1] = f.y;
            }
        }
    }
    pdl_wait();  // the router row is static; the tokens are the previous kernel's output
    // Passes of 16 tokens.  Each warp runs its tokens (tg, tg + 4, tg + 8, tg + 12) against its row; every dot product is
    // the same single-lane chain as in moe_router (element k of lane l, chunk c is column (l + 32 c) * 8 + k), so logits
    // are bit-identical.
    for (uint32_t t0 = 0; t0 < a.nb; t0 += 16) {
        const uint32_t nt = a.nb - t0 < 16 ? a.nb - t0 : 16;
        if (t0) __syncthreads();
        for (uint32_t e = threadIdx.x; e < nt * (D / 8); e += 512) {
            const uint4 v = __ldcg((const uint4 *)(x + (size_t)t0 * D) + e);
            const uint32_t tl = e / (D / 8), ce = e % (D / 8), c = ce >> 5, ln = ce & 31;
            const float2 f0 = __half22float2(*(const __half2 *)&v.x), f1 = __half22float2(*(const __half2 *)&v.y);
            const float2 f2 = __half22float2(*(const __half2 *)&v.z), f3 = __half22float2(*(const __half2 *)&v.w);
            xs[((tl * CH + c) * 2 + 0) * 32 + ln] = make_float4(f0.x, f0.y, f1.x, f1.y);
            xs[((tl * CH + c) * 2 + 1) * 32 + ln] = make_float4(f2.x, f2.y, f3.x, f3.y);
        }
        __syncthreads();
        if (r <= E) {
#pragma unroll 1
            for (uint32_t tl = tg; tl < nt; tl += 4) {
                const float4 *xt = xs + tl * CH * 64 + lane;
                float acc = 0.f;
#pragma unroll
                for (int c = 0; c < CH; c++) {
                    const float4 u = xt[c * 64], v = xt[c * 64 + 32];
                    acc = __fmaf_rn(wf[8 * c + 0], u.x, acc);
                    acc = __fmaf_rn(wf[8 * c + 1], u.y, acc);
                    acc = __fmaf_rn(wf[8 * c + 2], u.z, acc);
                    acc = __fmaf_rn(wf[8 * c + 3], u.w, acc);
                    acc = __fmaf_rn(wf[8 * c + 4], v.x, acc);
                    acc = __fmaf_rn(wf[8 * c + 5], v.y, acc);
                    acc = __fmaf_rn(wf[8 * c + 6], v.z, acc);
                    acc = __fmaf_rn(wf[8 * c + 7], v.w, acc);
                }
                const float s = warp_sum_canon(acc);
                if (lane == 0) logits[(size_t)(t0 + tl) * (E + 1) + r] = s;
            }
        }
    }
    pdl_wait();
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        last = atomicAdd(counter, 1u) == gridDim.x - 1;
        __threadfence();
    }
    __syncthreads();
    if (!last) return;
    moe_select_body<512>(logits, ms, E, topk, a);
    if (threadIdx.x == 0) *counter = 0;
}

template <int DD>
static cudaError_t moe_route_go(const QwLaunch &L, unsigned grid, uint32_t E, uint32_t topk, const sel_args &a) {
    cudaError_t e = cudaFuncSetAttribute(moe_route_k<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * DD * 4);
    if (e != cudaSuccess) return e;
    qw_launch(moe_route_k<DD>, grid, 512, 16 * DD * 4, L.stream, L.buf<__half>(0), L.buf<__half>(1), L.buf<__half>(2), L.buf<float>(3), L.buf<unsigned>(4),
              L.buf<moe_sel>(5), E, topk, a);
    return cudaGetLastError();
}

static cudaError_t launch_moe_route(const QwLaunch &L) {
    const uint32_t E = (uint32_t)L.def("E", 512), D = (uint32_t)L.def("D", 2048), topk = (uint32_t)L.def("TOPK", 10);
    sel_args a = L.bytes<sel_args>(14);
    QW_CHECK_ARG(L.has_bytes(14, 12) && a.nb >= 1 && a.nb <= MOE_MAXB);
    for (int i = 0; i <= 5; i++) QW_CHECK_ARG(L.buf<void>(i) != nullptr);
    QW_CHECK_ARG(E % 32 == 0 && (E == 512 || E <= 256) && topk >= 1 && topk < MOE_MAXK && topk <= E);  // E <= the block's 512 threads
    QW_CHECK_ARG(L.avail(0) >= (size_t)E * D * 2 && L.avail(1) >= (size_t)D * 2 && L.avail(2) >= (size_t)a.nb * D * 2 &&
                 L.avail(3) >= (size_t)a.nb * (E + 1) * 4 && L.avail(4) >= 4 && L.avail(5) >= sizeof(moe_sel));
    if (a.e_hi > E) a.e_hi = E;
    const unsigned grid = (E + 1 + 3) / 4;  // (the grid given by the host is ignored)
    if (D == 2048) return moe_route_go<2048>(L, grid, E, topk, a);
    if (D == 256) return moe_route_go<256>(L, grid, E, topk, a);
    return cudaErrorInvalidValue;
}
QW_FAMILY(moe_route, launch_moe_route, 1024)

// ------------------------------------------------------------------------------------------------ gate/up and down
// Persistent blocks of 8 warps; item = (group u, row tile).  Group U (one past the routed groups) is the
// shared expert with every token at rank topk.
struct MoeP {
    const uint8_t *Wa, *Wb;     // gate/up: routed gate and up [E][I][rb]; down: routed down [E][D][rb] in Wa
    const uint8_t *Sa, *Sb;     // shared expert's matrices (same shapes without the E axis); nullptr: no shared expert
    const __half *x;            // gate/up: tokens fp16 [nb][D]
    uint16_t *Hhi, *Hlo;        // [nb][topk+1][I] bf16 planes
    float *Pg;                  // down: [nb][topk+1][D]
    const moe_sel *ms;
    const QwTables *tab;
    unsigned *status;
    uint32_t D, I, rbD, rbI, tiles;
    uint32_t ebase;             // id of the first expert stored in Wa / Wb (expert-parallel slice)
    // expert-parallel exchange fused into the down projection (nranks > 1): every output row is stored into the Pg
    // buffer of every rank (peer memory), then the last block publishes this rank's sequence number to every rank
    float *PgR[8];              // Pg of rank r (PgR[rank] is the local one)
    EpPeers ep;                 // ep.nranks == 1: single GPU or NCCL exchange
};

constexpr int MOE_STG = 2;                             // staged tiles per team (28 KB each)
constexpr int MOE_TAB_BYTES = 512 * 16 * 8;
constexpr int MOE_RED_BYTES = 2 * 2 * 16 * 32 * 16;  // gate/up: per team two buffers (alternating by unit) of 16 x 32 float4
constexpr int MOE_DN_ROWS = 128;                       // rows of a down-projection tile: 16 per consumer warp

// Barrier among the 8 warps of a team, built on an mbarrier (one arrival per warp) so that the wait is bounded like every other
// wait of these kernels: a warp that gave up elsewhere and left cannot strand its team in a hardware barrier.  ph counts
// the team's barriers so far (its parity selects the phase).  False after about two seconds without the others.
__device__ __forceinline__ bool team_sync(uint64_t *bar, uint32_t &ph, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
    const bool ok = mbar_wait(bar, ph & 1);
    ph++;
    __syncwarp();
    return ok;
}

// Work units = (group, pass of 8 token columns, row tile), enumerated group-major, then pass, then tile, so that a team's
// contiguous range keeps one set of B fragments for many consecutive units and every team gets the same number of units
// whatever the group sizes.  Group U (one past the routed groups) is the shared expert with every token at rank topk.
// pre[g] = passes of all groups before g (shared memory, MOE_MAXE + 2 words).  Called by every thread of the block.
struct MoeSched {
    uint32_t U, nb, topk, groups, i0, i1;
};
template <int NTHR>
__device__ __forceinline__ MoeSched moe_sched(const moe_sel *ms, bool shared_expert, uint32_t tiles, uint32_t *pre, int tid, uint32_t team_id, uint32_t teams) {
    // the selection already left the prefix sums of passes over the routed groups (ms->pre[0..U]); all loads here are
    // independent of one another, so the table is in shared memory after one memory latency
    MoeSched w;
    for (uint32_t gi = tid; gi <= MOE_MAXE; gi += NTHR) pre[gi] = ms->pre[gi];
    w.U = ms->U;
    w.nb = ms->nb;
    w.topk = ms->topk;
    w.groups = w.U + (shared_expert ? 1u : 0u);
    __syncthreads();
    if (tid == 0 && shared_expert) pre[w.U + 1] = pre[w.U] + (w.nb + 7) / 8;
    __syncthreads();
    const uint32_t total = pre[w.groups] * tiles;
    w.i0 = (uint32_t)((uint64_t)total * team_id / teams);
    w.i1 = (uint32_t)((uint64_t)total * (team_id + 1) / teams);
    return w;
}
__device__ __forceinline__ void moe_locate(const uint32_t *pre, uint32_t groups, uint32_t tiles, uint32_t w, uint32_t &u, uint32_t &pass, uint32_t &tile) {
    const uint32_t q = w / tiles;
    tile = w % tiles;
    uint32_t lo = 0, hi = groups;  // largest u with pre[u] <= q
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (pre[mid] <= q) lo = mid;
        else hi = mid;
    }
    u = lo;
    pass = q - pre[lo];
}
// Column col of a unit's pass -> (token, rank); false when the pass has fewer columns.
__device__ __forceinline__ bool moe_entry(const moe_sel *ms, uint32_t u, uint32_t U, uint32_t e0, uint32_t c0, uint32_t cnt, uint32_t topk, uint32_t col,
                                          uint32_t &tok, uint32_t &rank) {
    if (c0 + col >= cnt) return false;
    if (u < U) {
        const uint32_t en = ms->ent[e0 + c0 + col];
        tok = en >> 8;
        rank = en & 255;
    } else {
        tok = c0 + col;
        rank = topk;
    }
    return true;
}

// ---- gate/up.  Persistent blocks of two teams of 8 warps; a unit is 16 gate rows + 16 up rows of one expert over the
// full K, warp = K-slice of 256: the same warp does the gate rows and then the up rows of its slice, so one set of B
// fragments (32 registers) serves both.  Partial sums of the 8 slices meet in shared memory; four warps finish the unit
// (SiLU(g) * u as bf16 high + low planes) while the other four already start on the next one.
__global__ void __launch_bounds__(512, 1) moe_gu_k(const MoeP p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = (uint64_t *)smem;  // [team * MOE_STG + stage], then the table's
    uint2 *tab = (uint2 *)(smem + 128);
    const int tid = threadIdx.x, team = tid >> 8, tt = tid & 255, warp = tt >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    float4 *red0 = (float4 *)(smem + 128 + MOE_TAB_BYTES) + team * 2 * 16 * 32;
    const uint32_t rb = p.rbD, units = p.D / 256;
    const uint32_t tile_bytes = 2 * 16 * rb, half_bytes = 16 * rb;
    const uint32_t stage_stride = (tile_bytes + 127) & ~127u;
    uint8_t *stage0 = smem + 128 + MOE_TAB_BYTES + MOE_RED_BYTES + (size_t)team * MOE_STG * stage_stride;
    const uint32_t KS = units < 8 ? units : 8, ks = warp;
    const bool active = ks < KS;
    // independent of earlier kernels: barriers and the codebook table (thread 0 both initialises and uses the table's
    // barrier here; the other threads see the initialised barriers after the __syncthreads in moe_sched)
    uint64_t *tab_bar = bars + 2 * MOE_STG, *team_bar = tab_bar + 1 + team;
    uint32_t team_ph = 0;
    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < 2 * MOE_STG + 1; s++) mbar_init(&bars[s], 1);
        mbar_init(tab_bar + 1, 8);
        mbar_init(tab_bar + 2, 8);
        mbar_init_fence();
        mbar_expect_tx(tab_bar, MOE_TAB_BYTES);
        bulk_g2s(tab, p.tab->grid_h4, MOE_TAB_BYTES, tab_bar);
    }
    pdl_wait();  // the selection record, the tokens and the H planes belong to earlier kernels
    const moe_sel *ms = p.ms;
    __shared__ uint32_t pre[MOE_MAXE + 2];
    const MoeSched w = moe_sched<512>(ms, p.Sa != nullptr, p.tiles, pre, tid, blockIdx.x * 2 + team, gridDim.x * 2);
    const uint32_t U = w.U, nb = w.nb, topk = w.topk, i0 = w.i0, i1 = w.i1;
    uint64_t *full = bars + team * MOE_STG;
    __shared__ uint4 meta[2][MOE_STG];  // per team and stage: {group, tile, first entry of the group, entries in the group}
    __shared__ uint32_t meta_c0[2][MOE_STG];
    auto issue = [&](uint32_t i) {  // team leader only: locate the unit, publish its description, start the copies
        if (i0 + i >= i1) return;
        uint32_t u, pass, tile;
        moe_locate(pre, w.groups, p.tiles, i0 + i, u, pass, tile);
        const uint32_t e0 = u < U ? ms->off[u] : 0, cnt = u < U ? ms->off[u + 1] - e0 : nb;
        meta[team][i % MOE_STG] = make_uint4(u, tile, e0, cnt);
        meta_c0[team][i % MOE_STG] = pass * 8;
        uint8_t *dst = stage0 + (size_t)(i % MOE_STG) * stage_stride;
        mbar_expect_tx(&full[i % MOE_STG], tile_bytes);
        const size_t o = u < U ? ((size_t)(ms->ue[u] - p.ebase) * p.I + (size_t)tile * 16) * rb : (size_t)tile * 16 * rb;
        bulk_g2s(dst, (u < U ? p.Wa : p.Sa) + o, half_bytes, &full[i % MOE_STG]);
        bulk_g2s(dst + half_bytes, (u < U ? p.Wb : p.Sb) + o, half_bytes, &full[i % MOE_STG]);
    };
    if (tt == 0)
        for (uint32_t i = 0; i + 1 < MOE_STG; i++) issue(i);
    bool ok = mbar_wait(tab_bar, 0);
    const uint32_t tabc = smem_u32(tab) + (lane & 15) * 8;  // this lane's copy of the interleaved codebook

    const ZeroRegs zr = zero_regs();
    uint4 xf[8];  // B fragments of the warp's K-slice: column g = entry c0 + g of the group
    uint32_t cur_u = 0xffffffffu, cur_c0 = 0;
    uint32_t oo = 0xffffffffu;  // element offset of the H row of this thread's epilogue column (~0 = column absent)

    for (uint32_t i = 0; ok && i0 + i < i1; i++) {
        if (tt == 0) issue(i + MOE_STG - 1);
        if (!mbar_wait(&full[i % MOE_STG], (i / MOE_STG) & 1)) {
            ok = false;
            break;
        }
        // the leader wrote the unit's description before its mbarrier arrive (release); the wait above acquires it
        const uint4 md = meta[team][i % MOE_STG];
        const uint32_t u = md.x, tile = md.y, e0 = md.z, cnt = md.w, c0 = meta_c0[team][i % MOE_STG];
        const uint32_t st = smem_u32(stage0) + (i % MOE_STG) * stage_stride;  // shared-space address of the staged tile
        // partial tiles alternate between two buffers, so one team barrier per unit is enough: a buffer is rewritten two
        // units later, after every thread has passed the next unit's barrier; the same barrier frees the stage for the
        // copy that the leader starts at the top of the next iteration
        float4 *red = red0 + (i & 1) * 16 * 32;
        if (u != cur_u || c0 != cur_c0) {  // new (group, pass): team-uniform
            cur_u = u;
            cur_c0 = c0;
            uint32_t tok = 0, rank = 0;
            // epilogue column of this thread: 2 * ((tt >> 2) & 3) + (tt & 1)
            oo = moe_entry(ms, u, U, e0, c0, cnt, topk, 2 * ((tt >> 2) & 3) + (tt & 1), tok, rank) ? (tok * (topk + 1) + rank) * p.I : 0xffffffffu;
            if (active) {
                tok = 0;
                const bool have = moe_entry(ms, u, U, e0, c0, cnt, topk, g, tok, rank);
                const uint4 zero = make_uint4(0, 0, 0, 0);
                const uint4 *xr = (const uint4 *)(p.x + (size_t)tok * p.D) + ks * 32 + t;
#pragma unroll
                for (int ib = 0; ib < 8; ib++) xf[ib] = have ? __ldcg(xr + 4 * ib) : zero;
            }
        }
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        if (active) {
#pragma unroll
            for (int j = 0; j < 2; j++) {  // gate rows, then up rows, of unit ks
                const uint32_t rows = st + j * half_bytes + g * rb + ks * 110;
                unit_mma1<false>(rows, rows + 8 * rb, tabc, t, zr, xf, xf, acc[j]);
            }
        }
        red[(warp * 2 + 0) * 32 + lane] = make_float4(acc[0][0], acc[0][1], acc[0][2], acc[0][3]);
        red[(warp * 2 + 1) * 32 + lane] = make_float4(acc[1][0], acc[1][1], acc[1][2], acc[1][3]);
        if (!team_sync(team_bar, team_ph, lane)) {
            ok = false;
            break;
        }
        if (tt < 128) {
            const int jj = tt & 3, ln = tt >> 2;
            float gs = 0.f, us = 0.f;
            for (uint32_t k2 = 0; k2 < KS; k2++) {
                gs += ((const float *)&red[(k2 * 2 + 0) * 32 + ln])[jj];
                us += ((const float *)&red[(k2 * 2 + 1) * 32 + ln])[jj];
            }
            if (oo != 0xffffffffu) {
                const uint32_t row = tile * 16 + (ln >> 2) + 8 * (jj >> 1);
                const float h = gs / (1.0f + expf(-gs)) * us;
                const __nv_bfloat16 hi = __float2bfloat16_rn(h);
                const __nv_bfloat16 lo = __float2bfloat16_rn(h - __bfloat162float(hi));
                const size_t ho = (size_t)oo + row;
                p.Hhi[ho] = __bfloat16_as_ushort(hi);
                p.Hlo[ho] = __bfloat16_as_ushort(lo);
            }
        }
    }
    if (!ok && lane == 0) set_status(p.status, ST_MBAR_TIMEOUT | 2);
}

// ---- down.  Persistent blocks of two teams; a team = 8 consumer warps + 1 producer warp.  A unit is 128 rows of one
// expert's down matrix over the full K (28 KB); consumer warp w owns rows 16w .. 16w+15 over all of K, so nothing is
// exchanged between warps and there is no team barrier per unit: the producer's copy completes the stage's "full"
// mbarrier, each consumer warp arrives on its "empty" mbarrier when it has read the tile, and a warp stores its
// 16 x 8 outputs straight from the accumulators.  The H rows of the pass (bf16 high and low planes of up to 8
// (token, rank) columns) sit in shared memory, padded so that the B-fragment loads of a quarter warp hit 8 different
// 16-byte bank groups; they are reloaded (two consumer barriers) only when (group, pass) changes.  MMA row g of a warp is
// tile row 16w + 2g, row g + 8 is 16w + 2g + 1: with 220-byte rows that keeps the raw-byte loads free of bank conflicts,
// and a lane's two rows of a column are one 8-byte store.
constexpr int MOE_DN_THREADS = 2 * 9 * 32;
template <int IB>
__device__ __forceinline__ void dn_sub(uint32_t u0, uint32_t u1, int t, const Iq3sHdr &h0, const Iq3sHdr &h1, uint32_t tabc, const ZeroRegs &zr, uint32_t hb_hi,
                                       uint32_t hb_lo, float (&acc)[4]) {
    const uint4 xv = lds_v4(hb_hi + IB * 64), xl = lds_v4(hb_lo + IB * 64);
    sub_mma1<true, IB, 128>(u0, u1, t, h0, h1, tabc, zr, xv, xl, acc);
}
__global__ void __launch_bounds__(MOE_DN_THREADS, 1) moe_dn_k(const MoeP p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = (uint64_t *)smem;  // full[team][stage], empty[team][stage], table
    uint2 *tab = (uint2 *)(smem + 128);
    const int tid = threadIdx.x, team = tid / 288, tt = tid % 288, warp = tt >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const uint32_t rb = p.rbI, units = p.I / 256;
    const uint32_t hs_stride = p.I * 2 + 64, hs_bytes = 16 * hs_stride;  // [plane][column] rows of I bf16 + 64 bytes of padding
    uint8_t *hs = smem + 128 + MOE_TAB_BYTES + (size_t)team * hs_bytes;
    const uint32_t tile_bytes = MOE_DN_ROWS * rb, stage_stride = (tile_bytes + 127) & ~127u;
    uint8_t *stage0 = smem + 128 + MOE_TAB_BYTES + 2 * hs_bytes + (size_t)team * MOE_STG * stage_stride;
    uint64_t *full = bars + team * MOE_STG, *empty = bars + 2 * MOE_STG + team * MOE_STG, *tab_bar = bars + 4 * MOE_STG, *team_bar = tab_bar + 1 + team;
    uint32_t team_ph = 0;
    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < 2 * MOE_STG; s++) {
            mbar_init(&bars[s], 1);
            mbar_init(&bars[2 * MOE_STG + s], 8);  // one arrival per consumer warp
        }
        mbar_init(tab_bar, 1);
        mbar_init(tab_bar + 1, 8);
        mbar_init(tab_bar + 2, 8);
        mbar_init_fence();
        mbar_expect_tx(tab_bar, MOE_TAB_BYTES);
        bulk_g2s(tab, p.tab->grid_b4, MOE_TAB_BYTES, tab_bar);
    }
    pdl_wait();  // the selection record, the H planes and the outputs belong to earlier kernels
    const moe_sel *ms = p.ms;
    __shared__ uint32_t pre[MOE_MAXE + 2];
    const MoeSched w = moe_sched<MOE_DN_THREADS>(ms, p.Sa != nullptr, p.tiles, pre, tid, blockIdx.x * 2 + team, gridDim.x * 2);
    const uint32_t U = w.U, nb = w.nb, topk = w.topk, i0 = w.i0, i1 = w.i1;
    __shared__ uint4 meta[2][MOE_STG];  // per team and stage: {group, tile, first entry of the group, entries in the group}
    __shared__ uint32_t meta_c0[2][MOE_STG];
    bool ok = true;
    if (warp == 8) {
        // ---- producer: one lane walks the team's units, reusing a stage as soon as all 8 consumer warps have left it
        if (lane == 0) {
            for (uint32_t i = 0; i0 + i < i1; i++) {
                const uint32_t s = i % MOE_STG;
                if (i >= MOE_STG && !mbar_wait(&empty[s], (i / MOE_STG - 1) & 1)) {
                    ok = false;
                    break;
                }
                uint32_t u, pass, tile;
                moe_locate(pre, w.groups, p.tiles, i0 + i, u, pass, tile);
                const uint32_t e0 = u < U ? ms->off[u] : 0, cnt = u < U ? ms->off[u + 1] - e0 : nb;
                meta[team][s] = make_uint4(u, tile, e0, cnt);
                meta_c0[team][s] = pass * 8;
                mbar_expect_tx(&full[s], tile_bytes);
                const uint8_t *src = u < U ? p.Wa + ((size_t)(ms->ue[u] - p.ebase) * p.D + (size_t)tile * MOE_DN_ROWS) * rb : p.Sa + (size_t)tile * MOE_DN_ROWS * rb;
                bulk_g2s(stage0 + (size_t)s * stage_stride, src, tile_bytes, &full[s]);
            }
            if (!ok) set_status(p.status, ST_MBAR_TIMEOUT | 4);
        }
    } else {
        // ---- consumers
        ok = mbar_wait(tab_bar, 0);
        const uint32_t tabc = smem_u32(tab) + (lane & 15) * 8;  // this lane's copy of the interleaved codebook
        const ZeroRegs zr = zero_regs();
        const uint32_t hb_hi = smem_u32(hs) + g * hs_stride + t * 16, hb_lo = hb_hi + 8 * hs_stride;
        uint32_t cur_u = 0xffffffffu, cur_c0 = 0;
        uint32_t oo[2] = {0xffffffffu, 0xffffffffu};  // element offsets of the output rows of columns 2t and 2t + 1 (~0 = absent)
        for (uint32_t i = 0; ok && i0 + i < i1; i++) {
            const uint32_t s = i % MOE_STG;
            if (!mbar_wait(&full[s], (i / MOE_STG) & 1)) {
                ok = false;
                break;
            }
            // the producer wrote the unit's description before its mbarrier arrive (release); the wait above acquires it
            const uint4 md = meta[team][s];
            const uint32_t u = md.x, tile = md.y, e0 = md.z, cnt = md.w, c0 = meta_c0[team][s];
            if (u != cur_u || c0 != cur_c0) {  // new (group, pass): uniform over the team's consumers
                cur_u = u;
                cur_c0 = c0;
                if (!team_sync(team_bar, team_ph, lane)) {  // every consumer warp is done with the previous pass's H rows
                    ok = false;
                    break;
                }
                const uint32_t i8 = p.I / 8;  // 16-byte pieces per row
                for (uint32_t idx = tt; idx < 16 * i8; idx += 256) {
                    const uint32_t pc = idx / i8, kk = idx - pc * i8, col = pc & 7;
                    uint32_t tok = 0, rank = 0;
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (moe_entry(ms, u, U, e0, c0, cnt, topk, col, tok, rank))
                        v = __ldcg((const uint4 *)((pc < 8 ? p.Hhi : p.Hlo) + ((size_t)tok * (topk + 1) + rank) * p.I) + kk);
                    *(uint4 *)(hs + (size_t)pc * hs_stride + kk * 16) = v;
                }
                uint32_t tok = 0, rank = 0;
                oo[0] = moe_entry(ms, u, U, e0, c0, cnt, topk, 2 * t, tok, rank) ? (tok * (topk + 1) + rank) * p.D : 0xffffffffu;
                oo[1] = moe_entry(ms, u, U, e0, c0, cnt, topk, 2 * t + 1, tok, rank) ? (tok * (topk + 1) + rank) * p.D : 0xffffffffu;
                if (!team_sync(team_bar, team_ph, lane)) {
                    ok = false;
                    break;
                }
            }
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t r0 = smem_u32(stage0) + s * stage_stride + (16 * warp + 2 * g) * rb;
#pragma unroll 1
            for (uint32_t ks = 0; ks < units; ks++) {
                const uint32_t u0 = r0 + ks * 110, u1 = u0 + rb, bh = hb_hi + ks * 512, bl = hb_lo + ks * 512;
                const Iq3sHdr h0 = iq3s_hdr(u0, t), h1 = iq3s_hdr(u1, t);
                dn_sub<0>(u0, u1, t, h0, h1, tabc, zr, bh, bl, acc);
                dn_sub<1>(u0, u1, t, h0, h1, tabc, zr, bh, bl, acc);
                dn_sub<2>(u0, u1, t, h0, h1, tabc, zr, bh, bl, acc);
                dn_sub<3>(u0, u1, t, h0, h1, tabc, zr, bh, bl, acc);
                dn_sub<4>(u0, u1, t, h0, h1, tabc, zr, bh, bl, acc);
                dn_sub<5>(u0, u1, t, h0, h1, tabc, zr, bh, bl, acc);
                dn_sub<6>(u0, u1, t, h0, h1, tabc, zr, bh, bl, acc);
                dn_sub<7>(u0, u1, t, h0, h1, tabc, zr, bh, bl, acc);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);  // this warp has read the tile
            // acc[0], acc[2] = rows 2g and 2g + 1 of column 2t; acc[1], acc[3] = the same rows of column 2t + 1
            const uint32_t row = tile * MOE_DN_ROWS + 16 * warp + 2 * g;
            if (p.ep.nranks > 1) {
                for (uint32_t r = 0; r < p.ep.nranks; r++) {
                    if (oo[0] != 0xffffffffu) *(float2 *)(p.PgR[r] + oo[0] + row) = make_float2(acc[0], acc[2]);
                    if (oo[1] != 0xffffffffu) *(float2 *)(p.PgR[r] + oo[1] + row) = make_float2(acc[1], acc[3]);
                }
            } else {
                if (oo[0] != 0xffffffffu) *(float2 *)(p.Pg + oo[0] + row) = make_float2(acc[0], acc[2]);
                if (oo[1] != 0xffffffffu) *(float2 *)(p.Pg + oo[1] + row) = make_float2(acc[1], acc[3]);
            }
        }
        if (!ok && lane == 0) set_status(p.status, ST_MBAR_TIMEOUT | 3);
    }
    if (p.ep.nranks > 1) ep_publish(p.ep);
}

// binds (gate/up): 0 = Wg, 1 = Wu, 2 = shared gate, 3 = shared up (used unless SHARED is defined 0), 4 = x, 5 = moe_sel,
//                  6 = Hhi, 7 = Hlo.   (down): 0 = Wd, 2 = shared down, 5 = moe_sel, 6 = Hhi, 7 = Hlo, 9 = Pg.
//                  both: 10 = id of the first expert held in the weight buffers (optional, default 0).
// defines: E, D, I, TOPK, EL (experts held locally, default E).  The host's grid and block are ignored (persistent: one block of 512 per SM).
static cudaError_t moe_fill(const QwLaunch &L, MoeP &p, uint32_t &E, uint32_t &topk, bool down) {
    E = (uint32_t)L.def("E", 512);
    topk = (uint32_t)L.def("TOPK", 10);
    p.D = (uint32_t)L.def("D", 2048);
    p.I = (uint32_t)L.def("I", 512);
    QW_CHECK_ARG(p.D % 256 == 0 && p.I % 256 == 0 && p.I % 16 == 0 && p.D % 128 == 0 && (L.tx == 256 || L.tx == 512));
    p.rbD = p.D / 256 * 110;
    p.rbI = p.I / 256 * 110;
    QW_CHECK_ARG((16 * p.rbD) % 16 == 0 && (MOE_DN_ROWS * p.rbI) % 16 == 0);
    p.Wa = L.buf<uint8_t>(0);
    p.Wb = L.buf<uint8_t>(1);
    const bool shared = L.def("SHARED", 1) != 0;  // bind slots persist across dispatches: optional inputs are opted into by a define
    p.Sa = shared ? L.buf<uint8_t>(2) : nullptr;
    p.Sb = shared && !down ? L.buf<uint8_t>(3) : nullptr;
    QW_CHECK_ARG(!shared || p.Sa);
    p.x = L.buf<__half>(4);
    p.ms = L.buf<moe_sel>(5);
    p.Hhi = L.buf<uint16_t>(6);
    p.Hlo = L.buf<uint16_t>(7);
    p.Pg = L.buf<float>(9);
    p.tab = (const QwTables *)L.tables;
    p.status = L.status;
    p.ep = EpPeers{};
    p.ep.nranks = 1;
    for (int r = 0; r < 8; r++) p.PgR[r] = nullptr;
    if (down && L.def("EPX", 0) > 1) {
        // binds 16 + r = Pg of rank r, 24 + r = flag array of rank r, 11 = {seq, done} counters (local, 8 bytes, zeroed),
        // 12 = {rank}; define EPX = number of ranks (2..8)
        p.ep.nranks = (uint32_t)L.def("EPX", 0);
        QW_CHECK_ARG(p.ep.nranks <= 8 && L.has_bytes(12, 4) && L.buf<unsigned>(11) && L.avail(11) >= 8);
        p.ep.rank = L.bytes<uint32_t>(12);
        QW_CHECK_ARG(p.ep.rank < p.ep.nranks);
        p.ep.seq = L.buf<unsigned>(11);
        p.ep.done = p.ep.seq + 1;
        for (uint32_t r = 0; r < p.ep.nranks; r++) {
            p.PgR[r] = L.buf<float>(16 + r);
            p.ep.flagR[r] = L.buf<unsigned>(24 + r);
            QW_CHECK_ARG(p.PgR[r] && p.ep.flagR[r] && L.avail(24 + r) >= p.ep.nranks * 4);
        }
    }
    // experts held in the bound weight buffers: EL of them starting at id bytes(10) (default: all E from 0);
    // moe_select must have been given the same range
    const uint32_t EL = (uint32_t)L.def("EL", E);
    p.ebase = L.has_bytes(10, 4) ? L.bytes<uint32_t>(10) : 0;
    QW_CHECK_ARG(EL >= 1 && p.ebase + EL <= E);
    const size_t wsz = (size_t)EL * p.I * p.rbD;  // == EL * D * rbI
    QW_CHECK_ARG(p.Wa && p.ms && p.Hhi && p.Hlo && L.avail(0) >= wsz && L.avail(5) >= sizeof(moe_sel));
    QW_CHECK_ARG(((uintptr_t)p.Wa & 15) == 0 && ((uintptr_t)p.Sa & 15) == 0 && ((uintptr_t)p.Hhi & 15) == 0 && ((uintptr_t)p.Hlo & 15) == 0);
    const size_t hsz = (size_t)MOE_MAXB * (topk + 1) * p.I * 2;
    QW_CHECK_ARG(L.avail(6) >= hsz && L.avail(7) >= hsz);
    if (p.Sa) QW_CHECK_ARG(L.avail(2) >= (size_t)p.I * p.rbD);
    if (!down) {
        QW_CHECK_ARG(p.Wb && p.x && L.avail(1) >= wsz && ((uintptr_t)p.Wb & 15) == 0 && ((uintptr_t)p.x & 15) == 0 && ((uintptr_t)p.Sb & 15) == 0);
        QW_CHECK_ARG((p.Sa == nullptr) == (p.Sb == nullptr));
        if (p.Sb) QW_CHECK_ARG(L.avail(3) >= (size_t)p.I * p.rbD);
        p.tiles = p.I / 16;
    } else {
        QW_CHECK_ARG(p.Pg && L.avail(9) >= (size_t)MOE_MAXB * (topk + 1) * p.D * 4);
        for (uint32_t r = 0; r < p.ep.nranks && p.ep.nranks > 1; r++) QW_CHECK_ARG(L.avail(16 + r) >= (size_t)MOE_MAXB * (topk + 1) * p.D * 4);
        p.tiles = p.D / MOE_DN_ROWS;
    }
    return cudaSuccess;
}

static cudaError_t moe_gu_go(const MoeP &p, int sm_count, cudaStream_t st) {
    const uint32_t tile_bytes = 2 * 16 * p.rbD;
    const size_t smem = 128 + MOE_TAB_BYTES + MOE_RED_BYTES + (size_t)2 * MOE_STG * ((tile_bytes + 127) & ~127u);
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(moe_gu_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    qw_launch(moe_gu_k, sm_count, 512, smem, st, p);
    return cudaGetLastError();
}
static cudaError_t moe_dn_go(const MoeP &p, int sm_count, cudaStream_t st) {
    const uint32_t tile_bytes = MOE_DN_ROWS * p.rbI;
    const size_t smem = 128 + MOE_TAB_BYTES + (size_t)2 * 16 * (p.I * 2 + 64) + (size_t)2 * MOE_STG * ((tile_bytes + 127) & ~127u);
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(moe_dn_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    qw_launch(moe_dn_k, sm_count, MOE_DN_THREADS, smem, st, p);
    return cudaGetLastError();
}

static cudaError_t launch_moe_gu(const QwLaunch &L) {
    MoeP p;
    uint32_t E, topk;
    cudaError_t e = moe_fill(L, p, E, topk, false);
    if (e != cudaSuccess) return e;
    const uint32_t units = p.D / 256;
    QW_CHECK_ARG(units == 1 || units == 2 || units == 4 || units == 8);
    return moe_gu_go(p, L.sm_count, L.stream);
}
QW_FAMILY(moe_gu, launch_moe_gu, 512)

static cudaError_t launch_moe_dn(const QwLaunch &L) {
    MoeP p;
    uint32_t E, topk;
    cudaError_t e = moe_fill(L, p, E, topk, true);
    if (e != cudaSuccess) return e;
    QW_CHECK_ARG(p.I / 256 <= 2);
    return moe_dn_go(p, L.sm_count, L.stream);
}
QW_FAMILY(moe_dn, launch_moe_dn, 512)

// ------------------------------------------------------------------------------------------------ combine
// out[t][r] = fp16( sum_{s < topk, rank order} w[t][s] * Pg[t][s][r]  +  w[t][topk] * Pg[t][topk][r] )
// binds: 3 = moe_sel, 4 = out fp16 [nb][D], 9 = Pg, 8 = nb; with RESID defined 1 also 5 = residual fp32 [nb][D]
// updated in place (h += out, the plain residual that stands in for the reference's hyper-connection mix).
// grid (D/256, nb) x 256
__global__ void __launch_bounds__(256) moe_cmb_k(const moe_sel *ms, __half *out, const float *Pg, float *resid, uint32_t D, uint32_t topk, uint32_t nb) {
    pdl_sync();
    const uint32_t row = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
    if (row >= D || t >= nb) return;
    float o = 0.f;
    for (uint32_t s = 0; s <= topk; s++) o = fmaf(ms->w[t][s], Pg[((size_t)t * (topk + 1) + s) * D + row], o);
    const __half h = __float2half_rn(o);
    out[(size_t)t * D + row] = h;
    if (resid) resid[(size_t)t * D + row] += __half2float(h);
}

static cudaError_t launch_moe_cmb(const QwLaunch &L) {
    const uint32_t D = (uint32_t)L.def("D", 2048), topk = (uint32_t)L.def("TOPK", 10);
    const uint32_t nb = L.bytes<uint32_t>(8);
    QW_CHECK_ARG(L.buf<void>(3) && L.buf<void>(4) && L.buf<void>(9) && nb >= 1 && nb <= MOE_MAXB);
    QW_CHECK_ARG(L.avail(3) >= sizeof(moe_sel) && L.avail(4) >= (size_t)nb * D * 2 && L.avail(9) >= (size_t)nb * (topk + 1) * D * 4);
    float *resid = L.def("RESID", 0) ? L.buf<float>(5) : nullptr;
    if (L.def("RESID", 0)) QW_CHECK_ARG(resid && L.avail(5) >= (size_t)nb * D * 4);
    qw_launch(moe_cmb_k, dim3((D + 255) / 256, nb), 256, 0, L.stream, L.buf<moe_sel>(3), L.buf<__half>(4), L.buf<float>(9), resid, D, topk, nb);
    return cudaGetLastError();
}
QW_FAMILY(moe_cmb, launch_moe_cmb, 256)

// size of struct moe_sel for hosts that allocate it (bind 1 of moe_select)
extern "C" size_t qw_moe_sel_bytes(void) { return sizeof(moe_sel); }
