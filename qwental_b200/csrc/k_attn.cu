// Ragged paged-KV gated GQA decode attention for all slots in one launch: split-K over the slot's pages with a
// log-sum-exp merge.
//
//   qsa_prep   per head: RMSNorm(q)*w, partial RoPE (first 64 dims, pairs (i, i+32), theta 1e7), write q;
//              RMSNorm(k)*w + RoPE -> K page, v -> V page at the slot's position
//              -- role of qsa_prep_f, kernels/qsa_dec.metal:68-127 (dense part: no indexer)
//   qsa_attn   one block per (page chunk, kv head, slot): online softmax over the chunk's tokens for the
//              GQA = QH/KVH query heads of that kv head, partial (acc, m, l) out
//              -- role of qsa_attn5 (dense branch), kernels/qsa_dec.metal:481-600
//   qsa_merge  log-sum-exp merge of a slot's partials in chunk order, y = fp16(fp16(o/L) * sigmoid(gate));
//              gate = second half of each head's q-projection output
//              -- role of qsa_merge4, kernels/qsa_dec.metal:609-645
//
// KV layout (new; the reference keeps one contiguous buffer per slot, src/engine.c:857-930): a pool of pages of
// 256 tokens; page p, attention layer l holds K [KVH][256][HD] then V [KVH][256][HD] in fp16, so one kv head's
// 256 keys are one contiguous 128 KB run.  A slot owns a list of page ids (its page table row).
// The reference launches the core once per slot (src/engine.c:8948-8959); here slot and chunk are grid
// dimensions, chunks past a slot's length exit at once, and the chunking of a slot depends only on its own
// length, so a slot's result is bit-identical alone or in any batch.
#include "common.cuh"
#include "qw_kern.h"
#include <cuda.h>
#include <cstdio>
#include <map>
#include <mutex>

using namespace qw;

#define QSA_EPS 1e-6f
#define QSA_PAGE 256

struct qsa_args {
    uint32_t nb, layer, nlayers, qkv_stride;  // qkv row: [QH x (q HD | gate HD)] [KVH x k HD] [KVH x v HD]
    uint32_t max_pages, max_chunks, pad0, pad1;
};

__device__ __forceinline__ size_t page_base(uint32_t page, uint32_t layer, uint32_t nlayers, uint32_t KVH, uint32_t HD) {
    return ((size_t)page * nlayers + layer) * 2 * KVH * QSA_PAGE * HD;  // in halves
}

// binds: 0 = qkv fp16 [nb][qkv_stride], 1 = q norm w fp32 [HD], 2 = k norm w fp32 [HD], 3 = q out fp16 [nb][QH][HD],
// 4 = KV pool fp16, 5 = page table int32 [slots][max_pages], 6 = pos int32 [nb] (tokens already in the cache),
// 7 = slot ids int32 [nb], 8 = qsa_args.   grid (QH + KVH, nb) x 256 (HD = 256)
__global__ void __launch_bounds__(256) qsa_prep_k(const __half *qkv, const float *qn, const float *kn, __half *q, __half *pool, const int32_t *pt,
                                                  const int32_t *posv, const int32_t *sids, qsa_args a, uint32_t QH, uint32_t KVH) {
    constexpr uint32_t HD = 256, RD = 64;
    __shared__ float tmp[8], v[HD];
    pdl_sync();
    const uint32_t hh = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t pos = (uint32_t)posv[t];
    const bool isq = hh < QH;
    const uint32_t kh = hh - QH;
    const __half *row = qkv + (size_t)t * a.qkv_stride;
    const float x = isq ? __half2float(row[hh * 2 * HD + tid]) : __half2float(row[QH * 2 * HD + kh * HD + tid]);
    const float p = warp_sum(x * x);
    if (lane == 0) tmp[warp] = p;
    __syncthreads();
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) ss += tmp[i];
    const float r = rsqrtf(ss / HD + QSA_EPS);
    v[tid] = x * r * (isq ? qn[tid] : kn[tid]);
    __syncthreads();
    if (tid < RD / 2) {
        const float f = powf(10000000.0f, -(float)(2 * tid) / (float)RD) * (float)pos;
        const float c = cosf(f), s = sinf(f);
        const float x1 = v[tid], x2 = v[tid + RD / 2];
        v[tid] = x1 * c - x2 * s;
        v[tid + RD / 2] = x2 * c + x1 * s;
    }
    __syncthreads();
    if (isq) {
        q[((size_t)t * QH + hh) * HD + tid] = __float2half_rn(v[tid]);
    } else {
        const uint32_t page = (uint32_t)pt[(size_t)sids[t] * a.max_pages + pos / QSA_PAGE];
        __half *pb = pool + page_base(page, a.layer, a.nlayers, KVH, HD);
        const size_t o = ((size_t)kh * QSA_PAGE + pos % QSA_PAGE) * HD + tid;
        pb[o] = __float2half_rn(v[tid]);
        pb[(size_t)KVH * QSA_PAGE * HD + o] = row[QH * 2 * HD + KVH * HD + kh * HD + tid];
    }
}

static bool qsa_dims(const QwLaunch &L, uint32_t &QH, uint32_t &KVH, uint32_t &HD) {
    QH = (uint32_t)L.def("QH", 16);
    KVH = (uint32_t)L.def("KVH", 2);
    HD = (uint32_t)L.def("HD", 256);
    return HD == 256 && QH % KVH == 0 && QH / KVH == 8;
}

static cudaError_t launch_qsa_prep(const QwLaunch &L) {
    uint32_t QH, KVH, HD;
    QW_CHECK_ARG(qsa_dims(L, QH, KVH, HD));
    qsa_args a = L.bytes<qsa_args>(8);
    QW_CHECK_ARG(L.has_bytes(8, 24) && a.nb >= 1 && a.nb <= 64 && a.layer < a.nlayers && a.qkv_stride >= QH * 2 * HD + 2 * KVH * HD);
    for (int i = 0; i <= 7; i++) QW_CHECK_ARG(L.buf<void>(i) != nullptr);
    QW_CHECK_ARG(L.avail(0) >= ((size_t)(a.nb - 1) * a.qkv_stride + QH * 2 * HD + 2 * KVH * HD) * 2 && L.avail(3) >= (size_t)a.nb * QH * HD * 2 &&
                 L.avail(6) >= (size_t)a.nb * 4 && L.avail(7) >= (size_t)a.nb * 4 && L.tx == 256);
    qw_launch(qsa_prep_k, dim3(QH + KVH, a.nb), 256, 0, L.stream, L.buf<__half>(0), L.buf<float>(1), L.buf<float>(2), L.buf<__half>(3), L.buf<__half>(4),
                                                          L.buf<int32_t>(5), L.buf<int32_t>(6), L.buf<int32_t>(7), a, QH, KVH);
    return cudaGetLastError();
}
QW_FAMILY(qsa_prep, launch_qsa_prep, 256)

// ------------------------------------------------------------------------------------------------ attention core
// Chunk = one page (256 tokens).  Block = 8 warps = the 8 query heads of one kv head; lane owns 8 of the 256
// dims; 4 tokens per iteration (scores by warp reduction, then the online-softmax update), the expression of
// kernels/qsa_dec.metal:520-539.  part [nb][max_chunks][QH][HD + 2] fp32 (acc, m, l).
// binds: 0 = q fp16 [nb][QH][HD], 1 = KV pool, 2 = page table, 3 = pos (tokens in the cache before this step;
// the step's own token was appended by qsa_prep, so the slot attends to pos + 1 tokens), 4 = slot ids,
// 5 = part, 6 = qsa_args.   grid (max_chunks, KVH, nb) x 256
__global__ void __launch_bounds__(256) qsa_attn_k(const __half *q, const __half *pool, const int32_t *pt, const int32_t *posv, const int32_t *sids,
                                                  float *part, qsa_args a, uint32_t QH, uint32_t KVH) {
    constexpr uint32_t HD = 256, PL = 8, U4 = 4;
    pdl_sync();
    const uint32_t ch = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const uint32_t ntok = (uint32_t)posv[t] + 1;
    if (ch * QSA_PAGE >= ntok) return;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, qh = kvh * 8 + warp;
    const uint32_t n = min((uint32_t)QSA_PAGE, ntok - ch * QSA_PAGE);
    const uint32_t page = (uint32_t)pt[(size_t)sids[t] * a.max_pages + ch];
    const __half *Kp = pool + page_base(page, a.layer, a.nlayers, KVH, HD) + (size_t)kvh * QSA_PAGE * HD + lane * PL;
    const __half *Vp = Kp + (size_t)KVH * QSA_PAGE * HD;
    const float scale = rsqrtf((float)HD);
    float qv[PL], acc[PL];
    {
        const uint4 qq = *(const uint4 *)(q + ((size_t)t * QH + qh) * HD + lane * PL);
        const uint32_t w4[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(*(const __half2 *)&w4[j]);
            qv[2 * j] = f.x * scale;
            qv[2 * j + 1] = f.y * scale;
        }
    }
#pragma unroll
    for (int d = 0; d < PL; d++) acc[d] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (uint32_t i = 0; i < n; i += U4) {
        float s[U4];
        uint4 vv[U4];
#pragma unroll
        for (uint32_t u = 0; u < U4; u++) {
            const bool ok = i + u < n;
            const uint32_t tk = ok ? i + u : i;
            const uint4 kk = __ldcg((const uint4 *)(Kp + (size_t)tk * HD));
            vv[u] = __ldcg((const uint4 *)(Vp + (size_t)tk * HD));
            const uint32_t w4[4] = {kk.x, kk.y, kk.z, kk.w};
            float d = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(*(const __half2 *)&w4[j]);
                d = fmaf(f.x, qv[2 * j], d);
                d = fmaf(f.y, qv[2 * j + 1], d);
            }
            d = warp_sum(d);
            s[u] = ok ? d : -INFINITY;
        }
        float mn = m;
#pragma unroll
        for (uint32_t u = 0; u < U4; u++) mn = fmaxf(mn, s[u]);
        const float alpha = expf(m - mn);
        l *= alpha;
#pragma unroll
        for (int d = 0; d < PL; d++) acc[d] *= alpha;
#pragma unroll
        for (uint32_t u = 0; u < U4; u++) {
            const float p = expf(s[u] - mn);
            l += p;
            const uint32_t w4[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(*(const __half2 *)&w4[j]);
                acc[2 * j] = fmaf(p, f.x, acc[2 * j]);
                acc[2 * j + 1] = fmaf(p, f.y, acc[2 * j + 1]);
            }
        }
        m = mn;
    }
    float *o = part + (((size_t)t * a.max_chunks + ch) * QH + qh) * (HD + 2);
#pragma unroll
    for (int d = 0; d < PL; d++) o[lane * PL + d] = acc[d];
    if (lane == 0) {
        o[HD] = m;
        o[HD + 1] = l;
    }
}

static cudaError_t launch_qsa_attn(const QwLaunch &L) {
    uint32_t QH, KVH, HD;
    QW_CHECK_ARG(qsa_dims(L, QH, KVH, HD));
    qsa_args a = L.bytes<qsa_args>(6);
    QW_CHECK_ARG(L.has_bytes(6, 24) && a.nb >= 1 && a.nb <= 64 && a.layer < a.nlayers && a.max_chunks >= 1 && a.max_chunks <= a.max_pages);
    for (int i = 0; i <= 5; i++) QW_CHECK_ARG(L.buf<void>(i) != nullptr);
    QW_CHECK_ARG(L.avail(0) >= (size_t)a.nb * QH * HD * 2 && L.avail(5) >= (size_t)a.nb * a.max_chunks * QH * (HD + 2) * 4 && L.tx == 256);
    qw_launch(qsa_attn_k, dim3(a.max_chunks, KVH, a.nb), 256, 0, L.stream, L.buf<__half>(0), L.buf<__half>(1), L.buf<int32_t>(2), L.buf<int32_t>(3),
                                                                   L.buf<int32_t>(4), L.buf<float>(5), a, QH, KVH);
    return cudaGetLastError();
}
QW_FAMILY(qsa_attn_simt, launch_qsa_attn, 256)

// ------------------------------------------------------------------------------------------------ attention core, tensor cores
// Same contract and partial format as qsa_attn_simt above, computed with warp MMAs on K / V tiles staged by 2-D
// tiled TMA copies (cp.async.bulk.tensor, 128-byte swizzle) -- this is the family the engine uses ("qsa_attn").
// Persistent warps: the (page chunk, kv head, slot) tasks of the launch are numbered slot-major and warp number w of the
// grid takes tasks w, w + W, w + 2W, ...  A warp owns a task completely: it walks the page's up to 256 tokens in steps
// of 16 with its own K and V tile and two mbarriers, keeps the online-softmax state of the 8 query heads in registers and
// writes the partial straight from them -- no block-wide synchronisation after the start, and the tiles of a warp's next
// task are requested while the current one finishes, so a warp always has a copy in flight.
//   scores   S^T[16 tokens][8 heads] = K[16][256] . Q^T            16 MMAs m16n8k16, A = K rows via ldmatrix
//   softmax  online, per head, over the token rows (lanes that share t = lane % 4 hold the same two heads)
//   output   O^T[256 dims][8 heads] += V^T[256][16 tokens] . P^T   16 MMAs, A = V via ldmatrix.trans,
//            B = the probabilities moved from accumulator layout to operand layout with four shuffles
// The 8 query heads of the kv head fill the MMA's N dimension exactly: nothing is padded.  What a task computes depends
// only on its slot's own length, never on which warp runs it or on the other slots of the batch.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *tm, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
                 "l"(tm), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

constexpr int AT_WARP_BYTES = 16384;  // per warp: K tile 8 KB + V tile 8 KB (4 swizzled boxes of 16 rows x 128 B each)
constexpr int AT_TAB_BYTES = 1024;    // per block: first task of every slot [65], tokens [64], slot id [64]
constexpr int AT_SMEM = 4 * AT_WARP_BYTES + 64 + AT_TAB_BYTES + 1024;
constexpr int AT_BLOCKS_PER_SM = 3;   // what the shared memory and the registers of the kernel allow

__global__ void __launch_bounds__(128) qsa_attn_mma_k(const __grid_constant__ CUtensorMap tm, const __half *q, const int32_t *pt, const int32_t *posv,
                                                      const int32_t *sids, float *part, qsa_args a, uint32_t QH, uint32_t KVH, unsigned *status) {
    constexpr uint32_t HD = 256;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    uint8_t *smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);  // swizzled boxes need 1024-byte alignment
    uint8_t *Kb = smem + warp * AT_WARP_BYTES, *Vb = Kb + 8192;
    uint64_t *bars = (uint64_t *)(smem + 4 * AT_WARP_BYTES) + warp * 2;
    uint32_t *first = (uint32_t *)(smem + 4 * AT_WARP_BYTES + 64), *ntokv = first + 65, *sidv = ntokv + 64;
    if (lane == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_init_fence();
    }
    pdl_sync();
    // pages of every slot and their running sum: slot s owns page numbers first[s] .. first[s + 1] - 1 of the launch
    if (warp == 0) {
        uint32_t c[2], nt[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t sl = lane + 32 * h;
            nt[h] = sl < a.nb ? (uint32_t)posv[sl] + 1 : 0;
            c[h] = min((nt[h] + QSA_PAGE - 1) / QSA_PAGE, a.max_chunks);
            ntokv[sl] = nt[h];
            sidv[sl] = sl < a.nb ? (uint32_t)sids[sl] : 0;
        }
        uint32_t s0 = c[0], s1 = c[1];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t u0 = __shfl_up_sync(0xffffffffu, s0, o), u1 = __shfl_up_sync(0xffffffffu, s1, o);
            if (lane >= (uint32_t)o) {
                s0 += u0;
                s1 += u1;
            }
        }
        const uint32_t tot0 = __shfl_sync(0xffffffffu, s0, 31);
        first[lane] = s0 - c[0];
        first[32 + lane] = tot0 + s1 - c[1];
        if (lane == 31) first[64] = tot0 + s1;
    }
    __syncthreads();
    const uint32_t tasks = first[64] * KVH, W = gridDim.x * 4;
    struct Task {
        uint32_t ts, kvh, ch, n;
        int rowK;
    };
    auto task_of = [&](uint32_t i) {  // i < tasks
        Task k;
        const uint32_t pi = i / KVH;
        k.kvh = i - pi * KVH;
        uint32_t lo = 0, hi = a.nb;  // largest slot with first[slot] <= pi (every slot of the step has at least one page)
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (first[mid] <= pi) lo = mid;
            else hi = mid;
        }
        k.ts = lo;
        k.ch = pi - first[lo];
        k.n = min((uint32_t)QSA_PAGE, ntokv[lo] - k.ch * QSA_PAGE);
        const uint32_t page = (uint32_t)pt[(size_t)sidv[lo] * a.max_pages + k.ch];
        k.rowK = (int)(((page * a.nlayers + a.layer) * 2) * KVH * QSA_PAGE + k.kvh * QSA_PAGE);
        return k;
    };
    auto load = [&](uint8_t *dst, uint64_t *bar, int row) {
        if (lane == 0) {
            fence_proxy_async();  // the warp's reads of this buffer (ordered by __syncwarp) before the async-proxy writes
            mbar_expect_tx(bar, 8192);
#pragma unroll
            for (int db = 0; db < 4; db++) tma_load_2d(dst + db * 2048, &tm, db * 64, row, bar);
        }
    };
    // ldmatrix lane roles: matrix mi = lane / 8, row r8 = lane % 8 (the swizzle key of that row)
    const uint32_t mi = lane >> 3, r8 = lane & 7;
    const uint32_t kbase = smem_u32(Kb) + ((mi & 1) * 8 + r8) * 128, vbase = smem_u32(Vb) + ((mi >> 1) * 8 + r8) * 128;
    const int vrows = (int)(KVH * QSA_PAGE);  // rows from a page's K tile to its V tile
    uint32_t kph = 0, vph = 0;  // copies waited for so far on the K / V barrier (their parity selects the phase)
    bool ok = true;
    uint32_t i = blockIdx.x * 4 + warp;
    Task cur{};
    if (i < tasks) {
        cur = task_of(i);
        load(Kb, &bars[0], cur.rowK);
        load(Vb, &bars[1], cur.rowK + vrows);
    }
    while (i < tasks && ok) {
        const uint32_t steps = (cur.n + 15) / 16;
        const bool more = i + W < tasks;
        Task nxt{};
        if (more) nxt = task_of(i + W);  // looked up now: its first tiles are requested as soon as this task's last ones are consumed
        // Q as B fragments (k = dim, n = head g), pre-scaled by HD^-1/2 = 1/16 (exact in fp16)
        uint32_t qf[16][2];
        {
            const __half *qp = q + ((size_t)cur.ts * QH + cur.kvh * 8 + g) * HD + 2 * t;
            const __half2 sc = __floats2half2_rn(0.0625f, 0.0625f);
#pragma unroll
            for (int ks = 0; ks < 16; ks++) {
                const __half2 v0 = __hmul2(*(const __half2 *)(qp + 16 * ks), sc), v1 = __hmul2(*(const __half2 *)(qp + 16 * ks + 8), sc);
                qf[ks][0] = *(const uint32_t *)&v0;
                qf[ks][1] = *(const uint32_t *)&v1;
            }
        }
        float o[16][4];
#pragma unroll
        for (int dt = 0; dt < 16; dt++) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
        for (uint32_t step = 0; step < steps; step++) {
            if (!mbar_wait(&bars[0], kph & 1)) { ok = false; break; }
            kph++;
            float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 16; ks++) {
                uint32_t af[4];
                ldsm_x4(af, kbase + (ks >> 2) * 2048 + ((((ks & 3) * 2 + (mi >> 1)) ^ r8) << 4));
                mma_f16(s, af, qf[ks][0], qf[ks][1], s);
            }
            __syncwarp();
            if (step + 1 < steps) load(Kb, &bars[0], cur.rowK + (int)(step + 1) * 16);
            else if (more) load(Kb, &bars[0], nxt.rowK);
            const uint32_t ta = step * 16 + g;
            if (ta >= cur.n) s[0] = s[1] = -INFINITY;
            if (ta + 8 >= cur.n) s[2] = s[3] = -INFINITY;
            float x0 = fmaxf(s[0], s[2]), x1 = fmaxf(s[1], s[3]);
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, off));
                x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, off));
            }
            const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);
            const float a0 = expf(m0 - n0), a1 = expf(m1 - n1);
            const float p0 = expf(s[0] - n0), p1 = expf(s[1] - n1), p2 = expf(s[2] - n0), p3 = expf(s[3] - n1);
            l0 = l0 * a0 + (p0 + p2);
            l1 = l1 * a1 + (p1 + p3);
            m0 = n0;
            m1 = n1;
#pragma unroll
            for (int dt = 0; dt < 16; dt++) {
                o[dt][0] *= a0;
                o[dt][1] *= a1;
                o[dt][2] *= a0;
                o[dt][3] *= a1;
            }
            // probabilities: accumulator layout (token g / g+8, heads 2t, 2t+1) -> B operand layout (tokens 2t, 2t+1 / +8,
            // head g).  Each probability travels as an fp16 high part plus an fp16 remainder (two MMAs per dim tile), so the
            // weighted sum keeps ~22 bits of p instead of 11.
            const __half2 h01 = __floats2half2_rn(p0, p1), h23 = __floats2half2_rn(p2, p3);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const __half2 r01 = __floats2half2_rn(p0 - f01.x, p1 - f01.y), r23 = __floats2half2_rn(p2 - f23.x, p3 - f23.y);
            const int srcA = (2 * t) * 4 + (g >> 1), srcB = srcA + 4;
            const uint32_t sel = (g & 1) ? 0x7632u : 0x5410u;
            auto to_b = [&](const __half2 &h) {
                const uint32_t u = *(const uint32_t *)&h;
                return __byte_perm(__shfl_sync(0xffffffffu, u, srcA), __shfl_sync(0xffffffffu, u, srcB), sel);
            };
            const uint32_t b0 = to_b(h01), b1 = to_b(h23), c0 = to_b(r01), c1 = to_b(r23);
            if (!mbar_wait(&bars[1], vph & 1)) { ok = false; break; }
            vph++;
#pragma unroll
            for (int dt = 0; dt < 16; dt++) {
                uint32_t af[4];
                ldsm_x4_t(af, vbase + (dt >> 2) * 2048 + ((((dt & 3) * 2 + (mi & 1)) ^ r8) << 4));
                mma_f16(o[dt], af, b0, b1, o[dt]);
                mma_f16(o[dt], af, c0, c1, o[dt]);
            }
            __syncwarp();
            if (step + 1 < steps) load(Vb, &bars[1], cur.rowK + vrows + (int)(step + 1) * 16);
            else if (more) load(Vb, &bars[1], nxt.rowK + vrows);
        }
        if (!ok) break;
        // the page's totals (the lanes that share t hold the same two heads), then the partial straight from the registers
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, off);
            l1 += __shfl_xor_sync(0xffffffffu, l1, off);
        }
        float *po0 = part + (((size_t)cur.ts * a.max_chunks + cur.ch) * QH + cur.kvh * 8 + 2 * t) * (HD + 2), *po1 = po0 + (HD + 2);
#pragma unroll
        for (int dt = 0; dt < 16; dt++) {
            po0[16 * dt + g] = o[dt][0];
            po1[16 * dt + g] = o[dt][1];
            po0[16 * dt + g + 8] = o[dt][2];
            po1[16 * dt + g + 8] = o[dt][3];
        }
        if (g == 0) {
            po0[HD] = m0;
            po0[HD + 1] = l0;
            po1[HD] = m1;
            po1[HD + 1] = l1;
        }
        cur = nxt;
        i += W;
    }
    if (!ok && lane == 0) set_status(status, ST_MBAR_TIMEOUT | 4);
}

// cuTensorMapEncodeTiled is a driver entry point; it is looked up through the runtime so that the library has no link
// dependency on libcuda (it must load, without running anything, on machines that have no driver).
typedef CUresult (*qw_encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                       const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                       CUtensorMapFloatOOBfill);
static bool attn_encode_map(CUtensorMap *tm, const void *pool, size_t bytes) {
    static qw_encode_tiled_fn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess || !p) return false;
        fn = (qw_encode_tiled_fn)p;
    }
    const cuuint64_t gdim[2] = {256, (cuuint64_t)(bytes / 512)};
    const cuuint64_t gstride[1] = {512};
    const cuuint32_t box[2] = {64, 16}, estr[2] = {1, 1};
    return fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)pool, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// One tensor map per KV pool: the pool seen as [rows of one token of one kv head][256 halves]
static const CUtensorMap *attn_tensor_map(void *pool, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<void *, size_t>, CUtensorMap> cache;
    std::lock_guard<std::mutex> lk(mu);
    auto key = std::make_pair(pool, bytes);
    auto it = cache.find(key);
    if (it != cache.end()) return &it->second;
    CUtensorMap tm;
    if (!attn_encode_map(&tm, pool, bytes)) return nullptr;
    return &(cache[key] = tm);
}

static cudaError_t launch_qsa_attn_mma(const QwLaunch &L) {
    uint32_t QH, KVH, HD;
    QW_CHECK_ARG(qsa_dims(L, QH, KVH, HD));
    qsa_args a = L.bytes<qsa_args>(6);
    QW_CHECK_ARG(L.has_bytes(6, 24) && a.nb >= 1 && a.nb <= 64 && a.layer < a.nlayers && a.max_chunks >= 1 && a.max_chunks <= a.max_pages);
    for (int i = 0; i <= 5; i++) QW_CHECK_ARG(L.buf<void>(i) != nullptr);
    QW_CHECK_ARG(L.avail(0) >= (size_t)a.nb * QH * HD * 2 && L.avail(5) >= (size_t)a.nb * a.max_chunks * QH * (HD + 2) * 4);
    QW_CHECK_ARG(((uintptr_t)L.buf<void>(1) & 15) == 0 && L.avail(1) >= 512 && L.avail(1) / 512 < 0x7fffffffull);
    const CUtensorMap *tm = attn_tensor_map(L.buf<void>(1), L.avail(1) / 512 * 512);
    QW_CHECK_ARG(tm != nullptr);
    const size_t smem = AT_SMEM;
    cudaError_t e = cudaFuncSetAttribute(qsa_attn_mma_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    // persistent: as many blocks as fit on the device at once, or fewer when the step cannot have that many tasks
    const uint32_t most = (a.nb * a.max_chunks * KVH + 3) / 4, cap = (uint32_t)L.sm_count * AT_BLOCKS_PER_SM;
    qw_launch(qsa_attn_mma_k, most < cap ? most : cap, 128, smem, L.stream, *tm, L.buf<__half>(0), L.buf<int32_t>(2), L.buf<int32_t>(3),
                                                                          L.buf<int32_t>(4), L.buf<float>(5), a, QH, KVH, L.status);
    return cudaGetLastError();
}
QW_FAMILY(qsa_attn, launch_qsa_attn_mma, 128)

// ------------------------------------------------------------------------------------------------ merge + output gate
// binds: 0 = part, 1 = qkv fp16 (gate = qkv[t][qh*2*HD + HD + d]), 2 = y fp16 [nb][QH*HD], 3 = pos, 4 = qsa_args.
// grid (QH, nb) x 512.  The chunk weights exp(m_c - M) are computed once per chunk (thread c); then the 16 warps take the
// chunks c = warp, warp + 16, ... (each in increasing order; a lane owns eight dims: four 8-byte loads per chunk -- a partial's 258
// floats keep rows 8-byte aligned, not 16 -- four chunks in flight per warp) and the 16 partial sums are added in warp order: o = sum_c w_c acc_c[d] / sum_c w_c l_c.  The order depends only on the slot's own chunk count.
#define QSA_MAXCH 1024
__global__ void __launch_bounds__(512) qsa_merge_k(const float *part, const __half *qkv, __half *y, const int32_t *posv, qsa_args a, uint32_t QH) {
    constexpr uint32_t HD = 256;
    __shared__ float wc[QSA_MAXCH], lc[QSA_MAXCH], tmp[16], ls[16];
    __shared__ float accs[16][HD];
    pdl_sync();
    const uint32_t qh = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the core wrote max_chunks partials per slot at most: a position beyond that (only a caller that passes its own device
    // positions can produce one) must not make the merge read another slot's partials or run off the buffer
    const uint32_t ntok = (uint32_t)posv[t] + 1, nch = min((ntok + QSA_PAGE - 1) / QSA_PAGE, min(a.max_chunks, (uint32_t)QSA_MAXCH));
    const float *base = part + ((size_t)t * a.max_chunks * QH + qh) * (HD + 2);
    const size_t cstride = (size_t)QH * (HD + 2);
    float mx = -INFINITY;
    for (uint32_t c = tid; c < nch; c += 512) {
        const float pm = base[c * cstride + HD], pl = base[c * cstride + HD + 1];
        wc[c] = pm;
        lc[c] = pl;
        if (pl > 0.f) mx = fmaxf(mx, pm);
    }
    mx = warp_max(mx);
    if (lane == 0) tmp[warp] = mx;
    __syncthreads();
    float M = tmp[0];
#pragma unroll
    for (int i = 1; i < 16; i++) M = fmaxf(M, tmp[i]);
    for (uint32_t c = tid; c < nch; c += 512) wc[c] = lc[c] > 0.f ? expf(wc[c] - M) : 0.f;
    __syncthreads();
    float l = 0.f;
    float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll 4
    for (uint32_t c = warp; c < nch; c += 16) {
        const float w = wc[c];
        const float2 *pv = (const float2 *)(base + c * cstride) + 4 * lane;
        const float2 v0 = pv[0], v1 = pv[1], v2 = pv[2], v3 = pv[3];
        l = fmaf(lc[c], w, l);
        acc[0].x = fmaf(v0.x, w, acc[0].x); acc[0].y = fmaf(v0.y, w, acc[0].y);
        acc[1].x = fmaf(v1.x, w, acc[1].x); acc[1].y = fmaf(v1.y, w, acc[1].y);
        acc[2].x = fmaf(v2.x, w, acc[2].x); acc[2].y = fmaf(v2.y, w, acc[2].y);
        acc[3].x = fmaf(v3.x, w, acc[3].x); acc[3].y = fmaf(v3.y, w, acc[3].y);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) *(float2 *)&accs[warp][8 * lane + 2 * i] = acc[i];
    if (lane == 0) ls[warp] = l;
    __syncthreads();
    if (tid < HD) {
        const uint32_t d = tid;
        float at = accs[0][d], lt = ls[0];
#pragma unroll
        for (int g2 = 1; g2 < 16; g2++) {
            at += accs[g2][d];
            lt += ls[g2];
        }
        const float g = __half2float(qkv[(size_t)t * a.qkv_stride + qh * 2 * HD + HD + d]);
        const float o = __half2float(__float2half_rn(at / lt));
        y[((size_t)t * QH + qh) * HD + d] = __float2half_rn(o * (1.0f / (1.0f + expf(-g))));
    }
}

static cudaError_t launch_qsa_merge(const QwLaunch &L) {
    uint32_t QH, KVH, HD;
    QW_CHECK_ARG(qsa_dims(L, QH, KVH, HD));
    qsa_args a = L.bytes<qsa_args>(4);
    QW_CHECK_ARG(L.has_bytes(4, 24) && a.nb >= 1 && a.nb <= 64 && a.max_chunks >= 1 && a.max_chunks <= QSA_MAXCH);
    for (int i = 0; i <= 3; i++) QW_CHECK_ARG(L.buf<void>(i) != nullptr);
    QW_CHECK_ARG(L.avail(0) >= (size_t)a.nb * a.max_chunks * QH * (HD + 2) * 4 && L.avail(2) >= (size_t)a.nb * QH * HD * 2 &&
                 L.avail(1) >= ((size_t)(a.nb - 1) * a.qkv_stride + QH * 2 * HD) * 2);
    qw_launch(qsa_merge_k, dim3(QH, a.nb), 512, 0, L.stream, L.buf<float>(0), L.buf<__half>(1), L.buf<__half>(2), L.buf<int32_t>(3), a, QH);
    return cudaGetLastError();
}
QW_FAMILY(qsa_merge, launch_qsa_merge, 256)

// ------------------------------------------------------------------------------------------------ no-allocation entry point
// qw_attn_decode_static: the attention core + merge for callers that must not allocate device memory at all --
// for example code running inside someone else's memory plan (a serving process whose whole HBM budget was handed
// out at start-up, or a host that calls in while a stream capture is open elsewhere and therefore cannot call
// cudaMalloc).  The split-K partials, which the batch path keeps in a caller-provided buffer, live here in a
// file-scope device array; every GPU that loads this library holds that array (8.45 MB) until the process exits.
//
//   limit     nb * max_chunks <= QW_ATTN_STATIC_MAX_CHUNK_SLOTS (512 page-chunks in flight, e.g. 16 slots of up to
//             8192 tokens, or 2 slots of 65536); QH = 16, KVH = 2, HD = 256 only.  Larger requests are rejected.
//   set-up    the first call on a device resolves the array's device address (cudaGetSymbolAddress, with that
//             device current) and remembers it; make that first call outside any stream capture.
//   contract  pos[t] + 1 <= max_chunks * 256 for every row: the core covers max_chunks pages per slot and the merge never
//             looks past them (a longer position is cut to the first max_chunks pages, not read out of bounds).
//   contents  nothing has to start at zero: the core writes every partial (accumulator, max, sum) that the merge
//             of the same call reads, so what an earlier call left behind is never looked at.
//   sharing   all calls on a device use the same array: two calls whose kernels overlap on the GPU (different
//             streams, or different host threads) race and corrupt each other's result.  Serialise them.
// No cudaMalloc / cudaFree / host allocation happens on this path: the tensor map is encoded on the stack, the
// per-device address table is a static array.
#define QW_ATTN_STATIC_MAX_CHUNK_SLOTS 512
static __device__ __align__(256) float g_attn_static_part[(size_t)QW_ATTN_STATIC_MAX_CHUNK_SLOTS * 16 * (256 + 2)];
static float *g_attn_static_ptr[64];  // per device: address of the array above (host code may not use the symbol itself)

extern "C" int qw_attn_decode_static(const void *q, const void *kv_pool, size_t kv_pool_bytes, const int32_t *page_table, const int32_t *pos,
                                     const int32_t *slot_ids, const void *qkv, void *y, uint32_t nb, uint32_t layer, uint32_t nlayers,
                                     uint32_t qkv_stride, uint32_t max_pages, uint32_t max_chunks, void *stream, char *err, size_t errlen) {
    auto fail = [&](int code, const char *msg) {
        if (err && errlen) snprintf(err, errlen, "qw_attn_decode_static: %s", msg);
        return code;
    };
    constexpr uint32_t QH = 16, KVH = 2, HD = 256;
    if (!q || !kv_pool || !page_table || !pos || !slot_ids || !qkv || !y) return fail(-1, "null pointer argument");
    if (nb < 1 || nb > 64 || max_chunks < 1 || max_chunks > max_pages || layer >= nlayers) return fail(-1, "bad nb / max_chunks / layer");
    if ((uint64_t)nb * max_chunks > QW_ATTN_STATIC_MAX_CHUNK_SLOTS)
        return fail(-2, "nb * max_chunks exceeds the static scratch (512 page-chunks); use the batch path with a caller-provided buffer");
    if (qkv_stride < QH * 2 * HD + 2 * KVH * HD || ((uintptr_t)kv_pool & 15) || kv_pool_bytes < 512 || kv_pool_bytes / 512 >= 0x7fffffffull)
        return fail(-1, "bad qkv stride or KV pool");
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(-3, "no current CUDA device");
    if (!g_attn_static_ptr[dev]) {  // once per device, with that device current
        float *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void **)&p, g_attn_static_part);
        if (e != cudaSuccess || !p) return fail(-3, cudaGetErrorString(e));
        g_attn_static_ptr[dev] = p;
    }
    float *part = g_attn_static_ptr[dev];
    CUtensorMap tm;  // encoded on the stack: no allocation
    if (!attn_encode_map(&tm, kv_pool, kv_pool_bytes / 512 * 512)) return fail(-3, "tensor map encoding failed");
    qsa_args a = {nb, layer, nlayers, qkv_stride, max_pages, max_chunks, 0, 0};
    const size_t smem = AT_SMEM;
    cudaError_t e = cudaFuncSetAttribute(qsa_attn_mma_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(-3, cudaGetErrorString(e));
    cudaStream_t st = (cudaStream_t)stream;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) return fail(-3, "cannot read the SM count");
    const uint32_t most = (nb * max_chunks * KVH + 3) / 4, cap = (uint32_t)sms * AT_BLOCKS_PER_SM;
    qsa_attn_mma_k<<<most < cap ? most : cap, 128, smem, st>>>(tm, (const __half *)q, page_table, pos, slot_ids, part, a, QH, KVH, nullptr);
    qsa_merge_k<<<dim3(QH, nb), 512, 0, st>>>(part, (const __half *)qkv, (__half *)y, pos, a, QH);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(-3, cudaGetErrorString(e));
    if (err && errlen) err[0] = 0;
    return 0;
}
