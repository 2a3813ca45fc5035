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
    qsa_prep_k<<<dim3(QH + KVH, a.nb), 256, 0, L.stream>>>(L.buf<__half>(0), L.buf<float>(1), L.buf<float>(2), L.buf<__half>(3), L.buf<__half>(4),
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
            const uint4 kk = __ldg((const uint4 *)(Kp + (size_t)tk * HD));
            vv[u] = __ldg((const uint4 *)(Vp + (size_t)tk * HD));
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
    qsa_attn_k<<<dim3(a.max_chunks, KVH, a.nb), 256, 0, L.stream>>>(L.buf<__half>(0), L.buf<__half>(1), L.buf<int32_t>(2), L.buf<int32_t>(3),
                                                                   L.buf<int32_t>(4), L.buf<float>(5), a, QH, KVH);
    return cudaGetLastError();
}
QW_FAMILY(qsa_attn, launch_qsa_attn, 256)

// ------------------------------------------------------------------------------------------------ merge + output gate
// binds: 0 = part, 1 = qkv fp16 (gate = qkv[t][qh*2*HD + HD + d]), 2 = y fp16 [nb][QH*HD], 3 = pos, 4 = qsa_args.
// grid (QH, nb) x 256.  The chunk weights exp(m_c - M) are computed once per chunk (thread c), then thread d sums
// dim d over the slot's chunks in chunk order: o = sum_c w_c acc_c[d] / sum_c w_c l_c.
#define QSA_MAXCH 1024
__global__ void __launch_bounds__(256) qsa_merge_k(const float *part, const __half *qkv, __half *y, const int32_t *posv, qsa_args a, uint32_t QH) {
    constexpr uint32_t HD = 256;
    __shared__ float wc[QSA_MAXCH], lc[QSA_MAXCH], tmp[8];
    const uint32_t qh = blockIdx.x, t = blockIdx.y, d = threadIdx.x, lane = d & 31, warp = d >> 5;
    const uint32_t ntok = (uint32_t)posv[t] + 1, nch = (ntok + QSA_PAGE - 1) / QSA_PAGE;
    const float *base = part + ((size_t)t * a.max_chunks * QH + qh) * (HD + 2);
    const size_t cstride = (size_t)QH * (HD + 2);
    float mx = -INFINITY;
    for (uint32_t c = d; c < nch; c += 256) {
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
    for (int i = 1; i < 8; i++) M = fmaxf(M, tmp[i]);
    for (uint32_t c = d; c < nch; c += 256) wc[c] = lc[c] > 0.f ? expf(wc[c] - M) : 0.f;
    __syncthreads();
    float l = 0.f, acc = 0.f;
#pragma unroll 4
    for (uint32_t c = 0; c < nch; c++) {
        const float w = wc[c];
        l = fmaf(lc[c], w, l);
        acc = fmaf(base[c * cstride + d], w, acc);
    }
    const float g = __half2float(qkv[(size_t)t * a.qkv_stride + qh * 2 * HD + HD + d]);
    const float o = __half2float(__float2half_rn(acc / l));
    y[((size_t)t * QH + qh) * HD + d] = __float2half_rn(o * (1.0f / (1.0f + expf(-g))));
}

static cudaError_t launch_qsa_merge(const QwLaunch &L) {
    uint32_t QH, KVH, HD;
    QW_CHECK_ARG(qsa_dims(L, QH, KVH, HD));
    qsa_args a = L.bytes<qsa_args>(4);
    QW_CHECK_ARG(L.has_bytes(4, 24) && a.nb >= 1 && a.nb <= 64 && a.max_chunks >= 1 && a.max_chunks <= QSA_MAXCH);
    for (int i = 0; i <= 3; i++) QW_CHECK_ARG(L.buf<void>(i) != nullptr);
    QW_CHECK_ARG(L.avail(0) >= (size_t)a.nb * a.max_chunks * QH * (HD + 2) * 4 && L.avail(2) >= (size_t)a.nb * QH * HD * 2 &&
                 L.avail(1) >= ((size_t)(a.nb - 1) * a.qkv_stride + QH * 2 * HD) * 2 && L.tx == 256);
    qsa_merge_k<<<dim3(QH, a.nb), 256, 0, L.stream>>>(L.buf<float>(0), L.buf<__half>(1), L.buf<__half>(2), L.buf<int32_t>(3), a, QH);
    return cudaGetLastError();
}
QW_FAMILY(qsa_merge, launch_qsa_merge, 256)
