// Small kernels around the four big ones: embedding gather, residual add + RMSNorm, greedy arg-max, slot
// bookkeeping, buffer fill.
//   kb_embed     h[t] = float(emb[tok[t]])                       -- role of gg_embed / kb_embed (src/engine.c:8887-8898)
//   add_rmsnorm  h += delta (optional); x = fp16(h * rsqrt(mean h^2 + 1e-6) * w): the plain residual + RMSNorm
//                that stands in for the reference's hyper-connection mix (eps as every reference norm,
//                kernels/engine.metal:11)
//   k_argmax     per token arg-max over the vocabulary, equal values -> smallest index
//                -- role of k_argmax1/2 (kernels/engine.metal:605-648) and argmax_cpu (src/engine.c:6144-6148)
//   par_advance  after a step: pos[t] += 1 and (optionally) tok[t] = the sampled id, so consecutive greedy steps
//                need no host round trip
//   qw_fill      zero / counter-based synthetic fill of a buffer (weights of the synthetic model)
#include "common.cuh"
#include "moe_sel.h"
#include "qw_kern.h"
#include <cooperative_groups.h>

using namespace qw;

// binds: 0 = emb fp16 [V][D], 1 = tok int32 [nb], 2 = h fp32 [nb][D], 3 = {nb, D, V}.  grid (ceil(D/256), nb) x 256
__global__ void kb_embed_k(const __half *emb, const int32_t *tok, float *h, uint32_t D, uint32_t V) {
    pdl_sync();
    const uint32_t d = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
    if (d >= D) return;
    uint32_t id = (uint32_t)tok[t];
    if (id >= V) id = 0;
    h[(size_t)t * D + d] = __half2float(emb[(size_t)id * D + d]);
}
static cudaError_t launch_kb_embed(const QwLaunch &L) {
    struct { uint32_t nb, D, V; } a = L.bytes<decltype(a)>(3);
    QW_CHECK_ARG(L.buf<void>(0) && L.buf<void>(1) && L.buf<void>(2) && L.has_bytes(3, 12) && a.nb >= 1 && a.nb <= 64);
    QW_CHECK_ARG(L.avail(0) >= (size_t)a.V * a.D * 2 && L.avail(1) >= a.nb * 4 && L.avail(2) >= (size_t)a.nb * a.D * 4);
    qw_launch(kb_embed_k, dim3((a.D + 255) / 256, a.nb), 256, 0, L.stream, L.buf<__half>(0), L.buf<int32_t>(1), L.buf<float>(2), a.D, a.V);
    return cudaGetLastError();
}
QW_FAMILY(kb_embed, launch_kb_embed, 256)

// binds: 0 = h fp32 [nb][D], 1 = delta fp16 [nb][D] (only with ADD defined 1: h is then updated in place),
// 2 = w fp32 [D], 3 = x out fp16 [nb][D], 4 = {nb, D}.  With CMB defined 1 the delta is not read from memory but is
// the MoE combine of moe_cmb (rank-ordered weighted sum of Pg plus the shared expert, rounded to fp16) computed on
// the fly: 5 = moe_sel, 6 = Pg fp32 [nb][TOPK+1][D], define TOPK.  grid nb x 256
template <int MODE>  // 0: norm only, 1: h += delta, 2: h += fp16(combine)
__global__ void __launch_bounds__(1024) add_rmsnorm_k(float *h, const __half *delta, const float *w, __half *x, uint32_t D, const moe_sel *ms,
                                                     const float *Pg, uint32_t topk, const unsigned *flags, const unsigned *seq, uint32_t nranks,
                                                     unsigned *status) {
    __shared__ float tmp[32];
    const uint32_t t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nth = blockDim.x;
    pdl_launch();
    float wv[4];  // the norm weights are static: read before the wait for the previous kernel
#pragma unroll
    for (int it = 0; it < 4; it++) wv[it] = tid + it * nth < D ? w[tid + it * nth] : 0.f;
    pdl_wait();
    // rows of Pg (MODE 2) or of delta (MODE 1) may have been stored by other ranks: wait until every rank has published
    if (nranks > 1) ep_wait(flags, seq, nranks, status);
    float *hr = h + (size_t)t * D;
    float wk[MOE_MAXK];
    if (MODE == 2) {
#pragma unroll
        for (uint32_t s = 0; s < MOE_MAXK; s++) wk[s] = s <= topk ? ms->w[t][s] : 0.f;
    }
    // a thread's values stay in registers between the two passes (D <= 4 * blockDim; beyond that they are read back)
    float vv[4] = {0.f, 0.f, 0.f, 0.f};
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < 4; it++) {
        const uint32_t d = tid + it * nth;
        if (d < D) {
            float v = hr[d];
            if (MODE == 1) {
                v += __half2float(delta[(size_t)t * D + d]);
                hr[d] = v;
            } else if (MODE == 2) {
                float pv[MOE_MAXK];  // all loads first (independent), then the rank-ordered chain
#pragma unroll
                for (uint32_t s = 0; s < MOE_MAXK; s++) pv[s] = s <= topk ? Pg[((size_t)t * (topk + 1) + s) * D + d] : 0.f;
                float o = 0.f;
#pragma unroll
                for (uint32_t s = 0; s < MOE_MAXK; s++)
                    if (s <= topk) o = fmaf(wk[s], pv[s], o);
                v += __half2float(__float2half_rn(o));
                hr[d] = v;
            }
            vv[it] = v;
            ss = fmaf(v, v, ss);
        }
    }
    for (uint32_t d = tid + 4 * nth; d < D; d += nth) {  // rows wider than the register copy
        float v = hr[d];
        if (MODE == 1) {
            v += __half2float(delta[(size_t)t * D + d]);
            hr[d] = v;
        } else if (MODE == 2) {
            float o = 0.f;
            for (uint32_t s = 0; s <= topk; s++) o = fmaf(wk[s], Pg[((size_t)t * (topk + 1) + s) * D + d], o);
            v += __half2float(__float2half_rn(o));
            hr[d] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) tmp[warp] = ss;
    __syncthreads();
    const float tot = warp_sum(lane < nth / 32 ? tmp[lane] : 0.f);  // every warp sums the same 32 values in the same order
    const float r = rsqrtf(tot / D + 1e-6f);
#pragma unroll
    for (int it = 0; it < 4; it++) {
        const uint32_t d = tid + it * nth;
        if (d < D) x[(size_t)t * D + d] = __float2half_rn(vv[it] * r * wv[it]);
    }
    for (uint32_t d = tid + 4 * nth; d < D; d += nth) x[(size_t)t * D + d] = __float2half_rn(hr[d] * r * w[d]);
}
// The MoE-combine form for D = 2048 (the step's hot case: it sits between the expert FFN and the next projection, and
// nothing else can run beside it).  A token is served by a cluster of 8 blocks of 256 threads, one column per thread: the
// twelve loads of a column are independent, the blocks are small enough to be resident next to the FFN's blocks while they
// wait for it, and the sum of squares of the row meets through the cluster's shared memory (every block pushes its partial sum to
// all eight; they are added in block order by every block, so the result does not depend on timing).  grid (8 nb) x 256, cluster 8.
__global__ void __cluster_dims__(8, 1, 1) __launch_bounds__(256) cmb_rmsnorm_cl_k(float *h, const float *w, __half *x, const moe_sel *ms, const float *Pg,
                                                                                    uint32_t topk, const unsigned *flags, const unsigned *seq,
                                                                                    uint32_t nranks, unsigned *rowcnt, unsigned *status) {
    constexpr uint32_t D = 2048;
    namespace cg = cooperative_groups;
    __shared__ float tmp[8];
    __shared__ float parts[8];  // the eight blocks' partial sums of squares, each written here by its owner
    cg::cluster_group cl = cg::this_cluster();
    const uint32_t t = blockIdx.x >> 3, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, d = (blockIdx.x & 7) * 256 + tid;
    pdl_launch();
    // first cluster barrier, split: arrive now, wait just before the partial sums are pushed (by then every block of the cluster
    // has long arrived, i.e. has started and owns its shared memory)
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    const float wd = w[d];  // the norm weights are static
    if (rowcnt) {
        // One GPU, the one-launch expert FFN before us: do not wait for its whole launch, only for this token's topk + 1 output rows
        // (each counted in by the warps that stored it; see moe_sel.h).  Everything read below was complete before the FFN stored
        // those rows, and the FFN no longer reads this token's x once they are.  Bounded like every wait of this library.
        if (tid <= topk) {
            const unsigned *c = rowcnt + t * (topk + 1) + tid;
            const uint64_t t0 = global_ns();
            while (ld_acquire_gpu(c) < MOE_FFN_ROW_DONE(D)) {
                __nanosleep(100);
                if (global_ns() - t0 > 2000000000ull) {
                    set_status(status, ST_PEER_TIMEOUT | 32);
                    break;
                }
            }
        }
        __syncthreads();
    } else {
        pdl_wait();
    }
    if (nranks > 1) ep_wait(flags, seq, nranks, status);
    float wk[MOE_MAXK], pv[MOE_MAXK];
#pragma unroll
    for (uint32_t s = 0; s < MOE_MAXK; s++) wk[s] = s <= topk ? ms->w[t][s] : 0.f;
#pragma unroll
    for (uint32_t s = 0; s < MOE_MAXK; s++) pv[s] = s <= topk ? __ldcg(Pg + ((size_t)t * (topk + 1) + s) * D + d) : 0.f;
    float v = h[(size_t)t * D + d];
    float o = 0.f;
#pragma unroll
    for (uint32_t s = 0; s < MOE_MAXK; s++)
        if (s <= topk) o = fmaf(wk[s], pv[s], o);  // rank order, as moe_cmb
    v += __half2float(__float2half_rn(o));
    h[(size_t)t * D + d] = v;
    const float ss = warp_sum(v * v);
    if (lane == 0) tmp[warp] = ss;
    __syncthreads();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (tid < 8) {  // thread r pushes this block's partial sum into block r's array: after the one cluster barrier nobody touches another block's memory
        float b = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) b += tmp[i];
        *cl.map_shared_rank(&parts[blockIdx.x & 7], tid) = b;
    }
    cl.sync();
    float tot = 0.f;
#pragma unroll
    for (unsigned r = 0; r < 8; r++) tot += parts[r];
    x[(size_t)t * D + d] = __float2half_rn(v * rsqrtf(tot / D + 1e-6f) * wd);
    if (rowcnt) {
        pdl_wait();  // this kernel's completion must imply the FFN's: later kernels rely on the chain of completed predecessors
        if ((blockIdx.x & 7) == 0 && tid <= topk) rowcnt[t * (topk + 1) + tid] = 0;  // cleared for the next layer's launch
    }
}
static cudaError_t launch_add_rmsnorm(const QwLaunch &L) {
    struct { uint32_t nb, D; } a = L.bytes<decltype(a)>(4);
    QW_CHECK_ARG(L.buf<void>(0) && L.buf<void>(2) && L.buf<void>(3) && L.has_bytes(4, 8) && a.nb >= 1 && a.nb <= 64);
    QW_CHECK_ARG(L.avail(0) >= (size_t)a.nb * a.D * 4 && L.avail(2) >= (size_t)a.D * 4 && L.avail(3) >= (size_t)a.nb * a.D * 2);
    if (L.def("CMB", 0)) {
        const uint32_t topk = (uint32_t)L.def("TOPK", 10);
        QW_CHECK_ARG(L.buf<void>(5) && L.buf<void>(6) && L.avail(5) >= sizeof(moe_sel) && L.avail(6) >= (size_t)a.nb * (topk + 1) * a.D * 4 && topk < MOE_MAXK);
        // EPX = number of expert-parallel ranks whose down projections store into Pg: 7 = this rank's flag array
        // (one sequence number per rank), 8 = this rank's sequence counter
        const uint32_t nranks = (uint32_t)L.def("EPX", 1);
        if (nranks > 1) QW_CHECK_ARG(nranks <= 8 && L.buf<void>(7) && L.avail(7) >= nranks * 4 && L.buf<void>(8) && L.avail(8) >= 4);
        if (a.D == 2048) {
            // ROWCNT defined 1 (one GPU, after moe_ffn): 9 = the FFN's scratch buffer, whose per-row counters replace the wait for the launch
            unsigned *rowcnt = nullptr;
            if (L.def("ROWCNT", 0)) {
                QW_CHECK_ARG(nranks == 1 && L.buf<unsigned>(9) && L.avail(9) >= MOE_FFN_SYNC_BYTES && (a.nb * (topk + 1)) <= MOE_MAXB * MOE_MAXK);
                rowcnt = L.buf<unsigned>(9) + MOE_FFN_ROWCNT;
            }
            qw_launch(cmb_rmsnorm_cl_k, a.nb * 8, 256, 0, L.stream, L.buf<float>(0), L.buf<float>(2), L.buf<__half>(3), L.buf<moe_sel>(5), L.buf<float>(6), topk,
                      nranks > 1 ? L.buf<unsigned>(7) : nullptr, nranks > 1 ? L.buf<unsigned>(8) : nullptr, nranks, rowcnt, (unsigned *)L.status);
            return cudaGetLastError();
        }
        qw_launch(add_rmsnorm_k<2>, a.nb, 1024, 0, L.stream, L.buf<float>(0), nullptr, L.buf<float>(2), L.buf<__half>(3), a.D, L.buf<moe_sel>(5), L.buf<float>(6), topk,
                  nranks > 1 ? L.buf<unsigned>(7) : nullptr, nranks > 1 ? L.buf<unsigned>(8) : nullptr, nranks, (unsigned *)L.status);
    } else if (L.def("ADD", 0)) {
        QW_CHECK_ARG(L.buf<void>(1) && L.avail(1) >= (size_t)a.nb * a.D * 2);
        const uint32_t nranks = (uint32_t)L.def("EPX", 1);  // the delta rows were stored by the ranks that own the slots: same binds 7, 8
        if (nranks > 1) QW_CHECK_ARG(nranks <= 8 && L.buf<void>(7) && L.avail(7) >= nranks * 4 && L.buf<void>(8) && L.avail(8) >= 4);
        qw_launch(add_rmsnorm_k<1>, a.nb, 512, 0, L.stream, L.buf<float>(0), L.buf<__half>(1), L.buf<float>(2), L.buf<__half>(3), a.D, nullptr, nullptr, 0,
                  nranks > 1 ? L.buf<unsigned>(7) : nullptr, nranks > 1 ? L.buf<unsigned>(8) : nullptr, nranks, (unsigned *)L.status);
    } else {
        qw_launch(add_rmsnorm_k<0>, a.nb, 512, 0, L.stream, L.buf<float>(0), nullptr, L.buf<float>(2), L.buf<__half>(3), a.D, nullptr, nullptr, 0, nullptr, nullptr, 1, nullptr);
    }
    return cudaGetLastError();
}
QW_FAMILY(add_rmsnorm, launch_add_rmsnorm, 256)

// A rank that has no row to contribute to an exchange still has to publish its sequence number.
// binds: 11 = {seq, done} counters, 12 = {rank}, 24 + r = flag array of rank r; define EPX = number of ranks.  grid 1 x 32
__global__ void ep_publish_k(const EpPeers ep) {
    pdl_sync();
    ep_publish(ep);
}
static cudaError_t launch_ep_publish(const QwLaunch &L) {
    EpPeers ep{};
    ep.nranks = (uint32_t)L.def("EPX", 0);
    QW_CHECK_ARG(ep.nranks >= 2 && ep.nranks <= 8 && L.has_bytes(12, 4) && L.buf<unsigned>(11) && L.avail(11) >= 8);
    ep.rank = L.bytes<uint32_t>(12);
    QW_CHECK_ARG(ep.rank < ep.nranks);
    ep.seq = L.buf<unsigned>(11);
    ep.done = ep.seq + 1;
    for (uint32_t r = 0; r < ep.nranks; r++) {
        ep.flagR[r] = L.buf<unsigned>(24 + r);
        QW_CHECK_ARG(ep.flagR[r] && L.avail(24 + r) >= ep.nranks * 4);
    }
    qw_launch(ep_publish_k, 1, 32, 0, L.stream, ep);
    return cudaGetLastError();
}
QW_FAMILY(ep_publish, launch_ep_publish, 32)

// binds: 0 = logits fp32 [nb][V], 1 = ids out int32 [nb], 2 = {nb, V}, 3 = second ids out (with IDS2 defined 1,
// e.g. a host-visible copy).  grid nb x 1024
__global__ void __launch_bounds__(1024) k_argmax_k(const float *lg, int32_t *ids, int32_t *ids2, uint32_t V) {
    __shared__ float bv[32];
    __shared__ uint32_t bi[32];
    pdl_sync();
    const uint32_t t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *r = lg + (size_t)t * V;
    float best = -INFINITY;
    uint32_t idx = 0xffffffffu;
    for (uint32_t i = tid; i < V; i += 1024) {
        const float v = r[i];
        if (v > best || idx == 0xffffffffu) { best = v; idx = i; }  // strictly greater: the lowest index of equals stays
    }
    auto better = [](float v, uint32_t i, float bv2, uint32_t bi2) { return v > bv2 || (v == bv2 && i < bi2); };
#pragma unroll
    for (int off = 16; off; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, off);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, off);
        if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = bv[lane];
        idx = bi[lane];
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, off);
            if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) {
            ids[t] = (int32_t)idx;
            if (ids2) ids2[t] = (int32_t)idx;
        }
    }
}
static cudaError_t launch_k_argmax(const QwLaunch &L) {
    struct { uint32_t nb, V; } a = L.bytes<decltype(a)>(2);
    QW_CHECK_ARG(L.buf<void>(0) && L.buf<void>(1) && L.has_bytes(2, 8) && a.nb >= 1 && a.nb <= 64 && a.V >= 1);
    QW_CHECK_ARG(L.avail(0) >= (size_t)a.nb * a.V * 4 && L.avail(1) >= a.nb * 4);
    int32_t *ids2 = L.def("IDS2", 0) ? L.buf<int32_t>(3) : nullptr;
    if (L.def("IDS2", 0)) QW_CHECK_ARG(ids2 && L.avail(3) >= a.nb * 4);
    qw_launch(k_argmax_k, a.nb, 1024, 0, L.stream, L.buf<float>(0), L.buf<int32_t>(1), ids2, a.V);
    return cudaGetLastError();
}
QW_FAMILY(k_argmax, launch_k_argmax, 1024)

// binds: 0 = pos int32 [nb], 3 = {nb}; with FEED defined 1 also 1 = tok int32 [nb], 2 = sampled ids int32 [nb]
__global__ void par_advance_k(int32_t *pos, int32_t *tok, const int32_t *ids, uint32_t nb) {
    pdl_sync();
    const uint32_t t = threadIdx.x;
    if (t >= nb) return;
    pos[t] += 1;
    if (tok && ids) tok[t] = ids[t];
}
static cudaError_t launch_par_advance(const QwLaunch &L) {
    const uint32_t nb = L.bytes<uint32_t>(3);
    QW_CHECK_ARG(L.buf<void>(0) && nb >= 1 && nb <= 64 && L.avail(0) >= nb * 4);
    const bool feed = L.def("FEED", 0) != 0;
    if (feed) QW_CHECK_ARG(L.buf<void>(1) && L.buf<void>(2) && L.avail(1) >= nb * 4 && L.avail(2) >= nb * 4);
    qw_launch(par_advance_k, 1, 64, 0, L.stream, L.buf<int32_t>(0), feed ? L.buf<int32_t>(1) : nullptr, feed ? L.buf<int32_t>(2) : nullptr, nb);
    return cudaGetLastError();
}
QW_FAMILY(par_advance, launch_par_advance, 64)

// The step's control block (token, slot id, position per row) is written by the host into pinned memory; this
// copies it into device memory once so that no other kernel reads across PCIe.
// binds: 0 = source int32, 1 = destination int32, 2 = {count}
__global__ void par_begin_k(const int32_t *src, int32_t *dst, uint32_t n) {
    pdl_sync();
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
}
static cudaError_t launch_par_begin(const QwLaunch &L) {
    const uint32_t n = L.bytes<uint32_t>(2);
    QW_CHECK_ARG(L.buf<void>(0) && L.buf<void>(1) && n >= 1 && L.avail(0) >= n * 4 && L.avail(1) >= n * 4);
    qw_launch(par_begin_k, 1, 256, 0, L.stream, L.buf<int32_t>(0), L.buf<int32_t>(1), n);
    return cudaGetLastError();
}
QW_FAMILY(par_begin, launch_par_begin, 256)

// ------------------------------------------------------------------------------------------------ fill
// Counter-based generator: byte i of a tensor with seed s is the low byte of mix64(s * 0x9E3779B97F4A7C15 + i)
// (qwental_b200/synth.py holds the same functions in numpy).
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ uint64_t hash_u64(uint64_t seed, uint64_t i) { return mix64(seed * 0x9E3779B97F4A7C15ull + i); }

struct fill_args {
    uint64_t seed, count;  // count: bytes (modes 0-2), elements (modes 3-5)
    uint64_t base;         // index of the first byte / element within the whole tensor (a rank's slice of a sharded tensor)
    uint32_t mode;         // 0 zero bytes, 1 IQ3_S blocks, 2 Q8_0 blocks, 3 fp16 normal, 4 fp32 normal, 5 fp32 constant
    float p0;              // multiplier of the block scale d (modes 1, 2), std (modes 3, 4) or the constant (mode 5)
    float p1;              // mean added (modes 3, 4)
};

__device__ __forceinline__ float hash_normal(uint64_t seed, uint64_t i) {
    const uint64_t h = hash_u64(seed, i);
    const float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777216.0f);
    const float u2 = (float)(uint32_t)((h >> 16) & 0xFFFFFF) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
}

__global__ void qw_fill_k(uint8_t *dst, fill_args a) {
    pdl_sync();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    if (a.mode == 0 && (((uintptr_t)dst | a.count) & 15) == 0) {  // zeroing: 16 bytes per store
        for (uint64_t li = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; li < a.count / 16; li += stride) ((uint4 *)dst)[li] = make_uint4(0, 0, 0, 0);
        return;
    }
    for (uint64_t li = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; li < a.count; li += stride) {
        const uint64_t i = a.base + li;
        if (a.mode == 0) dst[li] = 0;
        else if (a.mode == 1 || a.mode == 2) {
            const uint32_t bb = a.mode == 1 ? 110 : 34;
            const uint64_t blk = i / bb;
            const uint32_t off = (uint32_t)(i % bb);
            uint8_t by = (uint8_t)(hash_u64(a.seed, i) & 0xFF);
            if (a.mode == 2 && by == 0x80) by = 0x81;
            if (off < 2) {
                const float u = (float)(uint32_t)(hash_u64(a.seed ^ 0x5CA1Eull, blk) >> 40) * (1.0f / 16777216.0f);
                const float d = __fmul_rn(__fadd_rn(1e-3f, __fmul_rn(u, 1.9e-2f)), a.p0);
                const uint16_t hb = __half_as_ushort(__float2half_rn(d));
                by = off == 0 ? (uint8_t)(hb & 0xFF) : (uint8_t)(hb >> 8);
            }
            dst[li] = by;
        } else if (a.mode == 3) ((__half *)dst)[li] = __float2half_rn(hash_normal(a.seed, i) * a.p0 + a.p1);
        else if (a.mode == 4) ((float *)dst)[li] = hash_normal(a.seed, i) * a.p0 + a.p1;
        else ((float *)dst)[li] = a.p0;
    }
}
// binds: 0 = destination, 1 = fill_args
static cudaError_t launch_qw_fill(const QwLaunch &L) {
    fill_args a = L.bytes<fill_args>(1);
    QW_CHECK_ARG(L.buf<void>(0) && L.has_bytes(1, 36) && a.mode <= 5 && a.count > 0);
    const size_t esz = a.mode <= 2 ? 1 : a.mode == 3 ? 2 : 4;
    QW_CHECK_ARG(L.avail(0) >= a.count * esz);
    const uint64_t blocks = ((a.mode == 0 ? a.count / 16 : a.count) + 255) / 256 + 1;
    const unsigned grid = (unsigned)(blocks < (uint64_t)L.sm_count * 32 ? blocks : (uint64_t)L.sm_count * 32);
    qw_launch(qw_fill_k, grid, 256, 0, L.stream, L.buf<uint8_t>(0), a);
    return cudaGetLastError();
}
QW_FAMILY(qw_fill, launch_qw_fill, 256)
