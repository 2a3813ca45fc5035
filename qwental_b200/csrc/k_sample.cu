// Candidate selection for sampling: the k largest logits of every row (k <= 256), ordered by value descending and, among
// equal values, by token id ascending -- exactly the candidate list that make_dist builds with its insertion sort
// (src/engine.c:6098-6107), so the host can finish temperature / top-p / draw on 256 candidates instead of reading back and
// scanning the whole vocabulary row.  No counterpart kernel exists in the reference (it samples on the CPU from the full
// logits, src/engine.c:9410-9418); the host half that turns candidates into a token is qw_sample_candidates in engine.cpp.
//
// One block of 1024 threads per row.  Logits become order-preserving 32-bit keys; the k-th largest key is found by a
// three-pass radix select (11 + 11 + 10 bits, shared-memory histograms with warp-aggregated updates).  Usually exactly the
// wanted number of keys is >= the threshold and they are appended in one coalesced pass; when more keys equal the threshold
// than are wanted, every thread walks a contiguous range of the row instead, so that the lowest ids are kept by block-wide
// prefix sums.  A bitonic sort of the <= 256 survivors gives the final order.
#include "common.cuh"
#include "qw_kern.h"

using namespace qw;

namespace {
constexpr int TOPK_MAX = 256;

__device__ __forceinline__ uint32_t key_of(float v) {
    const uint32_t u = __float_as_uint(v + 0.0f);  // -0.0 becomes +0.0: the two compare equal in the reference's sort (ties -> lower id)
    return u ^ ((u >> 31) ? 0xffffffffu : 0x80000000u);
}
__device__ __forceinline__ float val_of(uint32_t k) { return __uint_as_float(k ^ ((k >> 31) ? 0x80000000u : 0xffffffffu)); }

// Block-wide exclusive prefix sums of two counters (1024 threads); totals returned through tot0 / tot1.
__device__ __forceinline__ void block_scan2(uint32_t a, uint32_t b, uint32_t &ea, uint32_t &eb, uint32_t &tot0, uint32_t &tot1, uint32_t (*ws)[32]) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t sa = a, sb = b;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t ta = __shfl_up_sync(0xffffffffu, sa, o), tb = __shfl_up_sync(0xffffffffu, sb, o);
        if (lane >= (uint32_t)o) { sa += ta; sb += tb; }
    }
    if (lane == 31) { ws[0][warp] = sa; ws[1][warp] = sb; }
    __syncthreads();
    if (warp == 0) {
        uint32_t xa = ws[0][lane], xb = ws[1][lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t ta = __shfl_up_sync(0xffffffffu, xa, o), tb = __shfl_up_sync(0xffffffffu, xb, o);
            if (lane >= (uint32_t)o) { xa += ta; xb += tb; }
        }
        ws[0][lane] = xa;
        ws[1][lane] = xb;
    }
    __syncthreads();
    ea = (warp ? ws[0][warp - 1] : 0) + sa - a;
    eb = (warp ? ws[1][warp - 1] : 0) + sb - b;
    tot0 = ws[0][31];
    tot1 = ws[1][31];
    __syncthreads();
}
}  // namespace

// binds: 0 = logits fp32 [nb][V], 1 = candidate ids out int32 [nb][256], 2 = candidate logits out fp32 [nb][256],
// 3 = {nb, V, k}.  Entries past k (or past V) are id -1 / logit -inf.  grid nb x 1024
__global__ void __launch_bounds__(1024) k_topk_k(const float *lg, int32_t *ids, float *vals, uint32_t V, uint32_t K) {
    __shared__ uint32_t hist[2048];
    __shared__ uint32_t ws[2][32];
    __shared__ unsigned long long cand[TOPK_MAX];
    __shared__ uint32_t sh_bin, sh_rem, sh_cnt, sh_n;
    pdl_sync();
    const uint32_t tid = threadIdx.x;
    const float *row = lg + (size_t)blockIdx.x * V;
    if (K > V) K = V;
    // ---- the K-th largest key: radix select over 11 + 11 + 10 bits
    uint32_t prefix = 0, rem = K;  // keys whose high bits equal `prefix` are still in play; rem of them (from the top) are wanted
    const int shifts[3] = {21, 10, 0}, widths[3] = {11, 11, 10};
    for (int ps = 0; ps < 3; ps++) {
        const int sh = shifts[ps], nb = 1 << widths[ps];
        for (uint32_t b = tid; b < 2048; b += 1024) hist[b] = 0;
        __syncthreads();
        for (uint32_t i = tid; i < V; i += 1024) {
            const uint32_t k = key_of(__ldcg(row + i));
            const bool in = ps == 0 || (k >> (sh + widths[ps])) == prefix;
            // logits crowd into a few bins: lanes with the same bin elect one to add their count (no serialised atomics)
            const uint32_t bin = in ? (k >> sh) & (nb - 1) : 0xffffffffu;
            const uint32_t peers = __match_any_sync(__activemask(), bin);
            if (in && (threadIdx.x & 31) == (uint32_t)__ffs(peers) - 1) atomicAdd(&hist[bin], (uint32_t)__popc(peers));
        }
        __syncthreads();
        // suffix sums over the bins (two bins per thread, highest bins first): bin b* = the highest bin whose suffix >= rem
        const uint32_t b1 = 2047 - 2 * tid, b0 = b1 - 1;  // this thread's bins, b1 > b0
        const uint32_t h1 = b1 < (uint32_t)nb ? hist[b1] : 0, h0 = b0 < (uint32_t)nb ? hist[b0] : 0;
        uint32_t e, dummy, tot, t2;
        block_scan2(h1 + h0, 0, e, dummy, tot, t2, ws);  // e = count in all bins above b1
        if (e < rem && e + h1 >= rem) { sh_bin = b1; sh_rem = rem - e; sh_cnt = h1; }
        else if (e + h1 < rem && e + h1 + h0 >= rem) { sh_bin = b0; sh_rem = rem - e - h1; sh_cnt = h0; }
        __syncthreads();
        prefix = (prefix << widths[ps]) | sh_bin;
        rem = sh_rem;
        __syncthreads();
    }
    const uint32_t T = prefix;  // rem = how many keys equal to T are wanted (the lowest ids)
    const uint32_t n_eq = sh_cnt;  // keys equal to T in the whole row (the last pass's bin holds exactly those)
    for (uint32_t j = tid; j < TOPK_MAX; j += 1024) cand[j] = 0;
    if (tid == 0) sh_n = 0;
    __syncthreads();
    if (n_eq == rem) {
        // ---- every key >= T is a winner (K of them): append in any order, the sort below orders them
        for (uint32_t i = tid; i < V; i += 1024) {
            const uint32_t k = key_of(__ldcg(row + i));
            if (k >= T) cand[atomicAdd(&sh_n, 1u)] = ((unsigned long long)k << 32) | (0xffffffffu - i);
        }
    } else {
        // ---- more keys equal T than are wanted: the lowest ids win.  Compaction in id order: thread t owns ids
        // [t*chunk, (t+1)*chunk) and block-wide prefix sums give every thread its output offsets
        const uint32_t chunk = (V + 1023) / 1024, i0 = tid * chunk, i1 = min(V, i0 + chunk);
        uint32_t ngt = 0, neq = 0;
        for (uint32_t i = i0; i < i1; i++) {
            const uint32_t k = key_of(__ldcg(row + i));
            ngt += k > T;
            neq += k == T;
        }
        uint32_t egt, eeq, tgt, teq;
        block_scan2(ngt, neq, egt, eeq, tgt, teq, ws);
        for (uint32_t i = i0; i < i1 && (ngt || neq); i++) {
            const uint32_t k = key_of(__ldcg(row + i));
            if (k > T) cand[egt++] = ((unsigned long long)k << 32) | (0xffffffffu - i);
            else if (k == T) {
                if (eeq < rem) cand[tgt + eeq] = ((unsigned long long)k << 32) | (0xffffffffu - i);
                eeq++;
            }
        }
    }
    __syncthreads();
    // ---- bitonic sort of 256 (key, ~id) words, descending: larger key first, then larger ~id = smaller id
    for (uint32_t size = 2; size <= TOPK_MAX; size <<= 1) {
        for (uint32_t stride = size >> 1; stride; stride >>= 1) {
            if (tid < TOPK_MAX / 2) {
                const uint32_t lo = 2 * tid - (tid & (stride - 1)), hi = lo + stride;
                const bool desc = (lo & size) == 0;
                const unsigned long long a = cand[lo], b = cand[hi];
                if ((a < b) == desc) { cand[lo] = b; cand[hi] = a; }
            }
            __syncthreads();
        }
    }
    if (tid < TOPK_MAX) {
        const unsigned long long c = cand[tid];
        const bool ok = tid < K;
        ids[(size_t)blockIdx.x * TOPK_MAX + tid] = ok ? (int32_t)(0xffffffffu - (uint32_t)c) : -1;
        vals[(size_t)blockIdx.x * TOPK_MAX + tid] = ok ? val_of((uint32_t)(c >> 32)) : -INFINITY;
    }
}

static cudaError_t launch_k_topk(const QwLaunch &L) {
    struct { uint32_t nb, V, k; } a = L.bytes<decltype(a)>(3);
    QW_CHECK_ARG(L.has_bytes(3, 12) && a.nb >= 1 && a.nb <= 64 && a.V >= 1 && a.k >= 1 && a.k <= (uint32_t)TOPK_MAX);
    QW_CHECK_ARG(L.buf<void>(0) && L.buf<void>(1) && L.buf<void>(2) && L.avail(0) >= (size_t)a.nb * a.V * 4 &&
                 L.avail(1) >= (size_t)a.nb * TOPK_MAX * 4 && L.avail(2) >= (size_t)a.nb * TOPK_MAX * 4);
    qw_launch(k_topk_k, a.nb, 1024, 0, L.stream, L.buf<float>(0), L.buf<int32_t>(1), L.buf<float>(2), a.V, a.k);
    return cudaGetLastError();
}
QW_FAMILY(k_topk, launch_k_topk, 1024)
