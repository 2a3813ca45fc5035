// Streaming probe: what a ring of bulk (TMA) copies into shared memory can pull out of HBM when nothing else limits it.
// Persistent blocks (one per SM); block b streams its own contiguous share of the buffer, `stage` bytes per copy, through a
// ring of `nst` stages; one producer lane issues the copies, the consumer warps wait for a stage, optionally read every
// byte of it once (16-byte shared-memory loads) and release it.  The role of the reference's pure-read probes
// (bench/moe_bw.c:1-3, bench/qmv.c:357-382) for the staging mechanism itself; timed from the host with CUDA events.
#include "common.cuh"
#include "qw_kern.h"

using namespace qw;

struct stream_probe_args {
    uint64_t bytes;   // total, a multiple of grid x stage
    uint32_t stage;   // bytes per copy, a multiple of 16
    uint32_t nst;     // stages of the ring (<= 16)
    uint32_t read;    // 1: the consumers read every staged byte; 0: they only wait and release
    uint32_t stride;  // 0: block b streams one contiguous share; 1: stage j of block b is stage j * grid + b of the buffer
};

__global__ void __launch_bounds__(544, 1) stream_probe_k(const uint8_t *src, unsigned *sink, stream_probe_args a, unsigned *status) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = (uint64_t *)smem, *empty = full + 16;
    uint8_t *st0 = smem + 256;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_sync();
    if (tid == 0) {
        for (uint32_t s = 0; s < a.nst; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 16);
        }
        mbar_init_fence();
    }
    __syncthreads();
    const uint64_t per = a.bytes / gridDim.x;
    const uint32_t n = (uint32_t)(per / a.stage);
    auto src_of = [&](uint32_t j) { return src + (a.stride ? ((uint64_t)j * gridDim.x + blockIdx.x) * a.stage : (uint64_t)blockIdx.x * per + (uint64_t)j * a.stage); };
    if (warp == 16) {
        if (lane == 0) {
            bool ok = true;
            for (uint32_t j = 0; j < n; j++) {
                const uint32_t s = j % a.nst;
                if (j >= a.nst && ok && !mbar_wait(&empty[s], (j / a.nst - 1) & 1)) {
                    ok = false;
                    set_status(status, ST_MBAR_TIMEOUT | 22);
                }
                fence_proxy_async();
                mbar_expect_tx(&full[s], a.stage);
                bulk_g2s(st0 + (size_t)s * a.stage, src_of(j), a.stage, &full[s]);
            }
        }
    } else {
        bool ok = true;
        unsigned acc = 0;
        for (uint32_t j = 0; j < n; j++) {
            const uint32_t s = j % a.nst;
            if (ok && !mbar_wait(&full[s], (j / a.nst) & 1)) {
                ok = false;
                if (lane == 0) set_status(status, ST_MBAR_TIMEOUT | 23);
            }
            if (a.read) {
                const uint4 *p = (const uint4 *)(st0 + (size_t)s * a.stage);
                for (uint32_t o = tid; o < a.stage / 16; o += 512) {
                    const uint4 v = p[o];
                    acc ^= v.x ^ v.y ^ v.z ^ v.w;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (acc == 0x9e3779b9u) *sink = acc;  // keeps the loads observable; practically never taken
    }
}

// binds: 0 = source buffer, 1 = sink (4 bytes), 2 = stream_probe_args
static cudaError_t launch_stream_probe(const QwLaunch &L) {
    const stream_probe_args a = L.bytes<stream_probe_args>(2);
    QW_CHECK_ARG(L.has_bytes(2, 24) && a.nst >= 1 && a.nst <= 16 && a.stage >= 16 && a.stage % 16 == 0 && (size_t)a.stage * a.nst + 256 <= 227 * 1024);
    QW_CHECK_ARG(L.buf<void>(0) && L.buf<void>(1) && L.avail(0) >= a.bytes && L.avail(1) >= 4 && ((uintptr_t)L.buf<void>(0) & 15) == 0);
    QW_CHECK_ARG(a.bytes % ((uint64_t)L.sm_count * a.stage) == 0 && a.bytes / ((uint64_t)L.sm_count * a.stage) < 0x7fffffffull);
    const size_t smem = 256 + (size_t)a.stage * a.nst;
    cudaError_t e = cudaFuncSetAttribute(stream_probe_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    qw_launch(stream_probe_k, L.sm_count, 544, smem, L.stream, L.buf<uint8_t>(0), L.buf<unsigned>(1), a, L.status);
    return cudaGetLastError();
}
QW_FAMILY(stream_probe, launch_stream_probe, 544)
