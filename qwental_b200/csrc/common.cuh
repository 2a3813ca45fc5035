// Device-side helpers shared by the kernel files: shared-memory addresses, mbarrier + 1-D bulk (TMA) copies
// with bounded waits, warp MMA wrappers, fixed-order warp reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qw {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- status word (pinned host memory mapped into the device): a kernel that gives up on a wait records
// where and returns, the host sees it at the batch's wait.
enum : unsigned { ST_OK = 0, ST_MBAR_TIMEOUT = 0x100, ST_BAD_ARG = 0x200, ST_PEER_TIMEOUT = 0x400 };
__device__ __forceinline__ void set_status(unsigned *status, unsigned code) {
    if (status) *(volatile unsigned *)status = code;  // plain store: the word lives in host memory
}

// ---- programmatic dependent launch: pdl_launch() lets the next kernel of the stream begin launching, pdl_wait() blocks
// until the previous kernel has completed and its writes are visible (a no-op when the launch carried no such
// attribute).  Rules of this library: nothing that another kernel of the same step reads or writes is touched before pdl_wait()
// (static weights and tables may be; so may per-slot state whose last writer ran one step earlier -- gdn_fstep_k says why); and data that
// an earlier kernel of the step produced is never read through the non-coherent path (__ldg / ld.global.nc) -- a kernel that
// started early is already running while its predecessor writes, so that path may serve stale lines.  Such loads use
// __ldcg (L2) or plain loads; __ldg is kept for weights and tables only.
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_sync() {
    pdl_launch();
    pdl_wait();
}

// ---- flags shared with other GPUs (peer memory over NVLink): system-scope release / acquire
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// ---- flags between the blocks of one kernel
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// ---- exchange between the ranks of one machine through peer memory: a producing kernel stores its rows into every rank's
// buffer and then publishes; the consuming kernel waits until every rank has published the same step.
struct EpPeers {
    unsigned *flagR[8];    // flag array of rank r (peer memory): slot [q] = sequence number rank q has completed
    unsigned *seq, *done;  // local: this rank's sequence counter, finished-block counter (both start at zero)
    uint32_t nranks, rank;
};
// Every thread of every block calls this after its last peer store.  The block barrier makes the block's stores visible to
// its first thread, whose one system-scope fence then orders them (fences are cumulative) before the counter update; the
// last block advances this rank's sequence number, fences once more and writes the number into slot [rank] of every rank
// with plain (relaxed) stores issued back to back -- together with the fence they are release stores, but none of them
// waits for the previous peer's store to be performed, so the publish costs one NVLink round trip, not one per rank.
__device__ __forceinline__ void st_relaxed_sys(unsigned *p, unsigned v) { asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void ep_publish(const EpPeers &ep) {
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        __threadfence_system();
        if (atomicAdd(ep.done, 1u) == gridDim.x * gridDim.y * gridDim.z - 1) {
            *ep.done = 0;
            const unsigned sv = *ep.seq + 1;
            *ep.seq = sv;
            __threadfence_system();  // every block's stores (observed through the counter) before the flags
            for (uint32_t r = 0; r < ep.nranks; r++) st_relaxed_sys(ep.flagR[r] + ep.rank, sv);
        }
    }
}
// ep_wait is defined after the status helpers below.

// ---- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: polls for at most about two seconds of wall time (the global nanosecond timer), then gives up
// with false; the caller records ST_MBAR_TIMEOUT and leaves.
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Every thread of the block calls this before it reads rows that other ranks stored: thread r < nranks waits (bounded,
// about 2 s, then ST_PEER_TIMEOUT through the status word) until rank r has published the sequence number this rank's own
// producing kernel has just reached; ends with a block barrier.
__device__ __forceinline__ void ep_wait(const unsigned *flags, const unsigned *seq, uint32_t nranks, unsigned *status) {
    if (threadIdx.x < nranks) {
        const unsigned want = *(volatile const unsigned *)seq;
        const uint64_t t0 = global_ns();
        while ((int)(ld_acquire_sys(flags + threadIdx.x) - want) < 0) {
            const uint64_t dt = global_ns() - t0;
            if (dt > 1000000ull && *(volatile unsigned *)status != 0) break;  // an earlier kernel already gave up: do not wait again
            if (dt > 2000000000ull) {
                set_status(status, ST_PEER_TIMEOUT | threadIdx.x);
                break;
            }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity) {
    for (int i = 0; i < 64; i++)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > 2000000000ull) return false;
    }
}

// ---- 1-D bulk copy global -> shared, completion counted on an mbarrier.  dst, src 16-byte aligned,
// bytes a multiple of 16.  No cluster multicast anywhere in this library.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- warp MMA m16n8k16, fp32 accumulate
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// ---- fixed-order warp sum: xor butterfly 16, 8, 4, 2, 1 with explicit round-to-nearest adds (every lane
// ends with the same value; the CPU oracle's lane_reduce() is the same expression)
__device__ __forceinline__ float warp_sum_canon(float v) {
#pragma unroll
    for (int off = 16; off; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t ldu16(const uint8_t *p) { return *(const uint16_t *)p; }

}  // namespace qw
