// Self-test of the tcgen05 helpers (umma.cuh): D[128][16] = A[128][K] * B[16][K]^T, fp16 operands laid out by the threads in
// the un-swizzled K-major form, fp32 accumulator in tensor memory, read back and written out.  Used by the parity tests to
// pin the descriptor conventions the expert-FFN kernel relies on.
#include "qw_kern.h"
#include "umma.cuh"

using namespace qw;

struct umma_test_args {
    uint32_t K;      // multiple of 16, <= 128
    uint32_t order;  // 0: core matrices stored [row group][K group] (K stride 128 bytes), 1: [K group][row group], 2: A in tensor memory
};

__global__ void __launch_bounds__(128) umma_test_k(const __half *A, const __half *B, float *out, umma_test_args a, unsigned *status) {
    __shared__ __align__(128) uint8_t sa[128 * 128 * 2];
    __shared__ __align__(128) uint8_t sb[16 * 128 * 2];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t slot;
    pdl_sync();
    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t KG = a.K / 8;
    // strides of the core matrices (bytes)
    const uint32_t a_k = a.order ? 16 * 128 : 128, a_mn = a.order ? 128 : KG * 128;
    const uint32_t b_k = a.order ? 2 * 128 : 128, b_mn = a.order ? 128 : KG * 128;
    if (warp == 0) tmem_alloc(&slot, 128);  // 32 accumulator columns, then up to 64 columns of A
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_init_fence();
    }
    for (uint32_t c = tid; c < 128 * KG && a.order < 2; c += 128) {  // 16-byte chunk (row, K group)
        const uint32_t row = c / KG, j = c % KG;
        *(uint4 *)(sa + (row >> 3) * a_mn + j * a_k + (row & 7) * 16) = *(const uint4 *)(A + (size_t)row * a.K + j * 8);
    }
    for (uint32_t c = tid; c < 16 * KG; c += 128) {
        const uint32_t row = c / KG, j = c % KG;
        *(uint4 *)(sb + (row >> 3) * b_mn + j * b_k + (row & 7) * 16) = *(const uint4 *)(B + (size_t)row * a.K + j * 8);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the generic stores above are read by the tensor core's proxy
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = slot;
    if (a.order == 2) {  // thread = row: its K values, two per column, into columns 32 ..
        for (uint32_t c0 = 0; c0 < a.K / 2; c0 += 16) {
            uint32_t v[16];
            for (int i = 0; i < 16; i++) v[i] = *(const uint32_t *)(A + (size_t)tid * a.K + 2 * (c0 + i));
            tmem_st16(tmem + ((uint32_t)(warp * 32) << 16) + 32 + c0, v);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncthreads();
        tc_fence_after_sync();
    }
    if (tid == 0) {
        const uint32_t idesc = umma_idesc_f16(128, 16);
        for (uint32_t k = 0; k < a.K / 16; k++) {
            const uint64_t bd = umma_desc(smem_u32(sb) + 2 * k * b_k, b_k, b_mn);
            if (a.order == 2) umma_f16_ts(tmem, tmem + 32 + 8 * k, bd, idesc, k > 0);
            else umma_f16(tmem, umma_desc(smem_u32(sa) + 2 * k * a_k, a_k, a_mn), bd, idesc, k > 0);
        }
        umma_commit(&bar);
    }
    const bool ok = mbar_wait(&bar, 0);
    tc_fence_after_sync();
    if (ok) {
        uint32_t v[16];
        tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16), v);
        tmem_ld_wait();
        for (int c = 0; c < 16; c++) out[(size_t)tid * 16 + c] = __uint_as_float(v[c]);
    } else if (tid == 0) set_status(status, ST_MBAR_TIMEOUT | 12);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

// binds: 0 = A fp16 [128][K], 1 = B fp16 [16][K], 2 = out fp32 [128][16], 3 = umma_test_args
static cudaError_t launch_umma_test(const QwLaunch &L) {
    const umma_test_args a = L.bytes<umma_test_args>(3);
    QW_CHECK_ARG(L.has_bytes(3, 8) && a.K >= 16 && a.K <= 128 && a.K % 16 == 0 && a.order <= 2 && (a.order < 2 || a.K % 32 == 0));
    QW_CHECK_ARG(L.buf<void>(0) && L.buf<void>(1) && L.buf<void>(2) && L.avail(0) >= 128 * a.K * 2 && L.avail(1) >= 16 * a.K * 2 && L.avail(2) >= 128 * 16 * 4);
    QW_CHECK_ARG((((uintptr_t)L.buf<void>(0) | (uintptr_t)L.buf<void>(1)) & 15) == 0);
    qw_launch(umma_test_k, 1, 128, 0, L.stream, L.buf<__half>(0), L.buf<__half>(1), L.buf<float>(2), a, L.status);
    return cudaGetLastError();
}
QW_FAMILY(umma_test, launch_umma_test, 128)

// Timing of back-to-back MMAs (operand contents do not matter): reps x 16 MMAs of M = 128, K = 16 and the given N, issued by
// one thread into `nacc` accumulators in rotation, A from tensor memory or shared memory.  out[0] = cycles from the first
// issue to the completion of the last MMA, out[1] = cycles spent issuing.
struct umma_bench_args {
    uint32_t reps, nacc, N, a_tmem;
};
__global__ void __launch_bounds__(128) umma_bench_k(unsigned long long *out, umma_bench_args a, unsigned *status) {
    extern __shared__ __align__(128) uint8_t sm[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t slot;
    pdl_sync();
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) tmem_alloc(&slot, 512);
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_init_fence();
    }
    for (uint32_t i = tid; i < (64 * 1024) / 16; i += 128) ((uint4 *)sm)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = slot;
    {  // zero the A columns (256 ..) so that no NaN patterns are multiplied
        uint32_t z[16];
        for (int i = 0; i < 16; i++) z[i] = 0;
        for (uint32_t c = 0; c < 256; c += 16) tmem_st16(tmem + ((uint32_t)(warp * 32) << 16) + 256 + c, z);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncthreads();
        tc_fence_after_sync();
    }
    if (tid == 0) {
        const uint32_t idesc = umma_idesc_f16(128, a.N);
        const uint32_t sb = smem_u32(sm), sa = sb + 16384;
        uint64_t bd[8], ad[8];  // descriptors prepared outside the timed loop
        for (uint32_t k = 0; k < 8; k++) {
            bd[k] = umma_desc(sb + k * 256, 128, 0);
            ad[k] = umma_desc(sa + k * 4096, 128, 256);  // A tile = 16 row groups x 256 bytes: all inside the 64 KB
        }
        const uint32_t mask = a.nacc - 1;  // nacc is a power of two
        const long long t0 = clock64();
        for (uint32_t r = 0; r < a.reps; r++) {
#pragma unroll
            for (uint32_t k = 0; k < 16; k++) {
                const uint32_t d = tmem + (k & mask) * a.N;  // nacc * N <= 256
                if (a.a_tmem) umma_f16_ts(d, tmem + 256 + 8 * k, bd[k & 7], idesc, 1);
                else umma_f16(d, ad[k & 7], bd[k & 7], idesc, 1);
            }
        }
        const long long t1 = clock64();
        umma_commit(&bar);
        const bool ok = mbar_wait(&bar, 0);
        const long long t2 = clock64();
        if (!ok) set_status(status, ST_MBAR_TIMEOUT | 12);
        out[0] = (unsigned long long)(t2 - t0);
        out[1] = (unsigned long long)(t1 - t0);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}
// binds: 0 = out (2 x u64), 1 = umma_bench_args
static cudaError_t launch_umma_bench(const QwLaunch &L) {
    const umma_bench_args a = L.bytes<umma_bench_args>(1);
    QW_CHECK_ARG(L.has_bytes(1, 16) && a.reps >= 1 && a.reps <= 4096 && a.nacc >= 1 && (a.nacc & (a.nacc - 1)) == 0 && a.N >= 16 && a.N <= 256 && a.N % 16 == 0 && a.nacc * a.N <= 256);
    QW_CHECK_ARG(L.buf<void>(0) && L.avail(0) >= 16);
    cudaError_t e = cudaFuncSetAttribute(umma_bench_k, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return e;
    qw_launch(umma_bench_k, 1, 128, 64 * 1024, L.stream, L.buf<unsigned long long>(0), a, L.status);
    return cudaGetLastError();
}
QW_FAMILY(umma_bench, launch_umma_bench, 128)
