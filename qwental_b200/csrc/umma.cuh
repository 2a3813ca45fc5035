// 5th-generation tensor core (tcgen05) helpers: tensor-memory allocation, shared-memory matrix descriptors for the
// un-swizzled K-major layout, the instruction descriptor of the fp16 x fp16 -> fp32 MMA, issue / commit, and loads of the
// accumulator from tensor memory.  One CTA per MMA (cta_group::1) everywhere in this library.
//
// Un-swizzled K-major operand in shared memory: the matrix is cut into core matrices of 8 rows x 16 bytes (8 fp16 values
// along K), each stored as 128 contiguous bytes (row r of the core matrix at + 16 r).  Core matrix (i, j) -- row group i,
// K group j -- lies at  start + i * MN_STRIDE + j * K_STRIDE;  both strides are multiples of 16 bytes and go into the
// descriptor.  One MMA consumes K = 16, i.e. two K groups; the next K step is the same descriptor with its start address
// advanced by 2 * K_STRIDE.
#pragma once
#include "common.cuh"

namespace qw {

// ---- tensor memory: columns of 128 lanes x 32 bits; allocation in powers of two >= 32 columns by one whole warp
__device__ __forceinline__ void tmem_alloc(uint32_t *slot_in_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors
// shared-memory matrix descriptor, no swizzle: bits 0-13 start >> 4, 16-29 leading-dimension byte offset >> 4 (stride between
// the two K groups of one MMA), 32-45 stride-dimension byte offset >> 4 (stride between row groups), 46-47 = 1, 61-63 = 0
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t k_stride, uint32_t mn_stride) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)((k_stride >> 4) & 0x3FFFu) << 16) | ((uint64_t)((mn_stride >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
// instruction descriptor, kind::f16: D = fp32 (bits 4-5 = 1), A = B = fp16 (formats 0), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr uint32_t umma_idesc_f16(uint32_t M, uint32_t N) { return (1u << 4) | ((N >> 3) << 17) | ((M >> 4) << 24); }

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the same with the A operand in tensor memory: lane = row, 32-bit column j of the operand = K elements 2j, 2j + 1 (K = 16 is 8 columns)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the mbarrier receives one arrival when every MMA issued so far by this thread has completed (and has read its operands)
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- accumulator -> registers: warp w % 4 owns lanes 32 (w % 4) .. + 31; thread l of the warp receives lane 32 (w % 4) + l,
// columns col .. col + N - 1.  Address = base + (lane << 16) + column.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                   "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr)
                 : "memory");
}
// registers -> tensor memory, same lane ownership as the loads
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr), "r"(v[0]), "r"(v[1]),
                 "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
                 "r"(v[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace qw
