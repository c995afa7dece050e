// The fifth-generation tensor core (tcgen05) as the kernels here use it: tensor memory
// (TMEM) allocation, shared-memory and instruction descriptors for bfloat16 operands in the
// 128-byte swizzled K-major layout that the bulk tensor copies write, the MMA itself, its
// commit to an mbarrier, and loads of the accumulator from TMEM.  One CTA per MMA
// (cta_group::1) throughout.
#pragma once
#include "tma.cuh"

// ------------------------------------------------------------------------------------------
// tensor memory: 128 lanes x 512 columns of 32 bits per SM; allocation by one whole warp,
// in powers of two of at least 32 columns.  The address lands in shared memory.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ------------------------------------------------------------------------------------------
// descriptors
// ------------------------------------------------------------------------------------------
// A tile of rows x 64 bfloat16 (128 bytes a row, rows of 8 in 1024-byte groups, 16-byte chunks
// xor-ed with the row: what a bulk tensor copy with the 128-byte swizzle writes), K-major.
// `address` is the tile's shared-memory address, 1024-byte aligned, plus 32 bytes for every
// 16 elements of K that an MMA starts further in.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t address) {
    uint64_t desc = 0;
    desc |= (uint64_t)((address & 0x3FFFF) >> 4);          // start address
    desc |= (uint64_t)1 << 16;                             // leading-dimension offset: unused with this swizzle
    desc |= (uint64_t)(1024 >> 4) << 32;                   // stride between groups of 8 rows
    desc |= (uint64_t)1 << 46;                             // descriptor version of this architecture
    desc |= (uint64_t)2 << 61;                             // 128-byte swizzle
    return desc;
}

// kind::f16 with bfloat16 A and B (both K-major) and a float32 accumulator of m x n.
__host__ __device__ constexpr uint32_t umma_idesc_bf16_f32(int m, int n) {
    return (1u << 4)                     // D: float32
           | (1u << 7)                   // A: bfloat16
           | (1u << 10)                  // B: bfloat16
           | ((uint32_t)(n >> 3) << 17)  // N / 8
           | ((uint32_t)(m >> 4) << 24); // M / 16
}

// D[tmem] (+)= A[smem] . B[smem]^T, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 16 consecutive columns of this thread's lane (lane = 32 * (warp % 4) + lane of the warp).
__device__ __forceinline__ void tmem_load_16(uint32_t address, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(address) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
