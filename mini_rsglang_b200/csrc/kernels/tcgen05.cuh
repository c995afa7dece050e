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

// A tile of k rows x n bfloat16 whose rows run along N (MN-major: what a copy of [keys][head size]
// gives a product that contracts over the keys): 64 columns (128 bytes) a row in the same swizzle,
// groups of 8 rows 1024 bytes apart, the next 64 columns `column_group_stride` bytes further.
// `address` moves by 16 rows (2048 bytes) for every 16 elements of K.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128_mn(uint32_t address, uint32_t column_group_stride) {
    uint64_t desc = 0;
    desc |= (uint64_t)((address & 0x3FFFF) >> 4);
    desc |= (uint64_t)((column_group_stride >> 4) & 0x3FFF) << 16;   // leading dimension: between groups of 64 columns
    desc |= (uint64_t)(1024 >> 4) << 32;                             // stride dimension: between groups of 8 rows
    desc |= (uint64_t)1 << 46;
    desc |= (uint64_t)2 << 61;
    return desc;
}

// kind::f16 with bfloat16 A and B and a float32 accumulator of m x n.  A is K-major; B is K-major
// unless `b_mn_major`.
__host__ __device__ constexpr uint32_t umma_idesc_bf16_f32(int m, int n, bool b_mn_major = false) {
    return (1u << 4)                     // D: float32
           | (1u << 7)                   // A: bfloat16
           | (1u << 10)                  // B: bfloat16
           | ((b_mn_major ? 1u : 0u) << 16)
           | ((uint32_t)(n >> 3) << 17)  // N / 8
           | ((uint32_t)(m >> 4) << 24); // M / 16
}

// D[tmem] (+)= A[smem] . B[smem]^T, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
// The same with the accumulator's old content not read (D = A . B^T) or always added to (D += A . B^T): no register
// carries the choice.  A descriptor moves by 2 for every 16 elements of K (32 bytes) within a swizzled row.
__device__ __forceinline__ void umma_bf16_first(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, 0, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc) : "memory");
}
__device__ __forceinline__ void umma_bf16_more(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile("{\n .reg .pred p;\n setp.eq.b32 p, 0, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc) : "memory");
}
// One lane of the (converged) warp: the lane that issues copies and MMAs while the whole warp walks the loop, so
// that addresses, coordinates and descriptors are the same in every lane.
__device__ __forceinline__ bool elect_one() {
    uint32_t chosen;
    asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(chosen));
    return chosen != 0;
}
// The same with A read from tensor memory (K-major: lane = row, two consecutive bfloat16 of K a column).
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 16 consecutive columns of this thread's lane; the values may be used after tmem_load_wait().
__device__ __forceinline__ void tmem_load_16_async(uint32_t address, float* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]),
                   "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15])
                 : "r"(address) : "memory");
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

// 32 consecutive columns of this thread's lane; the values may be used after tmem_load_wait().
__device__ __forceinline__ void tmem_load_32_async(uint32_t address, float* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]),
                   "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]),
                   "=f"(v[16]), "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]),
                   "=f"(v[24]), "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
                 : "r"(address) : "memory");
}
// 32 consecutive columns of this thread's lane.
__device__ __forceinline__ void tmem_load_32(uint32_t address, float* v) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(address) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// Writes 16 consecutive columns of this thread's lane (raw 32-bit words, e.g. pairs of bfloat16).
__device__ __forceinline__ void tmem_store_16_words(uint32_t address, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(address), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
                   "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
// Writes 16 consecutive columns of this thread's lane.
__device__ __forceinline__ void tmem_store_16(uint32_t address, const float (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(address), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
                   "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
                   "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
                   "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
                   "r"(__float_as_uint(v[15])) : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
