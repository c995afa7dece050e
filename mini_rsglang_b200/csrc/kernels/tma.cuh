// Bulk tensor copies (TMA), mbarriers and the error word of the kernels that wait on them.
//
// Every wait in these kernels is bounded: a wait that runs out of time sets a bit of the
// library's error word and returns, the kernel goes on to its end with whatever it has (its
// loops are bounded by sizes, never by a barrier), and the host reads the word after the step
// and fails the step loudly.  Nothing here spins without a limit.
#pragma once
#include <cuda.h>
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// error word: one per library that includes this header
// ------------------------------------------------------------------------------------------
#define MRS_ERR_BARRIER_TIMEOUT 1u     // an mbarrier wait ran out of time
#define MRS_ERR_TMEM 2u                // tensor memory could not be obtained
static __device__ unsigned int mrs_error_word = 0;
// A word in pinned host memory that mirrors the error word (set once by the host): the host then
// learns of an error by reading its own memory after a step, without a copy from the device.
static __device__ unsigned int* mrs_error_mirror = nullptr;

__device__ __forceinline__ void mrs_raise(unsigned int bits) {
    atomicOr(&mrs_error_word, bits);
    unsigned int* mirror = mrs_error_mirror;
    if (mirror) *reinterpret_cast<volatile unsigned int*>(mirror) = bits;
}

// `host_word`: an unsigned int in pinned (device-visible) host memory, zero while all is well.
static inline int mrs_set_error_mirror(unsigned int* host_word) {
    return (int)cudaMemcpyToSymbol(mrs_error_mirror, &host_word, sizeof(host_word));
}

// Reads and clears the library's error word (synchronises with the device).
static inline int mrs_take_error_word(unsigned int* out) {
    unsigned int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(out, mrs_error_word, sizeof(unsigned int));
    if (e != cudaSuccess) return (int)e;
    if (*out) e = cudaMemcpyToSymbol(mrs_error_word, &zero, sizeof(unsigned int));
    return (int)e;
}

// ------------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n .reg .b64 state;\n mbarrier.arrive.shared::cta.b64 state, [%0];\n}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("{\n .reg .b64 state;\n mbarrier.arrive.expect_tx.shared::cta.b64 state, [%0], %1;\n}"
                 ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Waits for the phase with the given parity to complete, for about a quarter of a second at
// most.  Returns false (and raises the error word) when the time ran out.  Once any wait of any
// CTA has given up, every later wait gives up at once, so a kernel whose barriers are stuck
// drains in a fraction of a second instead of a second per wait.
#define MRS_WAIT_CYCLES (1ll << 29)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long limit_cycles = MRS_WAIT_CYCLES) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    unsigned int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0 && *reinterpret_cast<volatile unsigned int*>(&mrs_error_word) != 0) return false;
        if (clock64() - start > limit_cycles) {
            mrs_raise(MRS_ERR_BARRIER_TIMEOUT);
            return false;
        }
    }
    return true;
}

// Orders writes of ordinary instructions to shared memory before reads by the copy and
// tensor-core units (the asynchronous proxy).
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ------------------------------------------------------------------------------------------
// tiled bulk tensor loads, global -> shared, completion on an mbarrier.  Never multicast.
// The innermost coordinate times the element size must be a multiple of 16 bytes.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3, int c4) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ------------------------------------------------------------------------------------------
// host: tensor maps.  The driver's encoder is looked up through the runtime, so the library
// does not link against the driver.
// ------------------------------------------------------------------------------------------
typedef CUresult (*mrs_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                        const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                        CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline mrs_encode_tiled_fn mrs_tensor_map_encoder() {
    static mrs_encode_tiled_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = (mrs_encode_tiled_fn)p;
    }
    return fn;
}

#define MRS_TENSOR_MAP_FAILED (-3)

// A bfloat16 tensor of `rank` dimensions, innermost first; strides in bytes for dimensions 1..rank-1.
static inline int mrs_make_tensor_map_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                                           const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
    mrs_encode_tiled_fn encode = mrs_tensor_map_encoder();
    if (!encode) return MRS_TENSOR_MAP_FAILED;
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        e[i] = 1;
        if (i + 1 < rank) s[i] = strides_bytes[i];
    }
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : MRS_TENSOR_MAP_FAILED;
}
