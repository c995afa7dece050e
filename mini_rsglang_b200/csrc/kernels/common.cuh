// Shared helpers of the engine's CUDA kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>
#include <stdlib.h>

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<bf16>(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` has 33 floats.
__device__ __forceinline__ float block_sum(float x, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    x = warp_sum(x);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    if (warp == 0) {
        float y = lane < warps ? scratch[lane] : 0.0f;
        y = warp_sum(y);
        if (lane == 0) scratch[32] = y;
    }
    __syncthreads();
    return scratch[32];
}

// Every launcher returns the CUDA error code of its launch (0 = success).
#define MRS_RETURN_LAUNCH_STATUS() return (int)cudaGetLastError()
#define MRS_EXPORT extern "C" __attribute__((visibility("default")))

// Status codes of the launchers' own argument checks (negative, so they cannot be CUDA codes).
#define MRS_BAD_ARGUMENT (-2)

// ------------------------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of the engine is launched with the attribute
// that lets it start while the kernel before it in the stream is still running; it must call
// pdl_wait() before it reads or writes anything that an earlier kernel may write or read
// (after the wait the earlier kernels are complete and their memory is visible), and calls
// pdl_launch_dependents() to let the kernel after it start in the same way.  What a kernel
// does before its wait (barrier set-up, fetching weights) overlaps its predecessors.  The
// kernels call pdl_launch_dependents() first: the kernel after a small kernel then becomes
// resident while the kernel before the small one still runs (a product fetches its first
// weight tiles under the product before it); its own wait still orders it after both.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Multiprocessors of the current device (asked once per device and kept): grids that loop over their
// work are capped by a multiple of it.
static inline int mrs_sm_count() {
    static int counts[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 1;
    if (counts[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 1;
        counts[device] = n;
    }
    return counts[device];
}

template <typename... KernelArgs, typename... Args>
static inline int mrs_launch(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    static const bool plain = getenv("MRS_PLAIN_LAUNCH") != nullptr;    // for measuring what the overlap gives
    config.attrs = &attribute;
    config.numAttrs = plain ? 0 : 1;
    cudaError_t e = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}

// Launches with the attribute above and returns from the enclosing launcher on failure.
#define MRS_LAUNCH(kernel, grid, block, smem, stream, ...)                                                        \
    do {                                                                                                          \
        const int mrs_status_ = mrs_launch(kernel, dim3(grid), dim3(block), (size_t)(smem), (cudaStream_t)(stream), \
                                           __VA_ARGS__);                                                          \
        if (mrs_status_ != 0) return mrs_status_;                                                                 \
    } while (0)
