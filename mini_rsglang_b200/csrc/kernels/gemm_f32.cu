// True float32 matrix product C[M,N] = A[M,K] . W[N,K]^T with float32 FMA on the CUDA cores:
// no tensor cores, no TF32.  It carries every projection of the 32-bit path.  The order in
// which the K terms of one output element are summed depends on K alone, never on M, so a
// token's result does not change with what else is in the batch.
//                                                   (reference: cuBLAS, kernels/src/lib.rs:298-321)
#include "common.cuh"

#define GF_BM 64
#define GF_BN 64
#define GF_BK 16

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                                                       float* __restrict__ C, int M, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float a_s[GF_BK][GF_BM + 4];
    __shared__ float w_s[GF_BK][GF_BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += GF_BK) {
        // 64 x 16 elements per tile, 256 threads: four elements each, consecutive k per thread group
        for (int idx = tid; idx < GF_BM * GF_BK; idx += 256) {
            const int row = idx / GF_BK, kk = idx % GF_BK;
            const int m = m0 + row, n = n0 + row, k = k0 + kk;
            a_s[kk][row] = (m < M && k < K) ? A[(size_t)m * K + k] : 0.0f;
            w_s[kk][row] = (n < N && k < K) ? W[(size_t)n * K + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GF_BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = a_s[kk][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = w_s[kk][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n < N) C[(size_t)m * N + n] = acc[i][j];
        }
    }
}

MRS_EXPORT int mrs_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return MRS_BAD_ARGUMENT;
    dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
    if (grid.y > 65535) return MRS_BAD_ARGUMENT;
    MRS_LAUNCH(gemm_f32_kernel, grid, 256, 0, stream,
        A, W, C, M, N, K);
    MRS_RETURN_LAUNCH_STATUS();
}
