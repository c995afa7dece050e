// The feed-forward's first product for many rows (prompt portions) on the tcgen05 tensor cores, bfloat16 in, float32
// accumulation, with the activation in its epilogue:
//   out[T, N / 2] = silu(x . gate^T) * (x . up^T)
//
// The library's product for these sizes runs near the tensor cores' peak, but it leaves its result in
// memory, which a second kernel reads again (2,048 tokens: 150 MB and 34 us a layer).  Here a CTA computes a
// tile of 128 tokens x 256 weight rows into one of two accumulators in tensor memory, and four warps turn a
// finished accumulator into the final values and store them while the next tile's MMAs run:
//   warp 0   fetches 128 x 64 token tiles and 256 x 64 weight tiles with bulk tensor copies (TMA,
//            128-byte swizzle) into a ring of stages;
//   warp 1   one thread issues tcgen05.mma (M 128, N 256, K 16) on the stages;
//   warps 2-5 a thread a token: the row's 256 sums from tensor memory.  A tile holds two blocks of 64 gate
//            and 64 up rows (the weights are stored so), so a thread has both factors of its outputs.
// CTAs are persistent; the tiles that share a weight tile are taken by neighbouring CTAs at the same
// time, so the weights come from HBM once.  Every wait is bounded (tma.cuh).
//   (reference: cuBLAS and a kernel of its own, crates/models/src/qwen3.rs:255-261; ops.cu:91-94)
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;              // tokens of a tile: the M of the MMA
constexpr int BN = 256;              // weight rows of a tile: two blocks of 64 gate + 64 up rows
constexpr int BK = 64;               // one 128-byte swizzled row of bfloat16
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLUMNS = 2 * BN;
constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * sizeof(uint64_t) + 16;

__global__ void __launch_bounds__(THREADS, 1) gemm_many_rows_kernel(
    const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map, bf16* __restrict__ out, int T, int N, int K) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + BK - 1) / BK;
    const int m_tiles = (T + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;          // tile t: weight tile t / m_tiles, token tile t % m_tiles

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLUMNS);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();

    // In the copy and MMA warps the whole warp walks the loop and one elected lane issues: addresses and descriptors
    // are then the same in every lane, which makes an issue cheap.
    if (warp == 0) {
        const bool leader = elect_one();
        if (leader) {
            tma_prefetch_descriptor(&x_map);
            tma_prefetch_descriptor(&w_map);
        }
        int it = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % STAGES;
                if (!(alive = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1))) break;
                unsigned char* stage = smem + s * STAGE_BYTES;
                if (leader) {
                    mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_2d(stage, &x_map, &full[s], kb * BK, m0);
                    tma_load_2d(stage + A_BYTES, &w_map, &full[s], kb * BK, n0);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        const bool leader = elect_one();
        constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, BN);
        int it = 0, round = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++round) {
            const int buffer = round & 1;
            if (!(alive = mbar_wait(&acc_empty[buffer], ((round >> 1) & 1) ^ 1))) break;
            tcgen05_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buffer * BN;
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % STAGES;
                if (!(alive = mbar_wait(&full[s], (it / STAGES) & 1))) break;
                tcgen05_fence_after_sync();
                const uint64_t a_desc = umma_smem_desc_sw128(smem_u32(smem + s * STAGE_BYTES));
                const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(smem + s * STAGE_BYTES + A_BYTES));
                if (leader) {
                    if (kb > 0) {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16_more(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc);
                    } else {
                        umma_bf16_first(d_tmem, a_desc, b_desc, idesc);
#pragma unroll
                        for (int k = 1; k < BK / UMMA_K; ++k) umma_bf16_more(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc);
                    }
                    umma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (leader) umma_commit(&acc_full[buffer]);
            __syncwarp();
        }
    } else {
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                 // token within the tile
        const int half_n = N >> 1;
        int round = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++round) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            const int buffer = round & 1;
            mbar_wait(&acc_full[buffer], (round >> 1) & 1);
            __syncwarp();
            tcgen05_fence_after_sync();
            const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + buffer * BN;
            const int token = m0 + row;
            bf16* dst = out + (size_t)token * half_n + (n0 >> 1);
#pragma unroll
            for (int block = 0; block < BN / 128; ++block) {          // 64 gate columns, then their 64 up columns
#pragma unroll
                for (int c = 0; c < 64; c += 32) {
                    float g[32], u[32];
                    tmem_load_32_async(acc + block * 128 + c, g);
                    tmem_load_32_async(acc + block * 128 + 64 + c, u);
                    tmem_load_wait();
                    if (token < T && n0 + block * 128 < N) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int p = 0; p < 4; ++p) {
                                const float g0 = g[e + 2 * p], g1 = g[e + 2 * p + 1];
                                __nv_bfloat162 pair = __floats2bfloat162_rn(g0 / (1.0f + __expf(-g0)) * u[e + 2 * p],
                                                                            g1 / (1.0f + __expf(-g1)) * u[e + 2 * p + 1]);
                                w[p] = *reinterpret_cast<uint32_t*>(&pair);
                            }
                            *reinterpret_cast<uint4*>(dst + block * 64 + c + e) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buffer]);
        }
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLUMNS);
    }
}

int launch(const void* x_map, const void* w_map, void* out, int T, int N, int K, int ctas, void* stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_many_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles = ((T + BM - 1) / BM) * ((N + BN - 1) / BN);
    MRS_LAUNCH(gemm_many_rows_kernel, ctas < tiles ? ctas : tiles, THREADS, SMEM_BYTES, stream, *reinterpret_cast<const CUtensorMap*>(x_map),
               *reinterpret_cast<const CUtensorMap*>(w_map), (bf16*)out, T, N, K);
    MRS_RETURN_LAUNCH_STATUS();
}

}  // namespace

// A tensor map of a row-major bfloat16 matrix [rows, cols] for copies of `box_rows` rows x 64 columns
// (128 rows for the activations, 256 for the weights).
MRS_EXPORT int mrs_gemm_many_rows_map(const void* base, long long rows, long long cols, int box_rows, void* map_out) {
    if (rows <= 0 || cols <= 0 || cols % 8 || box_rows <= 0 || box_rows > 256 || ((uintptr_t)base & 15)) return MRS_BAD_ARGUMENT;
    const uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
    const uint64_t strides[1] = {(uint64_t)cols * 2};
    const uint32_t box[2] = {BK, (uint32_t)box_rows};
    return mrs_make_tensor_map_bf16(reinterpret_cast<CUtensorMap*>(map_out), base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// out[T, N / 2] = silu(x . gate^T) * (x . up^T), bfloat16; w [N, K] holds in every block of 128 rows 64 gate rows and
// then the 64 matching up rows (N a multiple of 128).  `x_map`: map of x [T, K] with boxes of 128 rows; `w_map`: map
// of w with boxes of 256 rows.  `ctas`: the GPU's SMs.
MRS_EXPORT int mrs_gemm_gated_rows(const void* x_map, const void* w_map, void* out, int T, int N, int K, int ctas, void* stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || N % 128 || ctas < 1 || !x_map || !w_map || !out || ((uintptr_t)out & 15)) return MRS_BAD_ARGUMENT;
    return launch(x_map, w_map, out, T, N, K, ctas, stream);
}

MRS_EXPORT int mrs_gemm_many_rows_take_error(unsigned int* word) { return mrs_take_error_word(word); }
// Mirrors the error word into a word of pinned host memory from now on.
MRS_EXPORT int mrs_gemm_many_rows_mirror_errors(unsigned int* host_word) { return mrs_set_error_mirror(host_word); }

MRS_EXPORT const char* mrs_gemm_many_rows_error_string(int code) {
    if (code == MRS_BAD_ARGUMENT) return "arguments outside what the kernel supports (K no multiple of 8, N no multiple of 128, unaligned base)";
    if (code == MRS_TENSOR_MAP_FAILED) return "the driver refused the tensor map (address, sizes or strides)";
    return cudaGetErrorString((cudaError_t)code);
}
