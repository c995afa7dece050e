// Matrix products out[M, N] = x[M, K] . w[N, K]^T for few rows (M <= 128: decoded tokens and
// short portions), bfloat16 in, float32 accumulation, on the tcgen05 tensor cores.
//
// With few rows the product is bound by reading the weights once from HBM, so the kernel is a
// weight streamer: the roles of the operands are swapped (128 weight rows are the M of the MMA,
// the tokens its N, padded to 16/32/64/128), a producer warp fetches 128 x 64 weight tiles and
// the matching slice of x with bulk tensor copies (TMA, 128-byte swizzle) into a ring of
// shared-memory stages of two such blocks of K, a second warp issues tcgen05.mma on the stages
// into an accumulator in tensor memory (both warps walk their loops whole and one elected lane
// issues; a stage costs one barrier round and one tcgen05.commit), and four warps read finished
// accumulators back and store them transposed.
// CTAs are persistent: each walks its share of the work units (a unit = 128 weight rows x a
// range of K), with two accumulators in tensor memory, so copies and MMAs of the next unit run
// while the last one is stored.
//
// K is cut into `splits` ranges so that the units fill all SMs evenly.  The cut depends on N
// and K alone and partial sums are added in the order of the ranges by whichever CTA finishes
// a tile last, so a row's result does not depend on M or on what else is in the batch, bit for
// bit.                       (reference: cuBLAS in 32-row blocks, crates/kernels/src/lib.rs:241-322)
#include "tcgen05.cuh"

namespace {

constexpr int TILE_N = 128;          // weight rows of a unit: the M of the MMA
constexpr int BLOCK_K = 64;          // one 128-byte swizzled row of bfloat16
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;         // warp 0: copies, warp 1: MMA, warps 2..5: accumulator to memory
constexpr int W_TILE_BYTES = TILE_N * BLOCK_K * 2;
#ifndef MRS_GEMM_TC_BLOCKS
#define MRS_GEMM_TC_BLOCKS 2
#endif
#ifndef MRS_GEMM_TC_RING
#define MRS_GEMM_TC_RING 8
#endif

template <int MPAD> struct Shape {
    static constexpr int X_TILE_BYTES = MPAD * BLOCK_K * 2;
    static constexpr int BLOCK_BYTES = W_TILE_BYTES + X_TILE_BYTES;          // a block of K: its weight tile, then its rows of x
    // blocks of K in a stage: one barrier round and one commit for all of them (a commit holds the issuing lane
    // until the MMAs before it have drained, some 400 clocks whatever their number)
    static constexpr int BLOCKS = MRS_GEMM_TC_BLOCKS;
    static constexpr int STAGE_BYTES = BLOCKS * BLOCK_BYTES;
    // measured in the engine (decode step at batch 8, rings of 5, 6, 7, 8, 9, 10, 11 stages of 16 rows):
    // 4.51, 4.35, 4.27, 4.27, 4.32, 4.38, 4.42 ms
    static constexpr int STAGES = (MPAD <= 32 ? MRS_GEMM_TC_RING : (MPAD <= 64 ? 6 : 5)) / BLOCKS;
    static constexpr int TMEM_COLUMNS = 2 * MPAD < 32 ? 32 : 2 * MPAD;
    static constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * sizeof(uint64_t) + 16 +
                                         (size_t)MPAD * (MPAD <= 32 ? 128 : 64) * sizeof(float) + 4 * MPAD * sizeof(float) +
                                         (MPAD <= 32 ? (size_t)MPAD * (128 + 1) * sizeof(float) : 0) +   // cosines, sines, write slots
                                         MPAD * sizeof(float);                                           // the rows' norm factors
};

// How K is cut, as one number: ranges a tile (low 8 bits) for the first `tiles_first` tiles (bits 16 and up), and,
// where bits 8-15 are not zero, that many ranges for the tiles behind them: the tiles of a last round of units
// that would fill the GPU partly take more ranges, so that they fill it, and the round is shorter.
struct Ranges {
    int first, rest, tiles_first;
};
__host__ __device__ __forceinline__ Ranges ranges_of(int packed, int n_tiles) {
    Ranges r;
    r.first = packed & 0xFF;
    r.rest = (packed >> 8) & 0xFF;
    r.tiles_first = r.rest ? (packed >> 16) : n_tiles;
    if (r.tiles_first > n_tiles) r.tiles_first = n_tiles;
    return r;
}
__host__ __device__ __forceinline__ int units_of(const Ranges& r, int n_tiles) {
    return r.tiles_first * r.first + (n_tiles - r.tiles_first) * r.rest;
}
// A unit's tile, its range of K and the ranges of that tile.
__device__ __forceinline__ void unit_place(const Ranges& r, int unit, int& tile, int& split, int& splits) {
    const int units_first = r.tiles_first * r.first;
    if (unit < units_first) {
        tile = unit / r.first, split = unit % r.first, splits = r.first;
    } else {
        const int u = unit - units_first;
        tile = r.tiles_first + u / r.rest, split = u % r.rest, splits = r.rest;
    }
}

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

enum { EPI_PLAIN = 0, EPI_GATED = 1, EPI_HEADS = 2, EPI_RESIDUAL = 3 };

// How a product is tied to the RMSNorms around it, so that no kernel of their own runs for them.
// In: the activations are rows of the residual stream times the norm's weights, not yet divided by their
// root mean square; the sums of squares of the rows come in parts (one per 128 columns) and the product
// multiplies its sums by rsqrt(mean + eps) of their row, which gives the product of the normalised rows.
// Out (EPI_RESIDUAL): the product's result, rounded to bfloat16, is added to the float32 stream; `out`
// gets the new stream times the next norm's weights, and the parts of the rows' sums of squares are left
// for the product after it.  The parts are added in their order, so a row's factor does not depend on
// the batch.
struct NormLink {
    const float* in_square_sums;     // [in_parts][in_stride] or null
    int in_parts, in_stride;
    float in_inv_width, in_eps;
    float* stream;                   // [M, N] float32 (EPI_RESIDUAL)
    const float* next_weight;        // [N]
    float* out_square_sums;          // [tiles of N][MPAD]
};

// What the head epilogue needs beside the product: where q goes, the cache pages of k and v, the
// tokens' positions and write slots, the head norms' scales and the rotation's frequencies.
struct HeadEpilogue {
    bf16* q_out;             // [M, nq, 128]
    bf16* k_cache;           // [pages, nkv, page_size, 128]
    bf16* v_cache;
    const int* positions;    // [M]
    const int* slots;        // [M] page * page_size + offset, < 0 or null: no write
    const float* q_norm;     // [128] or null
    const float* k_norm;
    const float* inv_freq;   // [64] or null
    float eps;
    int nq, nkv, page_size;
};

template <int MPAD, typename OutT, int EPI>
__global__ void __launch_bounds__(THREADS, 1) gemm_small_m_kernel(
    const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map, OutT* __restrict__ out,
    float* __restrict__ partials, int* __restrict__ counters, int M, int N, int K, int splits, const HeadEpilogue heads,
    const NormLink link) {
    using S = Shape<MPAD>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE_BYTES);
    uint64_t* empty = full + S::STAGES;
    uint64_t* acc_full = empty + S::STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    float* exchange = reinterpret_cast<float*>(tmem_slot + 4);        // rows of a tile meet here: [MPAD][64] gated, [MPAD][128] + [4][MPAD] heads (up to 32 rows)
    __shared__ int is_last;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    const int n_tiles = (N + TILE_N - 1) / TILE_N;
    const Ranges ranges = ranges_of(splits, n_tiles);
    const int units = units_of(ranges, n_tiles);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) {
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
        tmem_alloc(tmem_slot, S::TMEM_COLUMNS);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------------ copies
        // The whole warp walks the loop and one elected lane issues: addresses and coordinates are then the same in
        // every lane, and an issue costs a fraction of what it costs a lone lane in divergent code.
        const bool leader = elect_one();
        if (leader) {
            tma_prefetch_descriptor(&w_map);
            tma_prefetch_descriptor(&x_map);
        }
        // The weights do not depend on the kernel before this one: the first ring of weight tiles is
        // asked for at once, and only the activations wait for that kernel to finish.
        int it = 0;
        int first_kb[S::STAGES], first_blocks[S::STAGES];
        bool waited = false;
        // the rows of x of a stage's blocks
        auto fetch_x = [&](int s, int kb, int blocks) {
            if (leader)
#pragma unroll
                for (int b = 0; b < S::BLOCKS; ++b)
                    if (b < blocks)
                        tma_load_2d(smem + s * S::STAGE_BYTES + b * S::BLOCK_BYTES + W_TILE_BYTES, &x_map, &full[s], (kb + b) * BLOCK_K, 0);
        };
        for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
            int tile, split, of;
            unit_place(ranges, unit, tile, split, of);
            const int kb0 = (int)((long long)split * k_blocks / of), kb1 = (int)((long long)(split + 1) * k_blocks / of);
            for (int kb = kb0; kb < kb1; kb += S::BLOCKS, ++it) {
                const int s = it % S::STAGES;
                const int blocks = min(S::BLOCKS, kb1 - kb);
                if (it == S::STAGES && !waited) {      // the ring is full of weights: now the activations
                    pdl_wait();
                    waited = true;
#pragma unroll
                    for (int j = 0; j < S::STAGES; ++j) fetch_x(j, first_kb[j], first_blocks[j]);
                }
                if (waited) mbar_wait(&empty[s], ((it / S::STAGES) & 1) ^ 1);
                if (leader) {
                    mbar_arrive_expect_tx(&full[s], blocks * S::BLOCK_BYTES);
#pragma unroll
                    for (int b = 0; b < S::BLOCKS; ++b)
                        if (b < blocks) tma_load_2d(smem + s * S::STAGE_BYTES + b * S::BLOCK_BYTES, &w_map, &full[s], (kb + b) * BLOCK_K, tile * TILE_N);
                }
                if (waited) fetch_x(s, kb, blocks);
                else {
#pragma unroll
                    for (int j = 0; j < S::STAGES; ++j)
                        if (j == it) first_kb[j] = kb, first_blocks[j] = blocks;
                }
                __syncwarp();
            }
        }
        if (!waited) {                                  // fewer steps than stages
            pdl_wait();
#pragma unroll
            for (int j = 0; j < S::STAGES; ++j)
                if (j < it) fetch_x(j, first_kb[j], first_blocks[j]);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA
        const bool leader = elect_one();
        constexpr uint32_t idesc = umma_idesc_bf16_f32(TILE_N, MPAD);
        int it = 0, round = 0;
        for (int unit = blockIdx.x; unit < units; unit += gridDim.x, ++round) {
            int tile, split, of;
            unit_place(ranges, unit, tile, split, of);
            const int kb0 = (int)((long long)split * k_blocks / of), kb1 = (int)((long long)(split + 1) * k_blocks / of);
            const int buffer = round & 1;
            mbar_wait(&acc_empty[buffer], ((round >> 1) & 1) ^ 1);
            tcgen05_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buffer * MPAD;
            for (int kb = kb0; kb < kb1; kb += S::BLOCKS, ++it) {
                const int s = it % S::STAGES;
                const int blocks = min(S::BLOCKS, kb1 - kb);
                mbar_wait(&full[s], (it / S::STAGES) & 1);
                tcgen05_fence_after_sync();
                if (leader) {
#pragma unroll
                    for (int b = 0; b < S::BLOCKS; ++b)
                        if (b < blocks) {
                            const uint64_t w_desc = umma_smem_desc_sw128(smem_u32(smem + s * S::STAGE_BYTES + b * S::BLOCK_BYTES));
                            const uint64_t x_desc = umma_smem_desc_sw128(smem_u32(smem + s * S::STAGE_BYTES + b * S::BLOCK_BYTES + W_TILE_BYTES));
                            if (kb > kb0 || b > 0) {
#pragma unroll
                                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) umma_bf16_more(d_tmem, w_desc + 2 * k, x_desc + 2 * k, idesc);
                            } else {
                                umma_bf16_first(d_tmem, w_desc, x_desc, idesc);
#pragma unroll
                                for (int k = 1; k < BLOCK_K / UMMA_K; ++k) umma_bf16_more(d_tmem, w_desc + 2 * k, x_desc + 2 * k, idesc);
                            }
                        }
                    umma_commit(&empty[s]);          // the stage is free once these MMAs have read it
                }
                __syncwarp();
            }
            if (leader) umma_commit(&acc_full[buffer]);
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------------ accumulator -> memory
        const int quarter = warp & 3;                      // the TMEM lanes this warp may read
        const int row = quarter * 32 + lane;               // weight row within the tile
        const int epi_thread = (warp - 2) * 32 + lane;
        // What the head epilogue needs beside the sums is fetched and computed now, under the first weight
        // tiles: the rotation's cosines and sines of every row, the write slots, this row's norm scales.
        float* cos_s = exchange + MPAD * 128 + 4 * MPAD;   // [MPAD][64]
        float* sin_s = cos_s + MPAD * 64;
        int* slot_s = reinterpret_cast<int*>(sin_s + MPAD * 64);
        float q_scale = 1.0f, k_scale = 1.0f;
        if (EPI == EPI_HEADS) {
            if (heads.inv_freq)
                for (int idx = epi_thread; idx < M * 64; idx += 128)
                    sincosf((float)heads.positions[idx >> 6] * heads.inv_freq[idx & 63], &sin_s[idx], &cos_s[idx]);
            if (epi_thread < M) slot_s[epi_thread] = heads.slots ? heads.slots[epi_thread] : -1;
            if (heads.q_norm) q_scale = heads.q_norm[row];
            if (heads.k_norm) k_scale = heads.k_norm[row];
            epilogue_sync();
        }
        float* row_factor = exchange + MPAD * (MPAD <= 32 ? 128 : 64) + 4 * MPAD + (MPAD <= 32 ? MPAD * (128 + 1) : 0);   // [MPAD]
        pdl_wait();                                        // `out`, `partials` and `counters` may still be in use before
        if (link.in_square_sums) {
            // the factor of each row's norm from the parts that the product before this one left
            if (epi_thread < MPAD) {
                float total = 0.0f;
                if (epi_thread < M) {
#pragma unroll 8
                    for (int p = 0; p < link.in_parts; ++p) total += __ldcg(link.in_square_sums + (size_t)p * link.in_stride + epi_thread);
                }
                row_factor[epi_thread] = rsqrtf(total * link.in_inv_width + link.in_eps);
            }
            epilogue_sync();
        }
        int round = 0;
        for (int unit = blockIdx.x; unit < units; unit += gridDim.x, ++round) {
            int tile, split, of;
            unit_place(ranges, unit, tile, split, of);
            const int buffer = round & 1;
            // the stream's old values and the next norm's weight of this thread's column: asked for early,
            // needed only by the CTA that finishes the tile
            float stream_old[EPI == EPI_RESIDUAL ? MPAD : 1];
            float next_weight = 0.0f;
            if (EPI == EPI_RESIDUAL) {
                const int column = tile * TILE_N + row;
                if (column < N) next_weight = __ldg(link.next_weight + column);
#pragma unroll
                for (int m = 0; m < MPAD; ++m) stream_old[m] = (m < M && column < N) ? __ldcg(link.stream + (size_t)m * N + column) : 0.0f;
            }
            mbar_wait(&acc_full[buffer], (round >> 1) & 1);
            __syncwarp();                    // the loads from tensor memory are collective
            tcgen05_fence_after_sync();
            float acc[MPAD];                   // one trip to tensor memory for the whole row
#pragma unroll
            for (int c = 0; c < MPAD; c += 16) tmem_load_16_async(tmem_base + ((uint32_t)(quarter * 32) << 16) + buffer * MPAD + c, acc + c);
            tmem_load_wait();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buffer]);      // the MMA warp may overwrite this accumulator

            const int n = tile * TILE_N + row;
            bool finished = of == 1;                      // does this CTA hold the tile's final sums?
            if (of > 1) {
                // partial sums of this range of K, then: the CTA that finishes the tile last adds all ranges in order
                constexpr int V = MPAD / 4;                                   // float4s of a padded row
                constexpr int RANGES_AT_ONCE = MPAD == 16 ? 4 : (MPAD == 32 ? 2 : 1);
                const int m4 = (M + 3) >> 2;
                float4* mine = reinterpret_cast<float4*>(partials) + ((size_t)unit * TILE_N + row) * m4;
#pragma unroll
                for (int j = 0; j < V; ++j)
                    if (j < m4) __stcg(mine + j, make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
                __threadfence();
                epilogue_sync();
                if (epi_thread == 0) {
                    const int arrived = atomicAdd(&counters[tile], 1);
                    is_last = arrived == of - 1;
                    if (is_last) counters[tile] = 0;           // ready for the next launch
                }
                epilogue_sync();
                finished = is_last;
                if (finished) {
                    __threadfence();
                    const float4* first = reinterpret_cast<const float4*>(partials) + ((size_t)(unit - split) * TILE_N + row) * m4;
#pragma unroll
                    for (int m = 0; m < MPAD; ++m) acc[m] = 0.0f;
                    for (int s0 = 0; s0 < of; s0 += RANGES_AT_ONCE) {
                        float4 v[RANGES_AT_ONCE][V];                      // all loads of a pass are in flight together
#pragma unroll
                        for (int u = 0; u < RANGES_AT_ONCE; ++u)
#pragma unroll
                            for (int j = 0; j < V; ++j)
                                v[u][j] = (s0 + u < of && j < m4) ? __ldcg(first + (size_t)(s0 + u) * TILE_N * m4 + j)
                                                                      : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                        for (int u = 0; u < RANGES_AT_ONCE; ++u)
#pragma unroll
                            for (int j = 0; j < V; ++j) {
                                acc[4 * j] += v[u][j].x;
                                acc[4 * j + 1] += v[u][j].y;
                                acc[4 * j + 2] += v[u][j].z;
                                acc[4 * j + 3] += v[u][j].w;
                            }
                    }
                }
            }
            if (finished && link.in_square_sums) {
#pragma unroll
                for (int m = 0; m < MPAD; ++m) acc[m] *= row_factor[m];
            }
            if (finished) {
                if (EPI == EPI_RESIDUAL) {
                    // stream += bfloat16(sum); out = bfloat16(stream * next norm's weight); this tile's part of
                    // the rows' sums of squares
                    float* warp_sums = exchange;                                                     // [4][MPAD]
#pragma unroll
                    for (int m = 0; m < MPAD; ++m)
                        if (m < M) {
                            float v = 0.0f;
                            if (n < N) {
                                v = stream_old[m] + __bfloat162float(__float2bfloat16_rn(acc[m]));
                                link.stream[(size_t)m * N + n] = v;
                                out[(size_t)m * N + n] = from_float<OutT>(v * next_weight);
                            }
                            const float sq = warp_sum(v * v);
                            if (lane == 0) warp_sums[(warp - 2) * MPAD + m] = sq;
                        }
                    epilogue_sync();
                    if (epi_thread < M)
                        link.out_square_sums[(size_t)tile * MPAD + epi_thread] =
                            (warp_sums[epi_thread] + warp_sums[MPAD + epi_thread]) + (warp_sums[2 * MPAD + epi_thread] + warp_sums[3 * MPAD + epi_thread]);
                } else if (EPI == EPI_GATED) {
                    // the tile's rows 0..63 are gate rows, rows 64..127 the matching up rows: the upper half
                    // hands its sums over and the lower half writes silu(gate) * up, 64 columns of [M, N / 2]
                    if (row >= 64) {
#pragma unroll
                        for (int m = 0; m < MPAD; ++m)
                            if (m < M) exchange[m * 64 + row - 64] = acc[m];
                    }
                    epilogue_sync();
                    if (row < 64) {
#pragma unroll
                        for (int m = 0; m < MPAD; ++m)
                            if (m < M) {
                                const float g = acc[m], u = exchange[m * 64 + row];
                                out[(size_t)m * (N >> 1) + tile * 64 + row] = from_float<OutT>(g / (1.0f + __expf(-g)) * u);
                            }
                    }
                } else if (EPI == EPI_HEADS) {
                    // The tile is one head of the fused q/k/v projection (128 rows = the head's elements): per-head
                    // RMSNorm of q and k, rotation of q and k by the tokens' positions, q to its tensor, k and v into
                    // the cache pages: what a kernel of its own does after the library's product.
                    const int head = tile, element = row;
                    const int kind = head < heads.nq ? 0 : (head < heads.nq + heads.nkv ? 1 : 2);      // q, k, v
                    const bool normed = kind == 0 ? heads.q_norm != nullptr : (kind == 1 ? heads.k_norm != nullptr : false);
                    float* warp_sums = exchange + MPAD * 128;                                        // [4][MPAD]
                    static_assert(EPI != EPI_HEADS || MPAD <= 32, "the head epilogue takes up to 32 rows");
                    if (normed) {
#pragma unroll
                        for (int m = 0; m < MPAD; ++m)
                            if (m < M) {
                                const float sq = warp_sum(acc[m] * acc[m]);
                                if (lane == 0) warp_sums[(warp - 2) * MPAD + m] = sq;
                            }
                        epilogue_sync();
                        const float w = kind == 0 ? q_scale : k_scale;
#pragma unroll
                        for (int m = 0; m < MPAD; ++m)
                            if (m < M) {
                                const float total = (warp_sums[m] + warp_sums[MPAD + m]) + (warp_sums[2 * MPAD + m] + warp_sums[3 * MPAD + m]);
                                acc[m] = acc[m] * rsqrtf(total / 128.0f + heads.eps) * w;
                            }
                    }
                    if (kind != 2 && heads.inv_freq) {
#pragma unroll
                        for (int m = 0; m < MPAD; ++m)
                            if (m < M) exchange[m * 128 + element] = acc[m];
                        epilogue_sync();
#pragma unroll
                        for (int m = 0; m < MPAD; ++m)
                            if (m < M) {
                                const float cs = cos_s[m * 64 + (element & 63)], sn = sin_s[m * 64 + (element & 63)];
                                const float partner = exchange[m * 128 + (element ^ 64)];
                                acc[m] = element < 64 ? acc[m] * cs - partner * sn : acc[m] * cs + partner * sn;
                            }
                    }
                    if (kind == 0) {
#pragma unroll
                        for (int m = 0; m < MPAD; ++m)
                            if (m < M) heads.q_out[((size_t)m * heads.nq + head) * 128 + element] = __float2bfloat16_rn(acc[m]);
                    } else if (heads.slots) {
                        bf16* cache = kind == 1 ? heads.k_cache : heads.v_cache;
                        const int g = kind == 1 ? head - heads.nq : head - heads.nq - heads.nkv;
#pragma unroll
                        for (int m = 0; m < MPAD; ++m)
                            if (m < M) {
                                const int slot = slot_s[m];
                                if (slot >= 0) {
                                    const int page = slot / heads.page_size, off = slot % heads.page_size;
                                    cache[(((size_t)page * heads.nkv + g) * heads.page_size + off) * 128 + element] = __float2bfloat16_rn(acc[m]);
                                }
                            }
                    }
                } else if (n < N) {
#pragma unroll
                    for (int m = 0; m < MPAD; ++m)
                        if (m < M) out[(size_t)m * N + n] = from_float<OutT>(acc[m]);
                }
            }
            epilogue_sync();                               // `is_last` is rewritten in the next round
        }
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, S::TMEM_COLUMNS);
    }
}

template <int MPAD, typename OutT, int EPI>
int launch(const CUtensorMap* w_map, const CUtensorMap* x_map, void* out, float* partials, int* counters, int M, int N,
           int K, int splits, int ctas, cudaStream_t stream, const NormLink& link, const HeadEpilogue& heads = HeadEpilogue{}) {
    using S = Shape<MPAD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_small_m_kernel<MPAD, OutT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return mrs_launch(gemm_small_m_kernel<MPAD, OutT, EPI>, dim3(ctas), dim3(THREADS), S::SMEM_BYTES, stream, *w_map, *x_map,
                      (OutT*)out, partials, counters, M, N, K, splits, heads, link);
}

}  // namespace

// A tensor map of a row-major bfloat16 matrix [rows, cols] for copies of `box_rows` rows x 64 columns.
MRS_EXPORT int mrs_gemm_tc_map(const void* base, long long rows, long long cols, int box_rows, void* map_out) {
    if (rows <= 0 || cols <= 0 || cols % 8 || box_rows <= 0 || box_rows > 256 || ((uintptr_t)base & 15)) return MRS_BAD_ARGUMENT;
    const uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
    const uint64_t strides[1] = {(uint64_t)cols * 2};
    const uint32_t box[2] = {BLOCK_K, (uint32_t)box_rows};
    return mrs_make_tensor_map_bf16(reinterpret_cast<CUtensorMap*>(map_out), base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// Ranges of K for a weight matrix [N, K] on a GPU with `sms` SMs, by a count of the time an SM
// spends: rounds of units x (64-column blocks of a unit + a unit's fixed cost + the cost of
// leaving and adding partial sums when there are several ranges), the costs in blocks' worth of
// time.  It depends on N, K and the GPU alone, never on the rows of the product.  The costs 4 and 8
// were measured in decode steps (with 2 and 2 the gate/up product of the 8B shape took 3 ranges
// instead of 2: batch 8 4.155 against 4.104 ms a step, batch 16 5.129 against 4.997 ms; 14B shape
// at batch 16 8.83 against 8.61 ms; 1 and 1, 3 and 4, 6 and 12, 4 and 16, 8 and 8 all slower).
MRS_EXPORT int mrs_gemm_tc_splits(int N, int K, int sms) {
    const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K, n_tiles = (N + TILE_N - 1) / TILE_N;
    int limit = k_blocks / 4;
    limit = limit < 1 ? 1 : (limit > 16 ? 16 : limit);
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= limit; ++s) {
        const long long rounds = ((long long)n_tiles * s + sms - 1) / sms;
        const long long cost = rounds * ((k_blocks + s - 1) / s + 4 + (s > 1 ? 8 : 0));
        if (best_cost < 0 || cost < best_cost) best = s, best_cost = cost;
    }
    // A last round of units that fills the GPU partly (after at least one full round): its tiles take as many ranges
    // as fill it, and the round is that much shorter.  The gate/up product of the 8B shape (192 tiles, 2 ranges: 2.6
    // rounds) gives its last 44 tiles 3 ranges; the head product (1,187 tiles, 8.02 rounds) its last 3 tiles 16.
    const long long units = (long long)n_tiles * best;
    const int rest_units = (int)(units % sms);
    if (units > sms && rest_units > 0 && rest_units % best == 0 && n_tiles < (1 << 15)) {
        const int rest_tiles = rest_units / best;
        int more = sms / rest_tiles;
        more = more > limit ? limit : more;
        if (more > best) return best | more << 8 | (n_tiles - rest_tiles) << 16;
    }
    return best;
}

// Floats of `partials` and ints of `counters` (zeroed once by the caller) that a product needs.
MRS_EXPORT long long mrs_gemm_tc_partial_floats(int M, int N, int splits) {
    const int n_tiles = (N + TILE_N - 1) / TILE_N;
    const Ranges r = ranges_of(splits, n_tiles);
    return r.first <= 1 && r.rest <= 1 ? 0 : (long long)units_of(r, n_tiles) * TILE_N * ((M + 3) / 4 * 4);
}
// Whether a count of ranges (or a plan of two counts, as mrs_gemm_tc_splits gives it) suits K.
static bool ranges_fit(int splits, int N, int K) {
    const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    const Ranges r = ranges_of(splits, (N + TILE_N - 1) / TILE_N);
    return splits > 0 && r.first >= 1 && r.first <= k_blocks && r.rest <= k_blocks && r.tiles_first >= 0;
}
MRS_EXPORT int mrs_gemm_tc_counters(int N) { return (N + TILE_N - 1) / TILE_N; }

// out[M, N] = x . w^T.  `w_map`: mrs_gemm_tc_map(w, N, K, 128); `x_map`: mrs_gemm_tc_map(x, M, K, mpad) with
// mpad = 16, 32, 64 or 128 >= M.  `out` is bfloat16 or float32 [M, N].  `ctas`: CTAs to launch (the GPU's SMs).
// With `gated`, w holds in every block of 128 rows 64 gate rows followed by the 64 matching up rows (N a
// multiple of 128), and out[M, N / 2] = silu(x . gate^T) * (x . up^T), bfloat16.
// `link` (or null): a NormLink.  With `in_square_sums` the sums are multiplied by their rows' norm factors; with
// `stream` (up to 32 rows, bfloat16 out, not gated) the result is added to the stream and `out` gets the stream
// times `next_weight`, with the parts of the rows' sums of squares in `out_square_sums` [ceil(N / 128)][mpad].
MRS_EXPORT int mrs_gemm_tc_small_m(const void* w_map, const void* x_map, void* out, int out_is_f32, int gated,
                                   float* partials, int* counters, int M, int N, int K, int splits, int mpad, int ctas,
                                   const void* link_in, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    NormLink link{};
    if (link_in) link = *reinterpret_cast<const NormLink*>(link_in);
    if (link.in_square_sums && (link.in_parts <= 0 || link.in_stride < M)) return MRS_BAD_ARGUMENT;
    if (link.stream && (gated || out_is_f32 || mpad > 32 || !link.next_weight || !link.out_square_sums)) return MRS_BAD_ARGUMENT;
    if (K <= 0 || K % 8 || M > mpad || !ranges_fit(splits, N, K) || ctas < 1) return MRS_BAD_ARGUMENT;
    if (splits > 1 && (!partials || !counters)) return MRS_BAD_ARGUMENT;
    const int units = units_of(ranges_of(splits, (N + TILE_N - 1) / TILE_N), (N + TILE_N - 1) / TILE_N);
    if (ctas > units) ctas = units;
    const CUtensorMap* wm = reinterpret_cast<const CUtensorMap*>(w_map);
    const CUtensorMap* xm = reinterpret_cast<const CUtensorMap*>(x_map);
    cudaStream_t st = (cudaStream_t)stream;
    if (gated && (out_is_f32 || N % TILE_N)) return MRS_BAD_ARGUMENT;
#define MRS_GEMM_CASE(P)                                                                                              \
    case P:                                                                                                           \
        if (gated) return launch<P, bf16, EPI_GATED>(wm, xm, out, partials, counters, M, N, K, splits, ctas, st, link);     \
        return out_is_f32 ? launch<P, float, EPI_PLAIN>(wm, xm, out, partials, counters, M, N, K, splits, ctas, st, link)   \
                          : launch<P, bf16, EPI_PLAIN>(wm, xm, out, partials, counters, M, N, K, splits, ctas, st, link);
    if (link.stream) {
        if (mpad == 16) return launch<16, bf16, EPI_RESIDUAL>(wm, xm, out, partials, counters, M, N, K, splits, ctas, st, link);
        return launch<32, bf16, EPI_RESIDUAL>(wm, xm, out, partials, counters, M, N, K, splits, ctas, st, link);
    }
    switch (mpad) {
        MRS_GEMM_CASE(16)
        MRS_GEMM_CASE(32)
        MRS_GEMM_CASE(64)
        MRS_GEMM_CASE(128)
    }
#undef MRS_GEMM_CASE
    return MRS_BAD_ARGUMENT;
}

// The fused q/k/v projection of an attention with heads of 128 elements, for up to 32 rows: the product, then per
// head the RMSNorm of q and k (scales `q_norm`, `k_norm`, or null), the rotation of q and k (`inv_freq` [64] or
// null; pairs (j, j + 64)), q into `q_out` [M, nq, 128] and k, v into the cache pages at `slots` (null: nothing
// is written).  `w_map` covers the weights [(nq + 2 nkv) * 128, K], q heads first, then k, then v.
// What the fused q/k/v projection takes: the head size (a weight tile is one head) and the most rows.
MRS_EXPORT int mrs_gemm_tc_qkv_head_dim() { return TILE_N; }
MRS_EXPORT int mrs_gemm_tc_qkv_max_rows() { return 32; }

MRS_EXPORT int mrs_gemm_tc_qkv_heads(const void* w_map, const void* x_map, void* q_out, void* k_cache, void* v_cache,
                                     const int* positions, const int* slots, const float* q_norm, const float* k_norm,
                                     const float* inv_freq, float eps, int nq, int nkv, int page_size, float* partials,
                                     int* counters, int M, int K, int splits, int mpad, int ctas, const void* link_in,
                                     void* stream) {
    if (M <= 0) return 0;
    NormLink link{};
    if (link_in) link = *reinterpret_cast<const NormLink*>(link_in);
    link.stream = nullptr;
    if (link.in_square_sums && (link.in_parts <= 0 || link.in_stride < M)) return MRS_BAD_ARGUMENT;
    const int N = (nq + 2 * nkv) * TILE_N;
    if (K <= 0 || K % 8 || M > mpad || mpad > 32 || !ranges_fit(splits, N, K) || ctas < 1 || nq <= 0 || nkv <= 0 ||
        page_size <= 0 || !q_out || !positions || (slots && (!k_cache || !v_cache)))
        return MRS_BAD_ARGUMENT;
    if (splits > 1 && (!partials || !counters)) return MRS_BAD_ARGUMENT;
    const int units = units_of(ranges_of(splits, N / TILE_N), N / TILE_N);
    if (ctas > units) ctas = units;
    HeadEpilogue heads{(bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, positions, slots, q_norm, k_norm, inv_freq, eps, nq, nkv, page_size};
    const CUtensorMap* wm = reinterpret_cast<const CUtensorMap*>(w_map);
    const CUtensorMap* xm = reinterpret_cast<const CUtensorMap*>(x_map);
    if (mpad == 16) return launch<16, bf16, EPI_HEADS>(wm, xm, nullptr, partials, counters, M, N, K, splits, ctas, (cudaStream_t)stream, link, heads);
    if (mpad == 32) return launch<32, bf16, EPI_HEADS>(wm, xm, nullptr, partials, counters, M, N, K, splits, ctas, (cudaStream_t)stream, link, heads);
    return MRS_BAD_ARGUMENT;
}

// A wait that runs out, for the tests of the error path: one warp waits on a barrier of its own at which nobody
// arrives, for `limit_cycles` clocks at most; the wait then gives up as every bounded wait of these kernels does
// (it raises the library's error word and returns), and the kernel ends.  Nothing else is touched.
__global__ void wait_probe_kernel(long long limit_cycles, int* gave_up) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        const bool arrived = mbar_wait(&bar, 0, limit_cycles);
        if (gave_up) *gave_up = arrived ? 0 : 1;
    }
}

MRS_EXPORT int mrs_gemm_tc_wait_probe(long long limit_cycles, int* gave_up, void* stream) {
    if (limit_cycles <= 0 || limit_cycles > (1ll << 24)) return MRS_BAD_ARGUMENT;      // a few milliseconds at most
    wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit_cycles, gave_up);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_gemm_tc_take_error(unsigned int* word) { return mrs_take_error_word(word); }
// Mirrors the error word into a word of pinned host memory from now on.
MRS_EXPORT int mrs_gemm_tc_mirror_errors(unsigned int* host_word) { return mrs_set_error_mirror(host_word); }

MRS_EXPORT const char* mrs_gemm_tc_error_string(int code) {
    if (code == MRS_BAD_ARGUMENT) return "arguments outside what the kernel supports (K no multiple of 8, M above the padded size, unaligned base, splits)";
    if (code == MRS_TENSOR_MAP_FAILED) return "the driver refused the tensor map (address, sizes or strides)";
    return cudaGetErrorString((cudaError_t)code);
}
