// Paged causal grouped-query attention for prompt portions on the tcgen05 tensor cores, for head
// sizes 64 and 128: -DMRS_HEAD_DIM=64|128.     (reference: ops.cu:101-147, one CTA per (token,
// head) on the CUDA cores)
//
// A tile is 128 query rows of one key/value head: 128 / group consecutive tokens of one request
// times the group's query heads, so a key is read once for all the heads that share it.  The
// tile's keys are walked in blocks of 128:
//   warp 0     one thread fetches the query tile and, page by page through the request's block
//              table, the keys and values of every block with bulk tensor copies (TMA, 128-byte
//              swizzle) into two-stage rings;
//   warp 1     one thread issues the MMAs: S = Q.K^T into one of two score buffers in tensor
//              memory (so the scores of the next block are computed while the softmax of this one
//              runs), then O += P.V with P read from shared memory and V taken as it lies in the
//              cache (rows of keys, the MN-major operand form);
//   warps 2-5  one thread per query row: scores from tensor memory, mask, running maximum and
//              sum in float32, probabilities as bfloat16 into shared memory in the operand layout.
//              The accumulator O stays in tensor memory; it is rescaled only when a row's maximum
//              grew by more than 2^8 since the last rescale (the sum uses the same reference, so
//              the quotient is exact), and is normalised and stored at the end.
// Every wait is bounded (tma.cuh).
#include "tcgen05.cuh"

#ifndef MRS_HEAD_DIM
#error "compile with -DMRS_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int D = MRS_HEAD_DIM;
static_assert(D == 64 || D == 128, "this kernel takes head sizes 64 and 128");
constexpr int HALVES = D / 64;
constexpr int BM = 128;                          // query rows of a tile
constexpr int BN = 128;                          // keys of a block
constexpr int THREADS = 192;
constexpr int Q_BYTES = BM * D * 2;
constexpr int KV_TILE_BYTES = BN * D * 2;        // keys (or values) of a block
constexpr int P_BYTES = BM * BN * 2;
constexpr int HALF_BYTES = 128 * 128;            // 128 rows of 128 bytes: one group of 64 columns of a tile
constexpr int TMEM_COLUMNS = 512;
constexpr int S_COLUMN = 0, O_COLUMN = 2 * BN;   // two score buffers, then the accumulator
constexpr float RESCALE_THRESHOLD = 8.0f;        // in powers of two

struct Tile {
    int seq, first_token, tokens, pad;
};

// 2^x in one instruction of the special-function unit (2 ulp; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct Barriers {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready, pv_done;
};

constexpr size_t SMEM_BYTES = 1024 + Q_BYTES + 4 * KV_TILE_BYTES + P_BYTES + sizeof(Barriers) + 16;

__global__ void __launch_bounds__(THREADS, 1) attention_prefill_kernel(
    const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
    const __grid_constant__ CUtensorMap v_map, const int* __restrict__ positions, const int* __restrict__ block_table,
    int table_width, const Tile* __restrict__ tiles, bf16* __restrict__ out, int nq, int nkv, int page_size,
    int page_shift, float scale_log2, int window) {
    extern __shared__ unsigned char smem_raw[];
    const Tile tile = tiles[blockIdx.x];
    if (tile.tokens <= 0) return;
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_smem = smem;
    unsigned char* k_smem = q_smem + Q_BYTES;               // two stages
    unsigned char* v_smem = k_smem + 2 * KV_TILE_BYTES;     // two stages
    unsigned char* p_smem = v_smem + 2 * KV_TILE_BYTES;
    Barriers* bars = reinterpret_cast<Barriers*>(p_smem + P_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);

    const int kv_head = blockIdx.y, group = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* pages = block_table + (size_t)tile.seq * table_width;
    const int rows = tile.tokens * group;
    const int first_pos = positions[tile.first_token], last_pos = positions[tile.first_token + tile.tokens - 1];
    const int key_end = last_pos + 1;
    const int key_begin = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int block_first = key_begin / BN, block_last = (key_end + BN - 1) / BN;
    const int blocks = block_last - block_first;

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars->k_full[s], 1);
            mbar_init(&bars->k_empty[s], 1);
            mbar_init(&bars->v_full[s], 1);
            mbar_init(&bars->v_empty[s], 1);
            mbar_init(&bars->s_full[s], 1);
        }
        mbar_init(&bars->p_ready, 4);
        mbar_init(&bars->pv_done, 1);
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
    pdl_wait();                  // queries and the newest keys come from the kernel before this one

    if (warp == 0) {
        // ------------------------------------------------------------------ copies
        // Every lane owns one page of a block: it reads the page's number a block ahead of its use and
        // issues the page's copies itself, so a block costs one trip to the block table and one round of
        // copies issued side by side.  Lane 0 also waits for the stage and arms its barrier.
        if (lane == 0) {
            tma_prefetch_descriptor(&q_map);
            tma_prefetch_descriptor(&k_map);
            tma_prefetch_descriptor(&v_map);
            mbar_arrive_expect_tx(&bars->q_full, Q_BYTES);
            for (int h = 0; h < HALVES; ++h)
                tma_load_3d(q_smem + h * HALF_BYTES, &q_map, &bars->q_full, h * 64, kv_head * group, tile.first_token);
        }
        const int rows_per_copy = min(page_size, BN);
        const int copies = BN / rows_per_copy;
        // keys past the end, before the window or on a page that was given back are masked by their
        // position; their copy reads page 0, which always exists and holds finite numbers
        auto page_of = [&](int j) {
            const int key = (block_first + j) * BN + lane * rows_per_copy;
            return (lane < copies && key < key_end) ? pages[key >> page_shift] : -1;
        };
        int next_page = page_of(0);
        for (int j = 0; j < blocks; ++j) {
            const int s = j & 1;
            const int my_page = next_page;
            if (j + 1 < blocks) next_page = page_of(j + 1);
            const uint32_t wait_parity = ((j >> 1) & 1) ^ 1;
            for (int which = 0; which < 2; ++which) {            // keys, then values
                uint64_t* full = which ? &bars->v_full[s] : &bars->k_full[s];
                if (lane == 0) {
                    mbar_wait(which ? &bars->v_empty[s] : &bars->k_empty[s], wait_parity);
                    mbar_arrive_expect_tx(full, KV_TILE_BYTES);
                }
                __syncwarp();                                    // the stage is free and the barrier armed
                unsigned char* dst = (which ? v_smem : k_smem) + s * KV_TILE_BYTES;
                const CUtensorMap* map = which ? &v_map : &k_map;
                if (lane < copies) {                             // every lane issues the copies of its own page
                    const int key = (block_first + j) * BN + lane * rows_per_copy;
                    const int row = my_page < 0 ? 0 : key & (page_size - 1);
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_5d(dst + h * HALF_BYTES + lane * rows_per_copy * 128, map, full, 0, row, h, kv_head, max(my_page, 0));
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16_f32(BM, BN);
            constexpr uint32_t idesc_o = umma_idesc_bf16_f32(BM, D, true);
            const uint32_t q_addr = smem_u32(q_smem), p_addr = smem_u32(p_smem);
            auto issue_scores = [&](int j) {
                const int s = j & 1;
                mbar_wait(&bars->k_full[s], (j >> 1) & 1);
                tcgen05_fence_after_sync();
                const uint32_t k_addr = smem_u32(k_smem + s * KV_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t offset = (k / 4) * HALF_BYTES + (k % 4) * 32;
                    umma_bf16(tmem_base + S_COLUMN + s * BN, umma_smem_desc_sw128(q_addr + offset),
                              umma_smem_desc_sw128(k_addr + offset), idesc_s, k > 0);
                }
                umma_commit(&bars->k_empty[s]);
                umma_commit(&bars->s_full[s]);
            };
            mbar_wait(&bars->q_full, 0);
            issue_scores(0);
            for (int j = 0; j < blocks; ++j) {
                const int s = j & 1;
                if (j + 1 < blocks) issue_scores(j + 1);
                mbar_wait(&bars->p_ready, j & 1);
                mbar_wait(&bars->v_full[s], (j >> 1) & 1);
                tcgen05_fence_after_sync();
                const uint32_t v_addr = smem_u32(v_smem + s * KV_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)
                    umma_bf16(tmem_base + O_COLUMN, umma_smem_desc_sw128(p_addr + (k / 4) * HALF_BYTES + (k % 4) * 32),
                              umma_smem_desc_sw128_mn(v_addr + k * 2048, HALF_BYTES), idesc_o, j > 0 || k > 0);
                umma_commit(&bars->v_empty[s]);
                umma_commit(&bars->pv_done);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax, one thread per query row
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int pos = row < rows ? positions[tile.first_token + row / group] : -1;
        const int lowest = window > 0 ? pos - window + 1 : 0;        // first key this row sees
        float reference = -CUDART_INF_F;     // the maximum that probabilities and the accumulator are scaled by
        float sum = 0.0f;
        for (int j = 0; j < blocks; ++j) {
            const int s = j & 1;
            const int key0 = (block_first + j) * BN;
            mbar_wait(&bars->s_full[s], (j >> 1) & 1);
            __syncwarp();                    // the loads below are collective: the warp goes on together
            tcgen05_fence_after_sync();
            float x[BN];
#pragma unroll
            for (int c = 0; c < BN; c += 32) tmem_load_32_async(lane_base + S_COLUMN + s * BN + c, x + c);
            tmem_load_wait();
            const bool edge = key0 + BN - 1 > first_pos || key0 < key_begin + (window > 0 ? BN : 0);   // a block that needs masks
            float part_max[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};   // four chains, not one of 128 links
            if (edge) {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int key = key0 + c;
                    x[c] = (key <= pos && key >= lowest) ? x[c] : -CUDART_INF_F;
                    part_max[c & 3] = fmaxf(part_max[c & 3], x[c]);
                }
            } else {
#pragma unroll
                for (int c = 0; c < BN; ++c) part_max[c & 3] = fmaxf(part_max[c & 3], x[c]);
            }
            // the scale is positive, so the maximum of the scaled scores is the scaled maximum
            const float block_max = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3])) * scale_log2;
            // the reference moves only when the maximum outgrew it by the threshold (always from -inf)
            float alpha = 1.0f;
            const bool moved = block_max > reference + RESCALE_THRESHOLD;
            if (moved) {
                alpha = exp2f(reference - block_max);          // 0 when the reference was -inf
                reference = block_max;
            }
            const float base = reference == -CUDART_INF_F ? 0.0f : reference;
            float part_sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t packed[BN / 2];
#pragma unroll
            for (int c = 0; c < BN; c += 2) {
                const float p0 = fast_exp2(fmaf(x[c], scale_log2, -base)), p1 = fast_exp2(fmaf(x[c + 1], scale_log2, -base));
                part_sum[(c >> 1) & 3] += p0 + p1;
                __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
                packed[c / 2] = *reinterpret_cast<uint32_t*>(&pair);
            }
            sum = sum * alpha + ((part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]));
            // the last block's P.V must be done before its probabilities are overwritten or O is rescaled
            if (j > 0) {
                mbar_wait(&bars->pv_done, (j - 1) & 1);
                __syncwarp();
                tcgen05_fence_after_sync();
                if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
                    for (int c = 0; c < D; c += 16) {
                        float o[16];
                        tmem_load_16(lane_base + O_COLUMN + c, o);
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] *= alpha;
                        tmem_store_16(lane_base + O_COLUMN + c, o);
                    }
                    tmem_store_wait();
                }
            }
            // probabilities of this row: 16-byte chunks of 8 keys, xor-ed with the row as the operand layout wants
#pragma unroll
            for (int chunk = 0; chunk < BN / 8; ++chunk) {
                unsigned char* dst = p_smem + (chunk / 8) * HALF_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
                *reinterpret_cast<uint4*>(dst) = make_uint4(packed[4 * chunk], packed[4 * chunk + 1], packed[4 * chunk + 2], packed[4 * chunk + 3]);
            }
            fence_async_shared();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->p_ready);
        }
        mbar_wait(&bars->pv_done, (blocks - 1) & 1);
        __syncwarp();
        tcgen05_fence_after_sync();
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        // loads from tensor memory are collective: every lane of the warp takes part, rows past the
        // tile's end drop what they read
        bf16* dst = out + ((size_t)(tile.first_token + (row < rows ? row / group : 0)) * nq + kv_head * group +
                           (row < rows ? row % group : 0)) * D;
#pragma unroll
        for (int c = 0; c < D; c += 16) {
            float o[16];
            tmem_load_16(lane_base + O_COLUMN + c, o);
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                __nv_bfloat162 pair = __floats2bfloat162_rn(o[2 * i] * inv, o[2 * i + 1] * inv);
                w[i] = *reinterpret_cast<uint32_t*>(&pair);
            }
            if (row < rows) {
                *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(dst + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
            }
        }
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLUMNS);
    }
}

int page_shift_of(int page_size) {
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    return (1 << shift) == page_size ? shift : -1;
}

}  // namespace

MRS_EXPORT int mrs_attention_prefill_tc_rows() { return BM; }

// Tensor map of one layer's key or value pages [pages, kv_heads, page_size, D] for copies of one
// group of 64 columns of up to 128 rows of a page.  `map_out`: 128 bytes, 64-byte aligned.
MRS_EXPORT int mrs_attention_prefill_tc_kv_map(const void* cache, long long pages, int nkv, int page_size, void* map_out) {
    if (page_shift_of(page_size) < 0 || page_size < 8 || pages <= 0 || nkv <= 0) return MRS_BAD_ARGUMENT;
    const uint64_t dims[5] = {64, (uint64_t)page_size, (uint64_t)HALVES, (uint64_t)nkv, (uint64_t)pages};
    const uint64_t strides[4] = {(uint64_t)D * 2, 128, (uint64_t)page_size * D * 2, (uint64_t)nkv * page_size * D * 2};
    const uint32_t box[5] = {64, (uint32_t)(page_size < BN ? page_size : BN), 1, 1, 1};
    return mrs_make_tensor_map_bf16(reinterpret_cast<CUtensorMap*>(map_out), cache, 5, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
}

// Tensor map of the step's queries [tokens, nq, D] for copies of 64 columns of (128 / group tokens) x (group heads).
MRS_EXPORT int mrs_attention_prefill_tc_q_map(const void* q, long long tokens, int nq, int group, void* map_out) {
    if (tokens <= 0 || nq <= 0 || group <= 0 || BM % group || nq % group) return MRS_BAD_ARGUMENT;
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)nq, (uint64_t)tokens};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)nq * D * 2};
    const uint32_t box[3] = {64, (uint32_t)group, (uint32_t)(BM / group)};
    return mrs_make_tensor_map_bf16(reinterpret_cast<CUtensorMap*>(map_out), q, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// Tiles of up to 128 / group tokens of one request each ((sequence, first token, tokens, 0) per tile).
MRS_EXPORT int mrs_attention_prefill_tc(const void* q_map, const void* k_map, const void* v_map, const int* positions,
                                        const int* block_table, int table_width, const int* tiles, int num_tiles,
                                        void* out, int nq, int nkv, int page_size, float scale, int window, void* stream) {
    if (num_tiles <= 0) return 0;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || page_size < 8 || nkv <= 0 || nq % nkv || BM % (nq / nkv)) return MRS_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    MRS_LAUNCH(attention_prefill_kernel, dim3(num_tiles, nkv), THREADS, SMEM_BYTES, stream,
               *reinterpret_cast<const CUtensorMap*>(q_map), *reinterpret_cast<const CUtensorMap*>(k_map),
               *reinterpret_cast<const CUtensorMap*>(v_map), positions, block_table, table_width, (const Tile*)tiles,
               (bf16*)out, nq, nkv, page_size, shift, scale * 1.4426950408889634f, window);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_attention_prefill_tc_take_error(unsigned int* word) { return mrs_take_error_word(word); }
// Mirrors the error word into a word of pinned host memory from now on.
MRS_EXPORT int mrs_attention_prefill_tc_mirror_errors(unsigned int* host_word) { return mrs_set_error_mirror(host_word); }

MRS_EXPORT const char* mrs_attention_prefill_tc_error_string(int code) {
    if (code == MRS_BAD_ARGUMENT) return "arguments outside what the kernel supports (page size below 8 or no power of two, a group of query heads that does not divide 128)";
    if (code == MRS_TENSOR_MAP_FAILED) return "the driver refused the tensor map (address, sizes or strides)";
    return cudaGetErrorString((cudaError_t)code);
}
