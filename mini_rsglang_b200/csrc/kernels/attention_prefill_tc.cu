// Paged causal grouped-query attention for prompt portions on the tcgen05 tensor cores, for head
// sizes 64 and 128: -DMRS_HEAD_DIM=64|128.     (reference: ops.cu:101-147, one CTA per (token,
// head) on the CUDA cores)
//
// A CTA works on two tiles of 128 query rows of one key/value head: a tile is 128 / group
// consecutive tokens of one request times the group's query heads, so a key is read once for all
// the heads that share it, and the second tile holds the tokens that follow the first, or, when
// the entry says so (its fourth number >> 16: tokens between the tiles), tokens further on in the
// same request: a late tile, whose walk is long, beside an early one, whose walk is short.  A group
// that does not divide 128 (5 query heads a key/value head: 25 tokens, 125 rows) leaves the tile's
// last rows empty: they are zeroed once, masked everywhere and never stored.  The keys
// are walked in blocks of 128:
//   warp 0      fetches the query tiles and, page by page through the request's block table, the
//               keys and values of every block with bulk tensor copies (TMA, 128-byte swizzle)
//               into two-stage rings; every lane owns one page of a block;
//   warp 1      walks its loop whole, one elected lane issues the MMAs (an issue is cheap when every
//               lane holds the same addresses): S = Q.K^T of each tile into the tile's score buffer in
//               tensor memory, then O += P.V with P read from tensor memory (it overwrites the
//               scores it came from) and V taken as it lies in the cache (rows of keys, the MN-major
//               operand form);
//   warps 2-5   softmax of the first tile, warps 6-9 of the second, one thread per query row:
//               scores from tensor memory, mask, running maximum and sum in float32, probabilities
//               back into tensor memory as pairs of bfloat16.
// The two tiles take turns: while one tile's exponentials run (the special-function unit makes 16
// a clock, as long as the block's MMAs take) the tensor cores work on the other tile.  Shared
// memory carries only Q, K and V: with P there too its bandwidth (128 bytes a clock) was the bound.
// The accumulators stay in tensor memory; one is rescaled only when a row's maximum grew by more
// than 2^8 since the last rescale (the sum uses the same reference, so the quotient is exact), and
// is normalised and stored at the end.
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
constexpr int TILES = 2;                         // tiles of a CTA
constexpr int BN = 128;                          // keys of a block
constexpr int STAGES = 2;                        // of the key and of the value ring
constexpr int THREADS = 64 + TILES * 128;
constexpr int Q_TILE_BYTES = BM * D * 2;
constexpr int Q_HALF_BYTES = BM * 128;           // 128 rows of 128 bytes: one group of 64 columns of a query tile
constexpr int KV_TILE_BYTES = BN * D * 2;        // keys (or values) of a block
constexpr int KV_HALF_BYTES = BN * 128;
constexpr int TMEM_COLUMNS = 512;
constexpr int S_COLUMNS = BN;                    // a tile's scores; its probabilities (pairs of bfloat16) take the first half
constexpr int O_COLUMN = TILES * S_COLUMNS;      // the score buffers, then the accumulators
static_assert(O_COLUMN + TILES * D <= TMEM_COLUMNS, "tensor memory");
constexpr float RESCALE_THRESHOLD = 8.0f;        // in powers of two

// A work entry: `tokens` consecutive tokens of request `seq` from row `first_token` of the step on.  `share` = 0:
// the CTA walks all keys.  Otherwise share = index | count << 8: the entry is one of `count` entries (which
// follow one another in the list) that walk one share of the key blocks each and leave their unnormalised
// accumulators, maxima and sums in `partials`; attention_prefill_merge_kernel puts them together.
struct Tile {
    int seq, first_token, tokens, share;
};
constexpr int PARTIAL_STRIDE = D + 4;            // floats of a row in `partials`: the accumulator, the maximum, the sum, 2 unused

// 2^x in one instruction of the special-function unit (2 ulp; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The softmax threads are bound by the instructions they issue, so two of sm_100's wider ones are used: the
// maximum of three numbers, and arithmetic on two floats at once (a pair of registers taken as one operand).
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n .reg .b64 ra, rb, rc, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mov.b64 rc, {%6, %7};\n"
        " fma.rn.f32x2 rd, ra, rb, rc;\n mov.b64 {%0, %1}, rd;\n}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n"
        " add.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

struct Barriers {
    uint64_t q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
    uint64_t s_full[TILES], p_ready[TILES], pv_done[TILES];
};

constexpr size_t SMEM_BYTES = 1024 + TILES * Q_TILE_BYTES + 2 * STAGES * KV_TILE_BYTES + sizeof(Barriers) + 16;

__global__ void __launch_bounds__(THREADS, 1) attention_prefill_kernel(
    const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
    const __grid_constant__ CUtensorMap v_map, const int* __restrict__ positions, const int* __restrict__ block_table,
    int table_width, const Tile* __restrict__ tiles, bf16* __restrict__ out, int nq, int nkv, int page_size,
    int page_shift, float scale_log2, int window, float* __restrict__ partials) {
    extern __shared__ unsigned char smem_raw[];
    // the grid runs over the key/value heads first: with the entries sorted by their work, all heavy CTAs start first
    const Tile work = tiles[blockIdx.y];
    if (work.tokens <= 0) return;
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_smem = smem;                                   // [tile][half][128 rows][64]
    unsigned char* k_smem = q_smem + TILES * Q_TILE_BYTES;          // [stage][half][128 keys][64]
    unsigned char* v_smem = k_smem + STAGES * KV_TILE_BYTES;
    Barriers* bars = reinterpret_cast<Barriers*>(v_smem + STAGES * KV_TILE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);

    const int kv_head = blockIdx.x, group = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* pages = block_table + (size_t)work.seq * table_width;
    const int tokens_per_tile = BM / group;
    // the tokens of the two tiles, their positions (a request's tokens of a step are consecutive) and their blocks of keys
    int tile_first[TILES], tile_tokens[TILES], tile_blocks[TILES], tile_first_pos[TILES];
    const int first_pos = positions[work.first_token];
    const int key_begin = window > 0 ? max(0, first_pos - window + 1) : 0;
    int block_first = key_begin / BN;
    int blocks = 0;
    // An entry may hold two tiles that are not neighbours: `gap` tokens of the request lie between them (other
    // entries take those).  The plan pairs an early tile, whose walk is short, with a late one, so that the CTAs of a
    // prompt take equally long; both read the same blocks of keys while the early one has any.
    const int gap = (int)((unsigned)work.share >> 16);
    int key_end = first_pos;
#pragma unroll
    for (int i = 0; i < TILES; ++i) {
        tile_first[i] = work.first_token + i * (tokens_per_tile + gap);
        tile_tokens[i] = max(0, min(tokens_per_tile, work.tokens - i * tokens_per_tile));
        tile_first_pos[i] = first_pos + i * (tokens_per_tile + gap);
        const int last_pos = tile_first_pos[i] + tile_tokens[i] - 1;
        tile_blocks[i] = tile_tokens[i] > 0 ? (last_pos + BN) / BN - block_first : 0;
        blocks = max(blocks, tile_blocks[i]);
        if (tile_tokens[i] > 0) key_end = last_pos + 1;
    }
    const int shares = (work.share >> 8) & 0xFF;
    if (shares > 1) {
        // this entry's share of the key blocks; a tile may have none of its blocks in it
        const int share = work.share & 0xFF;
        const int b0 = (int)((long long)blocks * share / shares), b1 = (int)((long long)blocks * (share + 1) / shares);
#pragma unroll
        for (int i = 0; i < TILES; ++i) tile_blocks[i] = max(0, min(tile_blocks[i], b1) - b0);
        block_first += b0;
        blocks = b1 - b0;
    }

    const int used_rows = tokens_per_tile * group;             // rows of a tile that a copy of queries fills
    if (used_rows < BM) {
        // the rows behind them belong to no token: zeros, so that nothing they yield is anything but finite
        for (int idx = threadIdx.x; idx < TILES * HALVES * (BM - used_rows) * 8; idx += THREADS) {
            const int chunk = idx & 7, line = (idx >> 3) % (BM - used_rows), part = (idx >> 3) / (BM - used_rows);
            *reinterpret_cast<uint4*>(q_smem + part * Q_HALF_BYTES + (used_rows + line) * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_async_shared();
    }
    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bars->k_full[s], 1);
            mbar_init(&bars->k_empty[s], 1);
            mbar_init(&bars->v_full[s], 1);
            mbar_init(&bars->v_empty[s], 1);
        }
        for (int i = 0; i < TILES; ++i) {
            mbar_init(&bars->s_full[i], 1);
            mbar_init(&bars->p_ready[i], 4);
            mbar_init(&bars->pv_done[i], 1);
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
            // rows past the last token arrive as zeros or as other tokens' queries, and are never stored
            mbar_arrive_expect_tx(&bars->q_full, TILES * HALVES * used_rows * 128);
            for (int i = 0; i < TILES; ++i)
                for (int h = 0; h < HALVES; ++h)
                    tma_load_3d(q_smem + i * Q_TILE_BYTES + h * Q_HALF_BYTES, &q_map, &bars->q_full, h * 64, kv_head * group,
                                tile_first[i]);
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
            const int s = j % STAGES;
            const int my_page = next_page;
            if (j + 1 < blocks) next_page = page_of(j + 1);
            const uint32_t wait_parity = ((j / STAGES) & 1) ^ 1;
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
                        tma_load_5d(dst + h * KV_HALF_BYTES + lane * rows_per_copy * 128, map, full, 0, row, h, kv_head, max(my_page, 0));
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA
        // The whole warp walks the loop and one elected lane issues: descriptors and addresses are then the same
        // in every lane, and an MMA costs its issuer some 40 clocks instead of 100 in divergent code.
        if (blocks > 0) {                                    // (a share of the keys can be empty)
            const bool leader = elect_one();
            constexpr uint32_t idesc_s = umma_idesc_bf16_f32(BM, BN);
            constexpr uint32_t idesc_o = umma_idesc_bf16_f32(BM, D, true);
            const uint32_t q_addr = smem_u32(q_smem);
            // scores of block j of tile i (the keys of block j are in their stage)
            auto issue_scores = [&](int i, int j) {
                const uint32_t k_addr = smem_u32(k_smem + (j % STAGES) * KV_TILE_BYTES);
                if (leader) {
                    const uint32_t s_tmem = tmem_base + i * S_COLUMNS;
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {
                        const uint64_t q_desc = umma_smem_desc_sw128(q_addr + i * Q_TILE_BYTES + (k / 4) * Q_HALF_BYTES + (k % 4) * 32);
                        const uint64_t k_desc = umma_smem_desc_sw128(k_addr + (k / 4) * KV_HALF_BYTES + (k % 4) * 32);
                        if (k == 0) umma_bf16_first(s_tmem, q_desc, k_desc, idesc_s);
                        else umma_bf16_more(s_tmem, q_desc, k_desc, idesc_s);
                    }
                    umma_commit(&bars->s_full[i]);
                }
                __syncwarp();
            };
            mbar_wait(&bars->q_full, 0);
            mbar_wait(&bars->k_full[0], 0);
            tcgen05_fence_after_sync();
#pragma unroll
            for (int i = 0; i < TILES; ++i)
                if (tile_blocks[i] > 0) issue_scores(i, 0);
            if (leader) umma_commit(&bars->k_empty[0]);
            __syncwarp();
            // The tiles take turns: P.V of a tile's block, then at once the scores of its next block (the
            // probabilities lie where the scores lay, and MMAs run in the order they are issued).
            for (int j = 0; j < blocks; ++j) {
                const int s = j % STAGES;
                bool waited_v = false, waited_k = false;
#pragma unroll
                for (int i = 0; i < TILES; ++i) {
                    if (j >= tile_blocks[i]) continue;
                    mbar_wait(&bars->p_ready[i], j & 1);
                    if (!waited_v) mbar_wait(&bars->v_full[s], (j / STAGES) & 1), waited_v = true;
                    tcgen05_fence_after_sync();
                    const uint32_t v_addr = smem_u32(v_smem + s * KV_TILE_BYTES);
                    if (leader) {
                        const uint32_t o_tmem = tmem_base + O_COLUMN + i * D, p_tmem = tmem_base + i * S_COLUMNS;
#pragma unroll
                        for (int k = 0; k < BN / 16; ++k) {
                            const uint64_t v_desc = umma_smem_desc_sw128_mn(v_addr + k * 2048, KV_HALF_BYTES);
                            if (k == 0 && j == 0) umma_bf16_a_tmem(o_tmem, p_tmem, v_desc, idesc_o, false);
                            else umma_bf16_a_tmem(o_tmem, p_tmem + k * 8, v_desc, idesc_o, true);
                        }
                    }
                    __syncwarp();
                    if (j + 1 < tile_blocks[i]) {
                        if (!waited_k) mbar_wait(&bars->k_full[(j + 1) % STAGES], ((j + 1) / STAGES) & 1), waited_k = true;
                        tcgen05_fence_after_sync();
                        issue_scores(i, j + 1);
                    } else {
                        if (leader) umma_commit(&bars->pv_done[i]);          // the tile's last block: its accumulator is final
                        __syncwarp();
                    }
                }
                if (leader) {
                    umma_commit(&bars->v_empty[s]);
                    if (waited_k) umma_commit(&bars->k_empty[(j + 1) % STAGES]);
                }
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax, one thread per query row of one tile
        const int i = (warp - 2) >> 2;                      // the tile of this warp group
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int rows = tile_tokens[i] * group;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int my_first_pos = tile_first_pos[i];
        const int pos = row < rows ? my_first_pos + row / group : -1;
        const int lowest = window > 0 ? pos - window + 1 : 0;        // first key this row sees
        const int my_blocks = tile_blocks[i];
        const uint32_t s_tmem = lane_base + i * S_COLUMNS;
        float reference = -CUDART_INF_F;     // the maximum that probabilities and the accumulator are scaled by
        float sum = 0.0f;
        for (int j = 0; j < my_blocks; ++j) {
            const int key0 = (block_first + j) * BN;
            // The scores of block j were issued after P.V of block j - 1, so when they are complete that
            // product has been added and the accumulator may be rescaled.
            mbar_wait(&bars->s_full[i], j & 1);
            __syncwarp();                    // the loads below are collective: the warp goes on together
            tcgen05_fence_after_sync();
            // a block needs masks when a key of it lies behind the tile's first position or before a row's window
            const bool edge = key0 + BN - 1 > my_first_pos || (window > 0 && key0 < my_first_pos + tile_tokens[i] - window + 1);
            // all scores of the row in one trip to tensor memory (a trip costs hundreds of clocks), then the row's maximum
            float x[BN];
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 32) tmem_load_32_async(s_tmem + c0, x + c0);
            tmem_load_wait();
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
                for (int c = 0; c < BN; c += 8) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) part_max[k] = max3(part_max[k], x[c + k], x[c + 4 + k]);
                }
            }
            // the scale is positive, so the maximum of the scaled scores is the scaled maximum
            const float block_max = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3])) * scale_log2;
            // the reference moves only when the maximum outgrew it by the threshold (always from -inf)
            float alpha = 1.0f;
            const bool moved = block_max > reference + RESCALE_THRESHOLD;
            if (moved) {
                alpha = fast_exp2(reference - block_max);      // 0 when the reference was -inf
                reference = block_max;
            }
            const float base = reference == -CUDART_INF_F ? 0.0f : reference;
            if (j > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll
                for (int c = 0; c < D; c += 16) {
                    float o[16];
                    tmem_load_16(lane_base + O_COLUMN + i * D + c, o);
#pragma unroll
                    for (int e = 0; e < 16; ++e) o[e] *= alpha;
                    tmem_store_16(lane_base + O_COLUMN + i * D + c, o);
                }
            }
            // probabilities, 32 scores at a time; their 16 words of bfloat16 pairs go where the scores lay
            float2 part_sum[4] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
            const float2 scale2 = make_float2(scale_log2, scale_log2), minus_base = make_float2(-base, -base);
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t packed[16];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const float2 t = fma2(make_float2(x[c0 + c], x[c0 + c + 1]), scale2, minus_base);
                    const float2 p = make_float2(fast_exp2(t.x), fast_exp2(t.y));
                    part_sum[(c >> 1) & 3] = add2(part_sum[(c >> 1) & 3], p);
                    __nv_bfloat162 pair = __floats2bfloat162_rn(p.x, p.y);
                    packed[c / 2] = *reinterpret_cast<uint32_t*>(&pair);
                }
                tmem_store_16_words(s_tmem + c0 / 2, packed);
            }
            sum = sum * alpha + (((part_sum[0].x + part_sum[0].y) + (part_sum[1].x + part_sum[1].y)) +
                                 ((part_sum[2].x + part_sum[2].y) + (part_sum[3].x + part_sum[3].y)));
            tmem_store_wait();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->p_ready[i]);
        }
        if (my_blocks > 0 || shares > 1) {
            float o[D];                        // one trip to tensor memory for the whole row
            if (my_blocks > 0) {
                mbar_wait(&bars->pv_done[i], 0);
                __syncwarp();
                tcgen05_fence_after_sync();
                // loads from tensor memory are collective: every lane of the warp takes part, rows past the
                // tile's end drop what they read
#pragma unroll
                for (int c = 0; c < D; c += 32) tmem_load_32_async(lane_base + O_COLUMN + i * D + c, o + c);
                tmem_load_wait();
            } else {                           // a share of the keys in which this tile has none
#pragma unroll
                for (int c = 0; c < D; ++c) o[c] = 0.0f;
            }
            if (shares > 1) {
                // one share of the keys: the row's accumulator as it stands, with the maximum it is scaled by and its sum
                float4* dst = reinterpret_cast<float4*>(
                    partials + ((((size_t)blockIdx.y * gridDim.x + blockIdx.x) * TILES + i) * BM + row) * PARTIAL_STRIDE);
#pragma unroll
                for (int c = 0; c < D; c += 4) dst[c / 4] = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
                dst[D / 4] = make_float4(reference, sum, 0.0f, 0.0f);
            } else if (row < rows) {
                const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
                bf16* dst = out + ((size_t)(tile_first[i] + row / group) * nq + kv_head * group + row % group) * D;
#pragma unroll
                for (int c = 0; c < D; c += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        __nv_bfloat162 pair = __floats2bfloat162_rn(o[c + 2 * e] * inv, o[c + 2 * e + 1] * inv);
                        w[e] = *reinterpret_cast<uint32_t*>(&pair);
                    }
                    *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
                }
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

// Puts the shares of an entry together: out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), M the largest maximum.
// A warp per query row (grid: key/value heads x entries x 32 groups of 8 rows); only the CTAs of an entry's first share work.
__global__ void __launch_bounds__(256) attention_prefill_merge_kernel(const Tile* __restrict__ tiles, const float* __restrict__ partials,
                                                                    bf16* __restrict__ out, int nq, int nkv) {
    pdl_launch_dependents();
    pdl_wait();
    const Tile work = tiles[blockIdx.y];
    const int shares = (work.share >> 8) & 0xFF;
    if (shares <= 1 || (work.share & 0xFF) != 0) return;
    const int group = nq / nkv, kv_head = blockIdx.x, tokens_per_tile = BM / group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int PER_LANE = D / 32;
    const int r = blockIdx.z * 8 + warp, i = r / BM, row = r % BM;
    const int tile_tokens = max(0, min(tokens_per_tile, work.tokens - i * tokens_per_tile));
    if (row >= tile_tokens * group) return;
    auto partial_of = [&](int s) {
        return partials + ((((size_t)(blockIdx.y + s) * gridDim.x + kv_head) * TILES + i) * BM + row) * PARTIAL_STRIDE;
    };
    // the maxima of all shares, a lane a share
    float best = -CUDART_INF_F;
    for (int s = lane; s < shares; s += 32) best = fmaxf(best, partial_of(s)[D]);
    best = warp_max(best);
    float acc[PER_LANE], total = 0.0f;
#pragma unroll
    for (int e = 0; e < PER_LANE; ++e) acc[e] = 0.0f;
#pragma unroll 4
    for (int s = 0; s < shares; ++s) {                 // in the order of the shares
        const float* p = partial_of(s);
        const float m = p[D];
        const float w = m == -CUDART_INF_F ? 0.0f : fast_exp2(m - best);      // a share without keys for this row counts nothing
        total += p[D + 1] * w;
#pragma unroll
        for (int e = 0; e < PER_LANE; ++e) acc[e] += p[lane * PER_LANE + e] * w;
    }
    const float inv = total > 0.0f ? 1.0f / total : 0.0f;
    bf16* dst = out + ((size_t)(work.first_token + i * tokens_per_tile + row / group) * nq + kv_head * group + row % group) * D +
                lane * PER_LANE;
#pragma unroll
    for (int e = 0; e < PER_LANE; ++e) dst[e] = __float2bfloat16_rn(acc[e] * inv);
}

int page_shift_of(int page_size) {
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    return (1 << shift) == page_size ? shift : -1;
}

}  // namespace

// Query rows of one CTA: two tiles of 128.
MRS_EXPORT int mrs_attention_prefill_tc_rows() { return TILES * BM; }
// Keys of one block that a CTA walks: the unit in which the host plans the shares of a long context.
MRS_EXPORT int mrs_attention_prefill_tc_key_block() { return BN; }

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

// Tensor map of the step's queries [tokens, nq, D] for copies of 64 columns of (128 / group tokens, rounded down) x (group heads).
MRS_EXPORT int mrs_attention_prefill_tc_q_map(const void* q, long long tokens, int nq, int group, void* map_out) {
    if (tokens <= 0 || nq <= 0 || group <= 0 || group > BM || nq % group) return MRS_BAD_ARGUMENT;
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)nq, (uint64_t)tokens};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)nq * D * 2};
    const uint32_t box[3] = {64, (uint32_t)group, (uint32_t)(BM / group)};
    return mrs_make_tensor_map_bf16(reinterpret_cast<CUtensorMap*>(map_out), q, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// Floats of `partials` for a list of `num_tiles` entries of which some are shares.
MRS_EXPORT long long mrs_attention_prefill_tc_partial_floats(int num_tiles, int nkv) {
    return (long long)num_tiles * nkv * TILES * BM * PARTIAL_STRIDE;
}

// Work entries of up to 2 x (128 / group, rounded down) consecutive tokens of one request each: (sequence, first token, tokens, share).
// share = 0: the entry walks all its keys.  share = index | count << 8 (count 2..255, the `count` entries of one
// portion one after the other): every entry walks one share of the key blocks; `partials`
// (mrs_attention_prefill_tc_partial_floats) carries their sums and `with_shares` must be set, so that the merge runs.
MRS_EXPORT int mrs_attention_prefill_tc(const void* q_map, const void* k_map, const void* v_map, const int* positions,
                                        const int* block_table, int table_width, const int* tiles, int num_tiles,
                                        void* out, int nq, int nkv, int page_size, float scale, int window,
                                        float* partials, int with_shares, void* stream) {
    if (num_tiles <= 0) return 0;
    if (with_shares && (!partials || num_tiles > 65535)) return MRS_BAD_ARGUMENT;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || page_size < 8 || nkv <= 0 || nq % nkv || nq / nkv > BM) return MRS_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    for (int done = 0; done < num_tiles; done += 65535) {         // a grid's second dimension ends at 65,535
        const int now = num_tiles - done < 65535 ? num_tiles - done : 65535;
        MRS_LAUNCH(attention_prefill_kernel, dim3(nkv, now), THREADS, SMEM_BYTES, stream,
                   *reinterpret_cast<const CUtensorMap*>(q_map), *reinterpret_cast<const CUtensorMap*>(k_map),
                   *reinterpret_cast<const CUtensorMap*>(v_map), positions, block_table, table_width, (const Tile*)tiles + done,
                   (bf16*)out, nq, nkv, page_size, shift, scale * 1.4426950408889634f, window, with_shares ? partials : nullptr);
    }
    if (with_shares)
        MRS_LAUNCH(attention_prefill_merge_kernel, dim3(nkv, num_tiles, TILES * BM / 8), 256, 0, stream, (const Tile*)tiles, (const float*)partials,
                   (bf16*)out, nq, nkv);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT int mrs_attention_prefill_tc_take_error(unsigned int* word) { return mrs_take_error_word(word); }
// Mirrors the error word into a word of pinned host memory from now on.
MRS_EXPORT int mrs_attention_prefill_tc_mirror_errors(unsigned int* host_word) { return mrs_set_error_mirror(host_word); }

MRS_EXPORT const char* mrs_attention_prefill_tc_error_string(int code) {
    if (code == MRS_BAD_ARGUMENT) return "arguments outside what the kernel supports (page size below 8 or no power of two, more than 128 query heads a key/value head)";
    if (code == MRS_TENSOR_MAP_FAILED) return "the driver refused the tensor map (address, sizes or strides)";
    return cudaGetErrorString((cudaError_t)code);
}
