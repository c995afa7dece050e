// Paged causal grouped-query attention on the tensor cores (bfloat16 in, float32 softmax and
// accumulation), compiled for one head size: -DMRS_HEAD_DIM=<multiple of 16, at most 256>.
// It serves prompts, decoded tokens and batches that mix both.   (reference: ops.cu:101-147,
// one CTA per (token, head) on the CUDA cores; here one CTA works on a tile of query rows
// that share a key/value head, so a key is read once for the whole group of query heads.)
//
// A *tile* is a run of consecutive tokens of ONE request.  Its query rows are the pairs
// (token, head within the group), row = token_in_tile * group + head_in_group.
//   rows mode  (64 rows, 4 warps x 16 rows): every warp walks all keys of the tile's range.
//   keys mode  (16 rows shared by 4 warps):  every warp takes 16 of each 64 keys and the four
//              partial results are merged at the end; for decoded tokens and short portions.
// Keys are walked in blocks of KV_BLOCK positions aligned to multiples of KV_BLOCK; with
// `splits` > 1 the blocks of a tile are dealt to `splits` CTAs that write unnormalised partial
// results (sum, running max, running sum) to scratch memory, and `combine` merges them.
// K and V blocks are gathered page by page through the request's block table with cp.async
// into shared memory (two stages), Q x K^T and P x V are mma.sync m16n8k16.
#include "common.cuh"

#ifndef MRS_HEAD_DIM
#error "compile with -DMRS_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int D = MRS_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16, at most 256");
constexpr int CHUNKS = D / 8;                 // 16-byte chunks in a row
constexpr bool SWIZZLE = (D % 64 == 0);       // rows of whole 128-byte lines: xor the chunk with the row
constexpr int THREADS = 128;
constexpr int ROWS_WIDE = 64, ROWS_NARROW = 16;
constexpr int KV_WIDE = D <= 128 ? 64 : 32;   // keys per block, rows mode
constexpr int KV_NARROW = 64;                 // keys per block, keys mode

__device__ __forceinline__ int tile_offset(int row, int col) {   // element offset in a [rows][D] tile
    const int chunk = col >> 3;
    return row * D + ((SWIZZLE ? (chunk ^ (row & 7)) : chunk) << 3) + (col & 7);
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;                // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct Tile {          // one entry of the tile list
    int seq;           // row of the block table
    int first_token;   // first row of q / out
    int tokens;        // tokens in the tile
    int pad;
};

// Copies keys [key0, key0 + KV) of one kv head into a [KV][D] shared tile.  Rows at or beyond
// `key_end`, before `key_begin`, or on a page that was given back are filled with zeros.
template <int KV>
__device__ __forceinline__ void load_kv_block(bf16* dst, const bf16* __restrict__ cache, const int* __restrict__ pages,
                                              int key0, int key_begin, int key_end, int kv_head, int nkv,
                                              int page_size, int page_shift) {
    for (int idx = threadIdx.x; idx < KV * CHUNKS; idx += THREADS) {
        const int row = idx / CHUNKS, chunk = idx % CHUNKS;
        const int key = key0 + row;
        bool valid = key >= key_begin && key < key_end;
        const bf16* src = cache;
        if (valid) {
            const int page = pages[key >> page_shift];
            valid = page >= 0;
            if (valid)
                src = cache + (((size_t)page * nkv + kv_head) * page_size + (key & (page_size - 1))) * D + chunk * 8;
        }
        cp_async16(dst + row * D + ((SWIZZLE ? (chunk ^ (row & 7)) : chunk) << 3), src, valid);
    }
}

// S[16 x 8*NT] += Q[16 x D] . K^T for the keys [key_row0, key_row0 + 8*NT) of the shared block.
template <int NT>
__device__ __forceinline__ void qk_product(float (&s)[NT][4], const bf16* q_tile, int q_row0, const bf16* k_tile,
                                           int key_row0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, q_tile + tile_offset(q_row0 + (lane & 15), kk * 16 + (lane >> 4) * 8));
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
            uint32_t b[4];
            ldmatrix_x4(b, k_tile + tile_offset(key_row0 + nt * 8 + (lane & 7) + ((lane >> 4) << 3),
                                                kk * 16 + ((lane >> 3) & 1) * 8));
            mma_bf16(s[nt], a, b[0], b[1]);
            mma_bf16(s[nt + 1], a, b[2], b[3]);
        }
    }
}

// O[16 x D] += P[16 x 8*NT] . V for the same keys; P is taken from the score registers.
template <int NT>
__device__ __forceinline__ void pv_product(float (&o)[D / 8][4], const float (&s)[NT][4], const bf16* v_tile,
                                           int key_row0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dt = 0; dt < D / 8; dt += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_tile + tile_offset(key_row0 + kk * 16 + (lane & 15), dt * 8 + (lane >> 4) * 8));
            mma_bf16(o[dt], a, b[0], b[1]);
            mma_bf16(o[dt + 1], a, b[2], b[3]);
        }
    }
}

// Masks the scores of one warp, updates the running max and sum of its two rows (lane / 4 and
// lane / 4 + 8), rescales the accumulator and turns the scores into probabilities.
template <int NT>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&o)[D / 8][4], float (&row_max)[2],
                                             float (&row_sum)[2], const int (&row_pos)[2], int key0, int key_end,
                                             int window, float scale_log2) {
    const int t = threadIdx.x & 3;
    float block_max[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int key = key0 + nt * 8 + 2 * t + (e & 1);
            const int pos = row_pos[e >> 1];
            const bool seen = key <= pos && key < key_end && (window <= 0 || key > pos - window);
            s[nt][e] = seen ? s[nt][e] * scale_log2 : -CUDART_INF_F;
            block_max[e >> 1] = fmaxf(block_max[e >> 1], s[nt][e]);
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        block_max[r] = fmaxf(block_max[r], __shfl_xor_sync(0xffffffffu, block_max[r], 1));
        block_max[r] = fmaxf(block_max[r], __shfl_xor_sync(0xffffffffu, block_max[r], 2));
        const float new_max = fmaxf(row_max[r], block_max[r]);
        const float base = new_max == -CUDART_INF_F ? 0.0f : new_max;   // a row that has seen no key yet
        const float alpha = exp2f(row_max[r] - base);
        row_max[r] = new_max;
        float sum = 0.0f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            s[nt][2 * r] = exp2f(s[nt][2 * r] - base);
            s[nt][2 * r + 1] = exp2f(s[nt][2 * r + 1] - base);
            sum += s[nt][2 * r] + s[nt][2 * r + 1];
        }
        row_sum[r] = row_sum[r] * alpha + sum;      // the sum over the quad's lanes is taken at the end
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            o[dt][2 * r] *= alpha;
            o[dt][2 * r + 1] *= alpha;
        }
    }
}

// Range of key blocks of a tile: [first, last) in units of KV positions, and the split's share.
__device__ __forceinline__ void block_range(int lo_key, int hi_key, int kv, int split, int splits, int& first, int& last) {
    const int b0 = lo_key / kv, b1 = (hi_key + kv - 1) / kv;
    const int per = (b1 - b0 + splits - 1) / splits;
    first = min(b1, b0 + split * per);
    last = min(b1, first + per);
}

// ---------------------------------------------------------------------------------------------
// rows mode: 64 query rows, every warp owns 16 of them and sees every key block.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS) attention_rows_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    const int* __restrict__ positions, const int* __restrict__ block_table, int table_width,
    const Tile* __restrict__ tiles, bf16* __restrict__ out, int nq, int nkv, int page_size, int page_shift,
    float scale_log2, int window) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_tile = reinterpret_cast<bf16*>(smem_raw);
    bf16* k_tiles = q_tile + ROWS_WIDE * D;
    bf16* v_tiles = k_tiles + 2 * KV_WIDE * D;
    constexpr int NT = KV_WIDE / 8;

    const Tile tile = tiles[blockIdx.x];
    if (tile.tokens <= 0) return;                    // a padding entry of the tile list
    const int kv_head = blockIdx.y, group = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* pages = block_table + (size_t)tile.seq * table_width;
    const int rows = tile.tokens * group;

    // query rows of the tile -> shared memory (rows past the tile's end are zeros)
    for (int idx = threadIdx.x; idx < ROWS_WIDE * CHUNKS; idx += THREADS) {
        const int row = idx / CHUNKS, chunk = idx % CHUNKS;
        const bool valid = row < rows;
        const bf16* src = q;
        if (valid) src = q + ((size_t)(tile.first_token + row / group) * nq + kv_head * group + row % group) * D + chunk * 8;
        cp_async16(q_tile + row * D + ((SWIZZLE ? (chunk ^ (row & 7)) : chunk) << 3), src, valid);
    }
    const int first_pos = positions[tile.first_token], last_pos = positions[tile.first_token + tile.tokens - 1];
    const int key_end = last_pos + 1;
    const int key_begin = window > 0 ? max(0, first_pos - window + 1) : 0;
    int block_first, block_last;
    block_range(key_begin, key_end, KV_WIDE, 0, 1, block_first, block_last);

    int row_pos[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + 8 * r;
        row_pos[r] = row < rows ? positions[tile.first_token + row / group] : last_pos;
    }
    float o[D / 8][4];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dt][e] = 0.0f;
    float row_max[2] = {-CUDART_INF_F, -CUDART_INF_F}, row_sum[2] = {0.0f, 0.0f};

    if (block_first < block_last) {
        load_kv_block<KV_WIDE>(k_tiles, k_cache, pages, block_first * KV_WIDE, key_begin, key_end, kv_head, nkv, page_size, page_shift);
        load_kv_block<KV_WIDE>(v_tiles, v_cache, pages, block_first * KV_WIDE, key_begin, key_end, kv_head, nkv, page_size, page_shift);
    }
    cp_async_commit();
    for (int block = block_first; block < block_last; ++block) {
        const int stage = (block - block_first) & 1;
        if (block + 1 < block_last) {
            load_kv_block<KV_WIDE>(k_tiles + (stage ^ 1) * KV_WIDE * D, k_cache, pages, (block + 1) * KV_WIDE, key_begin, key_end, kv_head, nkv, page_size, page_shift);
            load_kv_block<KV_WIDE>(v_tiles + (stage ^ 1) * KV_WIDE * D, v_cache, pages, (block + 1) * KV_WIDE, key_begin, key_end, kv_head, nkv, page_size, page_shift);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key0 = block * KV_WIDE;
        // a warp whose rows all lie before this block has nothing to add
        const int warp_last_pos = __shfl_sync(0xffffffffu, row_pos[1], 28);
        if (key0 <= warp_last_pos) {
            float s[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
            qk_product<NT>(s, q_tile, warp * 16, k_tiles + stage * KV_WIDE * D, 0);
            softmax_step<NT>(s, o, row_max, row_sum, row_pos, key0, key_end, window, scale_log2);
            pv_product<NT>(o, s, v_tiles + stage * KV_WIDE * D, 0);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = row_sum[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int row = warp * 16 + (lane >> 2) + 8 * r;
        if (row >= rows) continue;
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        bf16* dst = out + ((size_t)(tile.first_token + row / group) * nq + kv_head * group + row % group) * D;
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            const int col = dt * 8 + 2 * (lane & 3);
            *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[dt][2 * r] * inv, o[dt][2 * r + 1] * inv);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// keys mode: 16 query rows shared by the four warps; warp w takes keys [16w, 16w + 16) of every
// block of 64.  The four partial results are merged through shared memory; with splits > 1 the
// merged partial result goes to scratch memory for `combine`.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS) attention_keys_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    const int* __restrict__ positions, const int* __restrict__ block_table, int table_width,
    const Tile* __restrict__ tiles, bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    int nq, int nkv, int page_size, int page_shift, float scale_log2, int window, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_tile = reinterpret_cast<bf16*>(smem_raw);
    bf16* k_tiles = q_tile + ROWS_NARROW * D;
    bf16* v_tiles = k_tiles + 2 * KV_NARROW * D;
    constexpr int NT = 2;                                    // 16 keys per warp and block

    const Tile tile = tiles[blockIdx.x];
    if (tile.tokens <= 0) return;                    // a padding entry of the tile list
    const int kv_head = blockIdx.y, split = blockIdx.z, group = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* pages = block_table + (size_t)tile.seq * table_width;
    const int rows = tile.tokens * group;

    for (int idx = threadIdx.x; idx < ROWS_NARROW * CHUNKS; idx += THREADS) {
        const int row = idx / CHUNKS, chunk = idx % CHUNKS;
        const bool valid = row < rows;
        const bf16* src = q;
        if (valid) src = q + ((size_t)(tile.first_token + row / group) * nq + kv_head * group + row % group) * D + chunk * 8;
        cp_async16(q_tile + row * D + ((SWIZZLE ? (chunk ^ (row & 7)) : chunk) << 3), src, valid);
    }
    const int first_pos = positions[tile.first_token], last_pos = positions[tile.first_token + tile.tokens - 1];
    const int key_end = last_pos + 1;
    const int key_begin = window > 0 ? max(0, first_pos - window + 1) : 0;
    int block_first, block_last;
    block_range(key_begin, key_end, KV_NARROW, split, splits, block_first, block_last);

    int row_pos[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + 8 * r;
        row_pos[r] = row < rows ? positions[tile.first_token + row / group] : last_pos;
    }
    float o[D / 8][4];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dt][e] = 0.0f;
    float row_max[2] = {-CUDART_INF_F, -CUDART_INF_F}, row_sum[2] = {0.0f, 0.0f};

    if (block_first < block_last) {
        load_kv_block<KV_NARROW>(k_tiles, k_cache, pages, block_first * KV_NARROW, key_begin, key_end, kv_head, nkv, page_size, page_shift);
        load_kv_block<KV_NARROW>(v_tiles, v_cache, pages, block_first * KV_NARROW, key_begin, key_end, kv_head, nkv, page_size, page_shift);
    }
    cp_async_commit();
    for (int block = block_first; block < block_last; ++block) {
        const int stage = (block - block_first) & 1;
        if (block + 1 < block_last) {
            load_kv_block<KV_NARROW>(k_tiles + (stage ^ 1) * KV_NARROW * D, k_cache, pages, (block + 1) * KV_NARROW, key_begin, key_end, kv_head, nkv, page_size, page_shift);
            load_kv_block<KV_NARROW>(v_tiles + (stage ^ 1) * KV_NARROW * D, v_cache, pages, (block + 1) * KV_NARROW, key_begin, key_end, kv_head, nkv, page_size, page_shift);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key0 = block * KV_NARROW + warp * 16;
        if (key0 < key_end) {
            float s[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
            qk_product<NT>(s, q_tile, 0, k_tiles + stage * KV_NARROW * D, warp * 16);
            softmax_step<NT>(s, o, row_max, row_sum, row_pos, key0, key_end, window, scale_log2);
            pv_product<NT>(o, s, v_tiles + stage * KV_NARROW * D, warp * 16);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();

    // merge the four warps: shared memory now holds [4][16][D] sums and [4][16][2] (max, sum)
    float* merge_o = reinterpret_cast<float*>(k_tiles);
    float* merge_ml = merge_o + 4 * ROWS_NARROW * D;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = row_sum[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int row = (lane >> 2) + 8 * r;
        if ((lane & 3) == 0) {
            merge_ml[(warp * ROWS_NARROW + row) * 2] = row_max[r];
            merge_ml[(warp * ROWS_NARROW + row) * 2 + 1] = sum;
        }
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            const int col = dt * 8 + 2 * (lane & 3);
            merge_o[(warp * ROWS_NARROW + row) * D + col] = o[dt][2 * r];
            merge_o[(warp * ROWS_NARROW + row) * D + col + 1] = o[dt][2 * r + 1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS_NARROW * D; idx += THREADS) {
        const int row = idx / D, col = idx % D;
        if (row >= rows) continue;
        float m = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, merge_ml[(w * ROWS_NARROW + row) * 2]);
        const float base = m == -CUDART_INF_F ? 0.0f : m;
        float sum = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = exp2f(merge_ml[(w * ROWS_NARROW + row) * 2] - base);
            sum += merge_ml[(w * ROWS_NARROW + row) * 2 + 1] * f;
            acc += merge_o[(w * ROWS_NARROW + row) * D + col] * f;
        }
        if (splits == 1) {
            out[((size_t)(tile.first_token + row / group) * nq + kv_head * group + row % group) * D + col] =
                __float2bfloat16_rn(sum > 0.0f ? acc / sum : 0.0f);
        } else {
            const size_t slot = (((size_t)blockIdx.x * nkv + kv_head) * splits + split) * ROWS_NARROW + row;
            part_o[slot * D + col] = acc;
            if (col == 0) {
                part_ml[slot * 2] = m;
                part_ml[slot * 2 + 1] = sum;
            }
        }
    }
}

// Merges the `splits` partial results of every (tile, kv head, row).
__global__ void __launch_bounds__(THREADS) attention_combine_kernel(
    const float* __restrict__ part_o, const float* __restrict__ part_ml, const Tile* __restrict__ tiles,
    bf16* __restrict__ out, int nq, int nkv, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    const Tile tile = tiles[blockIdx.x];
    const int kv_head = blockIdx.y, group = nq / nkv, rows = tile.tokens * group;
    const size_t base_slot = ((size_t)blockIdx.x * nkv + kv_head) * splits * ROWS_NARROW;
    for (int idx = threadIdx.x; idx < rows * D; idx += THREADS) {
        const int row = idx / D, col = idx % D;
        float m = -CUDART_INF_F;
        for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(base_slot + (size_t)s * ROWS_NARROW + row) * 2]);
        const float base = m == -CUDART_INF_F ? 0.0f : m;
        float sum = 0.0f, acc = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const size_t slot = base_slot + (size_t)s * ROWS_NARROW + row;
            const float f = exp2f(part_ml[slot * 2] - base);
            sum += part_ml[slot * 2 + 1] * f;
            acc += part_o[slot * D + col] * f;
        }
        out[((size_t)(tile.first_token + row / group) * nq + kv_head * group + row % group) * D + col] =
            __float2bfloat16_rn(sum > 0.0f ? acc / sum : 0.0f);
    }
}

constexpr size_t smem_rows = (size_t)(ROWS_WIDE * D + 4 * KV_WIDE * D) * sizeof(bf16);
constexpr size_t smem_keys_tiles = (size_t)(ROWS_NARROW * D + 4 * KV_NARROW * D) * sizeof(bf16);
constexpr size_t smem_keys_merge = (size_t)ROWS_NARROW * D * sizeof(bf16) + (size_t)(4 * ROWS_NARROW * D + 4 * ROWS_NARROW * 2) * sizeof(float);
constexpr size_t smem_keys = smem_keys_tiles > smem_keys_merge ? smem_keys_tiles : smem_keys_merge;

int page_shift_of(int page_size) {
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    return (1 << shift) == page_size ? shift : -1;
}

}  // namespace

MRS_EXPORT int mrs_attention_mma_head_dim() { return D; }
MRS_EXPORT int mrs_attention_mma_rows(int narrow) { return narrow ? ROWS_NARROW : ROWS_WIDE; }

// Scratch floats that `mrs_attention_mma_keys` needs for `tiles` tiles, `nkv` heads, `splits` splits.
MRS_EXPORT long long mrs_attention_mma_scratch_floats(int tiles, int nkv, int splits) {
    return splits <= 1 ? 0 : (long long)tiles * nkv * splits * ROWS_NARROW * (D + 2);
}

// Tiles of up to 64 / group tokens each.
MRS_EXPORT int mrs_attention_mma_rows_mode(const void* q, const void* k_cache, const void* v_cache, const int* positions,
                                           const int* block_table, int table_width, const int* tiles, int num_tiles,
                                           void* out, int nq, int nkv, int page_size, float scale, int window,
                                           void* stream) {
    if (num_tiles <= 0) return 0;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || nkv <= 0 || nq % nkv || nq / nkv > ROWS_WIDE) return MRS_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rows);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    MRS_LAUNCH(attention_rows_kernel, dim3(num_tiles, nkv), THREADS, smem_rows, stream,
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, positions, block_table, table_width,
        (const Tile*)tiles, (bf16*)out, nq, nkv, page_size, shift, scale * 1.4426950408889634f, window);
    MRS_RETURN_LAUNCH_STATUS();
}

// Tiles of up to 16 / group tokens each; `splits` CTAs share a tile's keys.  `scratch` must hold
// mrs_attention_mma_scratch_floats(...) floats when splits > 1.
MRS_EXPORT int mrs_attention_mma_keys_mode(const void* q, const void* k_cache, const void* v_cache, const int* positions,
                                           const int* block_table, int table_width, const int* tiles, int num_tiles,
                                           void* out, float* scratch, int nq, int nkv, int page_size, float scale,
                                           int window, int splits, void* stream) {
    if (num_tiles <= 0) return 0;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || nkv <= 0 || nq % nkv || nq / nkv > ROWS_NARROW || splits < 1 || splits > 65535) return MRS_BAD_ARGUMENT;
    if (splits > 1 && !scratch) return MRS_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_keys_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_keys);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)num_tiles * nkv * splits * ROWS_NARROW * D : nullptr;
    MRS_LAUNCH(attention_keys_kernel, dim3(num_tiles, nkv, splits), THREADS, smem_keys, stream,
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, positions, block_table, table_width,
        (const Tile*)tiles, (bf16*)out, part_o, part_ml, nq, nkv, page_size, shift, scale * 1.4426950408889634f, window,
        splits);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (splits > 1)
        MRS_LAUNCH(attention_combine_kernel, dim3(num_tiles, nkv), THREADS, 0, stream,
            part_o, part_ml, (const Tile*)tiles, (bf16*)out, nq, nkv, splits);
    MRS_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------
// The same split attention with scratch memory that the library owns (see attention_no_alloc.h).
// ---------------------------------------------------------------------------------------------
#include "attention_no_alloc.h"

#include <atomic>
#include <mutex>

namespace {

// Device memory held by every GPU that loads this library.  In host code this name is only a
// stand-in for the symbol: its device address is looked up once per device below.
static __device__ __align__(256) float static_scratch[MRS_ATTENTION_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* static_scratch_address[kMaxDevices] = {};
std::atomic<bool> static_entry_ready[kMaxDevices];     // zero-initialised: false
std::mutex static_entry_setup;                         // two host threads may make a device's first call together

}  // namespace

MRS_EXPORT int mrs_attention_mma_keys_mode_static_scratch(const void* q, const void* k_cache, const void* v_cache,
                                                          const int* positions, const int* block_table,
                                                          int table_width, const int* tiles, int num_tiles, void* out,
                                                          int nq, int nkv, int page_size, float scale, int window,
                                                          int splits, void* stream) {
    if (num_tiles <= 0) return 0;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || nkv <= 0 || nq % nkv || nq / nkv > ROWS_NARROW || splits < 1 || splits > 65535) return MRS_BAD_ARGUMENT;
    const long long need = (long long)num_tiles * nkv * splits * ROWS_NARROW * (D + 2);
    if (splits > 1 && need > (long long)MRS_ATTENTION_STATIC_SCRATCH_FLOATS) return MRS_STATIC_SCRATCH_TOO_SMALL;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= kMaxDevices) return MRS_BAD_ARGUMENT;
    if (!static_entry_ready[device].load(std::memory_order_acquire)) {      // set-up, once per device, with that device current
        std::lock_guard<std::mutex> lock(static_entry_setup);
        if (!static_entry_ready[device].load(std::memory_order_relaxed)) {
            e = cudaGetSymbolAddress((void**)&static_scratch_address[device], static_scratch);
            if (e != cudaSuccess) return (int)e;
            e = cudaFuncSetAttribute(attention_keys_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_keys);
            if (e != cudaSuccess) return (int)e;
            static_entry_ready[device].store(true, std::memory_order_release);
        }
    }
    float* part_o = static_scratch_address[device];
    float* part_ml = part_o + (size_t)num_tiles * nkv * splits * ROWS_NARROW * D;
    MRS_LAUNCH(attention_keys_kernel, dim3(num_tiles, nkv, splits), THREADS, smem_keys, stream,
        (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, positions, block_table, table_width,
        (const Tile*)tiles, (bf16*)out, part_o, part_ml, nq, nkv, page_size, shift, scale * 1.4426950408889634f, window,
        splits);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (splits > 1)
        MRS_LAUNCH(attention_combine_kernel, dim3(num_tiles, nkv), THREADS, 0, stream,
            part_o, part_ml, (const Tile*)tiles, (bf16*)out, nq, nkv, splits);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT const char* mrs_attention_mma_error_string(int code) {
    if (code == MRS_STATIC_SCRATCH_TOO_SMALL)
        return "the call needs more scratch than the library's fixed array holds "
               "(tiles * kv_heads * splits * 16 * (head_dim + 2) floats must not exceed 4 Mi floats)";
    if (code == MRS_BAD_ARGUMENT) return "arguments outside what the kernel supports (page size, head grouping, splits, device)";
    return cudaGetErrorString((cudaError_t)code);
}
