// Paged grouped-query attention for decoded tokens and short portions (up to 16 query rows of
// one key/value head), for head sizes that are multiples of 64: -DMRS_HEAD_DIM=64|128|192|256.
// The step is bound by reading keys and values once from HBM, so this kernel is built around
// the copy: a producer warp walks the request's block table and fetches every page of a
// 64-key block with one bulk tensor copy (TMA) into a ring of shared-memory stages, 128-byte
// swizzled; four consumer warps wait on the stage's mbarrier, take 16 keys each with
// ldmatrix + mma.sync (float32 softmax and accumulation), and hand the stage back through a
// second mbarrier.  No thread computes an address of a key, and no block-wide barrier stands
// between two blocks of keys.                      (reference: ops.cu:101-147, one CTA per
// (token, head) walking the keys with scalar loads)
//
// Work is cut as in the plain tensor-core kernel: a tile is up to 16 / group consecutive tokens
// of one request; `splits` CTAs share the 64-key blocks of a tile.  When the splits are 2, 4, 8 or
// 16 they are launched as one thread-block cluster: every CTA sends each other CTA that CTA's
// slice of the head's columns of its unnormalised result (and all of them its maxima and sums)
// through distributed shared memory, counts the arrivals on an mbarrier of its own, and merges and
// stores its slice, in the order of the shares.  Nothing of the merge goes through global memory,
// whose dependent trips (result out, fence, counter, results in) cost microseconds each at the
// end of a kernel.  Other split counts leave their results in scratch memory, and the CTA that
// finishes a (tile, head) last merges them in order.
#include "tma.cuh"

#ifndef MRS_HEAD_DIM
#error "compile with -DMRS_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int D = MRS_HEAD_DIM;
static_assert(D % 64 == 0 && D >= 64 && D <= 256, "this kernel takes head sizes 64, 128, 192, 256");
constexpr int HALVES = D / 64;                  // 128-byte column groups of a row
constexpr int ROWS = 16;                        // query rows of a tile
constexpr int KV = 64;                          // keys per block
constexpr int STAGES = D <= 64 ? 6 : 3;
constexpr int CONSUMER_WARPS = 4;
constexpr int THREADS = 32 * (CONSUMER_WARPS + 1);
constexpr int STAGE_BYTES = 2 * KV * D * 2;     // keys and values of one block
constexpr int TILE_BYTES = KV * D * 2;

struct Tile {
    int seq, first_token, tokens, pad;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
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
// ---- distributed shared memory of a thread-block cluster
__device__ __forceinline__ uint32_t in_cta(uint32_t local_address, uint32_t rank) {      // the same place in CTA `rank`
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_address), "r"(rank));
    return a;
}
__device__ __forceinline__ void store_cluster(uint32_t address, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(address), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void store_cluster(uint32_t address, float2 v) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(address), "f"(v.x), "f"(v.y) : "memory");
}
__device__ __forceinline__ void arrive_in_cluster(uint32_t barrier_address) {          // after this thread's (and, through a CTA barrier, its CTA's) stores
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(barrier_address) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Bounded like mbar_wait; sees what the arriving CTAs of the cluster stored.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long start = clock64();
    unsigned int spins = 0;
    while (!mbar_try_wait_cluster(bar, parity)) {
        if ((++spins & 255u) == 0 && *reinterpret_cast<volatile unsigned int*>(&mrs_error_word) != 0) return false;
        if (clock64() - start > MRS_WAIT_CYCLES) {
            mrs_raise(MRS_ERR_BARRIER_TIMEOUT);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
constexpr int MAX_CLUSTER = 16;

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * CONSUMER_WARPS) : "memory"); }

__global__ void __launch_bounds__(THREADS) attention_decode_kernel(
    const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
    const bf16* __restrict__ q, const int* __restrict__ positions, const int* __restrict__ block_table, int table_width,
    const Tile* __restrict__ tiles, bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    int* __restrict__ counters, int nq, int nkv, int page_size, int page_shift, float scale_log2, int window, int splits,
    int in_cluster) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ int is_last;
    const Tile tile = tiles[blockIdx.x];
    if (tile.tokens <= 0) return;                    // a padding entry of the tile list
    // stages start on a 1024-byte boundary: the swizzle pattern of the copies is a function of the address
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    // what the other CTAs of a cluster send: their parts of this CTA's columns, and everybody's maxima and sums
    uint64_t* merge_bar = empty + STAGES;
    float* incoming_o = reinterpret_cast<float*>(merge_bar + 2);            // [splits][ROWS][D / splits]
    float* incoming_ml = incoming_o + ROWS * D;                            // [splits][ROWS][2]

    const int kv_head = blockIdx.y, split = blockIdx.z, group = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* pages = block_table + (size_t)tile.seq * table_width;
    const int rows = tile.tokens * group;
    const int first_pos = positions[tile.first_token], last_pos = positions[tile.first_token + tile.tokens - 1];
    const int key_end = last_pos + 1;
    const int key_begin = window > 0 ? max(0, first_pos - window + 1) : 0;
    // this split's share of the tile's 64-key blocks
    const int b0 = key_begin / KV, b1 = (key_end + KV - 1) / KV;
    const int per = (b1 - b0 + splits - 1) / splits;
    const int block_first = min(b1, b0 + split * per), block_last = min(b1, block_first + per);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        if (in_cluster) mbar_init(merge_bar, splits);
        mbar_fence_init();
    }
    __syncthreads();
    if (in_cluster) cluster_sync_all();          // every CTA's barrier stands before anybody can arrive at it
    pdl_launch_dependents();
    // The queries and the keys and values of this step's tokens come from the kernel before this one;
    // older keys lie in the cache since earlier steps.  The consumers wait before they read the
    // queries, the producer only before the first block that holds a key of this step: blocks of
    // older keys are fetched while the kernel before still runs.

    if (warp == CONSUMER_WARPS) {
        // ------------------------------------------------------------------ producer
        // Every lane owns one page of a block: it reads the page's number a block ahead of its use and
        // issues the page's copies itself, so a block costs one trip to the block table and one round of
        // copies issued side by side.  Lane 0 also waits for the stage and arms its barrier.
        if (lane == 0) {
            tma_prefetch_descriptor(&k_map);
            tma_prefetch_descriptor(&v_map);
        }
        const int rows_per_copy = min(page_size, KV);
        const int copies = KV / rows_per_copy;
        const int copy_bytes = rows_per_copy * D * 2;
        // keys past the end, before the window or on a page that was given back are masked by their
        // position; their copy reads page 0, which always exists and holds finite numbers
        auto page_of = [&](int block) {
            const int key = block * KV + lane * rows_per_copy;
            return (lane < copies && key < key_end) ? pages[key >> page_shift] : -1;
        };
        int next_page = block_first < block_last ? page_of(block_first) : -1;
        bool waited = false;
        for (int block = block_first; block < block_last; ++block) {
            const int it = block - block_first, s = it % STAGES;
            if (!waited && (block + 1) * KV > first_pos) {
                pdl_wait();
                waited = true;
            }
            const int my_page = next_page;
            if (block + 1 < block_last) next_page = page_of(block + 1);
            if (lane == 0) {
                if (it >= STAGES) mbar_wait(&empty[s], ((it / STAGES) - 1) & 1);
                mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
            }
            __syncwarp();                                    // the stage is free and the barrier armed
            unsigned char* k_dst = smem + s * STAGE_BYTES;
            unsigned char* v_dst = k_dst + TILE_BYTES;
            if (lane < copies) {                             // every lane issues the copies of its own page
                const int key = block * KV + lane * rows_per_copy;
                const int row = my_page < 0 ? 0 : key & (page_size - 1);
                tma_load_5d(k_dst + lane * copy_bytes, &k_map, &full[s], 0, row, 0, kv_head, max(my_page, 0));
                tma_load_5d(v_dst + lane * copy_bytes, &v_map, &full[s], 0, row, 0, kv_head, max(my_page, 0));
            }
        }
        if (in_cluster) cluster_sync_all();      // nobody leaves a cluster while a peer may still write into its shared memory
        return;
    }

    // ---------------------------------------------------------------------- consumers
    pdl_wait();
    // query rows as A fragments, kept in registers for every block of keys
    uint32_t qa[D / 16][4];
    {
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = g + 8 * half;
            const bool valid = row < rows;
            const bf16* src = q + ((size_t)(tile.first_token + (valid ? row / group : 0)) * nq + kv_head * group +
                                   (valid ? row % group : 0)) * D;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                qa[kk][half] = valid ? *reinterpret_cast<const uint32_t*>(src + kk * 16 + 2 * t) : 0u;
                qa[kk][half + 2] = valid ? *reinterpret_cast<const uint32_t*>(src + kk * 16 + 8 + 2 * t) : 0u;
            }
        }
    }
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

    // where this lane's ldmatrix rows lie in a stage: the copies put a page's rows as
    // [column group of 64][row][64 columns], 128 bytes a row, 16-byte chunks xor-ed with row % 8
    const int rows_per_copy = min(page_size, KV);
    const int sub_tile_bytes = rows_per_copy * 128;
    auto row_base = [&](int r) { return (r / rows_per_copy) * (rows_per_copy * D * 2) + (r % rows_per_copy) * 128; };
    const int k_row = warp * 16 + (lane & 7) + ((lane >> 4) << 3);     // Q.K^T: keys are the n index
    const int v_row = warp * 16 + (lane & 15);                         // P.V: keys are the k index
    const uint32_t k_row_off = row_base(k_row), v_row_off = row_base(v_row);
    const int swz = lane & 7;                                          // row % 8 of both rows above
    const uint32_t smem_base = smem_u32(smem);

    for (int block = block_first; block < block_last; ++block) {
        const int it = block - block_first, s = it % STAGES;
        mbar_wait(&full[s], (it / STAGES) & 1);
        const int key0 = block * KV + warp * 16;
        if (key0 < key_end) {
            const uint32_t k_tile = smem_base + s * STAGE_BYTES, v_tile = k_tile + TILE_BYTES;
            float sc[2][4] = {};
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t b[4];
                const int chunk = 2 * kk + ((lane >> 3) & 1);
                ldmatrix_x4(b, k_tile + k_row_off + (chunk >> 3) * sub_tile_bytes + (((chunk & 7) ^ swz) << 4));
                mma_bf16(sc[0], qa[kk], b[0], b[1]);
                mma_bf16(sc[1], qa[kk], b[2], b[3]);
            }
            // mask, running max and sum of the two rows of this lane (rows lane/4 and lane/4 + 8)
            const int t = lane & 3;
            float block_max[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + nt * 8 + 2 * t + (e & 1);
                    const int pos = row_pos[e >> 1];
                    const bool seen = key <= pos && key < key_end && (window <= 0 || key > pos - window);
                    sc[nt][e] = seen ? sc[nt][e] * scale_log2 : -CUDART_INF_F;
                    block_max[e >> 1] = fmaxf(block_max[e >> 1], sc[nt][e]);
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                block_max[r] = fmaxf(block_max[r], __shfl_xor_sync(0xffffffffu, block_max[r], 1));
                block_max[r] = fmaxf(block_max[r], __shfl_xor_sync(0xffffffffu, block_max[r], 2));
                const float new_max = fmaxf(row_max[r], block_max[r]);
                const float base = new_max == -CUDART_INF_F ? 0.0f : new_max;
                const float alpha = exp2f(row_max[r] - base);
                row_max[r] = new_max;
                float sum = 0.0f;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    sc[nt][2 * r] = exp2f(sc[nt][2 * r] - base);
                    sc[nt][2 * r + 1] = exp2f(sc[nt][2 * r + 1] - base);
                    sum += sc[nt][2 * r] + sc[nt][2 * r + 1];
                }
                row_sum[r] = row_sum[r] * alpha + sum;
#pragma unroll
                for (int dt = 0; dt < D / 8; ++dt) {
                    o[dt][2 * r] *= alpha;
                    o[dt][2 * r + 1] *= alpha;
                }
            }
            uint32_t pa[4] = {pack_bf16(sc[0][0], sc[0][1]), pack_bf16(sc[0][2], sc[0][3]),
                              pack_bf16(sc[1][0], sc[1][1]), pack_bf16(sc[1][2], sc[1][3])};
#pragma unroll
            for (int dt = 0; dt < D / 8; dt += 2) {
                uint32_t b[4];
                const int chunk = dt + (lane >> 4);
                ldmatrix_x4_trans(b, v_tile + v_row_off + (chunk >> 3) * sub_tile_bytes + (((chunk & 7) ^ swz) << 4));
                mma_bf16(o[dt], pa, b[0], b[1]);
                mma_bf16(o[dt + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    consumer_sync();      // every warp is done with the stages: their memory now carries the merge

    float* merge_o = reinterpret_cast<float*>(smem);
    float* merge_ml = merge_o + CONSUMER_WARPS * ROWS * D;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = row_sum[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int row = (lane >> 2) + 8 * r;
        if ((lane & 3) == 0) {
            merge_ml[(warp * ROWS + row) * 2] = row_max[r];
            merge_ml[(warp * ROWS + row) * 2 + 1] = sum;
        }
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            const int col = dt * 8 + 2 * (lane & 3);
            *reinterpret_cast<float2*>(&merge_o[(warp * ROWS + row) * D + col]) = make_float2(o[dt][2 * r], o[dt][2 * r + 1]);
        }
    }
    consumer_sync();
    if (in_cluster) {
        // ---- merge within the cluster.  This CTA's result, still scaled by its own maxima: columns
        // [j * cols, (j + 1) * cols) of every row go to CTA j, the maxima and sums to every CTA.
        const int cols = D / splits;
        const uint32_t o_here = smem_u32(incoming_o) + (uint32_t)split * ROWS * cols * 4, ml_here = smem_u32(incoming_ml) + (uint32_t)split * ROWS * 8;
        for (int idx = threadIdx.x; idx < rows * (D / 4); idx += 32 * CONSUMER_WARPS) {
            const int row = idx / (D / 4), col = (idx % (D / 4)) * 4;
            float m = -CUDART_INF_F;
#pragma unroll
            for (int w = 0; w < CONSUMER_WARPS; ++w) m = fmaxf(m, merge_ml[(w * ROWS + row) * 2]);
            const float base = m == -CUDART_INF_F ? 0.0f : m;
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < CONSUMER_WARPS; ++w) {
                const float f = exp2f(merge_ml[(w * ROWS + row) * 2] - base);
                const float4 v = *reinterpret_cast<const float4*>(&merge_o[(w * ROWS + row) * D + col]);
                acc.x += v.x * f, acc.y += v.y * f, acc.z += v.z * f, acc.w += v.w * f;
                sum += merge_ml[(w * ROWS + row) * 2 + 1] * f;
            }
            const int target = col / cols;
            store_cluster(in_cta(o_here + (uint32_t)(row * cols + col % cols) * 4, target), acc);
            if (col == 0)
                for (int j = 0; j < splits; ++j) store_cluster(in_cta(ml_here + (uint32_t)row * 8, j), make_float2(m, sum));
        }
        consumer_sync();                              // the CTA's stores are issued: one thread tells every CTA
        if (threadIdx.x == 0) {
            asm volatile("fence.acq_rel.cluster;" ::: "memory");
            for (int j = 0; j < splits; ++j) arrive_in_cluster(in_cta(smem_u32(merge_bar), j));
        }
        // all shares of this CTA's columns have arrived, or the time ran out: then nothing is stored (the error
        // word is raised and the host fails the step)
        const bool merged = mbar_wait_cluster(merge_bar, 0);
        for (int idx = threadIdx.x; merged && idx < rows * (cols / 4); idx += 32 * CONSUMER_WARPS) {
            const int row = idx / (cols / 4), col = (idx % (cols / 4)) * 4;
            float m = -CUDART_INF_F;
            for (int s = 0; s < splits; ++s) m = fmaxf(m, incoming_ml[(s * ROWS + row) * 2]);
            const float base = m == -CUDART_INF_F ? 0.0f : m;
            float sum = 0.0f;
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int s = 0; s < splits; ++s) {         // in the order of the shares
                const float f = exp2f(incoming_ml[(s * ROWS + row) * 2] - base);
                const float4 v = *reinterpret_cast<const float4*>(&incoming_o[(s * ROWS + row) * cols + col]);
                sum += incoming_ml[(s * ROWS + row) * 2 + 1] * f;
                acc.x += v.x * f, acc.y += v.y * f, acc.z += v.z * f, acc.w += v.w * f;
            }
            const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
            bf16* dst = out + ((size_t)(tile.first_token + row / group) * nq + kv_head * group + row % group) * D + split * cols + col;
            *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
            *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
        }
        // Every wait above is bounded, so every thread of the cluster gets here; a CTA whose wait ran out stays
        // until its peers have sent what they still had to send into its shared memory.
        cluster_sync_all();
        return;
    }
    const size_t first_slot = ((size_t)blockIdx.x * nkv + kv_head) * splits * ROWS;
    for (int idx = threadIdx.x; idx < rows * D; idx += 32 * CONSUMER_WARPS) {
        const int row = idx / D, col = idx % D;
        float m = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < CONSUMER_WARPS; ++w) m = fmaxf(m, merge_ml[(w * ROWS + row) * 2]);
        const float base = m == -CUDART_INF_F ? 0.0f : m;
        float sum = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < CONSUMER_WARPS; ++w) {
            const float f = exp2f(merge_ml[(w * ROWS + row) * 2] - base);
            sum += merge_ml[(w * ROWS + row) * 2 + 1] * f;
            acc += merge_o[(w * ROWS + row) * D + col] * f;
        }
        if (splits == 1) {
            out[((size_t)(tile.first_token + row / group) * nq + kv_head * group + row % group) * D + col] =
                __float2bfloat16_rn(sum > 0.0f ? acc / sum : 0.0f);
        } else {
            const size_t slot = first_slot + (size_t)split * ROWS + row;
            __stcg(&part_o[slot * D + col], acc);
            if (col == 0) {
                __stcg(&part_ml[slot * 2], m);
                __stcg(&part_ml[slot * 2 + 1], sum);
            }
        }
    }
    if (splits == 1) return;

    // The CTA that leaves its share last merges all shares of this (tile, head), in the order of the shares.
    __threadfence();
    consumer_sync();
    if (threadIdx.x == 0) {
        int* counter = &counters[blockIdx.x * nkv + kv_head];
        const int arrived = atomicAdd(counter, 1);
        is_last = arrived == splits - 1;
        if (is_last) *counter = 0;                   // ready for the next launch
    }
    consumer_sync();
    if (!is_last) return;
    __threadfence();
    float* all_ml = reinterpret_cast<float*>(smem);  // [splits][rows][2]: running max and sum of every share
    for (int idx = threadIdx.x; idx < splits * rows * 2; idx += 32 * CONSUMER_WARPS) {
        const int s = idx / (rows * 2), rest = idx % (rows * 2);
        all_ml[idx] = __ldcg(&part_ml[(first_slot + (size_t)s * ROWS) * 2 + rest]);
    }
    consumer_sync();
    for (int idx = threadIdx.x; idx < rows * (D / 4); idx += 32 * CONSUMER_WARPS) {
        const int row = idx / (D / 4), col = (idx % (D / 4)) * 4;
        float m = -CUDART_INF_F;
        for (int s = 0; s < splits; ++s) m = fmaxf(m, all_ml[(s * rows + row) * 2]);
        const float base = m == -CUDART_INF_F ? 0.0f : m;
        float sum = 0.0f;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int s0 = 0; s0 < splits; s0 += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                v[u] = s0 + u < splits ? __ldcg(reinterpret_cast<const float4*>(&part_o[(first_slot + (size_t)(s0 + u) * ROWS + row) * D + col]))
                                       : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (s0 + u < splits) {
                    const float f = exp2f(all_ml[((s0 + u) * rows + row) * 2] - base);
                    sum += all_ml[((s0 + u) * rows + row) * 2 + 1] * f;
                    acc.x += v[u].x * f, acc.y += v[u].y * f, acc.z += v[u].z * f, acc.w += v[u].w * f;
                }
        }
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        bf16* dst = out + ((size_t)(tile.first_token + row / group) * nq + kv_head * group + row % group) * D + col;
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
        *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    }
}

constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 2) * sizeof(uint64_t) +
                              (size_t)ROWS * D * sizeof(float) + (size_t)MAX_CLUSTER * ROWS * 2 * sizeof(float);
static_assert((size_t)STAGES * STAGE_BYTES >= (size_t)CONSUMER_WARPS * ROWS * (D + 2) * sizeof(float), "merge area");

int page_shift_of(int page_size) {
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    return (1 << shift) == page_size ? shift : -1;
}

}  // namespace

// A tensor map of one layer's key or value pages [pages, kv_heads, page_size, D]: written to
// `map_out` (128 bytes, 64-byte aligned), to be handed to the launcher with every call.
MRS_EXPORT int mrs_attention_decode_tma_map(const void* cache, long long pages, int nkv, int page_size, void* map_out) {
    if (page_shift_of(page_size) < 0 || page_size < 8 || pages <= 0 || nkv <= 0) return MRS_BAD_ARGUMENT;
    const uint64_t dims[5] = {64, (uint64_t)page_size, (uint64_t)HALVES, (uint64_t)nkv, (uint64_t)pages};
    const uint64_t strides[4] = {(uint64_t)D * 2, 128, (uint64_t)page_size * D * 2, (uint64_t)nkv * page_size * D * 2};
    const uint32_t box[5] = {64, (uint32_t)(page_size < KV ? page_size : KV), (uint32_t)HALVES, 1, 1};
    return mrs_make_tensor_map_bf16(reinterpret_cast<CUtensorMap*>(map_out), cache, 5, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
}

MRS_EXPORT long long mrs_attention_decode_tma_scratch_floats(int tiles, int nkv, int splits) {
    return splits <= 1 ? 0 : (long long)tiles * nkv * splits * ROWS * (D + 2);
}

// Tiles of up to 16 / group tokens each; `splits` (at most 256) CTAs share a tile's keys.  With
// splits > 1, `scratch` must hold mrs_attention_decode_tma_scratch_floats(...) floats and `counters`
// num_tiles * nkv ints that are zero before the first launch (the kernel leaves them zero).
MRS_EXPORT int mrs_attention_decode_tma(const void* k_map, const void* v_map, const void* q, const int* positions,
                                        const int* block_table, int table_width, const int* tiles, int num_tiles,
                                        void* out, float* scratch, int* counters, int nq, int nkv, int page_size,
                                        float scale, int window, int splits, void* stream) {
    if (num_tiles <= 0) return 0;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || page_size < 8 || nkv <= 0 || nq % nkv || nq / nkv > ROWS || splits < 1 || splits > 256)
        return MRS_BAD_ARGUMENT;
    if (splits > 1 && (!scratch || !counters)) return MRS_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)num_tiles * nkv * splits * ROWS * D : nullptr;
    const float scale_log2 = scale * 1.4426950408889634f;
    // 2, 4, 8 or 16 splits whose slices of the head's columns are whole float4s run as one cluster and merge among themselves
    static int largest_cluster = -1;
    if (largest_cluster < 0) {
        largest_cluster = 8;
        if (cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
            cudaLaunchConfig_t probe = {};
            probe.gridDim = dim3(1, 1, 16), probe.blockDim = dim3(THREADS), probe.dynamicSmemBytes = SMEM_BYTES;
            cudaLaunchAttribute shape;
            shape.id = cudaLaunchAttributeClusterDimension;
            shape.val.clusterDim.x = 1, shape.val.clusterDim.y = 1, shape.val.clusterDim.z = 16;
            probe.attrs = &shape, probe.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, attention_decode_kernel, &probe) == cudaSuccess && clusters > 0) largest_cluster = 16;
        }
        (void)cudaGetLastError();
    }
    const bool in_cluster = splits > 1 && (splits & (splits - 1)) == 0 && splits <= largest_cluster && D % (4 * splits) == 0;
    if (in_cluster) {
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(num_tiles, nkv, splits);
        config.blockDim = dim3(THREADS);
        config.dynamicSmemBytes = SMEM_BYTES;
        config.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attributes[2];
        attributes[0].id = cudaLaunchAttributeClusterDimension;
        attributes[0].val.clusterDim.x = 1, attributes[0].val.clusterDim.y = 1, attributes[0].val.clusterDim.z = splits;
        attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[1].val.programmaticStreamSerializationAllowed = 1;
        static const bool plain = getenv("MRS_PLAIN_LAUNCH") != nullptr;
        config.attrs = attributes;
        config.numAttrs = plain ? 1 : 2;
        return (int)cudaLaunchKernelEx(&config, attention_decode_kernel, *reinterpret_cast<const CUtensorMap*>(k_map),
                                       *reinterpret_cast<const CUtensorMap*>(v_map), (const bf16*)q, positions, block_table, table_width,
                                       (const Tile*)tiles, (bf16*)out, part_o, part_ml, counters, nq, nkv, page_size, shift, scale_log2,
                                       window, splits, 1);
    }
    MRS_LAUNCH(attention_decode_kernel, dim3(num_tiles, nkv, splits), THREADS, SMEM_BYTES, stream,
        *reinterpret_cast<const CUtensorMap*>(k_map), *reinterpret_cast<const CUtensorMap*>(v_map), (const bf16*)q,
        positions, block_table, table_width, (const Tile*)tiles, (bf16*)out, part_o, part_ml, counters, nq, nkv, page_size,
        shift, scale_log2, window, splits, 0);
    MRS_RETURN_LAUNCH_STATUS();
}

// Thread-block clusters of `splits` CTAs of this kernel that the GPU holds at once (0: no such cluster): what a
// plan may count on when it wants every share of every tile resident together.  Asked of the driver once a size.
MRS_EXPORT int mrs_attention_decode_tma_resident_clusters(int splits) {
    static int known[17] = {};
    if (splits < 2 || splits > 16 || (splits & (splits - 1))) return 0;
    if (known[splits] == 0) {
        known[splits] = -1;
        if (cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) == cudaSuccess &&
            (splits <= 8 || cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess)) {
            cudaLaunchConfig_t probe = {};
            probe.gridDim = dim3(64, 1, splits), probe.blockDim = dim3(THREADS), probe.dynamicSmemBytes = SMEM_BYTES;
            cudaLaunchAttribute shape;
            shape.id = cudaLaunchAttributeClusterDimension;
            shape.val.clusterDim.x = 1, shape.val.clusterDim.y = 1, shape.val.clusterDim.z = splits;
            probe.attrs = &shape, probe.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, attention_decode_kernel, &probe) == cudaSuccess && clusters > 0) known[splits] = clusters;
        }
        (void)cudaGetLastError();
    }
    return known[splits] > 0 ? known[splits] : 0;
}

// Reads and clears this library's error word (waits for the device).  0: no kernel gave up a wait.
MRS_EXPORT int mrs_attention_decode_tma_take_error(unsigned int* word) { return mrs_take_error_word(word); }
// Mirrors the error word into a word of pinned host memory from now on.
MRS_EXPORT int mrs_attention_decode_tma_mirror_errors(unsigned int* host_word) { return mrs_set_error_mirror(host_word); }

MRS_EXPORT const char* mrs_attention_decode_tma_error_string(int code) {
    if (code == MRS_BAD_ARGUMENT) return "arguments outside what the kernel supports (page size below 8 or no power of two, head grouping, splits)";
    if (code == MRS_TENSOR_MAP_FAILED) return "the driver refused the tensor map (address, sizes or strides)";
    return cudaGetErrorString((cudaError_t)code);
}
