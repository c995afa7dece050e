// Token selection on the device: arg-max, and seeded temperature / top-k / top-p sampling.
//
// The reference takes the arg-max on the GPU (ops.cu:152-162: larger logit wins, the smaller id
// on a tie) and samples on the host in float64 after sorting the whole row
// (crates/engine/src/lib.rs:207-244).  Here a row never leaves the device.  The set that may be
// drawn is the reference's: rows ordered by descending logit with ties by ascending id, cut to
// the first top_k, then to the shortest prefix whose weight exp((x - max)/T) reaches top_p times
// the weight of the top_k set.  Such a prefix is {x > threshold} plus the first few ids of
// {x == threshold}; the threshold is found by a radix descent over the float's bits (by count
// for top_k, by weight for top_p) in place of a sort.  The draw is the inverse CDF over the
// kept set in id order with u from a counter-based generator keyed by (seed, draw index), so a
// request's tokens do not depend on what else is in the batch.
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SAMPLE_THREADS 1024
#define SAMPLE_WARPS 32

__device__ __forceinline__ unsigned ordered_key(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(unsigned key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// u in [0, 1) from (seed, draw index): the splitmix64 finaliser over a Weyl sequence.
__host__ __device__ __forceinline__ float uniform_from_counter(unsigned long long seed, unsigned long long index) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (index + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

struct Best {
    float value;
    int id;
};
__device__ __forceinline__ Best better(Best a, Best b) {
    return (b.value > a.value || (b.value == a.value && b.id < a.id)) ? b : a;
}

// Arg-max of one row by the whole block; result valid in every thread.
__device__ Best block_argmax(const float* __restrict__ row, int vocab, Best* scratch) {
    Best best = {-CUDART_INF_F, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, Best{row[i], i});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other = {__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.id, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = best;
    __syncthreads();
    if (warp == 0) {
        Best b = lane < (int)(blockDim.x >> 5) ? scratch[lane] : Best{-CUDART_INF_F, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other = {__shfl_xor_sync(0xffffffffu, b.value, o), __shfl_xor_sync(0xffffffffu, b.id, o)};
            b = better(b, other);
        }
        if (lane == 0) scratch[32] = b;
    }
    __syncthreads();
    return scratch[32];
}

// One row per thread-block cluster: every block of the cluster takes a share of the row, block 0
// gathers the shares' results through distributed shared memory.  A row of 150k logits is then
// read by eight SMs instead of one.
__global__ void __launch_bounds__(SAMPLE_THREADS) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out,
                                                                int vocab) {
    __shared__ Best scratch[33];
    __shared__ Best shares[16];
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), blocks = cluster.num_blocks();
    const int row = blockIdx.x / blocks;
    const int share = (vocab + blocks - 1) / blocks;
    const int begin = min(vocab, (int)rank * share), end = min(vocab, begin + share);
    Best b = block_argmax(logits + (size_t)row * vocab + begin, end - begin, scratch);
    if (threadIdx.x == 0) {
        if (b.id != 0x7fffffff) b.id += begin;
        cluster.map_shared_rank(shares, 0)[rank] = b;
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        Best best = shares[0];
        for (unsigned r = 1; r < blocks; ++r) best = better(best, shares[r]);
        out[row] = best.id;
    }
}

MRS_EXPORT int mrs_argmax(const float* logits, int* out, int rows, int vocab, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return MRS_BAD_ARGUMENT;
    const unsigned blocks = vocab >= 65536 ? 8 : (vocab >= 16384 ? 4 : 1);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(rows * blocks);
    config.blockDim = dim3(SAMPLE_THREADS);
    config.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = blocks;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&config, argmax_kernel, logits, out, vocab);
    if (e != cudaSuccess) return (int)e;
    MRS_RETURN_LAUNCH_STATUS();
}

// Which elements are kept: keys above `low`, and the first `quota` ids among keys equal to `low`.
struct Cut {
    unsigned low;
    int quota;
};

struct SampleShared {
    Best best[33];
    float f[33];
    unsigned count[256];
    float weight[256];
    int warp_ties[SAMPLE_WARPS];
    int tie_base[SAMPLE_WARPS];
    float warp_weight[SAMPLE_WARPS];
    int sel;
    int remaining;
    float acc;
    int pick_warp;
    float pick_base;
};

// Per-warp exclusive offsets (in id order) of the elements whose key equals `key`.
__device__ void tie_offsets(const float* __restrict__ row, int vocab, int per_warp, unsigned key, SampleShared& s) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int begin = warp * per_warp, end = min(vocab, begin + per_warp);
    int ties = 0;
    for (int i = begin + lane; i < end; i += 32) ties += ordered_key(row[i]) == key;
    ties = (int)warp_sum((float)ties);   // counts stay far below 2^24
    __syncthreads();
    if (lane == 0) s.warp_ties[warp] = ties;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int w = 0; w < SAMPLE_WARPS; ++w) {
            s.tie_base[w] = run;
            run += s.warp_ties[w];
        }
    }
    __syncthreads();
}

// Walks this warp's id range in order and calls f(i, x, kept) for every element.
template <typename F>
__device__ __forceinline__ void walk(const float* __restrict__ row, int vocab, int per_warp, Cut cut, int tie_base,
                                     F f) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int begin = warp * per_warp, end = min(vocab, begin + per_warp);
    int seen = tie_base;
    for (int base = begin; base < end; base += 32) {
        const int i = base + lane;
        const bool live = i < end;
        const float x = live ? row[i] : 0.0f;
        const unsigned key = live ? ordered_key(x) : 0u;
        const bool tie = live && key == cut.low;
        const unsigned tie_mask = __ballot_sync(0xffffffffu, tie);
        const int rank = seen + __popc(tie_mask & ((1u << lane) - 1u));
        seen += __popc(tie_mask);
        const bool kept = live && (key > cut.low || (tie && rank < cut.quota));
        f(i, x, key, kept);
    }
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(
    const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
    const int* __restrict__ draw_index, int* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ SampleShared s;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float temp = temperature[r];
    const int k_raw = top_k[r];
    const float p_raw = top_p[r];

    // Largest logit (also the greedy answer) and a check that the row is finite.
    int bad = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = row[i];
        bad |= !(fabsf(x) <= 3.402823466e38f);
    }
    bad = __syncthreads_or(bad);
    const Best top = block_argmax(row, vocab, s.best);
    if (bad) {
        if (threadIdx.x == 0) out[r] = -1;
        return;
    }
    if (temp == 0.0f || k_raw == 1) {
        if (threadIdx.x == 0) out[r] = top.id;
        return;
    }
    const float inv_t = 1.0f / temp;
    const int per_warp = (((vocab + SAMPLE_WARPS - 1) / SAMPLE_WARPS) + 31) & ~31;

    // ---- top_k: the k-th largest key by count ------------------------------------------------
    Cut cut = {0u, 0x7fffffff};
    if (k_raw > 0 && k_raw < vocab) {
        unsigned prefix = 0u, mask = 0u;
        int remaining = k_raw;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = threadIdx.x; b < 256; b += blockDim.x) s.count[b] = 0u;
            __syncthreads();
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
                const unsigned key = ordered_key(row[i]);
                if ((key & mask) == prefix) atomicAdd(&s.count[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                int left = remaining, chosen = 0;
                for (int b = 255; b >= 0; --b) {
                    if ((int)s.count[b] >= left) { chosen = b; break; }
                    left -= (int)s.count[b];
                }
                s.sel = chosen;
                s.remaining = left;
            }
            __syncthreads();
            prefix |= (unsigned)s.sel << shift;
            mask |= 255u << shift;
            remaining = s.remaining;
            __syncthreads();
        }
        cut.low = prefix;
        cut.quota = remaining;
    }
    tie_offsets(row, vocab, per_warp, cut.low, s);
    int tie_base = s.tie_base[warp];

    // ---- weight of the top_k set ----------------------------------------------------------------
    float local = 0.0f;
    walk(row, vocab, per_warp, cut, tie_base, [&](int, float x, unsigned, bool kept) {
        if (kept) local += expf((x - top.value) * inv_t);
    });
    float total = block_sum(local, s.f);

    // ---- top_p: the key at which the running weight reaches top_p * total -----------------------
    if (p_raw < 1.0f) {
        const float target = p_raw * total;
        unsigned prefix = 0u, mask = 0u;
        float above = 0.0f;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = threadIdx.x; b < 256; b += blockDim.x) { s.weight[b] = 0.0f; s.count[b] = 0u; }
            __syncthreads();
            walk(row, vocab, per_warp, cut, tie_base, [&](int, float x, unsigned key, bool kept) {
                if (kept && (key & mask) == prefix) {
                    atomicAdd(&s.weight[(key >> shift) & 255u], expf((x - top.value) * inv_t));
                    atomicAdd(&s.count[(key >> shift) & 255u], 1u);
                }
            });
            __syncthreads();
            if (threadIdx.x == 0) {
                float acc = above;
                int chosen = -1, lowest = 0;
                for (int b = 255; b >= 0; --b) {
                    if (s.count[b] == 0u) continue;
                    lowest = b;
                    if (acc + s.weight[b] >= target) { chosen = b; break; }
                    acc += s.weight[b];
                }
                if (chosen < 0) {          // rounding left the sum a hair short: the last bin holds the edge
                    chosen = lowest;
                    acc -= s.weight[lowest];
                }
                s.sel = chosen;
                s.acc = acc;
            }
            __syncthreads();
            prefix |= (unsigned)s.sel << shift;
            mask |= 255u << shift;
            above = s.acc;
            __syncthreads();
        }
        const float each = expf((key_value(prefix) - top.value) * inv_t);
        int need = (int)ceilf((target - above) / each);
        if (need < 1) need = 1;
        if (prefix == cut.low) {
            cut.quota = min(cut.quota, need);
        } else {
            cut.low = prefix;
            cut.quota = need;
            tie_offsets(row, vocab, per_warp, cut.low, s);
            tie_base = s.tie_base[warp];
        }
    }

    // ---- inverse CDF over the kept set in id order ------------------------------------------------
    local = 0.0f;
    walk(row, vocab, per_warp, cut, tie_base, [&](int, float x, unsigned, bool kept) {
        if (kept) local += expf((x - top.value) * inv_t);
    });
    local = warp_sum(local);
    __syncthreads();
    if (lane == 0) s.warp_weight[warp] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        float retained = 0.0f;
        for (int w = 0; w < SAMPLE_WARPS; ++w) retained += s.warp_weight[w];
        const float u = uniform_from_counter(seed[r], (unsigned long long)draw_index[r]) * retained;
        float run = 0.0f;
        int chosen = -1, last = 0;
        for (int w = 0; w < SAMPLE_WARPS; ++w) {
            if (s.warp_weight[w] <= 0.0f) continue;
            last = w;
            if (run + s.warp_weight[w] > u) { chosen = w; break; }
            run += s.warp_weight[w];
        }
        if (chosen < 0) {
            chosen = last;
            run -= s.warp_weight[last];
        }
        s.pick_warp = chosen;
        s.pick_base = run;
        s.acc = u;
    }
    __syncthreads();
    if (warp != s.pick_warp) return;
    const float u = s.acc;
    float run = s.pick_base;
    int picked = -1, last_kept = -1;
    walk(row, vocab, per_warp, cut, tie_base, [&](int i, float x, unsigned, bool kept) {
        const float e = kept ? expf((x - top.value) * inv_t) : 0.0f;
        float cum = e;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, cum, o);
            if (lane >= o) cum += up;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, kept && run + cum > u);
        const unsigned kept_mask = __ballot_sync(0xffffffffu, kept);
        if (picked < 0 && hit) picked = i - lane + (__ffs(hit) - 1);
        if (kept_mask) last_kept = i - lane + (31 - __clz(kept_mask));
        run += __shfl_sync(0xffffffffu, cum, 31);
    });
    if (lane == 0) out[r] = picked >= 0 ? picked : last_kept;
}

// One row per block.  temperature, top_k (<= 0: off), top_p, seed and draw_index are per row.
// out[r] = the token, or -1 when the row holds a NaN or an infinity.
MRS_EXPORT int mrs_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                          const float* top_p, const unsigned long long* seed, const int* draw_index, int* out,
                          void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return MRS_BAD_ARGUMENT;
    MRS_LAUNCH(sample_kernel, rows, SAMPLE_THREADS, 0, stream,
        logits, vocab, temperature, top_k, top_p, seed,
                                                                     draw_index, out);
    MRS_RETURN_LAUNCH_STATUS();
}
