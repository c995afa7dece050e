// Paged causal grouped-query attention, plain SIMT version, float32 or bfloat16 storage.
// It is the attention of the 32-bit path and the device-side reference of the tensor-core
// kernels.  Any even head size up to 256, any number of heads and groups, any page size,
// optional sliding window.                               (reference: ops.cu:101-147)
//
// One warp per (token, query head).  Keys are taken 32 at a time: lane j scores key j with a
// full dot product, the warp reduces max and sum once per tile (online softmax, float32), then
// all lanes accumulate the 32 weighted value rows, each lane owning elements lane, lane+32, ...
#include "common.cuh"

#define ATTN_MAX_D 256
#define ATTN_WARPS 4

template <typename T>
__global__ void attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                                      const T* __restrict__ v_cache, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                      T* __restrict__ out, int tokens, int nq, int nkv, int d, int page_size,
                                      int table_width, float scale, int window) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float q_s[ATTN_WARPS][ATTN_MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * ATTN_WARPS + warp;
    if (unit >= (long long)tokens * nq) return;
    const int t = (int)(unit / nq), h = (int)(unit % nq);
    const int g = h / (nq / nkv);
    const int length = positions[t] + 1;
    const int first = window > 0 ? max(0, length - window) : 0;
    const int* pages = block_table + (size_t)seq_of_token[t] * table_width;
    const T* q_row = q + ((size_t)t * nq + h) * d;
    for (int e = lane; e < d; e += 32) q_s[warp][e] = to_float(q_row[e]);
    __syncwarp();

    float acc[ATTN_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < ATTN_MAX_D / 32; ++i) acc[i] = 0.0f;
    float running_max = -CUDART_INF_F, running_sum = 0.0f;

    for (int base = first; base < length; base += 32) {
        const int p = base + lane;
        float score = -CUDART_INF_F;
        if (p < length) {
            const int page = pages[p / page_size];
            const T* k_row = k_cache + (((size_t)page * nkv + g) * page_size + (p % page_size)) * d;
            float dot = 0.0f;
            for (int e = 0; e < d; ++e) dot += q_s[warp][e] * to_float(k_row[e]);
            score = dot * scale;
        }
        const float tile_max = warp_max(score);
        const float new_max = fmaxf(running_max, tile_max);
        const float alpha = expf(running_max - new_max);
        const float prob = p < length ? expf(score - new_max) : 0.0f;
        running_sum = running_sum * alpha + warp_sum(prob);
        running_max = new_max;
#pragma unroll
        for (int i = 0; i < ATTN_MAX_D / 32; ++i) acc[i] *= alpha;
        const int in_tile = min(32, length - base);
        for (int j = 0; j < in_tile; ++j) {
            const float pj = __shfl_sync(0xffffffffu, prob, j);
            const int pj_pos = base + j;
            const int page = pages[pj_pos / page_size];
            const T* v_row = v_cache + (((size_t)page * nkv + g) * page_size + (pj_pos % page_size)) * d;
#pragma unroll
            for (int i = 0; i < ATTN_MAX_D / 32; ++i) {
                const int e = lane + 32 * i;
                if (e < d) acc[i] += pj * to_float(v_row[e]);
            }
        }
    }
    T* o = out + ((size_t)t * nq + h) * d;
    const float inv = 1.0f / running_sum;
#pragma unroll
    for (int i = 0; i < ATTN_MAX_D / 32; ++i) {
        const int e = lane + 32 * i;
        if (e < d) o[e] = from_float<T>(acc[i] * inv);
    }
}

MRS_EXPORT int mrs_attention_simt(int is_bf16, const void* q, const void* k_cache, const void* v_cache,
                                  const int* positions, const int* seq_of_token, const int* block_table,
                                  void* out, int tokens, int nq, int nkv, int d, int page_size,
                                  int table_width, float scale, int window, void* stream) {
    if (tokens <= 0) return 0;
    if (d <= 0 || d > ATTN_MAX_D || nkv <= 0 || nq % nkv) return MRS_BAD_ARGUMENT;
    const long long units = (long long)tokens * nq;
    const unsigned blocks = (unsigned)((units + ATTN_WARPS - 1) / ATTN_WARPS);
    if (is_bf16)
        MRS_LAUNCH(attention_simt_kernel<bf16>, blocks, 32 * ATTN_WARPS, 0, stream,
            (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, positions, seq_of_token, block_table,
            (bf16*)out, tokens, nq, nkv, d, page_size, table_width, scale, window);
    else
        MRS_LAUNCH(attention_simt_kernel<float>, blocks, 32 * ATTN_WARPS, 0, stream,
            (const float*)q, (const float*)k_cache, (const float*)v_cache, positions, seq_of_token, block_table,
            (float*)out, tokens, nq, nkv, d, page_size, table_width, scale, window);
    MRS_RETURN_LAUNCH_STATUS();
}
