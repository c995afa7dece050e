// Embedding, residual-add + RMSNorm, per-head norm + rotary + cache write, SiLU-multiply.
// Every kernel exists for float32 and bfloat16 activations; statistics, angles and the
// residual stream are float32 in both.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// Tokens that the step before sampled and the host has not read yet: ids[rows[i]] = sampled[index[i]].
// A step can then be queued before its predecessor's tokens have reached the host.  A value that is no
// token (the sampler's mark of a row without finite logits, below zero) becomes token 0 here; the host
// sees the mark itself when it reads the step before, and fails the step.
// ---------------------------------------------------------------------------------------------
__global__ void patch_tokens_kernel(int* __restrict__ ids, const int* __restrict__ rows, const int* __restrict__ index,
                                    const int* __restrict__ sampled, int n, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int token = sampled[index[i]];
    ids[rows[i]] = token < 0 || token >= vocab ? 0 : token;
}

MRS_EXPORT int mrs_patch_tokens(int* ids, const int* rows, const int* index, const int* sampled, int n, int vocab, void* stream) {
    if (n <= 0) return 0;
    MRS_LAUNCH(patch_tokens_kernel, (n + 127) / 128, 128, 0, stream, ids, rows, index, sampled, n, vocab);
    MRS_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------
// Embedding: residual[t, :] = float(table[ids[t], :])      (reference: ops.cu:15-18)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ residual, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = table + (size_t)ids[t] * width;
    float* out = residual + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[i] = to_float(row[i]);
}

MRS_EXPORT int mrs_embed(int is_bf16, const void* table, const int* ids, float* residual,
                         int tokens, int width, void* stream) {
    if (tokens <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (is_bf16)
        MRS_LAUNCH(embed_kernel<bf16>, tokens, threads, 0, stream,
            (const bf16*)table, ids, residual, width);
    else
        MRS_LAUNCH(embed_kernel<float>, tokens, threads, 0, stream,
            (const float*)table, ids, residual, width);
    MRS_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------
// Residual add + RMSNorm                                   (reference: ops.cu:62-78)
//   v = residual[src] (+ delta[src]);  if write_back: residual[src] = v
//   out[r] = T(v * rsqrt(mean(v^2) + eps) * weight)
// `rows` (optional) picks the source rows, so the last norm runs only where logits are wanted.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ weight, float eps, T* __restrict__ out,
                                   const int* __restrict__ rows, int width, int write_back) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + src * width;
    const T* del = delta ? delta + src * width : nullptr;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        if (del) v += to_float(del[i]);
        if (write_back && del) res[i] = v;
        sum += v * v;
    }
    const float scale = rsqrtf(block_sum(sum, scratch) / (float)width + eps);
    T* o = out + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        if (del && !write_back) v += to_float(del[i]);
        o[i] = from_float<T>(v * scale * weight[i]);
    }
}

// The same with four elements a step and the row kept in registers between the two passes
// (width a multiple of 4, at most 4 * ROW_CHUNKS * blockDim.x).
#define ROW_CHUNKS 4
template <typename T, int VEC> struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                       const float* __restrict__ weight, float eps, T* __restrict__ out,
                                       const int* __restrict__ rows, int width, int write_back) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + src * width;
    const T* del = delta ? delta + src * width : nullptr;
    float4 v[ROW_CHUNKS];
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < ROW_CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        v[c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < width) {
            v[c] = Vec4<float>::load(res + i);
            if (del) {
                const float4 d = Vec4<T>::load(del + i);
                v[c].x += d.x, v[c].y += d.y, v[c].z += d.z, v[c].w += d.w;
                if (write_back) Vec4<float>::store(res + i, v[c]);
            }
            sum += v[c].x * v[c].x + v[c].y * v[c].y + v[c].z * v[c].z + v[c].w * v[c].w;
        }
    }
    float4 w[ROW_CHUNKS];                  // asked for before the block waits for its sum
#pragma unroll
    for (int c = 0; c < ROW_CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < width) w[c] = Vec4<float>::load(weight + i);
    }
    const float scale = rsqrtf(block_sum(sum, scratch) / (float)width + eps);
    T* o = out + (size_t)r * width;
#pragma unroll
    for (int c = 0; c < ROW_CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < width)
            Vec4<T>::store(o + i, make_float4(v[c].x * scale * w[c].x, v[c].y * scale * w[c].y, v[c].z * scale * w[c].z, v[c].w * scale * w[c].w));
    }
}

MRS_EXPORT int mrs_add_rmsnorm(int is_bf16, float* residual, const void* delta, const float* weight,
                               float eps, void* out, const int* rows, int n_rows, int width,
                               int write_back, void* stream) {
    if (n_rows <= 0) return 0;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    const bool aligned = (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
    if (width % 4 == 0 && aligned && width <= 4 * ROW_CHUNKS * 1024) {
        int vec_threads = ((width + 4 * ROW_CHUNKS - 1) / (4 * ROW_CHUNKS) + 31) / 32 * 32;     // the row fits the block's registers
        if (vec_threads < 64) vec_threads = 64;
        if (is_bf16)
            MRS_LAUNCH(add_rmsnorm_vec_kernel<bf16>, n_rows, vec_threads, 0, stream,
                residual, (const bf16*)delta, weight, eps, (bf16*)out, rows, width, write_back);
        else
            MRS_LAUNCH(add_rmsnorm_vec_kernel<float>, n_rows, vec_threads, 0, stream,
                residual, (const float*)delta, weight, eps, (float*)out, rows, width, write_back);
        MRS_RETURN_LAUNCH_STATUS();
    }
    if (is_bf16)
        MRS_LAUNCH(add_rmsnorm_kernel<bf16>, n_rows, threads, 0, stream,
            residual, (const bf16*)delta, weight, eps, (bf16*)out, rows, width, write_back);
    else
        MRS_LAUNCH(add_rmsnorm_kernel<float>, n_rows, threads, 0, stream,
            residual, (const float*)delta, weight, eps, (float*)out, rows, width, write_back);
    MRS_RETURN_LAUNCH_STATUS();
}

// Plain RMSNorm of activations of type T (no residual): out = T(x * rsqrt(mean(x^2)+eps) * w).
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const float* __restrict__ weight, float eps,
                               T* __restrict__ out, int width) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const T* row = x + (size_t)blockIdx.x * width;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = to_float(row[i]);
        sum += v * v;
    }
    const float scale = rsqrtf(block_sum(sum, scratch) / (float)width + eps);
    T* o = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        o[i] = from_float<T>(to_float(row[i]) * scale * weight[i]);
}

MRS_EXPORT int mrs_rmsnorm(int is_bf16, const void* x, const float* weight, float eps, void* out,
                           int n_rows, int width, void* stream) {
    if (n_rows <= 0) return 0;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (is_bf16)
        MRS_LAUNCH(rmsnorm_kernel<bf16>, n_rows, threads, 0, stream,
            (const bf16*)x, weight, eps, (bf16*)out, width);
    else
        MRS_LAUNCH(rmsnorm_kernel<float>, n_rows, threads, 0, stream,
            (const float*)x, weight, eps, (float*)out, width);
    MRS_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------
// Per-head RMSNorm of q and k, rotary position encoding of q and k, and the write of k and v
// into the paged cache, in one pass over the fused projection output.
//   (reference: split_columns ops.cu:29-32, rms 66-78, rope 79-90, scatter 95-98)
// qkv: [tokens, (nq + 2 nkv) * d]; q_out: [tokens, nq * d];
// caches: [pages, nkv, page_size, d]; slots[t] = page * page_size + offset (or < 0: no write).
// One warp per (token, head).  Norm weights and the frequency table are optional.
// ---------------------------------------------------------------------------------------------
#define MRS_MAX_HEAD_DIM 256

template <typename T>
__global__ void qk_norm_rope_store_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                          T* __restrict__ k_cache, T* __restrict__ v_cache,
                                          const int* __restrict__ positions, const int* __restrict__ slots,
                                          const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                          float eps, const float* __restrict__ inv_freq,
                                          int tokens, int nq, int nkv, int d, int page_size, int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float stage[4][MRS_MAX_HEAD_DIM];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = nq + 2 * nkv;
    const long long unit = (long long)blockIdx.x * 4 + warp;
    if (unit >= (long long)tokens * heads) return;
    const int t = (int)(unit / heads), h = (int)(unit % heads);
    const int kind = h < nq ? 0 : (h < nq + nkv ? 1 : 2);   // 0 q, 1 k, 2 v
    if (kind != 0 && !write_kv) return;
    const T* src = qkv + (size_t)t * heads * d + (size_t)h * d;
    float x[MRS_MAX_HEAD_DIM / 32];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < MRS_MAX_HEAD_DIM / 32; ++i) {
        const int e = lane + 32 * i;
        x[i] = e < d ? to_float(src[e]) : 0.0f;
        sum += x[i] * x[i];
    }
    const float* norm = kind == 0 ? q_norm : (kind == 1 ? k_norm : nullptr);
    if (norm) {
        const float scale = rsqrtf(warp_sum(sum) / (float)d + eps);
#pragma unroll
        for (int i = 0; i < MRS_MAX_HEAD_DIM / 32; ++i) {
            const int e = lane + 32 * i;
            if (e < d) x[i] = x[i] * scale * norm[e];
        }
    }
    if (kind != 2 && inv_freq) {
        const int half = d >> 1;
        const float pos = (float)positions[t];
#pragma unroll
        for (int i = 0; i < MRS_MAX_HEAD_DIM / 32; ++i) {
            const int e = lane + 32 * i;
            if (e < d) stage[warp][e] = x[i];
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < MRS_MAX_HEAD_DIM / 32; ++i) {
            const int e = lane + 32 * i;
            if (e < d) {
                const int j = e < half ? e : e - half;
                float s, c;
                sincosf(pos * inv_freq[j], &s, &c);
                const float partner = stage[warp][e < half ? e + half : e - half];
                x[i] = e < half ? x[i] * c - partner * s : x[i] * c + partner * s;
            }
        }
    }
    T* dst;
    if (kind == 0) {
        dst = q_out + (size_t)t * nq * d + (size_t)h * d;
    } else {
        const int slot = slots[t];
        if (slot < 0) return;
        const int page = slot / page_size, off = slot % page_size;
        const int g = kind == 1 ? h - nq : h - nq - nkv;
        T* base = kind == 1 ? k_cache : v_cache;
        dst = base + (((size_t)page * nkv + g) * page_size + off) * d;
    }
#pragma unroll
    for (int i = 0; i < MRS_MAX_HEAD_DIM / 32; ++i) {
        const int e = lane + 32 * i;
        if (e < d) dst[e] = from_float<T>(x[i]);
    }
}

// The cosines and sines of every token's angles, once a step for all layers that share the
// frequencies: out[t][j] = (cos, sin)(position[t] * inv_freq[j]), float32.
__global__ void rotation_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, long long total,
                                      int half, float2* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float s, c;
    sincosf((float)positions[i / half] * inv_freq[i % half], &s, &c);
    out[i] = make_float2(c, s);
}

MRS_EXPORT int mrs_rotation_table(const int* positions, const float* inv_freq, int tokens, int half, float* out, void* stream) {
    const long long total = (long long)tokens * half;
    if (total <= 0) return 0;
    if (!positions || !inv_freq || !out || ((uintptr_t)out & 15)) return MRS_BAD_ARGUMENT;
    MRS_LAUNCH(rotation_table_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, positions, inv_freq, total, half,
               reinterpret_cast<float2*>(out));
    MRS_RETURN_LAUNCH_STATUS();
}

// The norms, rotation and cache write of above for head sizes 64, 128 and 256.  A lane owns W = VEC / 2 consecutive elements of a head's lower half
// and the W elements that they rotate with in the upper half (two loads of 8 bytes, 16 for float32 heads of 256),
// so the rotation needs no other lane; LANES = d / VEC lanes a head add their squares for the norm, and one load
// of a warp covers 32 / LANES heads.  The cosines and sines come from the step's table (`rotations`
// [tokens][d / 2] of (cos, sin); null: no rotation), so a warp's loads depend on nothing before them; a warp takes
// four such loads of a token's heads at a time, all in flight together, and goes on with the grid's stride.
#define ROPE_LOADS_PER_STEP 4
#define ROPE_BLOCKS_PER_SM 3

// One head's elements of a lane: RMSNorm over the head (the head's lanes add their squares), the rotation of the
// pairs (j, j + d / 2), rounding, store.  `weights`: the norm's weights from this lane's first element on, or null.
template <typename T, int W, int LANES>
__device__ __forceinline__ void store_normed_rotated(const Pack<T, W>& lo, const Pack<T, W>& hi, T* dst, const float* weights, float eps,
                                                     bool rotate, const float (&cs)[W], const float (&sn)[W], unsigned mask) {
    constexpr int half = W * LANES;
    float a[W], b[W];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < W; ++i) {
        a[i] = to_float(lo.v[i]);
        b[i] = to_float(hi.v[i]);
        sum += a[i] * a[i] + b[i] * b[i];
    }
    if (weights) {
#pragma unroll
        for (int offset = LANES / 2; offset > 0; offset >>= 1) sum += __shfl_xor_sync(mask, sum, offset);
        const float scale = rsqrtf(sum / (float)(2 * half) + eps);
        const Pack<float, W> wa = *reinterpret_cast<const Pack<float, W>*>(weights);
        const Pack<float, W> wb = *reinterpret_cast<const Pack<float, W>*>(weights + half);
#pragma unroll
        for (int i = 0; i < W; ++i) {
            a[i] = a[i] * scale * wa.v[i];
            b[i] = b[i] * scale * wb.v[i];
        }
    }
    Pack<T, W> out_lo, out_hi;
#pragma unroll
    for (int i = 0; i < W; ++i) {
        out_lo.v[i] = from_float<T>(rotate ? a[i] * cs[i] - b[i] * sn[i] : a[i]);
        out_hi.v[i] = from_float<T>(rotate ? b[i] * cs[i] + a[i] * sn[i] : b[i]);
    }
    *reinterpret_cast<Pack<T, W>*>(dst) = out_lo;
    *reinterpret_cast<Pack<T, W>*>(dst + half) = out_hi;
}

template <typename T, int VEC, int LANES>
__global__ void __launch_bounds__(256, ROPE_BLOCKS_PER_SM) qk_norm_rope_store_vec_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
    const int* __restrict__ slots, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
    const float2* __restrict__ rotations, int tokens, int nq, int nkv, int page_size, int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int d = VEC * LANES, half = d / 2, W = VEC / 2, G = ROPE_LOADS_PER_STEP, HEADS_PER_LOAD = 32 / LANES;
    const int lane = threadIdx.x & 31;
    const int first = lane % LANES * W;                     // this lane's first element in each half of its head
    // the lanes of this lane's head: they shuffle among themselves, whatever the warp's other heads do
    const unsigned mask = LANES == 32 ? 0xffffffffu : ((1u << (LANES & 31)) - 1u) << (lane / LANES * LANES);
    const int heads = nq + 2 * nkv, heads_per_step = HEADS_PER_LOAD * G;
    const int steps_per_token = (heads + heads_per_step - 1) / heads_per_step;
    const int steps = tokens * steps_per_token;
    const int warps = gridDim.x * (blockDim.x >> 5);
    __shared__ __align__(16) float scales[2][d];            // the head norms' weights of q and k
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        scales[0][e] = q_norm ? q_norm[e] : 1.0f;
        scales[1][e] = k_norm ? k_norm[e] : 1.0f;
    }
    __syncthreads();
    for (int step = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); step < steps; step += warps) {
        const int t = step / steps_per_token;
        const int h0 = (step - t * steps_per_token) * heads_per_step + lane / LANES;      // this lane's head of the first load
        const T* row = qkv + (size_t)t * heads * d + first;
        Pack<T, W> lo[G], hi[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const int h = h0 + g * HEADS_PER_LOAD;
            if (h < heads && (h < nq || write_kv)) {
                lo[g] = *reinterpret_cast<const Pack<T, W>*>(row + (size_t)h * d);
                hi[g] = *reinterpret_cast<const Pack<T, W>*>(row + (size_t)h * d + half);
            }
        }
        float cs[W], sn[W];
        if (rotations && h0 < nq + nkv) {
            const Pack<float2, W> angles = *reinterpret_cast<const Pack<float2, W>*>(rotations + (size_t)t * half + first);
#pragma unroll
            for (int i = 0; i < W; ++i) cs[i] = angles.v[i].x, sn[i] = angles.v[i].y;
        }
        int page = 0, off = 0;
        bool writes = false;                                // does this token have a place in the cache?
        if (write_kv && h0 + (G - 1) * HEADS_PER_LOAD >= nq) {
            const int slot = slots[t];
            writes = slot >= 0;
            if (writes) page = slot / page_size, off = slot - page * page_size;
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const int h = h0 + g * HEADS_PER_LOAD;
            if (h >= heads) continue;
            if (h >= nq) {
                if (!writes) continue;
                const bool is_k = h < nq + nkv;
                T* dst = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + (is_k ? h - nq : h - nq - nkv)) * page_size + off) * d + first;
                if (!is_k) {                                // v: as it came
                    *reinterpret_cast<Pack<T, W>*>(dst) = lo[g];
                    *reinterpret_cast<Pack<T, W>*>(dst + half) = hi[g];
                    continue;
                }
                store_normed_rotated<T, W, LANES>(lo[g], hi[g], dst, k_norm ? scales[1] + first : nullptr, eps, rotations != nullptr, cs, sn, mask);
            } else {
                store_normed_rotated<T, W, LANES>(lo[g], hi[g], q_out + ((size_t)t * nq + h) * d + first, q_norm ? scales[0] + first : nullptr, eps,
                                                  rotations != nullptr, cs, sn, mask);
            }
        }
    }
}

template <typename T, int VEC, int LANES>
static int launch_rope_vec(const void* qkv, void* q_out, void* k_cache, void* v_cache, const int* slots, const float* q_norm,
                           const float* k_norm, float eps, const float* rotations, int tokens, int nq, int nkv, int page_size,
                           int write_kv, void* stream) {
    const int heads_per_step = 32 / LANES * ROPE_LOADS_PER_STEP;
    const long long steps = (long long)tokens * ((nq + 2 * nkv + heads_per_step - 1) / heads_per_step);
    if (steps > 0x7fffffffLL) return MRS_BAD_ARGUMENT;
    const long long want = (steps + 7) / 8;
    const long long most = (long long)mrs_sm_count() * 2 * ROPE_BLOCKS_PER_SM;
    MRS_LAUNCH((qk_norm_rope_store_vec_kernel<T, VEC, LANES>), (unsigned)(want > most ? most : want), 256, 0, stream, (const T*)qkv,
               (T*)q_out, (T*)k_cache, (T*)v_cache, slots, q_norm, k_norm, eps, reinterpret_cast<const float2*>(rotations), tokens, nq,
               nkv, page_size, write_kv);
    MRS_RETURN_LAUNCH_STATUS();
}

// `rotations` (or null): the step's table of `mrs_rotation_table` for these positions and frequencies; with it (or without
// any rotation) heads of 64, 128 and 256 elements take the vector kernel.
MRS_EXPORT int mrs_qk_norm_rope_store(int is_bf16, const void* qkv, void* q_out, void* k_cache, void* v_cache,
                                      const int* positions, const int* slots, const float* q_norm,
                                      const float* k_norm, float eps, const float* inv_freq, const float* rotations, int tokens,
                                      int nq, int nkv, int d, int page_size, int write_kv, void* stream) {
    if (tokens <= 0) return 0;
    if (d <= 0 || d > MRS_MAX_HEAD_DIM || (d & 1)) return MRS_BAD_ARGUMENT;
    const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)rotations) & 31) == 0;
    if (aligned && (d == 64 || d == 128 || d == 256) && (rotations || !inv_freq)) {
#define MRS_ROPE_VEC(T, V, L)                                                                                      \
    return launch_rope_vec<T, V, L>(qkv, q_out, k_cache, v_cache, slots, q_norm, k_norm, eps, rotations, tokens, nq, nkv, \
                                    page_size, write_kv, stream)
        if (is_bf16) {
            if (d == 64) MRS_ROPE_VEC(bf16, 8, 8);
            if (d == 128) MRS_ROPE_VEC(bf16, 8, 16);
            MRS_ROPE_VEC(bf16, 8, 32);
        } else {
            if (d == 64) MRS_ROPE_VEC(float, 4, 16);
            if (d == 128) MRS_ROPE_VEC(float, 4, 32);
            MRS_ROPE_VEC(float, 8, 32);
        }
#undef MRS_ROPE_VEC
    }
    const long long units = (long long)tokens * (nq + 2 * nkv);
    const unsigned blocks = (unsigned)((units + 3) / 4);
    if (is_bf16)
        MRS_LAUNCH(qk_norm_rope_store_kernel<bf16>, blocks, 128, 0, stream,
            (const bf16*)qkv, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, positions, slots, q_norm, k_norm,
            eps, inv_freq, tokens, nq, nkv, d, page_size, write_kv);
    else
        MRS_LAUNCH(qk_norm_rope_store_kernel<float>, blocks, 128, 0, stream,
            (const float*)qkv, (float*)q_out, (float*)k_cache, (float*)v_cache, positions, slots, q_norm, k_norm,
            eps, inv_freq, tokens, nq, nkv, d, page_size, write_kv);
    MRS_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------
// SiLU-multiply over the fused gate/up projection: out[t, i] = silu(gu[t, i]) * gu[t, I + i]
//   (reference: ops.cu:91-94)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total, int inter, int block) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / inter;
        const int c = (int)(i % inter);
        // all gate columns, then all up columns; or blocks of gate columns each followed by its up columns
        const long long gate_at = block ? (long long)(c / block) * 2 * block + c % block : c;
        const long long up_at = block ? gate_at + block : (long long)inter + c;
        const float g = to_float(gate_up[t * 2 * inter + gate_at]);
        const float u = to_float(gate_up[t * 2 * inter + up_at]);
        out[i] = from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

// The same with one 16-byte vector a thread and token (width and block multiples of VEC).  A thread keeps its
// columns and walks down the tokens of the grid's second dimension, so no index is divided in the loop; when the
// result is rounded to bfloat16 the exponential and the quotient are the fast ones.
template <typename T, int VEC>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int tokens, int inter, int block) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (c >= inter) return;
    const int gate_at = block ? c / block * 2 * block + c % block : c;
    const int up_at = block ? gate_at + block : inter + c;
    for (int t = blockIdx.y; t < tokens; t += gridDim.y) {
        const T* row = gate_up + (size_t)t * 2 * inter;
        const Pack<T, VEC> g = *reinterpret_cast<const Pack<T, VEC>*>(row + gate_at);
        const Pack<T, VEC> u = *reinterpret_cast<const Pack<T, VEC>*>(row + up_at);
        Pack<T, VEC> o;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const float gj = to_float(g.v[j]);
            // the 32-bit path takes the accurate exponential and quotient, as the scalar kernel does: the same bits either way
            const float silu = sizeof(T) == 2 ? __fdividef(gj, 1.0f + __expf(-gj)) : gj / (1.0f + expf(-gj));
            o.v[j] = from_float<T>(silu * to_float(u.v[j]));
        }
        *reinterpret_cast<Pack<T, VEC>*>(out + (size_t)t * inter + c) = o;
    }
}

MRS_EXPORT int mrs_silu_mul(int is_bf16, const void* gate_up, void* out, int tokens, int inter, int block, void* stream) {
    const long long total = (long long)tokens * inter;
    if (total <= 0) return 0;
    if (block < 0 || (block && inter % block)) return MRS_BAD_ARGUMENT;
    const int threads = 256;
    const bool aligned = (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0;
    const int vec = is_bf16 ? 8 : 4;
    if (inter % vec == 0 && block % vec == 0 && aligned) {
        const dim3 grid((unsigned)((inter / vec + threads - 1) / threads), (unsigned)(tokens < 65535 ? tokens : 65535));
        if (is_bf16)
            MRS_LAUNCH((silu_mul_vec_kernel<bf16, 8>), grid, threads, 0, stream, (const bf16*)gate_up, (bf16*)out, tokens, inter, block);
        else
            MRS_LAUNCH((silu_mul_vec_kernel<float, 4>), grid, threads, 0, stream, (const float*)gate_up, (float*)out, tokens, inter, block);
        MRS_RETURN_LAUNCH_STATUS();
    }
    long long want = (total + threads - 1) / threads;
    const long long most = (long long)mrs_sm_count() * 16;
    const unsigned blocks = (unsigned)(want > most ? most : want);
    if (is_bf16)
        MRS_LAUNCH(silu_mul_kernel<bf16>, blocks, threads, 0, stream, (const bf16*)gate_up, (bf16*)out, total, inter, block);
    else
        MRS_LAUNCH(silu_mul_kernel<float>, blocks, threads, 0, stream, (const float*)gate_up, (float*)out, total, inter, block);
    MRS_RETURN_LAUNCH_STATUS();
}

MRS_EXPORT const char* mrs_error_string(int code) {
    if (code == MRS_BAD_ARGUMENT) return "kernel launcher refused its arguments (size outside what the kernel supports)";
    return cudaGetErrorString((cudaError_t)code);
}
