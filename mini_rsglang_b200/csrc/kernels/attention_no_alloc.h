// Split attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (mirthfulLee/mini-rsglang allocates a
// fresh buffer for every intermediate result).  It exists for programs that embed this library
// where device allocation is off limits: a host that hands the library a fixed set of buffers
// and forbids cudaMalloc (for instance because another component owns the whole device heap, or
// because an allocation would stall a latency-critical loop), or a
// plain C caller that has no allocator of this engine at hand.  Such a caller still passes its
// inputs and its output; only the scratch memory that the split kernel needs between its two
// launches comes from the library itself.
//
// The scratch is one file-scope array in device memory of
//     MRS_ATTENTION_STATIC_SCRATCH_FLOATS floats (16 MiB),
// which every GPU that loads the library holds until the process exits.  A call needs
//     tiles * kv_heads * splits * 16 * (head_dim + 2) floats
// (ask mrs_attention_mma_scratch_floats); a call that needs more is refused with
// MRS_STATIC_SCRATCH_TOO_SMALL and launches nothing.
//
// The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
// raises the kernels' shared-memory limit; make that first call outside any stream capture.
// That set-up runs under a lock, so two host threads may make a device's first call at the same
// time (their launches still must not overlap on the GPU, see below).
// The function itself calls no cudaMalloc, cudaFree or any allocating routine.
//
// All calls share the one array and it keeps the last call's contents.  Nothing in it has to be
// zero at the start (every value that is read was written by the same call), but two calls that
// overlap on the GPU (different streams, or the same stream from two host threads without
// ordering) would write the same floats: run them one after the other.
#pragma once

#define MRS_ATTENTION_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define MRS_STATIC_SCRATCH_TOO_SMALL (-3)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as mrs_attention_mma_keys_mode, without the scratch pointer:
//   q [tokens, nq * head_dim], caches [pages, nkv, page_size, head_dim], out like q (bfloat16);
//   positions [tokens], block_table [sequences, table_width], tiles [num_tiles][4]
//   = (sequence, first token, tokens, 0), each of at most 16 / (nq / nkv) tokens (int32);
//   splits >= 1 CTAs share the keys of a tile.  Returns 0, a CUDA error code, or a negative
//   refusal (mrs_attention_mma_error_string explains all of them).
int mrs_attention_mma_keys_mode_static_scratch(const void* q, const void* k_cache, const void* v_cache,
                                               const int* positions, const int* block_table, int table_width,
                                               const int* tiles, int num_tiles, void* out, int nq, int nkv,
                                               int page_size, float scale, int window, int splits, void* stream);

const char* mrs_attention_mma_error_string(int code);

#ifdef __cplusplus
}
#endif
