// Decode attention over the paged cache without any allocation, for callers that cannot
// allocate device memory when they call.
//
// This entry point has no counterpart in the reference project (which has no kernels of
// its own and lets PyTorch allocate whatever its library calls need).
//
// Who needs it. The regular entry point, pae_paged_attention_decode, takes a scratch
// buffer for the per-slice partial results, and somebody has to allocate that buffer.
// Three kinds of callers of this library cannot do that at call time:
//   - a serving process that gave the cache pool everything that was left of device
//     memory at start-up: a later cudaMalloc fails, or succeeds only by chance;
//   - a latency-bound decode loop: cudaMalloc and cudaFree synchronise the device and
//     stall the stream they were supposed to feed;
//   - a host program that uses these libraries through their C symbols alone, without
//     torch, and so has no caching allocator to ask.
// For them the scratch lives in a fixed array inside the library.
//
// What it costs and where it stops. The array holds PAE_NOALLOC_SCRATCH_FLOATS floats
// (8 MiB) in the global memory of every GPU on which the library is loaded, until the
// process exits. A call that needs more scratch (requests x heads x slices x (head_dim + 2)
// floats) is refused with an error message; nothing is launched.
//
// Sharing. Every call uses the same array, and the array keeps what the last call left in
// it. Nothing in it has to start at zero: each call writes every partial result that its
// merge step reads before it reads it. Two calls that overlap on the GPU (different
// streams, or different host threads on one device) race on the array and must be
// ordered by the caller.
//
// Set-up. The first call on a device looks up the device address of the array
// (cudaGetSymbolAddress, with that device current) and keeps it; it should be made
// before any stream capture begins on that device. No call allocates: no cudaMalloc,
// cudaFree, or allocating library routine is used.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Floats of scratch held inside the library (8 MiB).
#define PAE_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

// Same arguments and result as pae_paged_attention_decode, without `scratch`:
// out [tokens, heads, d] bfloat16 for every request that brings exactly one token.
// Returns 0, or a non-zero code after storing a message for pae_last_error().
int pae_paged_attention_decode_noalloc(void* out, const void* qkv, const void* keys, const void* values,
                                       const int* block_table, int table_width, const int* q_start, const int* kv_len,
                                       int seqs, int heads, int kv_heads, int d, int page_size, float scale, int window,
                                       int slice_keys, int max_slices, void* stream);

// The most floats of scratch a call may need (PAE_NOALLOC_SCRATCH_FLOATS).
long long pae_noalloc_scratch_capacity(void);

const char* pae_last_error(void);

#ifdef __cplusplus
}
#endif
