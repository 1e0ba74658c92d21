// Allocation-free decode attention entry point (exported C symbol).
//
// This entry point has no counterpart in the reference implementation.
//
// Who it is for: code that may not allocate device memory at the moment it needs
// paged decode attention.  Examples are a host thread that runs inside somebody
// else's memory pool and must not touch cudaMalloc (an allocation there can
// synchronise the whole device or fail under a pool that already owns all free
// memory), a latency-critical serving loop where every allocation is forbidden after
// start-up, and plain C or ctypes callers that have raw device pointers but no torch
// allocator to lend this library a workspace.
//
// What it does: the same computation as the extension's `decode_attention` with an
// explicit split count, i.e. split-KV paged decode attention followed by the merge
// of the splits.  The per-split partial outputs and their log-sum-exp values, which
// the regular entry point keeps in a workspace tensor, live here in two file-scope
// `static __device__` arrays inside the shared object:
//     FC_NOALLOC_MAX_PART_FLOATS (2 Mi floats = 8 MiB)  partial outputs  [B, Hq, splits, D]
//     FC_NOALLOC_MAX_LSE_FLOATS  (64 Ki floats = 256 KiB) log-sum-exp    [B, Hq, splits]
// Every GPU on which the library is loaded holds these 8.25 MiB until the process exits.
//
// Rules for callers
//  * Inputs and outputs are the caller's: q [B, Hq, D] bf16, k_cache / v_cache
//    [num_blocks, Hkv, block_size, D] bf16, block_tables [B, max_blocks] int32,
//    context_lens [B] int32, out [B, Hq, D] bf16, all on the current device.
//  * B * Hq * splits * D must not exceed FC_NOALLOC_MAX_PART_FLOATS and B * Hq * splits must
//    not exceed FC_NOALLOC_MAX_LSE_FLOATS; larger requests are rejected with
//    FC_NOALLOC_TOO_LARGE and a message, nothing is launched.
//  * The first call on a device resolves the device addresses of the two arrays
//    (cudaGetSymbolAddress with that device current) and remembers them.  Make that
//    first call before any stream capture begins.
//  * All calls share the two arrays, and the arrays keep whatever the previous call left.
//    Nothing in them has to start at zero: every cell that the merge reads is written
//    by the attention kernel of the same call first, also when one of its bounded waits
//    runs out (that split is then written with weight zero and `status` receives the code;
//    pass a status word if such a call must not go unnoticed).  Two calls whose kernels
//    overlap on the GPU (different streams, no ordering between them) race on the arrays.
//  * No cudaMalloc, cudaFree or allocating library routine is called.
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FC_NOALLOC_MAX_PART_FLOATS (2u << 20)
#define FC_NOALLOC_MAX_LSE_FLOATS (64u << 10)

enum {
  FC_NOALLOC_OK = 0,
  FC_NOALLOC_BAD_ARGUMENT = 1,   // null pointer, unsupported head_dim / group size / block size, splits < 1
  FC_NOALLOC_TOO_LARGE = 2,      // the request needs more scratch than the static arrays hold
  FC_NOALLOC_CUDA_ERROR = 3,     // a CUDA call failed (message says which)
};

// Returns one of the codes above.  `err` (may be NULL) receives a NUL-terminated message of at
// most `err_len` bytes on failure.  `stream` is a cudaStream_t (NULL = the default stream);
// `status` (may be NULL) is a device word that receives a non-zero code if a bounded wait in
// the kernel runs out or a block-table entry is out of range.
int fc_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                const int* context_lens, void* out, int B, int Hq, int Hkv, int D, int block_size,
                                int max_blocks, int num_blocks, int splits, float scale, unsigned int* status,
                                void* stream, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
