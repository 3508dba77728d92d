// Split-key decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for hosts
// of this library that cannot call cudaMalloc at the time they need attention: code
// running inside a CUDA-graph capture (allocation is illegal there), a real-time loop
// that may not take the allocator's locks or its unbounded latency, a process whose
// whole device-memory budget was handed to another allocator at start-up, or a thin
// C shim without any allocator of its own.  They still pass inputs and outputs; what
// they cannot provide is the kernel's scratch (the partial results of the key splits
// and the per-tile arrival counters), so that scratch lives in a fixed array inside
// the library image instead.
//
// Limits and rules:
//  * The array is BSPEC_NOALLOC_SCRATCH_BYTES (16 MiB + 64 KiB) of device memory per GPU
//    that loads the library, held until the process exits.
//  * A call needs n_tokens * Hq * n_splits * (head_dim + 2) floats of it and
//    n_entries * Hkv * row_tiles counters; a call that needs more than
//    BSPEC_NOALLOC_MAX_PARTIAL_FLOATS floats or BSPEC_NOALLOC_MAX_COUNTERS counters is
//    refused with BSPEC_NOALLOC_TOO_LARGE and nothing is launched.
//  * The first call on each device looks the array's device address up once
//    (cudaGetSymbolAddress, with that device current).  Make that first call outside
//    of any stream capture; later calls only enqueue work on `stream`.
//  * All calls share the one array and it keeps the previous call's contents.  The
//    counters are cleared on the stream at the start of every call; the partial results
//    are fully rewritten before they are read.  Two calls whose work overlaps on the GPU
//    (different streams, or graphs replayed concurrently) race on it: serialise them.
//  * Only requests with few new tokens (q_len <= 16 / (Hq / Hkv), i.e. decode steps) are
//    served; head_dim must be 64, 128 or 256; bfloat16 only.
#pragma once
#include <cuda_runtime.h>

#define BSPEC_NOALLOC_MAX_PARTIAL_FLOATS (4u * 1024u * 1024u)
#define BSPEC_NOALLOC_MAX_COUNTERS (16u * 1024u)
#define BSPEC_NOALLOC_SCRATCH_BYTES (BSPEC_NOALLOC_MAX_PARTIAL_FLOATS * 4u + BSPEC_NOALLOC_MAX_COUNTERS * 4u)

#define BSPEC_NOALLOC_OK 0
#define BSPEC_NOALLOC_TOO_LARGE (-1)      // the sizes need more scratch than the array holds
#define BSPEC_NOALLOC_BAD_ARGUMENT (-2)   // unsupported head_dim, group size, split count or q_len
#define BSPEC_NOALLOC_SETUP_FAILED (-3)   // the array's address could not be obtained on this device

#ifdef __cplusplus
extern "C" {
#endif
// Causal attention of the step's (decode) tokens over their requests' paged keys and values.
// q: bfloat16 rows of `q_row_stride` elements, the Hq query heads first; out: bfloat16 [n_tokens, Hq * head_dim];
// cache: one layer's pages [pages][2][Hkv][page_size][head_dim]; the int arrays as in the step's metadata.
// Returns BSPEC_NOALLOC_OK, one of the codes above, or a positive cudaError_t of the launch.  If `message` is not
// null, a one-line description of a refusal is written to it (at most `message_len` bytes).
int bspec_attention_decode_noalloc(const void* q, long long q_row_stride, void* out, const void* cache,
                                   const int* qo_indptr, const int* positions, const int* tok_entry,
                                   const int* kv_indptr, const int* kv_indices, int n_entries, int n_tokens,
                                   int max_q_len, int Hq, int Hkv, int head_dim, int page_size, float scale,
                                   int window, int n_splits, cudaStream_t stream, char* message, int message_len);
#ifdef __cplusplus
}
#endif
