// Split-KV decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for hosts that drive
// the library through its C symbols and have no allocator to offer.
//
// thn_attention_decode_bf16 needs float32 scratch for the partial results of its key
// splits, and leaves it to the caller to provide.  Some callers cannot: a process that
// has handed every spare byte of the GPU to a cache or to another runtime at start-up,
// so that cudaMalloc would fail or stall the device in the middle of serving; a plug-in
// called from a thread that must not block on the driver's allocation lock; a C host
// without any pool of its own.  For them this variant keeps the scratch inside the
// library, in a fixed array in device memory that every GPU holds from the moment it
// loads the library until the process exits.
//
// Limits and rules:
//  * The array holds THN_NO_ALLOC_SCRATCH_FLOATS floats (4 MiB).  A call needs
//    n_seqs * n_q * n_splits * (head_dim + 2) floats when n_splits > 1 and none otherwise;
//    a call that needs more is refused with THN_BAD_ARGUMENT and a message, nothing runs.
//  * The first call on each device looks up the array's device address (with that device
//    current).  It launches nothing extra, but it is a runtime query: make the first call
//    on a device before any stream capture begins on it.
//  * The call allocates nothing: no cudaMalloc, no cudaFree, no library routine that does.
//  * All calls share the one array, and it keeps whatever the last call left.  Nothing in
//    it has to start at zero: every split writes its own partial (an empty split writes
//    "no keys") before the merge reads it.  Two calls that overlap on the GPU, on different
//    streams, would write the same array and race: keep calls to this entry point on one
//    stream, or order them with events.
//
// Inputs and outputs are the caller's, exactly as for thn_attention_decode_bf16: q and out
// [n_seqs, n_q * head_dim] bfloat16, one row per sequence; row_slot and row_pos int32
// [n_seqs]; the cache entry by its base pointer, block table and geometry; err an optional
// device error word.
#pragma once

#include <cuda_runtime.h>

#define THN_NO_ALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default"))) int thn_attention_decode_bf16_no_alloc(
    void* out, const void* q, const int* row_slot, const int* row_pos, const void* kv_base, const int* block_table,
    int bt_stride, int n_kv, int page_size, int head_dim, int n_seqs, int n_q, int n_splits, float scale, int window,
    int* err, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
