// Decode attention over the paged cache for callers that must not allocate.
//
// This entry point has no counterpart in the upstream project: upstream's decode
// attention allocates its partial-result buffers with torch on every call
// (paged_attention_kernels.py:245-250).
//
// Who needs it.  The regular entry point, tis_attn_mma, takes its scratch memory (the
// per-split partial outputs and their log-sums) from the caller, and the engine gets that
// memory from torch's caching allocator.  Some callers cannot do that: a host program
// that hands this library raw device pointers and owns all device memory itself under a
// fixed budget, with no allocator the library could call into; and code that runs where a
// device allocation is not permitted at all because it may synchronise the whole device
// or fail once memory is tight -- a latency-critical serving loop after its start-up
// phase, for instance.  For them the scratch lives inside the library.
//
// How.  The scratch is one file-scope  static __device__ __align__(256) float  array of
// TIS_NOALLOC_SCRATCH_FLOATS floats (8 MiB).  Every GPU on which the library is loaded
// holds those 8 MiB until the process exits.  The first call on a device looks the
// array's device address up (cudaGetSymbolAddress, with that device current) and keeps it;
// that first call should therefore come before any stream capture.  Later calls launch
// kernels and nothing else: no cudaMalloc, no cudaFree, no library routine that allocates.
//
// With two to eight splits the kernel merges the splits inside a thread-block cluster and
// needs no scratch at all; the built-in array serves calls with more splits than that.
//
// Limits.  Only decode-style tiles (at most 16 / G rows each, G = query heads per kv
// head).  The call is refused with a clear error (TIS_BAD_SIZE, text in tis_last_error())
// when  n_rows * H * num_splits * (head size + 1)  exceeds TIS_NOALLOC_SCRATCH_FLOATS.
//
// Sharing.  All calls of a process on one device use the same array.  Nothing in it has to
// be cleared between calls: every partial result that the merge step reads is written
// earlier in the same call.  But two calls that overlap on the GPU (different streams, or
// graphs replayed concurrently) write the same memory and corrupt each other: order them
// on one stream.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#define TIS_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and meaning as tis_attn_mma in keys mode, minus the scratch pointer.
// Returns 0 when the kernels were launched on `stream`.
int tis_attn_decode_noalloc(const void* q, int q_stride, void* out, int out_stride, const void* plane,
                            const int* block_table, int bt_stride, int num_pages, const int* positions,
                            const int* row_slot, const int* tile_row0, const int* tile_rows, int num_tiles,
                            int n_rows, int H, int KVH, int page_size, int window, float scale,
                            int keys_per_split, int num_splits, int* fault, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
