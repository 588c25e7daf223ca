// nib_attention_decode_static: split-KV decode attention for callers that cannot allocate.
//
// This entry point has no counterpart in the reference project.  It exists for hosts that drive
// this library from a context in which device memory may not be requested: a runtime that handed
// the whole GPU to its own pool at start-up, a plug-in that runs inside somebody else's stream
// callback or real-time loop, a sandbox whose policy forbids cudaMalloc after initialisation.
// Such a caller owns its inputs and outputs already, but nib_attention_decode also wants scratch
// memory for the partial results of its key splits and for the arrival counters of its merge, and
// would have to be given an allocation for them.
//
// Here that scratch is a fixed array inside the library itself (file scope, device memory,
// NIB_STATIC_SCRATCH_FLOATS floats plus NIB_STATIC_COUNTERS counters, about 4.1 MiB).  Every GPU
// that loads the library carries the array until the process exits, whether or not this function
// is ever called.  The function allocates nothing: no cudaMalloc, no cudaFree, no library call that
// allocates.  The caller still passes the inputs, the output and the stream.
//
// Sizes.  The call needs  n_rows * n_head * n_splits * (head_dim + 2)  floats and  n_rows * n_head
// counters.  A call that needs more than the array holds is refused with
// NIB_ERR_STATIC_SCRATCH_TOO_SMALL and launches nothing; nib_attention_decode_static_limits()
// reports the two limits so that a caller can test beforehand.
//
// First call on a device.  The array's address on the current device is looked up once, on the
// first call made with that device current (cudaGetSymbolAddress; its error code is returned if it
// fails).  Make that first call outside any stream capture.
//
// Sharing.  All calls use the same array, and the array keeps whatever the last call left in it.
// The function clears the counters (the only part that must start at zero) on `stream` before it
// launches; the partial results are overwritten before they are read.  Two calls whose kernels
// overlap on the GPU (different streams without an order between them, or different host threads
// doing so) race on the array and produce garbage: serialise them.
#pragma once

#include <cuda_runtime.h>

#define NIB_STATIC_SCRATCH_FLOATS (1 << 20)
#define NIB_STATIC_COUNTERS (1 << 14)
#define NIB_ERR_STATIC_SCRATCH_TOO_SMALL (-4)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as nib_attention_decode (see api.h), without the scratch and counter
// pointers.  Returns 0, a positive cudaError_t, or a negative NIB_ERR_* code.
int nib_attention_decode_static(int dtype, const void* q, int ldq, const void* cache, void* out, int ldo,
                                const int* block_table, int max_blocks, const int* rows,
                                const int* row_entry, const int* positions, int n_rows, int n_head,
                                int n_kv_head, int head_dim, int page_size, int n_pages, float scale,
                                int window, int chunk, int n_splits, int* status, cudaStream_t stream);

// The capacity of the built-in scratch: floats for partial results, counters for (row, head) pairs.
void nib_attention_decode_static_limits(long long* max_floats, long long* max_counters);

#ifdef __cplusplus
}
#endif
