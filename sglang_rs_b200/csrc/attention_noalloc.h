// srb_paged_attention_noalloc: split-key paged attention for callers that cannot allocate.
//
// This entry point has no counterpart in the reference; it exists for programs that embed
// this library where device allocation is off the table: a host that handed all device
// memory to its own pools at start-up, a plug-in that runs inside someone else's allocator
// and must not call cudaMalloc behind its back, or code that runs where an allocation would
// synchronise the device at a bad moment.  Such a caller still owns its inputs and outputs
// (q, the page pools, the block table, out); what it cannot provide is the scratch that the
// split run needs for its partial results.  Here that scratch is a fixed array inside the
// library's device image.
//
// Limits and rules:
//  * The array holds SRB_NOALLOC_SCRATCH_FLOATS floats (8 MiB).  Every GPU on which the
//    library is loaded carries it until the process exits.
//  * A call needs rows * n_q * max_splits * (head_dim + 2) floats; a larger request is refused
//    with a message and nothing is launched.
//  * The first call on a device looks up the array's device address (once per device, with
//    that device current).  Make that first call before any stream capture begins.
//  * All calls share the one array and it keeps whatever the last call left.  Nothing in it
//    has to start at zero: each call writes every partial it later reads.  Two calls whose
//    kernels may run at the same time (different streams, different threads) race on it;
//    keep calls to this entry point ordered on the device.
//  * max_splits must cover the row with the most keys: positions[r] / split_size + 1 (fewer with a
//    window).  The host cannot see positions that live on the device, so a row that needs more is
//    reported from the device instead: bit SRB_FLAG_TOO_FEW_SPLITS (16) is set in *error_word and the
//    row's output lacks its newest keys.  Rows with a negative position are padding and are left alone.
//  * It calls no cudaMalloc, cudaFree or other allocating routine, of CUDA or of any library.
//
// Arguments are those of srb_paged_attention without the two scratch pointers; split_size
// must be positive.  Returns 0, or a negative status with the text in srb_last_error().
#pragma once

#define SRB_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif
int srb_paged_attention_noalloc(const void* q, const void* k_pool, const void* v_pool, void* out,
                                const int* positions, const int* row_request, const int* block_table,
                                int table_stride, int rows, int n_q, int n_kv, int head_dim, int page_size,
                                int num_pages, int window, int split_size, int max_splits, float scale,
                                int* error_word, int dtype, void* stream);
int srb_noalloc_scratch_floats(void);
const char* srb_last_error(void);
#ifdef __cplusplus
}
#endif
