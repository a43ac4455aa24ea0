// ullm_decode_attention_static: decode attention for callers that cannot allocate.
//
// This entry point has no counterpart in the reference (izmttk/ullm): it exists
// for hosts that embed this library where device allocation is off limits: code
// that runs under a memory budget fixed at start-up, inside another framework's
// allocator-free section, or behind a plug-in interface that hands in buffers
// and forbids cudaMalloc.  The regular entry point, ullm_decode_attention, needs
// a scratch buffer for the partial results of its key-range splits and leaves
// its allocation to the caller; this variant keeps that scratch in a fixed array
// inside the library instead.
//
// What the caller passes: the same inputs and the same output as for
// ullm_decode_attention, minus the scratch pointer.  What it must know:
//
//   * The scratch is one file-scope device array of
//     ULLM_STATIC_SCRATCH_FLOATS floats (4 MiB).  Every GPU on which the
//     library is loaded holds it from load until the process exits.
//   * A call with two or more splits needs batch * num_q * num_splits *
//     (head_dim + 2) floats (ullm_decode_attention_scratch_floats).  A call
//     that needs more is refused with ULLM_ERR_SCRATCH_TOO_LARGE (5) and
//     launches nothing; use fewer splits, a smaller batch, or the regular
//     entry point.  With num_splits == 1 no partials exist, the array is not
//     touched and any batch is taken.
//   * The first call on a device looks up the array's device address (once per
//     device, with that device current).  Make that first call before any
//     stream capture begins on that device.  The address is the CURRENT
//     device's: `stream` must belong to the device that is current at the call.
//   * All calls share the one array and it keeps the previous call's contents.
//     Nothing in it has to start at zero: every element a call reads was
//     written by the same call.  Two calls that overlap on the GPU (different
//     streams, or graphs replayed side by side) race on it; order them.
//   * It calls no cudaMalloc, no cudaFree and no library routine that allocates.
//
// Returns 0 on success, otherwise one of the ULLM_ERR_* codes.
#pragma once

#define ULLM_STATIC_SCRATCH_FLOATS (1 << 20)
#define ULLM_ERR_SCRATCH_TOO_LARGE 5

#ifdef __cplusplus
extern "C" {
#endif

int ullm_decode_attention_static(const void* q, long long q_row_stride, const void* k_cache, const void* v_cache,
                                 const int* block_table, int max_pages, const int* req_slots, const int* kv_len,
                                 void* out, int batch, int num_q, int num_kv, int head_dim, int page_size, int window,
                                 float scale, int num_splits, long long num_pages, int* status, void* stream);

// The limit, for callers that want to size their batches against it.
long long ullm_decode_attention_static_capacity(void);

#ifdef __cplusplus
}
#endif
