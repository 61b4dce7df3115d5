// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in LockStep; it exists for hosts that
// embed the library without torch's allocator and cannot call cudaMalloc where
// the engine's step function would: a process that handed all device memory to
// a pool of its own at start-up (a later cudaMalloc fails or eats into another
// tenant's share), or a latency-bound loop in which cudaMalloc's implicit
// device-wide synchronisation is not acceptable.
//
// ls_attention_decode_noalloc does what ls_attention_decode followed by
// ls_attention_combine do (split-KV attention of single query tokens over the
// paged cache, then the fold of the splits in ascending order), but keeps the
// partial results in a fixed array that lives in the library's device image
// instead of in buffers the caller allocates.  The caller still passes every
// input and the output.
//
// Limits and rules:
//  - The scratch holds LS_NOALLOC_SCRATCH_FLOATS floats (8 MiB).  A call needs
//    n_slots * nq * (d + 2) of them, where n_slots is one more than the largest
//    slot a work item names; a larger call is refused with LS_E_NOALLOC_TOO_LARGE
//    and launches nothing.  The work and combine items live on the device, so the
//    host cannot read them: the kernels themselves compare every slot an item
//    names with n_slots, record LS_DEV_ROW_RANGE in the error word for one that
//    lies outside, and skip it, so a wrong item cannot write past the array.
//    Every GPU that loads the library holds these 8 MiB until the process exits.
//  - The first call on a device looks up the scratch's device address (once per
//    device, with that device current).  Make that first call outside any
//    stream capture.
//  - It calls no cudaMalloc, cudaFree or other allocating routine.
//  - All calls share the one array, and it keeps what the last call left.  The
//    split kernel overwrites every float a call's combine reads, so nothing has
//    to start at zero.  Two calls that overlap on the GPU (different streams,
//    or different host threads without ordering) race on the array: order them.
#pragma once

#include <cuda_runtime.h>

#define LS_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define LS_E_NOALLOC_TOO_LARGE (-10)   // the call needs more scratch than the array holds
#define LS_E_NOALLOC_SETUP (-11)       // the scratch's device address could not be obtained

#ifdef __cplusplus
extern "C" {
#endif

// q, out: [tokens, nq, d]; pages: [num_pages, 2, nkv, page_size, d] (dtype: 0
// float32, 1 bfloat16); work: n_work items of 8 ints and combine: n_combine
// items of 4 ints, as for ls_attention_decode and ls_attention_combine;
// n_slots: number of partial slots the work items use.  Returns 0, a negative
// LS_E_* refusal, or the positive cudaError_t of a failed launch.
int ls_attention_decode_noalloc(const void* q, const void* pages, void* out, int dtype,
                                const int* work, int n_work, const int* combine, int n_combine,
                                int n_slots, const int* block_table, int table_stride, int nq,
                                int nkv, int d, int page_size, int num_pages, int window,
                                float scale, int* err, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
