// Allocation-free entry point of the routing-plan builder.
//
// This function has no counterpart in the reference.  It exists for callers that must not allocate
// device memory while they run: code inside a memory pool it may not grow, a host thread that is not
// allowed to call into the CUDA allocator (cudaMalloc and cudaFree serialise against the whole device
// and may block behind other work), or a runtime that has handed all free memory to another library.
// `mdt_make_plan` needs (num_slots / 256 + 1) * num_experts ints of scratch, which its Python binding
// allocates per call; this variant keeps that scratch in a fixed array inside the library instead.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch array covers.  Every GPU that loads the library holds the
// array ((MDT_NOALLOC_MAX_SLOTS / 256 + 1) * 64 ints = 256.25 KiB) until the process exits.
#define MDT_NOALLOC_MAX_SLOTS 262144
#define MDT_NOALLOC_MAX_EXPERTS 64

// error codes (negative); 0 = launched
#define MDT_NOALLOC_TOO_LARGE (-20)      // num_slots or num_experts beyond the maxima above
#define MDT_NOALLOC_BAD_DEVICE (-21)     // current device ordinal beyond the table of this library
#define MDT_NOALLOC_NO_SYMBOL (-22)      // cudaGetSymbolAddress failed on the current device
#define MDT_NOALLOC_BAD_ARGUMENT (-23)   // block < 1, negative sizes or a null pointer

// Same results as mdt_make_plan (csrc/api.h): a stable counting sort of `num_slots` expert ids into
// expert groups padded to `block` rows.  All pointers are device pointers supplied by the caller:
//   counts[num_experts], padded_offsets[num_experts + 1], dest_row[num_slots], src_slot[capacity].
// The function enqueues on `stream` and calls no cudaMalloc, cudaFree or any allocating routine.
//
// The scratch array that a call uses is the one of the device that is current when the call is made, so
// `stream` must be a stream of that device.  The first call on a device looks up the address of the
// scratch array for that device (cudaGetSymbolAddress, with that device current); make that first call
// before any stream capture.
// All calls on a device share the one scratch array and it keeps the previous call's contents; every
// entry a call reads is written by that call first, so nothing needs clearing, but two calls that
// overlap on the GPU (different streams without an ordering between them) race on it.
int mdt_make_plan_noalloc(const int* expert_ids, int num_slots, int num_experts, int block, int capacity,
                          int* counts, int* padded_offsets, int* dest_row, int* src_slot, cudaStream_t stream);

// Human-readable text for the codes above (and for 0).
const char* mdt_make_plan_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
