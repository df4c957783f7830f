// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference engine: it exists for hosts that embed this
// library and cannot call cudaMalloc while they serve, for one of two reasons. Some hand the whole
// device to an arena of their own at start-up, so a later cudaMalloc simply fails; others run a
// latency-critical loop in which a call that may synchronise the device or take a driver lock
// (cudaMalloc and cudaFree do both) is forbidden by their own rules. Such a caller owns q, the
// cache, the index arrays and the output, but has nowhere to put the kernel's scratch.
//
// ib_attention_decode_noalloc is ib_attention_decode with the split-context partial results kept
// in a fixed array inside the library instead of caller-provided scratch. It computes the same
// values with the same kernels.
//
// Limits and rules:
//  * The array holds IB_DECODE_NOALLOC_MAX_FLOATS float32 values (8 MiB), and every GPU that loads
//    the library holds that much until the process exits. A call needs
//    n_dec * heads * max_slices * (head_dim + 2) values; a larger call is refused with an error
//    message, nothing is launched.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress) with that
//    device current. Make that first call before any stream capture begins on the device.
//  * The function calls no cudaMalloc, cudaFree or any other allocating routine.
//  * All calls share the one array, and it keeps what the last call left in it. Nothing in it has
//    to start at zero: the first kernel writes every entry the second one reads. Two calls whose
//    kernels may overlap on the GPU (different streams, no dependency between them) race on it:
//    order them.
#pragma once
#include <cuda_runtime.h>

#include "kv_view.cuh"

#define IB_DECODE_NOALLOC_MAX_FLOATS (2u * 1024u * 1024u)

// Arguments as ib_attention_decode, without part_o and part_ml. Returns 0, or 1 after storing a
// message that ib_last_error() returns.
extern "C" int ib_attention_decode_noalloc(const void* q, const IbKvView* kv, const int* dec_tokens, int n_dec, const int* positions,
                                           const int* seg_of_token, int window, float scale, void* out, int heads, int max_slices,
                                           int tiles_per_slice, unsigned* status, cudaStream_t stream);
