// An entry point for callers that must not allocate device memory.
//
// This has no counterpart in hoenza/DELTA.  It exists for programs that embed this library
// in a place where cudaMalloc is off limits: a plug-in that runs inside somebody else's
// capture or real-time loop, a host that has handed all device memory to one arena and
// forbids further driver allocations, a process whose allocator may not be re-entered from
// the thread that calls us.  The split-key decode attention normally needs a scratch buffer
// for the partial results of its blocks, which the caller allocates (in this package: torch).
// dk_attention_decode_static does the same work with the scratch inside the library.
#pragma once
#include <cuda_runtime.h>
#include "attention_params.h"

#ifdef __cplusplus
extern "C" {
#endif

// Floats of built-in scratch (2 Mi floats = 8 MiB, held by every GPU that loads the library
// until the process exits).  A launch needs rows * H * splits * (hd + 2) floats when
// splits > 1 and none when splits == 1.
#define DK_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

// Same arguments, same kernels and same result as dk_attention_decode, except that
// p->scratch is ignored: the partial results of the blocks go to an array that lives in the
// library.  It calls no cudaMalloc, cudaFree or any other allocating routine.
//
//  * A launch that needs more than DK_STATIC_SCRATCH_FLOATS floats is refused with
//    DK_ERR_ARG (-1) and a message in dk_last_error(); use fewer splits or rows.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress)
//    and keeps it; make that first call before any stream capture begins.  "The device" is
//    the one that is current when the call is made: make the stream's device current first.
//  * All calls share the one array per device.  It still holds what the last call left, but
//    nothing has to be cleared: every block writes its own slot before the merge reads it.
//    Two calls that overlap on the GPU (different streams) would write the same slots and
//    race; keep calls on one stream or order them yourself.
int dk_attention_decode_static(const DkAttnParams* p, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
