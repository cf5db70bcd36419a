// Sum of squares of a bf16 array for callers that must not allocate.
//
// This entry point has no counterpart in the reference library.  It exists for code that runs where device
// allocation is forbidden or impossible: a region being captured into a CUDA graph, a callback on a thread
// that may not take the allocator's locks, a process whose memory is fully handed to another allocator.
// Such callers cannot provide the work memory that mcclSumSquaresBf16 asks for, and cannot let the library
// call cudaMalloc on their behalf.  Here the work memory is a fixed array inside the library image.
#pragma once

#include <stdint.h>

#include "mccl.h"

#ifdef __cplusplus
extern "C" {
#endif

// Largest element count one call accepts (4096 tiles of 65536 elements).
#define MCCL_SUM_SQUARES_NOALLOC_MAX_ELEMS (4096ull * 65536ull)

// out (one float on the device) = [out +] sum(x[i]^2), x = n bf16 values on the current device.
//  * Allocates nothing: no cudaMalloc/cudaFree, no allocating library call.  The partial sums live in a
//    static device array of (64 + 4096) floats, about 16.6 KB, which every GPU that loads the library
//    holds until the process exits.
//  * n above MCCL_SUM_SQUARES_NOALLOC_MAX_ELEMS is refused with mcclInvalidArgument (and a WARN log line).
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
//    first call before starting any stream capture on that device.
//  * All calls on a device share the one array.  Calls ordered on one stream are fine; calls that can run
//    at the same time on the GPU (different streams, different threads) race on it and give wrong sums.
mcclResult_t mcclSumSquaresBf16NoAlloc(const void* x, uint64_t n, float* out, int accumulate, mcclStream_t stream);

#ifdef __cplusplus
}
#endif
