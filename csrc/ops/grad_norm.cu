// C entry point of the sum-of-squares kernel with caller-provided scratch memory.
#include <cuda_runtime.h>

#include "../core/core.h"
#include "grad_norm.cuh"
#include "mccl.h"
#include "mccl_ops.h"

using namespace mccl;

// Floats of scratch a call over n elements needs.
extern "C" uint64_t mcclSumSquaresScratchFloats(uint64_t n) { return kNormHeader + normBlocks(n); }

// out (device float) = [out +] sum(x[i]^2).  `scratch` is device memory of at least
// mcclSumSquaresScratchFloats(n) floats whose first word is zero before the first use (the kernel leaves it
// zero again); calls that share scratch must be ordered on one stream.
extern "C" mcclResult_t mcclSumSquaresBf16(const void* x, uint64_t n, float* scratch, uint64_t scratchFloats, float* out,
                                           int accumulate, mcclStream_t stream) {
  if (out == nullptr || (n > 0 && (x == nullptr || scratch == nullptr))) return mcclInvalidArgument;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (n == 0) {
    if (!accumulate && cudaMemsetAsync(out, 0, sizeof(float), s) != cudaSuccess) return mcclSystemError;
    return mcclSuccess;
  }
  if (scratchFloats < mcclSumSquaresScratchFloats(n)) {
    MCCL_WARN("mcclSumSquaresBf16: %llu floats of scratch given, %llu needed", (unsigned long long)scratchFloats,
              (unsigned long long)mcclSumSquaresScratchFloats(n));
    return mcclInvalidArgument;
  }
  sumSquaresKernel<<<(unsigned)normBlocks(n), kNormThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, scratch, out, accumulate);
  return cudaGetLastError() == cudaSuccess ? mcclSuccess : mcclSystemError;
}
