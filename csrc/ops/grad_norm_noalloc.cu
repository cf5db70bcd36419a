// Allocation-free variant of mcclSumSquaresBf16: same kernel, work memory in a file-scope device array.
#include <cuda_runtime.h>
#include <mutex>

#include "../core/core.h"
#include "grad_norm.cuh"
#include "grad_norm_noalloc.h"

using namespace mccl;

namespace {

constexpr uint64_t kMaxBlocks = MCCL_SUM_SQUARES_NOALLOC_MAX_ELEMS / kNormTile;

// Ticket counter in the first word, then one partial sum per block.  In host code this name is only a
// stand-in for the symbol; the address a kernel can use comes from cudaGetSymbolAddress, per device.
static __device__ __align__(256) float g_normScratch[kNormHeader + kMaxBlocks];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratchAddr[kMaxDevices] = {nullptr};

// Device address of the array on the current device, looked up once per device.
mcclResult_t scratchForCurrentDevice(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return mcclSystemError;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratchAddr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_normScratch);
    if (e != cudaSuccess || p == nullptr) {
      MCCL_WARN("cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      cudaGetLastError();
      return mcclSystemError;
    }
    g_scratchAddr[dev] = static_cast<float*>(p);
  }
  *out = g_scratchAddr[dev];
  return mcclSuccess;
}

}  // namespace

extern "C" mcclResult_t mcclSumSquaresBf16NoAlloc(const void* x, uint64_t n, float* out, int accumulate, mcclStream_t stream) {
  if (out == nullptr || (n > 0 && x == nullptr)) return mcclInvalidArgument;
  if (n > MCCL_SUM_SQUARES_NOALLOC_MAX_ELEMS) {
    MCCL_WARN("mcclSumSquaresBf16NoAlloc: %llu elements exceed the fixed work area (%llu at most); use mcclSumSquaresBf16",
              (unsigned long long)n, (unsigned long long)MCCL_SUM_SQUARES_NOALLOC_MAX_ELEMS);
    return mcclInvalidArgument;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (n == 0) {
    if (!accumulate && cudaMemsetAsync(out, 0, sizeof(float), s) != cudaSuccess) return mcclSystemError;
    return mcclSuccess;
  }
  float* scratch = nullptr;
  MCCLCHECK(scratchForCurrentDevice(&scratch));
  // The array keeps whatever the previous call left.  Only the ticket counter has to start at zero (every
  // partial that is read is written first); clear it here in case an earlier launch never finished.
  if (cudaMemsetAsync(scratch, 0, sizeof(unsigned), s) != cudaSuccess) return mcclSystemError;
  sumSquaresKernel<<<(unsigned)normBlocks(n), kNormThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, scratch, out, accumulate);
  return cudaGetLastError() == cudaSuccess ? mcclSuccess : mcclSystemError;
}
