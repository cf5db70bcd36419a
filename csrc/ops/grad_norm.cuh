// Sum of squares of a bf16 array (the global gradient norm of a training step, accumulated bucket by
// bucket).  Two stages inside one launch: every block folds one fixed tile into a partial sum in scratch
// memory; the block that finishes last (a ticket counter, also in scratch) adds the partials in index
// order, so the result does not depend on which block finished when.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace mccl {

constexpr int kNormThreads = 256;
constexpr uint64_t kNormTile = 65536;          // elements per block
constexpr uint64_t kNormHeader = 64;           // floats reserved in front of the partials (ticket counter)

// scratch layout: [0] ticket counter (as unsigned), [kNormHeader ...) one partial per block.
static __global__ void __launch_bounds__(kNormThreads) sumSquaresKernel(const __nv_bfloat16* x, uint64_t n, float* scratch,
                                                                 float* out, int accumulate) {
  __shared__ float warpSums[kNormThreads / 32];
  __shared__ unsigned ticket;
  const uint64_t lo = (uint64_t)blockIdx.x * kNormTile;
  const uint64_t hi = lo + kNormTile < n ? lo + kNormTile : n;
  float acc = 0.f;
  const bool vec = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  if (vec) {
    const uint64_t v0 = lo / 8, v1 = hi / 8;                 // lo is a multiple of the tile, hence of 8
    for (uint64_t i = v0 + threadIdx.x; i < v1; i += kNormThreads) {
      const uint4 q = reinterpret_cast<const uint4*>(x)[i];
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
      for (int k = 0; k < 8; ++k) { const float f = __bfloat162float(e[k]); acc += f * f; }
    }
    for (uint64_t i = v1 * 8 + threadIdx.x; i < hi; i += kNormThreads) { const float f = __bfloat162float(x[i]); acc += f * f; }
  } else {
    for (uint64_t i = lo + threadIdx.x; i < hi; i += kNormThreads) { const float f = __bfloat162float(x[i]); acc += f * f; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warpSums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < kNormThreads / 32; ++w) s += warpSums[w];
    scratch[kNormHeader + blockIdx.x] = s;
    __threadfence();
    ticket = atomicAdd(reinterpret_cast<unsigned*>(scratch), 1u);
  }
  __syncthreads();
  if (ticket != gridDim.x - 1) return;
  // Last block: every partial is visible (each writer fenced before taking its ticket).
  __threadfence();
  float s = 0.f;
  for (unsigned i = threadIdx.x; i < gridDim.x; i += kNormThreads) s += reinterpret_cast<volatile float*>(scratch)[kNormHeader + i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) warpSums[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kNormThreads / 32; ++w) t += warpSums[w];
    *out = accumulate ? *out + t : t;
    *reinterpret_cast<unsigned*>(scratch) = 0u;            // ready for the next launch
  }
}

inline uint64_t normBlocks(uint64_t n) { return (n + kNormTile - 1) / kNormTile; }

}  // namespace mccl
