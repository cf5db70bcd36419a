// LayerNorm forward and backward for bf16 activations with rows of 256, 512 or 1024 elements (wider rows
// would spill the per-lane column sums out of registers; callers fall back to the framework's kernel).
// One warp per row, each lane holding VPL 16-byte vectors of the row in registers.
//   forward : mean / rstd by warp shuffles, y = (x - mean) * rstd * gamma + beta, mean and rstd saved in fp32.
//   backward: dx per row from two warp reductions; every lane also accumulates dgamma / dbeta of its columns
//             over the rows its warp walks, the CTA folds its warps through shared memory and writes one
//             partial per CTA; a second small kernel adds the partials.  One pass over x and dy instead of
//             the separate (and slow) column-reduction kernel of an unfused backward.
// No counterpart in the reference (it has no model code).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mccl.h"
#include "mccl_ops.h"

namespace {

constexpr int kLnWarps = 4;
constexpr int kLnThreads = kLnWarps * 32;

__device__ __forceinline__ float warpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int VPL>
__global__ void __launch_bounds__(kLnThreads) lnForwardKernel(const __nv_bfloat16* x, const __nv_bfloat16* gamma,
                                                              const __nv_bfloat16* beta, __nv_bfloat16* y, float* mean,
                                                              float* rstd, int64_t rows, float eps) {
  constexpr int D = VPL * 256;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float g[VPL * 8], b[VPL * 8];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const uint4 gq = reinterpret_cast<const uint4*>(gamma)[lane + 32 * j], bq = reinterpret_cast<const uint4*>(beta)[lane + 32 * j];
    const __nv_bfloat16* ge = reinterpret_cast<const __nv_bfloat16*>(&gq);
    const __nv_bfloat16* be = reinterpret_cast<const __nv_bfloat16*>(&bq);
#pragma unroll
    for (int k = 0; k < 8; ++k) { g[j * 8 + k] = __bfloat162float(ge[k]); b[j * 8 + k] = __bfloat162float(be[k]); }
  }
  for (int64_t row = (int64_t)blockIdx.x * kLnWarps + warp; row < rows; row += (int64_t)gridDim.x * kLnWarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
    float v[VPL * 8];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const uint4 q = xr[lane + 32 * j];
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
      for (int k = 0; k < 8; ++k) { v[j * 8 + k] = __bfloat162float(e[k]); s += v[j * 8 + k]; }
    }
    const float mu = warpSum(s) * (1.0f / D);
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPL * 8; ++i) { const float d = v[i] - mu; sq += d * d; }
    const float rs = rsqrtf(warpSum(sq) * (1.0f / D) + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + row * D);
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      uint4 q;
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&q);
#pragma unroll
      for (int k = 0; k < 8; ++k) e[k] = __float2bfloat16_rn((v[j * 8 + k] - mu) * rs * g[j * 8 + k] + b[j * 8 + k]);
      yr[lane + 32 * j] = q;
    }
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
  }
}

template <int VPL>
__global__ void __launch_bounds__(kLnThreads) lnBackwardKernel(const __nv_bfloat16* x, const __nv_bfloat16* dy,
                                                               const __nv_bfloat16* gamma, const float* mean, const float* rstd,
                                                               __nv_bfloat16* dx, float* partial, int64_t rows) {
  constexpr int D = VPL * 256;
  __shared__ float red[kLnWarps][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float g[VPL * 8], dg[VPL * 8], db[VPL * 8];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const uint4 gq = reinterpret_cast<const uint4*>(gamma)[lane + 32 * j];
    const __nv_bfloat16* ge = reinterpret_cast<const __nv_bfloat16*>(&gq);
#pragma unroll
    for (int k = 0; k < 8; ++k) { g[j * 8 + k] = __bfloat162float(ge[k]); dg[j * 8 + k] = 0.f; db[j * 8 + k] = 0.f; }
  }
  for (int64_t row = (int64_t)blockIdx.x * kLnWarps + warp; row < rows; row += (int64_t)gridDim.x * kLnWarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
    const uint4* dr = reinterpret_cast<const uint4*>(dy + row * D);
    uint4 xq[VPL], dq[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) { xq[j] = xr[lane + 32 * j]; dq[j] = dr[lane + 32 * j]; }
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const __nv_bfloat16* xe = reinterpret_cast<const __nv_bfloat16*>(&xq[j]);
      const __nv_bfloat16* de = reinterpret_cast<const __nv_bfloat16*>(&dq[j]);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float xh = (__bfloat162float(xe[k]) - mu) * rs, d = __bfloat162float(de[k]), gd = d * g[j * 8 + k];
        s1 += gd; s2 += gd * xh;
        dg[j * 8 + k] += d * xh; db[j * 8 + k] += d;
      }
    }
    s1 = warpSum(s1) * (1.0f / D);
    s2 = warpSum(s2) * (1.0f / D);
    uint4* outr = reinterpret_cast<uint4*>(dx + row * D);
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const __nv_bfloat16* xe = reinterpret_cast<const __nv_bfloat16*>(&xq[j]);
      const __nv_bfloat16* de = reinterpret_cast<const __nv_bfloat16*>(&dq[j]);
      uint4 q;
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&q);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float xh = (__bfloat162float(xe[k]) - mu) * rs, gd = __bfloat162float(de[k]) * g[j * 8 + k];
        e[k] = __float2bfloat16_rn(rs * (gd - s1 - xh * s2));
      }
      outr[lane + 32 * j] = q;
    }
  }
  // Fold the four warps' column sums, dgamma first, then dbeta, through shared memory.
  float* out = partial + (int64_t)blockIdx.x * 2 * D;
  for (int pass = 0; pass < 2; ++pass) {
    __syncthreads();
#pragma unroll
    for (int j = 0; j < VPL; ++j)
#pragma unroll
      for (int k = 0; k < 8; ++k) red[warp][(lane + 32 * j) * 8 + k] = pass == 0 ? dg[j * 8 + k] : db[j * 8 + k];
    __syncthreads();
    for (int c = threadIdx.x; c < D; c += kLnThreads) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < kLnWarps; ++w) t += red[w][c];
      out[pass * D + c] = t;
    }
  }
}

__global__ void lnReducePartialsKernel(const float* partial, int nPartials, int D, __nv_bfloat16* dgamma, __nv_bfloat16* dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= 2 * D) return;
  float t = 0.f;
  for (int p = 0; p < nPartials; ++p) t += partial[(int64_t)p * 2 * D + c];
  if (c < D) dgamma[c] = __float2bfloat16_rn(t); else dbeta[c - D] = __float2bfloat16_rn(t);
}

int lnGrid(int64_t rows) {
  int64_t ctas = (rows + kLnWarps * 8 - 1) / (kLnWarps * 8);     // about eight rows per warp
  if (ctas > 148 * 4) ctas = 148 * 4;
  return ctas < 1 ? 1 : (int)ctas;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// Number of CTAs the backward pass uses for `rows` rows = number of fp32 partials of 2*D floats it writes.
extern "C" int mcclLayerNormPartials(int64_t rows) { return lnGrid(rows); }

extern "C" mcclResult_t mcclLayerNormForward(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                                             int64_t rows, int D, float eps, mcclStream_t stream) {
  if (!x || !gamma || !beta || !y || !mean || !rstd || rows < 0) return mcclInvalidArgument;
  if (!aligned16(x) || !aligned16(gamma) || !aligned16(beta) || !aligned16(y)) return mcclInvalidArgument;
  if (rows == 0) return mcclSuccess;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto* X = static_cast<const __nv_bfloat16*>(x); auto* G = static_cast<const __nv_bfloat16*>(gamma);
  auto* B = static_cast<const __nv_bfloat16*>(beta); auto* Y = static_cast<__nv_bfloat16*>(y);
  const int grid = lnGrid(rows);
  switch (D) {
    case 256:  lnForwardKernel<1><<<grid, kLnThreads, 0, s>>>(X, G, B, Y, mean, rstd, rows, eps); break;
    case 512:  lnForwardKernel<2><<<grid, kLnThreads, 0, s>>>(X, G, B, Y, mean, rstd, rows, eps); break;
    case 1024: lnForwardKernel<4><<<grid, kLnThreads, 0, s>>>(X, G, B, Y, mean, rstd, rows, eps); break;
    default: return mcclInvalidArgument;
  }
  return cudaGetLastError() == cudaSuccess ? mcclSuccess : mcclSystemError;
}

// partial: fp32 work memory of mcclLayerNormPartials(rows) * 2 * D floats.
extern "C" mcclResult_t mcclLayerNormBackward(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd,
                                              void* dx, void* dgamma, void* dbeta, float* partial, int64_t rows, int D,
                                              mcclStream_t stream) {
  if (!x || !dy || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta || !partial || rows <= 0) return mcclInvalidArgument;
  if (!aligned16(x) || !aligned16(dy) || !aligned16(gamma) || !aligned16(dx)) return mcclInvalidArgument;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto* X = static_cast<const __nv_bfloat16*>(x); auto* DY = static_cast<const __nv_bfloat16*>(dy);
  auto* G = static_cast<const __nv_bfloat16*>(gamma); auto* DX = static_cast<__nv_bfloat16*>(dx);
  const int grid = lnGrid(rows);
  switch (D) {
    case 256:  lnBackwardKernel<1><<<grid, kLnThreads, 0, s>>>(X, DY, G, mean, rstd, DX, partial, rows); break;
    case 512:  lnBackwardKernel<2><<<grid, kLnThreads, 0, s>>>(X, DY, G, mean, rstd, DX, partial, rows); break;
    case 1024: lnBackwardKernel<4><<<grid, kLnThreads, 0, s>>>(X, DY, G, mean, rstd, DX, partial, rows); break;
    default: return mcclInvalidArgument;
  }
  if (cudaGetLastError() != cudaSuccess) return mcclSystemError;
  lnReducePartialsKernel<<<(2 * D + 255) / 256, 256, 0, s>>>(partial, grid, D, static_cast<__nv_bfloat16*>(dgamma),
                                                             static_cast<__nv_bfloat16*>(dbeta));
  return cudaGetLastError() == cudaSuccess ? mcclSuccess : mcclSystemError;
}
