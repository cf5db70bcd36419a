// Fused softmax cross-entropy over bf16 logits for the language-model head.
//   forward : one CTA per row, one pass (online max / sum-of-exponentials in fp32) -> per-row loss and
//             log-sum-exp; the 8192 x 50304 logits are read once and never widened to an fp32 tensor.
//   backward: dlogits = (exp(logit - lse) - [j == target]) * grad / rows, written in bf16 over the logits
//             (they are not needed afterwards); padding columns beyond the vocabulary get zero.
// Replaces the cast + log_softmax + nll_loss kernels (and their fp32 temporaries of rows x vocab) of an
// unfused loss.  No counterpart in the reference (it has no model code).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mccl.h"
#include "mccl_ops.h"

namespace {

constexpr int kCeThreads = 256;

struct MaxSum { float m, s; };
__device__ __forceinline__ MaxSum combine(MaxSum a, MaxSum b) {
  const float m = fmaxf(a.m, b.m);
  if (m == -INFINITY) return MaxSum{m, 0.f};
  return MaxSum{m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}
__device__ __forceinline__ void push(MaxSum& a, float x) {
  if (x > a.m) { a.s = a.s * __expf(a.m - x) + 1.f; a.m = x; }
  else a.s += __expf(x - a.m);
}

__global__ void __launch_bounds__(kCeThreads) ceForwardKernel(const __nv_bfloat16* logits, int64_t ld, int vocab,
                                                              const int64_t* targets, float* loss, float* lse) {
  __shared__ MaxSum warpAcc[kCeThreads / 32];
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* x = logits + row * ld;
  MaxSum acc{-INFINITY, 0.f};
  const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
  const int nVec = vec ? vocab / 8 : 0;
  for (int i = threadIdx.x; i < nVec; i += kCeThreads) {
    const uint4 q = reinterpret_cast<const uint4*>(x)[i];
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
    for (int k = 0; k < 8; ++k) push(acc, __bfloat162float(e[k]));
  }
  for (int i = nVec * 8 + threadIdx.x; i < vocab; i += kCeThreads) push(acc, __bfloat162float(x[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other{__shfl_xor_sync(0xffffffffu, acc.m, o), __shfl_xor_sync(0xffffffffu, acc.s, o)};
    acc = combine(acc, other);
  }
  if ((threadIdx.x & 31) == 0) warpAcc[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    MaxSum t = warpAcc[0];
    for (int w = 1; w < kCeThreads / 32; ++w) t = combine(t, warpAcc[w]);
    const float l = t.m + logf(t.s);
    const int64_t tgt = targets[row];
    lse[row] = l;
    loss[row] = (tgt >= 0 && tgt < vocab) ? l - __bfloat162float(x[tgt]) : 0.f;     // out-of-range target: ignored row
  }
}

__global__ void __launch_bounds__(kCeThreads) ceBackwardKernel(__nv_bfloat16* logits, int64_t ld, int vocab, int width,
                                                               const int64_t* targets, const float* lse, const float* gradOut,
                                                               float invRows) {
  const int64_t row = blockIdx.x;
  __nv_bfloat16* x = logits + row * ld;
  const float l = lse[row];
  const int64_t tgt = targets[row];
  const bool live = tgt >= 0 && tgt < vocab;
  const float scale = live ? (*gradOut) * invRows : 0.f;
  const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
  const int nVec = vec ? width / 8 : 0;
  for (int i = threadIdx.x; i < nVec; i += kCeThreads) {
    uint4 q = reinterpret_cast<const uint4*>(x)[i];
    __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&q);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int j = i * 8 + k;
      float g = 0.f;
      if (j < vocab) g = (__expf(__bfloat162float(e[k]) - l) - (j == tgt ? 1.f : 0.f)) * scale;
      e[k] = __float2bfloat16_rn(g);
    }
    reinterpret_cast<uint4*>(x)[i] = q;
  }
  for (int j = nVec * 8 + threadIdx.x; j < width; j += kCeThreads) {
    float g = 0.f;
    if (j < vocab) g = (__expf(__bfloat162float(x[j]) - l) - (j == tgt ? 1.f : 0.f)) * scale;
    x[j] = __float2bfloat16_rn(g);
  }
}

}  // namespace

// loss[row] = logsumexp(logits[row, :vocab]) - logits[row, target[row]]; lse[row] keeps the log-sum-exp.
extern "C" mcclResult_t mcclCrossEntropyForward(const void* logits, int64_t rows, int64_t ld, int vocab, const int64_t* targets,
                                                float* loss, float* lse, mcclStream_t stream) {
  if (logits == nullptr || targets == nullptr || loss == nullptr || lse == nullptr || rows < 0 || vocab <= 0 || ld < vocab)
    return mcclInvalidArgument;
  if (rows == 0) return mcclSuccess;
  ceForwardKernel<<<(unsigned)rows, kCeThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, vocab, targets, loss, lse);
  return cudaGetLastError() == cudaSuccess ? mcclSuccess : mcclSystemError;
}

// In place: logits[row, j] <- d(mean loss)/d(logit) * gradOut for j < vocab, 0 for vocab <= j < width.
extern "C" mcclResult_t mcclCrossEntropyBackward(void* logits, int64_t rows, int64_t ld, int vocab, int width,
                                                 const int64_t* targets, const float* lse, const float* gradOut,
                                                 mcclStream_t stream) {
  if (logits == nullptr || targets == nullptr || lse == nullptr || gradOut == nullptr || rows < 0 || vocab <= 0 || width < vocab ||
      ld < width) return mcclInvalidArgument;
  if (rows == 0) return mcclSuccess;
  ceBackwardKernel<<<(unsigned)rows, kCeThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), ld, vocab, width, targets, lse, gradOut, 1.0f / (float)rows);
  return cudaGetLastError() == cudaSuccess ? mcclSuccess : mcclSystemError;
}
