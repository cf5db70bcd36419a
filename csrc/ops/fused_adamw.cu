// Fused AdamW over one flat gradient bucket: reads the (already averaged) bf16 gradients in place in the
// bucket the all-reduce wrote, updates fp32 master weights and both moments, and writes the bf16 working
// copy of the parameters: one pass over memory instead of the dozen elementwise kernels of an unfused step.
// Exposed through the C ABI so the Python side can call it with raw pointers on any stream.
// No counterpart in the reference (it has no training code); this is the optimizer half of the
// data-parallel step its benchmark describes (docs/perf-scaling.png: "compute on batch + gradient all-reduce").
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mccl.h"
#include "mccl_ops.h"

namespace {

struct AdamArgs {
  __nv_bfloat16* param;      // bf16 working weights (what the model reads)
  float* master;             // fp32 master weights
  float* expAvg;
  float* expAvgSq;
  const __nv_bfloat16* grad; // bf16 gradients (bucket)
  uint64_t n;
  float lr, beta1, beta2, eps, weightDecay, gradScale, biasCorr1, biasCorr2Sqrt;
  int zeroGrad;              // clear the gradient after use, ready for the next accumulation
  const float* normSq;       // optional device scalar: squared global gradient norm (for clipping)
  float maxNorm;             // clip threshold; used only when normSq is set
  const float* hyper;        // optional device array {lr, 1 - beta1^t, sqrt(1 - beta2^t)}: read at run time, so a
                             // launch recorded in a CUDA graph follows the schedule when it is replayed
};

__global__ void __launch_bounds__(256) adamwKernel(AdamArgs a) {
  if (a.hyper != nullptr) { a.lr = a.hyper[0]; a.biasCorr1 = a.hyper[1]; a.biasCorr2Sqrt = a.hyper[2]; }
  if (a.normSq != nullptr) {   // global-norm clipping: scale = min(1, maxNorm / ||g||), read on the device (no host sync)
    const float norm = sqrtf(*a.normSq) * a.gradScale;
    if (norm > a.maxNorm) a.gradScale *= a.maxNorm / (norm + 1e-6f);
  }
  const uint64_t nVec = a.n / 8;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = tid; i < nVec; i += nth) {
    uint4 gq = reinterpret_cast<const uint4*>(a.grad)[i];
    const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(&gq);
    float4 w[2], m[2], v[2];
    w[0] = reinterpret_cast<float4*>(a.master)[2 * i]; w[1] = reinterpret_cast<float4*>(a.master)[2 * i + 1];
    m[0] = reinterpret_cast<float4*>(a.expAvg)[2 * i]; m[1] = reinterpret_cast<float4*>(a.expAvg)[2 * i + 1];
    v[0] = reinterpret_cast<float4*>(a.expAvgSq)[2 * i]; v[1] = reinterpret_cast<float4*>(a.expAvgSq)[2 * i + 1];
    float* wf = reinterpret_cast<float*>(w);
    float* mf = reinterpret_cast<float*>(m);
    float* vf = reinterpret_cast<float*>(v);
    uint4 pq;
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(&pq);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gr = __bfloat162float(g[k]) * a.gradScale;
      mf[k] = a.beta1 * mf[k] + (1.f - a.beta1) * gr;
      vf[k] = a.beta2 * vf[k] + (1.f - a.beta2) * gr * gr;
      const float denom = sqrtf(vf[k]) / a.biasCorr2Sqrt + a.eps;
      wf[k] = wf[k] * (1.f - a.lr * a.weightDecay) - (a.lr / a.biasCorr1) * (mf[k] / denom);
      p[k] = __float2bfloat16_rn(wf[k]);
    }
    reinterpret_cast<float4*>(a.master)[2 * i] = w[0]; reinterpret_cast<float4*>(a.master)[2 * i + 1] = w[1];
    reinterpret_cast<float4*>(a.expAvg)[2 * i] = m[0]; reinterpret_cast<float4*>(a.expAvg)[2 * i + 1] = m[1];
    reinterpret_cast<float4*>(a.expAvgSq)[2 * i] = v[0]; reinterpret_cast<float4*>(a.expAvgSq)[2 * i + 1] = v[1];
    reinterpret_cast<uint4*>(a.param)[i] = pq;
    if (a.zeroGrad) reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(a.grad))[i] = make_uint4(0, 0, 0, 0);
  }
  // tail (n not a multiple of 8)
  for (uint64_t i = nVec * 8 + tid; i < a.n; i += nth) {
    const float gr = __bfloat162float(a.grad[i]) * a.gradScale;
    const float m = a.beta1 * a.expAvg[i] + (1.f - a.beta1) * gr;
    const float v = a.beta2 * a.expAvgSq[i] + (1.f - a.beta2) * gr * gr;
    const float denom = sqrtf(v) / a.biasCorr2Sqrt + a.eps;
    const float w = a.master[i] * (1.f - a.lr * a.weightDecay) - (a.lr / a.biasCorr1) * (m / denom);
    a.expAvg[i] = m; a.expAvgSq[i] = v; a.master[i] = w;
    a.param[i] = __float2bfloat16_rn(w);
    if (a.zeroGrad) const_cast<__nv_bfloat16*>(a.grad)[i] = __float2bfloat16_rn(0.f);
  }
}

}  // namespace

static mcclResult_t adamwLaunch(void* param, float* master, float* expAvg, float* expAvgSq, const void* grad,
                                uint64_t n, float lr, float beta1, float beta2, float eps, float weightDecay,
                                float gradScale, int step, int zeroGrad, const float* normSq, float maxNorm,
                                const float* hyper, mcclStream_t stream) {
  if (param == nullptr || master == nullptr || expAvg == nullptr || expAvgSq == nullptr || grad == nullptr || step < 1)
    return mcclInvalidArgument;
  if (n == 0) return mcclSuccess;
  // All five arrays are walked with 16/32-byte vectors.
  if (((uintptr_t)param | (uintptr_t)grad) & 15u || ((uintptr_t)master | (uintptr_t)expAvg | (uintptr_t)expAvgSq) & 15u)
    return mcclInvalidArgument;
  AdamArgs a;
  a.param = static_cast<__nv_bfloat16*>(param);
  a.master = master; a.expAvg = expAvg; a.expAvgSq = expAvgSq;
  a.grad = static_cast<const __nv_bfloat16*>(grad);
  a.n = n;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weightDecay = weightDecay; a.gradScale = gradScale;
  a.biasCorr1 = 1.f - powf(beta1, (float)step);
  a.biasCorr2Sqrt = sqrtf(1.f - powf(beta2, (float)step));
  a.zeroGrad = zeroGrad;
  a.normSq = normSq;
  a.maxNorm = maxNorm;
  a.hyper = hyper;
  const uint64_t vec = (n + 7) / 8;
  int blocks = (int)((vec + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  adamwKernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? mcclSuccess : mcclSystemError;
}

extern "C" mcclResult_t mcclFusedAdamW(void* param, float* master, float* expAvg, float* expAvgSq, const void* grad,
                                       uint64_t n, float lr, float beta1, float beta2, float eps, float weightDecay,
                                       float gradScale, int step, int zeroGrad, const float* normSq, float maxNorm,
                                       mcclStream_t stream) {
  return adamwLaunch(param, master, expAvg, expAvgSq, grad, n, lr, beta1, beta2, eps, weightDecay, gradScale, step, zeroGrad,
                     normSq, maxNorm, nullptr, stream);
}

// The same step with the learning rate and the two bias corrections read from device memory when the kernel
// runs: hyper = {lr, 1 - beta1^t, sqrt(1 - beta2^t)}.  For launches recorded in a CUDA graph.
extern "C" mcclResult_t mcclFusedAdamWDeviceHyper(void* param, float* master, float* expAvg, float* expAvgSq, const void* grad,
                                                  uint64_t n, const float* hyper, float beta1, float beta2, float eps,
                                                  float weightDecay, float gradScale, int zeroGrad, const float* normSq,
                                                  float maxNorm, mcclStream_t stream) {
  if (hyper == nullptr) return mcclInvalidArgument;
  return adamwLaunch(param, master, expAvg, expAvgSq, grad, n, 0.f, beta1, beta2, eps, weightDecay, gradScale, 1, zeroGrad,
                     normSq, maxNorm, hyper, stream);
}
