/*
 * mccl-b200 compute entry points that go with the collectives: the tcgen05 GEMM and its fused tensor-parallel
 * forms, the fused expert-parallel token exchange, and the kernels of the data-parallel training step (fused
 * AdamW with global-norm clipping, sum of squares, cross-entropy, LayerNorm).  sm_100a only; every pointer is a
 * device pointer on the current device unless stated otherwise; calls are enqueued on `stream`.
 * None of these has a counterpart in the reference (a communication library without compute or model code).
 */
#ifndef MCCL_OPS_H_
#define MCCL_OPS_H_

#include "mccl.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- bf16 GEMM on the 5th-generation tensor cores: C[M,N] = act(A[M,K] * B[N,K]^T) --------------------------- */
#define MCCL_EPILOGUE_NONE 0
#define MCCL_EPILOGUE_SILU 1
/* M % 128 == 0, N % 64 == 0, K % 64 == 0.  maxCtas = 0: one CTA per SM. */
mcclResult_t mcclTpGemm(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int maxCtas, mcclStream_t stream);
/* The same product by pairs of SMs on 256-row tiles (M % 256 == 0). */
mcclResult_t mcclTpGemm2(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int maxCtas, mcclStream_t stream);
/* Error code the last GEMM kernel on the current device recorded (0 = none); reading clears it. */
int mcclTpGemmLastError(void);

/* Fused all-gather -> GEMM -> activation.  xShard [M/n, K] in symmetric memory, xFull [M, K] local workspace,
 * W [N, K] local weight shard, out [M, N], flags >= 16 uint64 of device memory.  Collective over comm. */
mcclResult_t mcclTpAllGatherGemm(mcclComm_t comm, const void* xShard, void* xFull, const void* W, void* out, void* flags,
                                 int M, int N, int K, int epilogue, mcclStream_t stream);
/* Fused GEMM -> reduce-scatter over rows.  H [M, K], W [N, K], partial [M, N] and flags (16 + M/128 + M/128 uint64,
 * zeroed once) in symmetric memory, out [M/n, N], accum [M/n, N] fp32; callIndex = 1, 2, ... per flags buffer. */
mcclResult_t mcclTpGemmReduceScatter(mcclComm_t comm, const void* H, const void* W, void* partial, void* flags, void* out,
                                     float* accum, int M, int N, int K, uint64_t callIndex, mcclStream_t stream);

/* ---- expert-parallel token exchange fused with the routing gather / scatter --------------------------------------- */
/* exchange: symmetric memory, [ranks][expertsPerRank][capacity][rowBytes] on every rank.  flat[t] = expert * capacity +
 * slot of token t, negative for a dropped token.  scale (nullable): one float per token. */
mcclResult_t mcclMoeScatter(mcclComm_t comm, const void* tokens, const int32_t* flat, const float* scale, void* exchange,
                            int nTokens, int rowBytes, int expertsPerRank, int capacity, mcclDataType_t dt, mcclStream_t stream);
mcclResult_t mcclMoeGather(mcclComm_t comm, const void* exchange, const int32_t* flat, const float* scale, void* out,
                           int nTokens, int rowBytes, int expertsPerRank, int capacity, mcclDataType_t dt, mcclStream_t stream);

/* ---- training-step kernels (bf16 parameters and gradients, fp32 state) --------------------------------------------- */
/* AdamW on n elements; normSq / maxNorm (nullable / 0): clip by the global gradient norm held on the device. */
mcclResult_t mcclFusedAdamW(void* param, float* master, float* expAvg, float* expAvgSq, const void* grad, uint64_t n, float lr,
                            float beta1, float beta2, float eps, float weightDecay, float gradScale, int step, int zeroGrad,
                            const float* normSq, float maxNorm, mcclStream_t stream);
/* The same step with {lr, 1 - beta1^t, sqrt(1 - beta2^t)} read from the device array `hyper` when the kernel runs, so a
   launch recorded in a CUDA graph follows the schedule on every replay. */
mcclResult_t mcclFusedAdamWDeviceHyper(void* param, float* master, float* expAvg, float* expAvgSq, const void* grad, uint64_t n,
                                       const float* hyper, float beta1, float beta2, float eps, float weightDecay, float gradScale,
                                       int zeroGrad, const float* normSq, float maxNorm, mcclStream_t stream);
uint64_t     mcclSumSquaresScratchFloats(uint64_t n);
/* out = [out +] sum(x^2) over n bf16 values; scratch: mcclSumSquaresScratchFloats(n) floats, first word zero. */
mcclResult_t mcclSumSquaresBf16(const void* x, uint64_t n, float* scratch, uint64_t scratchFloats, float* out, int accumulate,
                                mcclStream_t stream);
/* Cross-entropy over bf16 logits [rows, ld] (vocab <= ld): per-row loss and log-sum-exp; backward in place. */
mcclResult_t mcclCrossEntropyForward(const void* logits, int64_t rows, int64_t ld, int vocab, const int64_t* targets, float* loss,
                                     float* lse, mcclStream_t stream);
mcclResult_t mcclCrossEntropyBackward(void* logits, int64_t rows, int64_t ld, int vocab, int width, const int64_t* targets,
                                      const float* lse, const float* gradOut, mcclStream_t stream);
/* LayerNorm over bf16 rows of D in {256, 512, 1024}. */
int          mcclLayerNormPartials(int64_t rows);
mcclResult_t mcclLayerNormForward(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int64_t rows,
                                  int D, float eps, mcclStream_t stream);
/* partial: mcclLayerNormPartials(rows) x 2 x D floats of work memory. */
mcclResult_t mcclLayerNormBackward(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd, void* dx,
                                   void* dgamma, void* dbeta, float* partial, int64_t rows, int D, mcclStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MCCL_OPS_H_ */
