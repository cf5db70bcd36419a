/* C user of the cuda transport: one process per GPU of an NVSwitch box, symmetric buffers, grouped calls.
 *
 *   gcc -Iinclude -I/usr/local/cuda/include examples/allreduce_cuda.c -Lmccl_b200/lib -lmccl \
 *       -L/usr/local/cuda/lib64 -lcudart -Wl,-rpath,$PWD/mccl_b200/lib -o allreduce_cuda
 *   for r in 0 1; do MCCL_BOOTSTRAP_PORT=53811 MCCL_WORLD_SIZE=2 MCCL_RANK=$r ./allreduce_cuda & done; wait
 *
 * Rank r uses GPU r.  The buffer comes from mcclMemAlloc, so the all-reduce runs on it in place (NVLS when the
 * box has it); the all-gather and the reduce-scatter are issued inside one group.
 */
#include <stdio.h>
#include <stdlib.h>

#include <cuda_runtime.h>

#include "mccl.h"

#define CHECK(call) do { mcclResult_t r_ = (call); if (r_ != mcclSuccess) { \
  fprintf(stderr, "%s failed: %s\n", #call, mcclGetErrorString(r_)); return 1; } } while (0)
#define CUDA(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { \
  fprintf(stderr, "%s failed: %s\n", #call, cudaGetErrorString(e_)); return 1; } } while (0)

int main(void) {
  const int rank = atoi(getenv("MCCL_RANK") ? getenv("MCCL_RANK") : "0");
  const int world = atoi(getenv("MCCL_WORLD_SIZE") ? getenv("MCCL_WORLD_SIZE") : "1");
  enum { N = 1 << 20 };
  CUDA(cudaSetDevice(rank));
  cudaStream_t stream;
  CUDA(cudaStreamCreate(&stream));

  mcclUniqueId id;
  mcclComm_t comm;
  mcclConfig_t cfg = {1, "cuda"};
  CHECK(mcclGetUniqueId(&id));
  CHECK(mcclCommInitRankConfig(&comm, world, id, rank, &cfg));

  float *x = NULL, *gathered = NULL, *mine = NULL;
  CHECK(mcclMemAlloc(comm, N * sizeof(float), (void**)&x));                    /* collective, same size everywhere */
  CHECK(mcclMemAlloc(comm, (size_t)N * world * sizeof(float), (void**)&gathered));
  CUDA(cudaMalloc((void**)&mine, (N / world) * sizeof(float)));                /* plain memory is staged */
  float* host = (float*)malloc(N * sizeof(float));
  for (int i = 0; i < N; ++i) host[i] = (float)(rank + 1);
  CUDA(cudaMemcpyAsync(x, host, N * sizeof(float), cudaMemcpyHostToDevice, stream));

  CHECK(mcclAllReduce(comm, x, x, N, mcclFloat32, mcclAvg, (mcclStream_t)stream));
  CHECK(mcclGroupStart());
  CHECK(mcclAllGather(comm, x, gathered, N, mcclFloat32, (mcclStream_t)stream));
  CHECK(mcclReduceScatter(comm, x, mine, N / world, mcclFloat32, mcclSum, (mcclStream_t)stream));
  CHECK(mcclGroupEnd());
  float avg = 0.f, sum = 0.f;
  CUDA(cudaMemcpyAsync(&avg, gathered + (size_t)N * (world - 1), sizeof(float), cudaMemcpyDeviceToHost, stream));
  CUDA(cudaMemcpyAsync(&sum, mine, sizeof(float), cudaMemcpyDeviceToHost, stream));
  CUDA(cudaStreamSynchronize(stream));

  mcclResult_t async = mcclSuccess;
  CHECK(mcclCommGetAsyncError(comm, &async));
  int algo = -1, nvls = 0;
  CHECK(mcclCommLastAlgo(comm, &algo));
  CHECK(mcclCommNvlsEnabled(comm, &nvls));
  const float wantAvg = (float)(world + 1) / 2.0f;
  printf("rank %d of %d (nvls %d, last algo %s): avg %.2f (expected %.2f), reduce-scatter %.2f (expected %.2f), async %s\n",
         rank, world, nvls, mcclAlgoStr(algo), avg, wantAvg, sum, wantAvg * world, mcclGetErrorString(async));
  CHECK(mcclMemFree(comm, gathered));
  CHECK(mcclMemFree(comm, x));
  cudaFree(mine);
  free(host);
  CHECK(mcclCommFinalize(comm));
  CHECK(mcclCommDestroy(comm));
  return (avg == wantAvg && sum == wantAvg * world && async == mcclSuccess) ? 0 : 1;
}
