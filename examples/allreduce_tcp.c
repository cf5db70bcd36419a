/* Minimal C user of the library: N ranks on loopback over the tcp transport (one process per rank).
 *
 *   cc -Iinclude examples/allreduce_tcp.c -Lbuild/cmake -lmccl -Wl,-rpath,$PWD/build/cmake -o allreduce_tcp
 *   MCCL_BOOTSTRAP_PORT=53801 MCCL_WORLD_SIZE=2 MCCL_RANK=0 ./allreduce_tcp &
 *   MCCL_BOOTSTRAP_PORT=53801 MCCL_WORLD_SIZE=2 MCCL_RANK=1 ./allreduce_tcp
 *
 * With MCCL_BOOTSTRAP_PORT set, every rank builds the same id from the environment (mcclGetUniqueId).
 */
#include <stdio.h>
#include <stdlib.h>

#include "mccl.h"

#define CHECK(call) do { mcclResult_t r_ = (call); if (r_ != mcclSuccess) { \
  fprintf(stderr, "%s failed: %s\n", #call, mcclGetErrorString(r_)); return 1; } } while (0)

int main(void) {
  const int rank = atoi(getenv("MCCL_RANK") ? getenv("MCCL_RANK") : "0");
  const int world = atoi(getenv("MCCL_WORLD_SIZE") ? getenv("MCCL_WORLD_SIZE") : "1");
  mcclUniqueId id;
  mcclComm_t comm;
  mcclConfig_t cfg = {1, "tcp"};
  CHECK(mcclGetUniqueId(&id));
  CHECK(mcclCommInitRankConfig(&comm, world, id, rank, &cfg));
  enum { N = 1 << 16 };
  static float x[N];
  for (int i = 0; i < N; ++i) x[i] = (float)(rank + 1);
  CHECK(mcclAllReduce(comm, x, x, N, mcclFloat32, mcclSum, NULL));
  int algo = -1;
  CHECK(mcclCommLastAlgo(comm, &algo));
  printf("rank %d of %d: all-reduce(%s) -> %.0f (expected %d)\n", rank, world, mcclAlgoStr(algo), x[0], world * (world + 1) / 2);
  CHECK(mcclCommFinalize(comm));
  CHECK(mcclCommDestroy(comm));
  return x[0] == (float)(world * (world + 1) / 2) ? 0 : 1;
}
