// Three ranks as threads of one process over the tcp transport, exercising init, every collective with
// every algorithm, grouped Send/Recv, split, a non-blocking communicator and abort from another thread.
// Built against a ThreadSanitizer flavour of the library (cmake -DMCCL_SANITIZE_THREAD=ON) it is the
// race detector for the host code: bootstrap, acceptor thread, worker queue, pools, connection maps.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "mccl.h"

#define CHECK(call)                                                                      \
  do {                                                                                   \
    mcclResult_t rc_ = (call);                                                           \
    if (rc_ != mcclSuccess) { fprintf(stderr, "%s:%d %s -> %s\n", __FILE__, __LINE__, #call, mcclGetErrorString(rc_)); failures++; return; } \
  } while (0)

static std::atomic<int> failures{0};
static const int kRanks = 3;

static void rankMain(int rank, mcclUniqueId id, int blocking) {
  mcclConfig_t cfg = {blocking, "tcp"};
  mcclComm_t comm = nullptr;
  CHECK(mcclCommInitRankConfig(&comm, kRanks, id, rank, &cfg));
  const size_t n = 70001;
  std::vector<float> x(n), y(n), big(n * kRanks);
  for (int algo = -1; algo < 3; ++algo) {
    mcclSetForcedAlgo(algo);
    for (size_t i = 0; i < n; ++i) x[i] = (float)(rank + 1);
    CHECK(mcclAllReduce(comm, x.data(), y.data(), n, mcclFloat32, mcclSum, nullptr));
    CHECK(mcclCommSynchronize(comm));
    if (y[0] != 6.0f || y[n - 1] != 6.0f) { fprintf(stderr, "rank %d algo %d allreduce %f\n", rank, algo, y[0]); failures++; }
    CHECK(mcclAllGather(comm, x.data(), big.data(), n, mcclFloat32, nullptr));
    CHECK(mcclReduceScatter(comm, big.data(), y.data(), n, mcclFloat32, mcclMax, nullptr));
    CHECK(mcclBroadcast(comm, x.data(), y.data(), n, mcclFloat32, 1, nullptr));
    CHECK(mcclReduce(comm, x.data(), y.data(), n, mcclFloat32, mcclAvg, 2, nullptr));
    CHECK(mcclCommSynchronize(comm));
  }
  mcclSetForcedAlgo(mcclAlgoAuto);
  CHECK(mcclGroupStart());
  CHECK(mcclSend(comm, x.data(), n, mcclFloat32, (rank + 1) % kRanks, nullptr));
  CHECK(mcclRecv(comm, y.data(), n, mcclFloat32, (rank + kRanks - 1) % kRanks, nullptr));
  CHECK(mcclGroupEnd());
  CHECK(mcclCommSynchronize(comm));
  mcclComm_t sub = nullptr;
  CHECK(mcclCommSplit(comm, rank == 0 ? MCCL_SPLIT_NOCOLOR : 1, rank, &sub, nullptr));
  if (sub != nullptr) {
    int one = 1, sum = 0;
    CHECK(mcclAllReduce(sub, &one, &sum, 1, mcclInt32, mcclSum, nullptr));
    CHECK(mcclCommSynchronize(sub));
    if (sum != 2) failures++;
    CHECK(mcclCommFinalize(sub));
    CHECK(mcclCommDestroy(sub));
  }
  mcclResult_t async = mcclSuccess;
  CHECK(mcclCommGetAsyncError(comm, &async));
  CHECK(mcclCommFinalize(comm));
  // Abort from a second thread while this one is (possibly) still inside the communicator's API.
  std::thread killer([comm] { mcclCommAbort(comm); });
  killer.join();
  CHECK(mcclCommDestroy(comm));
}

int main() {
  for (int blocking = 1; blocking >= 0; --blocking) {
    mcclUniqueId id;
    if (mcclGetUniqueId(&id) != mcclSuccess) return 2;
    std::vector<std::thread> ts;
    for (int r = 0; r < kRanks; ++r) ts.emplace_back(rankMain, r, id, blocking);
    for (auto& t : ts) t.join();
  }
  printf("tsan_tcp: %d failures\n", failures.load());
  return failures.load() ? 1 : 0;
}
