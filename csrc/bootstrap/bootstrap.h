// Control plane: a star of persistent TCP connections to rank 0 that provides all-gather and barrier.
// Parity: mcclBootstrapAllGather (src/bootstrap.h:10-11, src/bootstrap.cc:16-84) of the reference.  The
// reference re-dials rank 0 for every round; here each rank keeps one connection for the communicator's
// lifetime, every round carries a sequence number and size so a desynchronised rank is detected instead
// of mis-parsed, and all sockets carry deadlines so a rank that dies mid-round fails the round.
#pragma once

#include <atomic>
#include <cstdint>
#include <mutex>
#include <vector>

#include "../core/core.h"

namespace mccl {

struct BootstrapId {       // contents of mcclUniqueId.internal
  char     ip[64];
  uint16_t port;
  uint16_t pad[3];
  uint64_t nonce;
};

struct Bootstrap {
  int rank = 0, n = 1;
  uint64_t nonce = 0;
  int listenFd = -1;            // rank 0 only, closed once every rank has joined
  int rootFd = -1;              // ranks > 0
  std::vector<int> fds;         // rank 0: fds[r] for r > 0
  uint32_t seq = 0;
  std::mutex mu;                // one round at a time
  std::atomic<bool> aborted{false};   // set by Abort from any thread
};

MCCL_PARAM(BootstrapTimeoutSec);

// Open a listener for a future rank 0 of this process and describe it in *id (ephemeral port unless
// MCCL_BOOTSTRAP_PORT is set, in which case nothing is opened and every rank can build the same id).
// `ip` = address to listen on (nullptr: MCCL_BOOTSTRAP_IP, else 127.0.0.1); `alwaysListen` ignores the env port.
mcclResult_t bootstrapCreateId(BootstrapId* id, const char* ip = nullptr, bool alwaysListen = false);
// Local IPv4 address (host order) of this rank's connection to rank 0; 0 for rank 0 itself.
uint32_t     bootstrapLocalIp(const Bootstrap* bs);
// Rank 0 adopts (or opens) the listener and waits for n-1 dialers; other ranks dial with retries.
mcclResult_t bootstrapInit(const BootstrapId& id, int rank, int n, Bootstrap** out);
mcclResult_t bootstrapAllGather(Bootstrap* bs, const void* send, void* recv, size_t bytesPerRank);
mcclResult_t bootstrapBarrier(Bootstrap* bs);
void         bootstrapAbort(Bootstrap* bs);   // shutdown sockets, keep memory
void         bootstrapClose(Bootstrap* bs);   // close and free

}  // namespace mccl
