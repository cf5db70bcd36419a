// Striped-TCP data path used by the CPU transport (and available to a future multi-node backend).
// One logical connection is a bundle of MCCL_NSOCKS sockets; a message is cut into one contiguous shard
// per socket and the shards move in parallel on the stripe pool; both ends derive the split from the
// byte count, so no length travels.  A per-communicator endpoint owns a persistent listener whose accept
// thread sorts interleaved dials into bundles by (peer, kind).
// Parity: src/transport/m2m.h:10-33, src/transport/m2m.cc:25-368 of the reference.
#pragma once

#include <condition_variable>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "../core/core.h"

namespace mccl {

constexpr int kMaxStripes = 8;

enum ConnKind : uint32_t {
  CONN_COLL_A = 0,  // collectives, first ring direction / first tree
  CONN_COLL_B = 1,  // counter-rotating ring / second tree: never shares a socket with set A
  CONN_P2P    = 2,  // user Send/Recv, one bundle per direction (the sender dials)
};

struct TcpConn {
  int peer = -1;
  uint32_t kind = 0;
  int nSocks = 0;
  int fds[kMaxStripes];
};

struct TcpEndpoint {
  int rank = 0;
  uint64_t nonce = 0;
  int listenFd = -1;
  uint16_t port = 0;
  std::thread acceptor;
  std::mutex mu;
  std::condition_variable cv;
  bool stop = false;
  // key = (peer << 8) | kind, plus a direction bit for p2p so that a->b and b->a stay distinct.
  std::map<uint64_t, TcpConn*> conns;
  std::map<uint64_t, TcpConn*> partial;
  uint64_t arrivals = 0;   // bumped whenever a bundle completes (RecvAny waits on it)
};

MCCL_PARAM(NSocks);
MCCL_PARAM(StripeMinBytes);
MCCL_PARAM(ConnectTimeoutMs);
MCCL_PARAM(AcceptTimeoutMs);
MCCL_PARAM(KeepaliveIdleSec);

mcclResult_t tcpEndpointStart(int rank, uint64_t nonce, TcpEndpoint** out);
// Unblock every thread parked in this endpoint's sockets; nothing is freed.
void         tcpEndpointShutdown(TcpEndpoint* ep);
void         tcpEndpointClose(TcpEndpoint* ep);

// Outbound bundle to `peer` (dials on first use).
mcclResult_t tcpDial(TcpEndpoint* ep, int peer, uint32_t kind, const char* ip, uint16_t port, TcpConn** out);
// Inbound bundle from `peer`: waits until the acceptor has every stripe (accept timeout applies).
mcclResult_t tcpAwait(TcpEndpoint* ep, int peer, uint32_t kind, TcpConn** out);
// Symmetric helper for collective bundles: the lower rank dials, the higher one waits.
mcclResult_t tcpConnectPair(TcpEndpoint* ep, int peer, uint32_t kind, const char* ip, uint16_t port, TcpConn** out);

mcclResult_t tcpSend(TcpConn* c, const void* buf, size_t bytes);
mcclResult_t tcpRecv(TcpConn* c, void* buf, size_t bytes);
// Shard i of a `bytes`-long message over n stripes is [bytes*i/n, bytes*(i+1)/n).
inline size_t stripeOffset(size_t bytes, int n, int i) { return (size_t)((__uint128_t)bytes * (unsigned)i / (unsigned)n); }

// Inbound p2p bundles currently known (for RecvAny) and the arrival counter to wait on.
void         tcpInboundP2p(TcpEndpoint* ep, std::vector<TcpConn*>* out, uint64_t* arrivals);

}  // namespace mccl
