#include "tcp.h"

#include <chrono>
#include <cstring>

#include "../os/pool.h"
#include "../os/socket.h"

namespace mccl {

DEFINE_MCCL_PARAM(NSocks, "NSOCKS", 2);
DEFINE_MCCL_PARAM(StripeMinBytes, "STRIPE_MIN_BYTES", 256 * 1024);
DEFINE_MCCL_PARAM(ConnectTimeoutMs, "CONNECT_TIMEOUT_MS", 5000);
DEFINE_MCCL_PARAM(AcceptTimeoutMs, "ACCEPT_TIMEOUT_MS", 30000);
DEFINE_MCCL_PARAM(KeepaliveIdleSec, "KEEPALIVE_IDLE_SEC", 10);

namespace {
struct StripeHello {
  uint64_t nonce;
  int32_t  srcRank;
  uint32_t kind;
  uint32_t shard;
  uint32_t nSocks;
};

int stripeCount() {
  int64_t n = mcclParamNSocks();
  if (n < 1) n = 1;
  if (n > kMaxStripes) n = kMaxStripes;
  return (int)n;
}

// Outbound and inbound p2p bundles to the same peer are different flows.
uint64_t connKey(int peer, uint32_t kind, bool inbound) {
  return ((uint64_t)(uint32_t)peer << 8) | (kind << 1) | ((kind == CONN_P2P && inbound) ? 1u : 0u);
}

void tuneData(int fd, int nSocks) {
  // The per-connection buffer budget is split across the stripes.
  sockSetBuffers(fd, (int)(mcclParamSocketBufKb() * 1024 / nSocks));
  sockSetKeepalive(fd, (int)mcclParamKeepaliveIdleSec());
}

void acceptLoop(TcpEndpoint* ep) {
  for (;;) {
    {
      std::lock_guard<std::mutex> lk(ep->mu);
      if (ep->stop) return;
    }
    int fd = -1;
    mcclResult_t rc = sockAccept(ep->listenFd, 200, &fd);
    if (rc == mcclInProgress) continue;
    if (rc != mcclSuccess) {
      std::lock_guard<std::mutex> lk(ep->mu);
      if (ep->stop) return;
      continue;
    }
    // A dialer that connects and then stalls must not wedge the listener: bounded header read.
    sockSetDeadline(fd, 5);
    StripeHello h;
    if (sockRecv(fd, &h, sizeof(h)) != mcclSuccess || h.nonce != ep->nonce || h.nSocks == 0 ||
        h.nSocks > (uint32_t)kMaxStripes || h.shard >= h.nSocks) {
      MCCL_WARN("tcp: dropping a data connection with a bad preamble");
      sockClose(fd);
      continue;
    }
    sockSetDeadline(fd, 0);
    tuneData(fd, (int)h.nSocks);
    std::lock_guard<std::mutex> lk(ep->mu);
    const uint64_t key = connKey(h.srcRank, h.kind, true);
    TcpConn*& c = ep->partial[key];
    if (c == nullptr) {
      c = new TcpConn();
      c->peer = h.srcRank;
      c->kind = h.kind;
      c->nSocks = (int)h.nSocks;
      for (int i = 0; i < kMaxStripes; ++i) c->fds[i] = -1;
    }
    c->fds[h.shard] = fd;
    bool whole = true;
    for (int i = 0; i < c->nSocks; ++i) whole = whole && c->fds[i] >= 0;
    if (whole) {
      ep->conns[key] = c;
      ep->partial.erase(key);
      ++ep->arrivals;
      ep->cv.notify_all();
    }
  }
}
}  // namespace

mcclResult_t tcpEndpointStart(int rank, uint64_t nonce, TcpEndpoint** out) {
  TcpEndpoint* ep = new TcpEndpoint();
  ep->rank = rank;
  ep->nonce = nonce;
  mcclResult_t rc = sockListen(nullptr, 0, &ep->listenFd, &ep->port);
  if (rc != mcclSuccess) {
    delete ep;
    return rc;
  }
  ep->acceptor = std::thread(acceptLoop, ep);
  *out = ep;
  return mcclSuccess;
}

void tcpEndpointShutdown(TcpEndpoint* ep) {
  if (ep == nullptr) return;
  std::lock_guard<std::mutex> lk(ep->mu);
  ep->stop = true;
  for (auto& kv : ep->conns)
    for (int i = 0; i < kv.second->nSocks; ++i) sockShutdown(kv.second->fds[i]);
  for (auto& kv : ep->partial)
    for (int i = 0; i < kv.second->nSocks; ++i) sockShutdown(kv.second->fds[i]);
  ep->cv.notify_all();
}

void tcpEndpointClose(TcpEndpoint* ep) {
  if (ep == nullptr) return;
  tcpEndpointShutdown(ep);
  if (ep->acceptor.joinable()) ep->acceptor.join();
  sockClose(ep->listenFd);
  for (auto* m : {&ep->conns, &ep->partial})
    for (auto& kv : *m) {
      for (int i = 0; i < kv.second->nSocks; ++i) sockClose(kv.second->fds[i]);
      delete kv.second;
    }
  delete ep;
}

mcclResult_t tcpDial(TcpEndpoint* ep, int peer, uint32_t kind, const char* ip, uint16_t port, TcpConn** out) {
  const uint64_t key = connKey(peer, kind, false);
  {
    std::lock_guard<std::mutex> lk(ep->mu);
    if (ep->stop) MCCLFAIL(mcclInvalidUsage);
    auto it = ep->conns.find(key);
    if (it != ep->conns.end()) { *out = it->second; return mcclSuccess; }
  }
  TcpConn* c = new TcpConn();
  c->peer = peer;
  c->kind = kind;
  c->nSocks = stripeCount();
  for (int i = 0; i < kMaxStripes; ++i) c->fds[i] = -1;
  mcclResult_t rc = mcclSuccess;
  for (int i = 0; i < c->nSocks && rc == mcclSuccess; ++i) {
    rc = sockConnect(ip, port, (int)mcclParamConnectTimeoutMs(), 50, &c->fds[i]);
    if (rc != mcclSuccess) break;
    tuneData(c->fds[i], c->nSocks);
    StripeHello h = {ep->nonce, ep->rank, kind, (uint32_t)i, (uint32_t)c->nSocks};
    rc = sockSend(c->fds[i], &h, sizeof(h));
  }
  if (rc != mcclSuccess) {
    for (int i = 0; i < c->nSocks; ++i) sockClose(c->fds[i]);
    delete c;
    return noteFailure(rc, __FILE__, __LINE__);
  }
  std::lock_guard<std::mutex> lk(ep->mu);
  ep->conns[key] = c;
  *out = c;
  return mcclSuccess;
}

mcclResult_t tcpAwait(TcpEndpoint* ep, int peer, uint32_t kind, TcpConn** out) {
  const uint64_t key = connKey(peer, kind, true);
  std::unique_lock<std::mutex> lk(ep->mu);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(mcclParamAcceptTimeoutMs());
  for (;;) {
    if (ep->stop) MCCLFAIL(mcclInvalidUsage);
    auto it = ep->conns.find(key);
    if (it != ep->conns.end()) { *out = it->second; return mcclSuccess; }
    if (ep->cv.wait_until(lk, deadline) == std::cv_status::timeout) {
      MCCL_WARN("tcp: rank %d never connected (kind %u)", peer, kind);
      return mcclSystemError;
    }
  }
}

mcclResult_t tcpConnectPair(TcpEndpoint* ep, int peer, uint32_t kind, const char* ip, uint16_t port, TcpConn** out) {
  if (ep->rank < peer) return tcpDial(ep, peer, kind, ip, port, out);
  return tcpAwait(ep, peer, kind, out);
}

static mcclResult_t stripedXfer(TcpConn* c, char* buf, size_t bytes, bool isSend) {
  if (bytes == 0) return mcclSuccess;
  if (c->nSocks == 1 || bytes < (size_t)mcclParamStripeMinBytes()) {
    return isSend ? sockSend(c->fds[0], buf, bytes) : sockRecv(c->fds[0], buf, bytes);
  }
  return parallelFor(stripePool(), c->nSocks, [&](int i) -> mcclResult_t {
    const size_t lo = stripeOffset(bytes, c->nSocks, i), hi = stripeOffset(bytes, c->nSocks, i + 1);
    return isSend ? sockSend(c->fds[i], buf + lo, hi - lo) : sockRecv(c->fds[i], buf + lo, hi - lo);
  });
}

mcclResult_t tcpSend(TcpConn* c, const void* buf, size_t bytes) {
  return stripedXfer(c, const_cast<char*>(static_cast<const char*>(buf)), bytes, true);
}
mcclResult_t tcpRecv(TcpConn* c, void* buf, size_t bytes) {
  return stripedXfer(c, static_cast<char*>(buf), bytes, false);
}

void tcpInboundP2p(TcpEndpoint* ep, std::vector<TcpConn*>* out, uint64_t* arrivals) {
  std::lock_guard<std::mutex> lk(ep->mu);
  out->clear();
  for (auto& kv : ep->conns)
    if (kv.second->kind == CONN_P2P && (kv.first & 1u)) out->push_back(kv.second);
  if (arrivals) *arrivals = ep->arrivals;
}

}  // namespace mccl
