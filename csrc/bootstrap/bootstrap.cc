#include "bootstrap.h"

#include <cstdlib>
#include <cstring>
#include <map>
#include <random>
#include <arpa/inet.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <unistd.h>

#include "../os/pool.h"
#include "../os/socket.h"

namespace mccl {

DEFINE_MCCL_PARAM(BootstrapTimeoutSec, "BOOTSTRAP_TIMEOUT_SEC", 30);

namespace {
constexpr uint32_t kMagic = 0x6d63636cu;  // "mccl"
struct Hello { uint32_t magic; int32_t rank; int32_t n; uint32_t pad; uint64_t nonce; };
struct RoundHdr { uint32_t seq; uint32_t pad; uint64_t bytes; };

std::mutex gPendingMu;
std::map<uint64_t, int> gPendingListeners;  // nonce -> listening fd opened by bootstrapCreateId

uint64_t freshNonce() {
  std::random_device rd;
  uint64_t v = ((uint64_t)rd() << 32) ^ rd() ^ ((uint64_t)getpid() << 17);
  return v ? v : 1;
}
}  // namespace

mcclResult_t bootstrapCreateId(BootstrapId* id, const char* ip, bool alwaysListen) {
  memset(id, 0, sizeof(*id));
  if (ip == nullptr) ip = envStr("MCCL_BOOTSTRAP_IP");
  snprintf(id->ip, sizeof(id->ip), "%s", ip ? ip : "127.0.0.1");
  int64_t port = alwaysListen ? 0 : envInt("MCCL_BOOTSTRAP_PORT", 0);
  if (port > 0) {  // shared-by-convention id: every rank derives the same one from the environment
    id->port = (uint16_t)port;
    id->nonce = 0;
    return mcclSuccess;
  }
  int fd = -1;
  uint16_t bound = 0;
  MCCLCHECK(sockListen(id->ip, 0, &fd, &bound));
  id->port = bound;
  id->nonce = freshNonce();
  std::lock_guard<std::mutex> lk(gPendingMu);
  gPendingListeners[id->nonce] = fd;
  return mcclSuccess;
}

uint32_t bootstrapLocalIp(const Bootstrap* bs) {
  if (bs == nullptr || bs->rootFd < 0) return 0;
  struct sockaddr_in a;
  socklen_t len = sizeof(a);
  if (getsockname(bs->rootFd, (struct sockaddr*)&a, &len) != 0 || a.sin_family != AF_INET) return 0;
  return ntohl(a.sin_addr.s_addr);
}

static mcclResult_t rootCollect(Bootstrap* bs) {
  const int deadlineMs = (int)mcclParamBootstrapTimeoutSec() * 1000;
  int joined = 0;
  while (joined < bs->n - 1) {
    int fd = -1;
    mcclResult_t rc = sockAccept(bs->listenFd, deadlineMs, &fd);
    if (rc == mcclInProgress) {
      MCCL_WARN("bootstrap: only %d of %d ranks joined within %d ms", joined + 1, bs->n, deadlineMs);
      return mcclSystemError;
    }
    MCCLCHECK(rc);
    sockSetDeadline(fd, (int)mcclParamBootstrapTimeoutSec());
    Hello h;
    if (sockRecv(fd, &h, sizeof(h)) != mcclSuccess || h.magic != kMagic || h.nonce != bs->nonce ||
        h.n != bs->n || h.rank <= 0 || h.rank >= bs->n || bs->fds[h.rank] >= 0) {
      MCCL_WARN("bootstrap: dropping a dialer with a bad hello");
      sockClose(fd);
      continue;
    }
    bs->fds[h.rank] = fd;
    ++joined;
  }
  // Acknowledge only after everyone is in, so a successful init on any rank means the world is whole.
  for (int r = 1; r < bs->n; ++r) {
    uint32_t ok = kMagic;
    MCCLCHECK(sockSend(bs->fds[r], &ok, sizeof(ok)));
  }
  sockClose(bs->listenFd);
  bs->listenFd = -1;
  return mcclSuccess;
}

mcclResult_t bootstrapInit(const BootstrapId& id, int rank, int n, Bootstrap** out) {
  if (n < 1 || rank < 0 || rank >= n) MCCLFAIL(mcclInvalidArgument);
  Bootstrap* bs = new Bootstrap();
  bs->rank = rank;
  bs->n = n;
  bs->nonce = id.nonce;
  bs->fds.assign(n, -1);
  mcclResult_t rc = mcclSuccess;
  if (rank == 0) {
    {
      std::lock_guard<std::mutex> lk(gPendingMu);
      auto it = gPendingListeners.find(id.nonce);
      if (id.nonce != 0 && it != gPendingListeners.end()) {
        bs->listenFd = it->second;
        gPendingListeners.erase(it);
      }
    }
    if (bs->listenFd < 0) rc = sockListen(id.ip, id.port, &bs->listenFd, nullptr);
    if (rc == mcclSuccess && n > 1) rc = rootCollect(bs);
    if (rc == mcclSuccess && bs->listenFd >= 0) { sockClose(bs->listenFd); bs->listenFd = -1; }
  } else {
    const int retries = (int)mcclParamBootstrapTimeoutSec() * 10;  // 100 ms apart
    rc = sockConnect(id.ip, id.port, 1000, retries, &bs->rootFd);
    if (rc == mcclSuccess) {
      sockSetDeadline(bs->rootFd, (int)mcclParamBootstrapTimeoutSec());
      Hello h = {kMagic, rank, n, 0, id.nonce};
      rc = sockSend(bs->rootFd, &h, sizeof(h));
    }
    if (rc == mcclSuccess) {
      uint32_t ok = 0;
      rc = sockRecv(bs->rootFd, &ok, sizeof(ok));
      if (rc == mcclSuccess && ok != kMagic) rc = mcclRemoteError;
    }
  }
  if (rc != mcclSuccess) {
    bootstrapClose(bs);
    return noteFailure(rc == mcclInProgress ? mcclSystemError : rc, __FILE__, __LINE__);
  }
  *out = bs;
  return mcclSuccess;
}

mcclResult_t bootstrapAllGather(Bootstrap* bs, const void* send, void* recv, size_t bytes) {
  std::lock_guard<std::mutex> lk(bs->mu);
  if (bs->aborted) MCCLFAIL(mcclInvalidUsage);
  char* table = static_cast<char*>(recv);
  if (send != table + (size_t)bs->rank * bytes) memcpy(table + (size_t)bs->rank * bytes, send, bytes);
  const uint32_t seq = ++bs->seq;
  if (bs->n == 1) return mcclSuccess;
  if (faultInject("bootstrap")) MCCLFAIL(mcclSystemError);
  if (bs->rank == 0) {
    mcclResult_t rc = parallelFor(fanoutPool(), bs->n - 1, [&](int i) -> mcclResult_t {
      const int r = i + 1;
      RoundHdr h;
      mcclResult_t e = sockRecv(bs->fds[r], &h, sizeof(h));
      if (e != mcclSuccess) return e;
      if (h.seq != seq || h.bytes != bytes) {
        MCCL_WARN("bootstrap: rank %d is at round %u/%zu bytes, root at %u/%zu", r, h.seq, (size_t)h.bytes, seq, bytes);
        return mcclRemoteError;
      }
      return sockRecv(bs->fds[r], table + (size_t)r * bytes, bytes);
    });
    MCCLCHECK(rc);
    rc = parallelFor(fanoutPool(), bs->n - 1, [&](int i) -> mcclResult_t {
      return sockSend(bs->fds[i + 1], table, bytes * (size_t)bs->n);
    });
    MCCLCHECK(rc);
  } else {
    RoundHdr h = {seq, 0, bytes};
    MCCLCHECK(sockSend(bs->rootFd, &h, sizeof(h)));
    MCCLCHECK(sockSend(bs->rootFd, table + (size_t)bs->rank * bytes, bytes));
    MCCLCHECK(sockRecv(bs->rootFd, table, bytes * (size_t)bs->n));
  }
  return mcclSuccess;
}

mcclResult_t bootstrapBarrier(Bootstrap* bs) {
  std::vector<int32_t> v(bs->n, 0);
  int32_t mine = bs->rank;
  return bootstrapAllGather(bs, &mine, v.data(), sizeof(int32_t));
}

void bootstrapAbort(Bootstrap* bs) {
  if (bs == nullptr) return;
  bs->aborted = true;
  sockShutdown(bs->rootFd);
  sockShutdown(bs->listenFd);
  for (int fd : bs->fds) sockShutdown(fd);
}

void bootstrapClose(Bootstrap* bs) {
  if (bs == nullptr) return;
  sockClose(bs->rootFd);
  sockClose(bs->listenFd);
  for (int fd : bs->fds) sockClose(fd);
  delete bs;
}

}  // namespace mccl
