// Send / Recv / RecvAny and call grouping.
// Inside mcclGroupStart/End nothing runs: Send/Recv and collectives are recorded per thread and issued
// by the outermost GroupEnd.  Per communicator: first the all-reduce calls that can share a kernel, as ONE
// launch (cuda transport); then the other recorded collectives, in program order; then all Send/Recv as one
// batch in which every (peer, direction) flow progresses concurrently, so a rank may post Send(p) and Recv(p)
// in either order without deadlock.  The calls of a group are independent of one another by contract (none may
// consume another's result), and on the cuda transport they must all name the same stream.  Batches of different communicators are
// issued concurrently so that two ranks that order their communicators differently cannot block each
// other.  Errors raised while recording are latched and returned by GroupEnd.
// Parity: src/p2p.cc:20-321 of the reference (which defers only Send/Recv; collectives there run at once).
#include <algorithm>
#include <chrono>
#include <cstring>
#include <map>
#include <arpa/inet.h>
#include <poll.h>
#include <thread>

#include "comm.h"
#include "../os/pool.h"

namespace mccl {

namespace {
struct GroupEntry {
  mcclComm* comm;
  bool isColl;
  P2pOp op;
  std::function<mcclResult_t()> launch;
  CollCall call;
};
struct GroupState {
  int depth = 0;
  mcclResult_t error = mcclSuccess;
  std::vector<GroupEntry> entries;
};
thread_local GroupState g_group;
}  // namespace

bool groupActive() { return g_group.depth > 0; }

mcclResult_t groupRecord(const P2pOp& op) {
  g_group.entries.push_back(GroupEntry{op.comm, false, op, nullptr, CollCall()});
  return mcclSuccess;
}
mcclResult_t groupRecordColl(mcclComm* comm, std::function<mcclResult_t()> launch, const CollCall& call) {
  g_group.entries.push_back(GroupEntry{comm, true, P2pOp{}, std::move(launch), call});
  return mcclSuccess;
}

// One batch on the tcp transport: outbound bundles are dialled by the sender, inbound ones awaited, then
// each (peer, direction) flow moves its messages in program order on its own thread.
mcclResult_t cpuRunP2pBatch(mcclComm* c, const std::vector<P2pOp>& ops) {
  std::map<std::pair<int, int>, std::vector<const P2pOp*>> flows;
  for (const P2pOp& op : ops) {
    if (op.peer == c->rank) continue;
    flows[{op.peer, op.isSend ? 1 : 0}].push_back(&op);
  }
  // Self sends pair with self receives in order.
  std::vector<const P2pOp*> selfS, selfR;
  for (const P2pOp& op : ops) if (op.peer == c->rank) (op.isSend ? selfS : selfR).push_back(&op);
  if (selfS.size() != selfR.size()) MCCLFAIL(mcclInvalidUsage);
  for (size_t i = 0; i < selfS.size(); ++i) {
    if (selfS[i]->bytes != selfR[i]->bytes) MCCLFAIL(mcclInvalidUsage);
    memmove(selfR[i]->buf, selfS[i]->buf, selfS[i]->bytes);
  }
  std::vector<std::pair<std::pair<int, int>, std::vector<const P2pOp*>>> list(flows.begin(), flows.end());
  // Dial first (never blocks on the peer), then wait for inbound bundles.
  std::vector<TcpConn*> conns(list.size(), nullptr);
  for (size_t i = 0; i < list.size(); ++i) {
    if (list[i].first.second != 1) continue;
    const int peer = list[i].first.first;
    struct in_addr a;
    a.s_addr = htonl(c->infos[peer].ip);
    char ip[64];
    inet_ntop(AF_INET, &a, ip, sizeof(ip));
    MCCLCHECK(tcpDial(c->ep, peer, CONN_P2P, ip, c->infos[peer].dataPort, &conns[i]));
  }
  for (size_t i = 0; i < list.size(); ++i)
    if (list[i].first.second == 0) MCCLCHECK(tcpAwait(c->ep, list[i].first.first, CONN_P2P, &conns[i]));
  return parallelFor(fanoutPool(), (int)list.size(), [&](int i) -> mcclResult_t {
    for (const P2pOp* op : list[i].second) {
      mcclResult_t rc = op->isSend ? tcpSend(conns[i], op->buf, op->bytes) : tcpRecv(conns[i], op->buf, op->bytes);
      if (rc != mcclSuccess) return rc;
    }
    return mcclSuccess;
  });
}

// First inbound p2p flow with data wins.  Polls the known inbound bundles in one-second ticks so that
// abort is noticed and bundles that arrive meanwhile are picked up.
mcclResult_t cpuRecvAny(mcclComm* c, void* buf, size_t bytes, int* src) {
  for (;;) {
    if (c->aborted.load()) MCCLFAIL(mcclInvalidUsage);
    std::vector<TcpConn*> in;
    tcpInboundP2p(c->ep, &in, nullptr);
    if (in.empty()) {
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
      continue;
    }
    std::vector<struct pollfd> pf(in.size());
    for (size_t i = 0; i < in.size(); ++i) pf[i] = {in[i]->fds[0], POLLIN, 0};
    int rc = poll(pf.data(), pf.size(), in.size() < (size_t)c->nRanks - 1 ? 50 : 1000);
    if (rc <= 0) continue;
    for (size_t i = 0; i < in.size(); ++i) {
      if (!(pf[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
      MCCLCHECK(tcpRecv(in[i], buf, bytes));
      *src = in[i]->peer;
      return mcclSuccess;
    }
  }
}

static mcclResult_t issueComm(mcclComm* comm, std::vector<GroupEntry>& entries) {
  mcclResult_t first = mcclSuccess;
  std::vector<P2pOp> batch;
  mcclStream_t stream = nullptr;
  // On the cuda transport a group is issued on ONE stream: its fused launches cannot honour an order between
  // streams, so a group that names several is refused rather than silently reordered.
  if (comm->cuda) {
    bool have = false;
    mcclStream_t seen = nullptr;
    for (GroupEntry& e : entries) {
      if (e.comm != comm) continue;
      const mcclStream_t s = e.isColl ? e.call.stream : e.op.stream;
      if (have && s != seen) {
        MCCL_WARN("the calls of one group on one communicator must use one stream");
        return noteFailure(mcclInvalidUsage, __FILE__, __LINE__);
      }
      have = true; seen = s;
    }
  }
  // The all-reduce calls of the group that can share a kernel go out as one launch, at the place of the first.
  std::vector<CollCall> calls;
  std::vector<size_t> callEntry;
  if (comm->cuda && comm->nRanks > 1) {
    for (size_t i = 0; i < entries.size(); ++i)
      if (entries[i].comm == comm && entries[i].isColl && entries[i].call.coll == mcclCollAllReduce) { calls.push_back(entries[i].call); callEntry.push_back(i); }
  }
  std::vector<char> fused(entries.size(), 0);
  if (calls.size() > 1) {
    std::vector<char> done;
    mcclResult_t rc = commLaunch(comm, [&]() { return cudaGroupAllReduce(comm, calls, &done); });
    if (rc != mcclSuccess) return rc;
    for (size_t k = 0; k < done.size(); ++k) if (done[k]) fused[callEntry[k]] = 1;
  }
  for (size_t i = 0; i < entries.size(); ++i) {
    GroupEntry& e = entries[i];
    if (e.comm != comm || fused[i]) continue;
    if (e.isColl) {
      mcclResult_t rc = e.launch();
      if (rc != mcclSuccess && first == mcclSuccess) first = rc;
    } else {
      batch.push_back(e.op);
      stream = e.op.stream;
    }
  }
  if (!batch.empty() && first == mcclSuccess) {
    mcclResult_t rc;
    if (comm->cuda) rc = commLaunch(comm, [=]() { return cudaP2pBatch(comm, batch, stream); });
    else rc = commLaunch(comm, [=]() { return cpuRunP2pBatch(comm, batch); });
    if (rc != mcclSuccess) first = rc;
  }
  return first;
}

}  // namespace mccl

using namespace mccl;

extern "C" {

mcclResult_t mcclGroupStart(void) {
  ++g_group.depth;
  return mcclSuccess;
}

mcclResult_t mcclGroupEnd(void) {
  if (g_group.depth <= 0) MCCLFAIL(mcclInvalidUsage);
  if (--g_group.depth > 0) return mcclSuccess;
  std::vector<GroupEntry> entries;
  entries.swap(g_group.entries);
  mcclResult_t latched = g_group.error;
  g_group.error = mcclSuccess;
  if (latched != mcclSuccess) return latched;
  std::vector<mcclComm*> comms;
  for (GroupEntry& e : entries)
    if (std::find(comms.begin(), comms.end(), e.comm) == comms.end()) comms.push_back(e.comm);
  if (comms.empty()) return mcclSuccess;
  if (comms.size() == 1) return issueComm(comms[0], entries);
  std::vector<mcclResult_t> rcs(comms.size(), mcclSuccess);
  std::vector<std::thread> threads;
  for (size_t i = 1; i < comms.size(); ++i)
    threads.emplace_back([&, i] { rcs[i] = issueComm(comms[i], entries); });
  rcs[0] = issueComm(comms[0], entries);
  for (auto& t : threads) t.join();
  for (mcclResult_t rc : rcs) if (rc != mcclSuccess) return rc;
  return mcclSuccess;
}

mcclResult_t mcclGroupAbort(void) {
  g_group.depth = 0;
  g_group.entries.clear();
  g_group.error = mcclSuccess;
  return mcclSuccess;
}

static mcclResult_t p2pCommon(mcclComm_t comm, void* buf, size_t count, mcclDataType_t dt, int peer, bool isSend,
                              mcclStream_t stream) {
  mcclResult_t bad = mcclSuccess;
  if (comm == nullptr) bad = mcclInvalidArgument;
  else if (mcclDataSize(dt) == 0 || peer < 0 || peer >= comm->nRanks || (buf == nullptr && count > 0)) bad = mcclInvalidArgument;
  else if (comm->aborted.load()) bad = mcclInvalidUsage;
  if (bad != mcclSuccess) {
    if (groupActive() && g_group.error == mcclSuccess) g_group.error = bad;
    return noteFailure(bad, __FILE__, __LINE__);
  }
  P2pOp op{comm, isSend, peer, buf, count * mcclDataSize(dt), stream};
  if (groupActive()) return groupRecord(op);
  std::vector<P2pOp> one{op};
  if (comm->cuda) return commLaunch(comm, [=]() { return cudaP2pBatch(comm, one, stream); });
  return commLaunch(comm, [=]() { return cpuRunP2pBatch(comm, one); });
}

mcclResult_t mcclSend(mcclComm_t comm, const void* sendbuff, size_t count, mcclDataType_t dt, int peer, mcclStream_t stream) {
  return p2pCommon(comm, const_cast<void*>(sendbuff), count, dt, peer, true, stream);
}
mcclResult_t mcclRecv(mcclComm_t comm, void* recvbuff, size_t count, mcclDataType_t dt, int peer, mcclStream_t stream) {
  return p2pCommon(comm, recvbuff, count, dt, peer, false, stream);
}

mcclResult_t mcclRecvAny(mcclComm_t comm, void* recvbuff, size_t count, mcclDataType_t dt, int* srcRank, mcclStream_t stream) {
  if (comm == nullptr || srcRank == nullptr || mcclDataSize(dt) == 0 || (recvbuff == nullptr && count > 0))
    MCCLFAIL(mcclInvalidArgument);
  if (groupActive()) MCCLFAIL(mcclInvalidUsage);     // the source is only known once it completes
  if (comm->aborted.load()) MCCLFAIL(mcclInvalidUsage);
  if (comm->nRanks < 2) MCCLFAIL(mcclInvalidUsage);
  const size_t bytes = count * mcclDataSize(dt);
  // The caller needs *srcRank on return, so this call is synchronous even on a non-blocking communicator.
  MCCLCHECK(mcclCommSynchronize(comm));
  if (comm->cuda) return cudaRecvAny(comm, recvbuff, bytes, srcRank, stream);
  mcclResult_t rc = cpuRecvAny(comm, recvbuff, bytes, srcRank);
  if (resultFatal(rc)) comm->asyncState.store((int)rc);
  return rc;
}

}  // extern "C"
