// Collective algorithms of the tcp transport: ring (single and counter-rotating dual), tree (hub star,
// spanning tree or double-binary tree) and direct one-shot, for all five collectives, on host buffers.
// Index math follows the reference so that results are reproducible across the two libraries:
// ring all-reduce src/device/all_reduce.h:63-144, tree all-reduce :148-225, direct :17-60; all-gather
// src/device/all_gather.h:18-139; reduce-scatter src/device/reduce_scatter.h:19-210; broadcast
// src/device/broadcast.h:16-104; reduce src/device/reduce.h:20-179; subtree packing
// src/device/treeflow.h:9-27.  Every fold runs in ascending rank order so all ranks get identical bytes.
#include <algorithm>
#include <cstring>

#include "../comm/comm.h"
#include "../device/host_reduce.h"
#include "../os/pool.h"

namespace mccl {

DEFINE_MCCL_PARAM(DualRings, "DUAL_RINGS", 1);
DEFINE_MCCL_PARAM(DualRingMinBytes, "DUAL_RING_MIN_BYTES", 1 << 20);
DEFINE_MCCL_PARAM(PipelineChunks, "PIPELINE_CHUNKS", 4);

namespace {

inline int wrap(int v, int n) { v %= n; return v < 0 ? v + n : v; }

struct Ctx {
  mcclComm* c;
  int n, r;
  size_t es;
  mcclDataType_t dt;
  mcclRedOp_t op;   // avg already mapped to sum
};

mcclResult_t sendTo(mcclComm* c, int peer, uint32_t kind, const void* buf, size_t bytes) {
  TcpConn* conn = nullptr;
  MCCLCHECK(commPeerConn(c, peer, kind, &conn));
  return tcpSend(conn, buf, bytes);
}
mcclResult_t recvFrom(mcclComm* c, int peer, uint32_t kind, void* buf, size_t bytes) {
  TcpConn* conn = nullptr;
  MCCLCHECK(commPeerConn(c, peer, kind, &conn));
  return tcpRecv(conn, buf, bytes);
}

// send || recv, the two halves of one ring step.
mcclResult_t sendRecv(mcclComm* c, uint32_t kind, int sendPeer, const void* sbuf, size_t sbytes,
                      int recvPeer, void* rbuf, size_t rbytes) {
  TcpConn *sc = nullptr, *rc = nullptr;
  // Connections are resolved before the parallel section so that dial/accept order is deterministic.
  MCCLCHECK(commPeerConn(c, sendPeer, kind, &sc));
  MCCLCHECK(commPeerConn(c, recvPeer, kind, &rc));
  return parallelFor(fanoutPool(), 2, [&](int i) -> mcclResult_t {
    return i == 0 ? tcpSend(sc, sbuf, sbytes) : tcpRecv(rc, rbuf, rbytes);
  });
}

struct RingLeg {
  uint32_t kind;
  int dir;          // +1: along ring.next, -1: against it
  int sendPeer, recvPeer;
};

RingLeg makeLeg(const mcclComm* c, int dir) {
  RingLeg l;
  l.dir = dir;
  l.kind = dir > 0 ? CONN_COLL_A : CONN_COLL_B;
  l.sendPeer = dir > 0 ? c->chan.ring.next : c->chan.ring.prev;
  l.recvPeer = dir > 0 ? c->chan.ring.prev : c->chan.ring.next;
  return l;
}

bool useDualRing(const mcclComm* c, size_t bytes, size_t count) {
  return mcclParamDualRings() != 0 && c->nRanks >= 3 && bytes >= (size_t)mcclParamDualRingMinBytes() &&
         count >= 2 * (size_t)c->nRanks;
}

// ---------------------------------------------------------------------------------------------------
// all-reduce
// ---------------------------------------------------------------------------------------------------
mcclResult_t ringAllReduceLeg(const Ctx& x, const RingLeg& leg, char* buf, size_t cnt, char* staging) {
  const int n = x.n, r = x.r, d = leg.dir;
  auto off = [&](int i) { return chunkOff(cnt, n, i) * x.es; };
  auto len = [&](int i) { return (chunkOff(cnt, n, i + 1) - chunkOff(cnt, n, i)); };
  for (int i = 0; i < n - 1; ++i) {            // reduce phase
    const int s = wrap(r - d * i, n), t = wrap(r - d * (i + 1), n);
    MCCLCHECK(sendRecv(x.c, leg.kind, leg.sendPeer, buf + off(s), len(s) * x.es, leg.recvPeer, staging, len(t) * x.es));
    MCCLCHECK(hostReduce(buf + off(t), staging, len(t), x.dt, x.op));
  }
  for (int i = 0; i < n - 1; ++i) {            // gather phase
    const int s = wrap(r - d * (i - 1), n), t = wrap(r - d * i, n);
    MCCLCHECK(sendRecv(x.c, leg.kind, leg.sendPeer, buf + off(s), len(s) * x.es, leg.recvPeer, buf + off(t), len(t) * x.es));
  }
  return mcclSuccess;
}

mcclResult_t ringAllReduce(const Ctx& x, char* buf, size_t count) {
  const size_t bytes = count * x.es;
  void* st = nullptr;
  if (useDualRing(x.c, bytes, count)) {
    const size_t half = count / 2;
    const size_t legStage = ((count - half) / x.n + 2) * x.es;
    MCCLCHECK(commReserveStaging(x.c, 2 * legStage, &st));
    char* sp = static_cast<char*>(st);
    return parallelFor(fanoutPool(), 2, [&](int k) -> mcclResult_t {
      return k == 0 ? ringAllReduceLeg(x, makeLeg(x.c, +1), buf, half, sp)
                    : ringAllReduceLeg(x, makeLeg(x.c, -1), buf + half * x.es, count - half, sp + legStage);
    });
  }
  MCCLCHECK(commReserveStaging(x.c, (count / x.n + 2) * x.es, &st));
  return ringAllReduceLeg(x, makeLeg(x.c, +1), buf, count, static_cast<char*>(st));
}

// Fold the children's data for [buf, buf+cnt) into buf: receive from all children in parallel into
// staging slices, then fold them in child order.
mcclResult_t reduceFromChildren(const Ctx& x, uint32_t kind, const std::vector<int>& down, char* buf, size_t cnt, char* staging) {
  const int nc = (int)down.size();
  if (nc == 0 || cnt == 0) return mcclSuccess;
  std::vector<TcpConn*> conns(nc);
  for (int k = 0; k < nc; ++k) MCCLCHECK(commPeerConn(x.c, down[k], kind, &conns[k]));
  MCCLCHECK(parallelFor(fanoutPool(), nc, [&](int k) -> mcclResult_t {
    return tcpRecv(conns[k], staging + (size_t)k * cnt * x.es, cnt * x.es);
  }));
  return hostReduceMulti(buf, staging, cnt, nc, cnt, x.dt, x.op);
}

mcclResult_t sendToChildren(const Ctx& x, uint32_t kind, const std::vector<int>& down, const char* buf, size_t bytes) {
  const int nc = (int)down.size();
  if (nc == 0 || bytes == 0) return mcclSuccess;
  std::vector<TcpConn*> conns(nc);
  for (int k = 0; k < nc; ++k) MCCLCHECK(commPeerConn(x.c, down[k], kind, &conns[k]));
  return parallelFor(fanoutPool(), nc, [&](int k) -> mcclResult_t { return tcpSend(conns[k], buf, bytes); });
}

mcclResult_t treeUp(const Ctx& x, uint32_t kind, const TreeView& t, char* buf, size_t cnt, char* staging) {
  MCCLCHECK(reduceFromChildren(x, kind, t.down, buf, cnt, staging));
  if (t.up >= 0) MCCLCHECK(sendTo(x.c, t.up, kind, buf, cnt * x.es));
  return mcclSuccess;
}
mcclResult_t treeDown(const Ctx& x, uint32_t kind, const TreeView& t, char* buf, size_t cnt) {
  if (t.up >= 0) MCCLCHECK(recvFrom(x.c, t.up, kind, buf, cnt * x.es));
  return sendToChildren(x, kind, t.down, buf, cnt * x.es);
}

mcclResult_t treeAllReduce(const Ctx& x, char* buf, size_t count) {
  const Channel& ch = x.c->chan;
  void* st = nullptr;
  if (ch.dtree && count >= 2) {
    // Two complementary trees, each reducing one half over its own connection set.
    const size_t half = count / 2;
    const size_t a = std::max(ch.tree.down.size(), (size_t)1) * half * x.es;
    const size_t b = std::max(ch.treeB.down.size(), (size_t)1) * (count - half) * x.es;
    MCCLCHECK(commReserveStaging(x.c, a + b, &st));
    char* sp = static_cast<char*>(st);
    return parallelFor(fanoutPool(), 2, [&](int k) -> mcclResult_t {
      if (k == 0) {
        MCCLCHECK(treeUp(x, CONN_COLL_A, ch.tree, buf, half, sp));
        return treeDown(x, CONN_COLL_A, ch.tree, buf, half);
      }
      MCCLCHECK(treeUp(x, CONN_COLL_B, ch.treeB, buf + half * x.es, count - half, sp + a));
      return treeDown(x, CONN_COLL_B, ch.treeB, buf + half * x.es, count - half);
    });
  }
  // Single tree, pipelined: chunk i+1 climbs while chunk i descends.
  int K = (count * x.es >= (1u << 20)) ? (int)mcclParamPipelineChunks() : 1;
  if (K < 1) K = 1;
  if ((size_t)K > count) K = (int)std::max<size_t>(count, 1);
  const size_t maxChunk = count / K + 1;
  const size_t fan = std::max(ch.tree.down.size(), (size_t)1);
  MCCLCHECK(commReserveStaging(x.c, fan * maxChunk * x.es, &st));
  char* sp = static_cast<char*>(st);
  auto off = [&](int i) { return chunkOff(count, K, i); };
  auto up = [&](int i) { return treeUp(x, CONN_COLL_A, ch.tree, buf + off(i) * x.es, off(i + 1) - off(i), sp); };
  auto down = [&](int i) { return treeDown(x, CONN_COLL_A, ch.tree, buf + off(i) * x.es, off(i + 1) - off(i)); };
  MCCLCHECK(up(0));
  for (int i = 0; i < K; ++i) {
    if (i + 1 < K) {
      MCCLCHECK(parallelFor(fanoutPool(), 2, [&](int k) -> mcclResult_t { return k == 0 ? up(i + 1) : down(i); }));
    } else {
      MCCLCHECK(down(i));
    }
  }
  return mcclSuccess;
}

// One-shot: everyone sends its whole buffer to everyone; slot k holds rank k's contribution and the fold
// runs over slots 0..n-1 in that order on every rank.
mcclResult_t directAllReduce(const Ctx& x, const char* send, char* recv, size_t count) {
  const size_t bytes = count * x.es;
  void* st = nullptr;
  MCCLCHECK(commReserveStaging(x.c, bytes * x.n, &st));
  char* slots = static_cast<char*>(st);
  std::vector<TcpConn*> conns(x.n, nullptr);
  for (int p = 0; p < x.n; ++p) if (p != x.r) MCCLCHECK(commPeerConn(x.c, p, CONN_COLL_A, &conns[p]));
  memcpy(slots + (size_t)x.r * bytes, send, bytes);
  MCCLCHECK(parallelFor(fanoutPool(), 2 * x.n, [&](int i) -> mcclResult_t {
    const int p = i / 2;
    if (p == x.r) return mcclSuccess;
    return (i & 1) ? tcpRecv(conns[p], slots + (size_t)p * bytes, bytes) : tcpSend(conns[p], slots + (size_t)x.r * bytes, bytes);
  }));
  memcpy(recv, slots, bytes);
  return hostReduceMulti(recv, slots + bytes, count, x.n - 1, count, x.dt, x.op);
}

// ---------------------------------------------------------------------------------------------------
// all-gather
// ---------------------------------------------------------------------------------------------------
mcclResult_t ringAllGatherLeg(const Ctx& x, const RingLeg& leg, char* recv, size_t slotBytes, size_t lo, size_t hi) {
  // Moves bytes [lo, hi) of every slot.
  const int n = x.n, r = x.r, d = leg.dir;
  for (int i = 0; i < n - 1; ++i) {
    const int s = wrap(r - d * i, n), t = wrap(r - d * (i + 1), n);
    MCCLCHECK(sendRecv(x.c, leg.kind, leg.sendPeer, recv + (size_t)s * slotBytes + lo, hi - lo,
                       leg.recvPeer, recv + (size_t)t * slotBytes + lo, hi - lo));
  }
  return mcclSuccess;
}

mcclResult_t ringAllGather(const Ctx& x, char* recv, size_t sendcount) {
  const size_t slot = sendcount * x.es;
  if (useDualRing(x.c, slot * x.n, sendcount)) {
    const size_t half = (sendcount / 2) * x.es;
    return parallelFor(fanoutPool(), 2, [&](int k) -> mcclResult_t {
      return k == 0 ? ringAllGatherLeg(x, makeLeg(x.c, +1), recv, slot, 0, half)
                    : ringAllGatherLeg(x, makeLeg(x.c, -1), recv, slot, half, slot);
    });
  }
  return ringAllGatherLeg(x, makeLeg(x.c, +1), recv, slot, 0, slot);
}

mcclResult_t directAllGather(const Ctx& x, char* recv, size_t slot) {
  std::vector<TcpConn*> conns(x.n, nullptr);
  for (int p = 0; p < x.n; ++p) if (p != x.r) MCCLCHECK(commPeerConn(x.c, p, CONN_COLL_A, &conns[p]));
  return parallelFor(fanoutPool(), 2 * x.n, [&](int i) -> mcclResult_t {
    const int p = i / 2;
    if (p == x.r) return mcclSuccess;
    return (i & 1) ? tcpRecv(conns[p], recv + (size_t)p * slot, slot) : tcpSend(conns[p], recv + (size_t)x.r * slot, slot);
  });
}

// Ranks of the subtree rooted at `node` (ascending), from the global parent table.
std::vector<int> subtreeRanks(const std::vector<int>& parent, int node) {
  const int n = (int)parent.size();
  std::vector<int> out;
  for (int r = 0; r < n; ++r) {
    int a = r, guard = 0;
    while (a >= 0 && a != node && guard++ <= n) a = parent[a];
    if (a == node) out.push_back(r);
  }
  return out;
}

// Tree all-gather: packed subtree slots climb (ascending rank order on both ends), the full buffer descends.
mcclResult_t treeAllGather(const Ctx& x, char* recv, size_t slot) {
  const Channel& ch = x.c->chan;
  const std::vector<int>& parent = ch.treeParent;
  void* st = nullptr;
  MCCLCHECK(commReserveStaging(x.c, slot * x.n, &st));
  char* pack = static_cast<char*>(st);
  std::vector<std::vector<int>> sub;
  for (int child : ch.tree.down) sub.push_back(subtreeRanks(parent, child));
  const int nc = (int)ch.tree.down.size();
  std::vector<TcpConn*> conns(nc);
  std::vector<size_t> offs(nc + 1, 0);
  for (int k = 0; k < nc; ++k) {
    MCCLCHECK(commPeerConn(x.c, ch.tree.down[k], CONN_COLL_A, &conns[k]));
    offs[k + 1] = offs[k] + sub[k].size() * slot;
  }
  MCCLCHECK(parallelFor(fanoutPool(), nc, [&](int k) -> mcclResult_t {
    return tcpRecv(conns[k], pack + offs[k], sub[k].size() * slot);
  }));
  for (int k = 0; k < nc; ++k)
    for (size_t j = 0; j < sub[k].size(); ++j) memcpy(recv + (size_t)sub[k][j] * slot, pack + offs[k] + j * slot, slot);
  if (ch.tree.up >= 0) {
    std::vector<int> mineSub = subtreeRanks(parent, x.r);
    for (size_t j = 0; j < mineSub.size(); ++j) memcpy(pack + j * slot, recv + (size_t)mineSub[j] * slot, slot);
    MCCLCHECK(sendTo(x.c, ch.tree.up, CONN_COLL_A, pack, mineSub.size() * slot));
    MCCLCHECK(recvFrom(x.c, ch.tree.up, CONN_COLL_A, recv, slot * x.n));
  }
  return sendToChildren(x, CONN_COLL_A, ch.tree.down, recv, slot * x.n);
}

// ---------------------------------------------------------------------------------------------------
// reduce-scatter
// ---------------------------------------------------------------------------------------------------
mcclResult_t ringReduceScatterLeg(const Ctx& x, const RingLeg& leg, const char* send, char* recv, size_t blk,
                                  size_t lo, size_t hi, char* scratch) {
  // Elements [lo, hi) of every block.  Three scratch buffers: receive staging and two alternating folds,
  // so the caller's send buffer is never written.
  const int n = x.n, r = x.r, d = leg.dir;
  const size_t cnt = hi - lo, bytes = cnt * x.es;
  char* recvS = scratch;
  char* fold[2] = {scratch + bytes, scratch + 2 * bytes};
  const char* prevFold = nullptr;
  for (int i = 0; i < n - 1; ++i) {
    const int sIdx = wrap(r - d * (i + 1), n), dIdx = wrap(r - d * (i + 2), n);
    const char* sp = (i == 0) ? send + ((size_t)sIdx * blk + lo) * x.es : prevFold;
    MCCLCHECK(sendRecv(x.c, leg.kind, leg.sendPeer, sp, bytes, leg.recvPeer, recvS, bytes));
    char* dst = (i == n - 2) ? recv + lo * x.es : fold[i & 1];
    MCCLCHECK(hostReduceOut(dst, send + ((size_t)dIdx * blk + lo) * x.es, recvS, cnt, x.dt, x.op));
    prevFold = dst;
  }
  return mcclSuccess;
}

mcclResult_t ringReduceScatter(const Ctx& x, const char* send, char* recv, size_t recvcount) {
  void* sc = nullptr;
  if (useDualRing(x.c, recvcount * x.es * x.n, recvcount)) {
    const size_t half = recvcount / 2;
    const size_t legBytes = 3 * (recvcount - half) * x.es;
    MCCLCHECK(commReserveScratch(x.c, 2 * legBytes, &sc));
    char* sp = static_cast<char*>(sc);
    return parallelFor(fanoutPool(), 2, [&](int k) -> mcclResult_t {
      return k == 0 ? ringReduceScatterLeg(x, makeLeg(x.c, +1), send, recv, recvcount, 0, half, sp)
                    : ringReduceScatterLeg(x, makeLeg(x.c, -1), send, recv, recvcount, half, recvcount, sp + legBytes);
    });
  }
  MCCLCHECK(commReserveScratch(x.c, 3 * recvcount * x.es, &sc));
  return ringReduceScatterLeg(x, makeLeg(x.c, +1), send, recv, recvcount, 0, recvcount, static_cast<char*>(sc));
}

mcclResult_t directReduceScatter(const Ctx& x, const char* send, char* recv, size_t recvcount) {
  const size_t blk = recvcount * x.es;
  void* st = nullptr;
  MCCLCHECK(commReserveStaging(x.c, blk * x.n, &st));
  char* slots = static_cast<char*>(st);
  std::vector<TcpConn*> conns(x.n, nullptr);
  for (int p = 0; p < x.n; ++p) if (p != x.r) MCCLCHECK(commPeerConn(x.c, p, CONN_COLL_A, &conns[p]));
  memcpy(slots + (size_t)x.r * blk, send + (size_t)x.r * blk, blk);
  MCCLCHECK(parallelFor(fanoutPool(), 2 * x.n, [&](int i) -> mcclResult_t {
    const int p = i / 2;
    if (p == x.r) return mcclSuccess;
    return (i & 1) ? tcpRecv(conns[p], slots + (size_t)p * blk, blk) : tcpSend(conns[p], send + (size_t)p * blk, blk);
  }));
  memcpy(recv, slots, blk);
  return hostReduceMulti(recv, slots + blk, recvcount, x.n - 1, recvcount, x.dt, x.op);
}

// Tree reduce-scatter: the whole input is folded up the tree, then each child receives the packed
// blocks of its subtree and keeps its own.
mcclResult_t treeReduceScatter(const Ctx& x, const char* send, char* recv, size_t recvcount) {
  const Channel& ch = x.c->chan;
  const size_t blk = recvcount * x.es, total = recvcount * x.n;
  void *sc = nullptr, *st = nullptr;
  MCCLCHECK(commReserveScratch(x.c, 2 * total * x.es, &sc));
  MCCLCHECK(commReserveStaging(x.c, std::max(ch.tree.down.size(), (size_t)1) * total * x.es, &st));
  char* work = static_cast<char*>(sc);
  char* pack = work + total * x.es;
  memcpy(work, send, total * x.es);
  MCCLCHECK(treeUp(x, CONN_COLL_A, ch.tree, work, total, static_cast<char*>(st)));
  // Down: my subtree's blocks arrive packed in ascending rank order.
  std::vector<int> mineSub = subtreeRanks(ch.treeParent, x.r);
  if (ch.tree.up >= 0) {
    MCCLCHECK(recvFrom(x.c, ch.tree.up, CONN_COLL_A, pack, mineSub.size() * blk));
    for (size_t j = 0; j < mineSub.size(); ++j) memcpy(work + (size_t)mineSub[j] * blk, pack + j * blk, blk);
  }
  memcpy(recv, work + (size_t)x.r * blk, blk);
  const int nc = (int)ch.tree.down.size();
  std::vector<TcpConn*> conns(nc);
  std::vector<std::vector<int>> sub(nc);
  std::vector<size_t> offs(nc + 1, 0);
  for (int k = 0; k < nc; ++k) {
    MCCLCHECK(commPeerConn(x.c, ch.tree.down[k], CONN_COLL_A, &conns[k]));
    sub[k] = subtreeRanks(ch.treeParent, ch.tree.down[k]);
    offs[k + 1] = offs[k] + sub[k].size() * blk;
    for (size_t j = 0; j < sub[k].size(); ++j) memcpy(pack + offs[k] + j * blk, work + (size_t)sub[k][j] * blk, blk);
  }
  return parallelFor(fanoutPool(), nc, [&](int k) -> mcclResult_t {
    return tcpSend(conns[k], pack + offs[k], sub[k].size() * blk);
  });
}

// ---------------------------------------------------------------------------------------------------
// broadcast
// ---------------------------------------------------------------------------------------------------
mcclResult_t ringBroadcast(const Ctx& x, char* buf, size_t bytes, int root) {
  const int n = x.n;
  const RingLeg leg = makeLeg(x.c, +1);
  const int dist = wrap(x.r - root, n);
  int K = (n > 2 && bytes >= (1u << 20)) ? (int)mcclParamPipelineChunks() : 1;
  if (K < 1) K = 1;
  if ((size_t)K > bytes) K = 1;
  auto off = [&](int i) { return chunkOff(bytes, K, i); };
  if (dist == 0) {
    for (int i = 0; i < K; ++i) MCCLCHECK(sendTo(x.c, leg.sendPeer, leg.kind, buf + off(i), off(i + 1) - off(i)));
    return mcclSuccess;
  }
  if (dist == n - 1) {   // the rank before the root only receives
    for (int i = 0; i < K; ++i) MCCLCHECK(recvFrom(x.c, leg.recvPeer, leg.kind, buf + off(i), off(i + 1) - off(i)));
    return mcclSuccess;
  }
  MCCLCHECK(recvFrom(x.c, leg.recvPeer, leg.kind, buf + off(0), off(1) - off(0)));
  for (int i = 0; i + 1 < K; ++i)
    MCCLCHECK(sendRecv(x.c, leg.kind, leg.sendPeer, buf + off(i), off(i + 1) - off(i),
                       leg.recvPeer, buf + off(i + 1), off(i + 2) - off(i + 1)));
  return sendTo(x.c, leg.sendPeer, leg.kind, buf + off(K - 1), off(K) - off(K - 1));
}

// Tree broadcast from an arbitrary root: the root hands the data to the tree's root (one hop) unless it
// is the tree's root itself; then the data flows down.  A parent skips a child that is the broadcast root
// (it already has the data), and the broadcast root forwards to its own children without receiving.
mcclResult_t treeBroadcast(const Ctx& x, char* buf, size_t bytes, int root) {
  const Channel& ch = x.c->chan;
  int hub = 0;
  for (int r = 0; r < x.n; ++r) if (ch.treeParent[r] < 0) hub = r;
  if (root != hub) {
    if (x.r == root) MCCLCHECK(sendTo(x.c, hub, CONN_COLL_B, buf, bytes));
    if (x.r == hub) MCCLCHECK(recvFrom(x.c, root, CONN_COLL_B, buf, bytes));
  }
  if (x.r != root && x.r != hub) MCCLCHECK(recvFrom(x.c, ch.tree.up, CONN_COLL_A, buf, bytes));
  std::vector<int> kids;
  for (int k : ch.tree.down) if (k != root) kids.push_back(k);
  return sendToChildren(x, CONN_COLL_A, kids, buf, bytes);
}

// ---------------------------------------------------------------------------------------------------
// reduce
// ---------------------------------------------------------------------------------------------------
mcclResult_t treeReduce(const Ctx& x, const char* send, char* recv, size_t count, int root, bool avg) {
  const Channel& ch = x.c->chan;
  const size_t bytes = count * x.es;
  int hub = 0;
  for (int r = 0; r < x.n; ++r) if (ch.treeParent[r] < 0) hub = r;
  void *sc = nullptr, *st = nullptr;
  char* work = recv;
  if (x.r != root || recv == nullptr) {   // non-roots fold in scratch: their send buffer stays intact
    MCCLCHECK(commReserveScratch(x.c, bytes, &sc));
    work = static_cast<char*>(sc);
  }
  MCCLCHECK(commReserveStaging(x.c, std::max(ch.tree.down.size(), (size_t)1) * bytes, &st));
  if (work != send) memcpy(work, send, bytes);
  MCCLCHECK(treeUp(x, CONN_COLL_A, ch.tree, work, count, static_cast<char*>(st)));
  if (root != hub) {
    if (x.r == hub) MCCLCHECK(sendTo(x.c, root, CONN_COLL_B, work, bytes));
    if (x.r == root) MCCLCHECK(recvFrom(x.c, hub, CONN_COLL_B, recv, bytes));
  }
  if (x.r == root && avg) MCCLCHECK(hostScale(recv, count, x.dt, x.n));
  return mcclSuccess;
}

mcclResult_t directReduce(const Ctx& x, const char* send, char* recv, size_t count, int root, bool avg) {
  const size_t bytes = count * x.es;
  if (x.r != root) return sendTo(x.c, root, CONN_COLL_A, send, bytes);
  void* st = nullptr;
  MCCLCHECK(commReserveStaging(x.c, bytes * x.n, &st));
  char* slots = static_cast<char*>(st);
  std::vector<TcpConn*> conns(x.n, nullptr);
  for (int p = 0; p < x.n; ++p) if (p != x.r) MCCLCHECK(commPeerConn(x.c, p, CONN_COLL_A, &conns[p]));
  memcpy(slots + (size_t)x.r * bytes, send, bytes);
  MCCLCHECK(parallelFor(fanoutPool(), x.n, [&](int p) -> mcclResult_t {
    return p == x.r ? mcclSuccess : tcpRecv(conns[p], slots + (size_t)p * bytes, bytes);
  }));
  memcpy(recv, slots, bytes);
  MCCLCHECK(hostReduceMulti(recv, slots + bytes, count, x.n - 1, count, x.dt, x.op));
  return avg ? hostScale(recv, count, x.dt, x.n) : mcclSuccess;
}

// Ring reduce: the reduce phase of the ring all-reduce in scratch, then every rank ships the chunk it
// owns straight to the root, which receives them all in parallel.
mcclResult_t ringReduce(const Ctx& x, const char* send, char* recv, size_t count, int root, bool avg) {
  const int n = x.n, r = x.r;
  const size_t bytes = count * x.es;
  void *sc = nullptr, *st = nullptr;
  MCCLCHECK(commReserveScratch(x.c, bytes, &sc));
  MCCLCHECK(commReserveStaging(x.c, (count / n + 2) * x.es, &st));
  char* work = static_cast<char*>(sc);
  memcpy(work, send, bytes);
  const RingLeg leg = makeLeg(x.c, +1);
  auto off = [&](int i) { return chunkOff(count, n, i) * x.es; };
  auto len = [&](int i) { return chunkOff(count, n, i + 1) - chunkOff(count, n, i); };
  for (int i = 0; i < n - 1; ++i) {
    const int s = wrap(r - i, n), t = wrap(r - (i + 1), n);
    MCCLCHECK(sendRecv(x.c, leg.kind, leg.sendPeer, work + off(s), len(s) * x.es, leg.recvPeer, st, len(t) * x.es));
    MCCLCHECK(hostReduce(work + off(t), st, len(t), x.dt, x.op));
  }
  const int owned = wrap(r + 1, n);   // the fully reduced chunk this rank holds after the reduce phase
  if (r != root) return sendTo(x.c, root, CONN_COLL_B, work + off(owned), len(owned) * x.es);
  std::vector<TcpConn*> conns(n, nullptr);
  for (int p = 0; p < n; ++p) if (p != r) MCCLCHECK(commPeerConn(x.c, p, CONN_COLL_B, &conns[p]));
  memcpy(recv + off(owned), work + off(owned), len(owned) * x.es);
  MCCLCHECK(parallelFor(fanoutPool(), n, [&](int p) -> mcclResult_t {
    if (p == r) return mcclSuccess;
    const int ch = wrap(p + 1, n);
    return tcpRecv(conns[p], recv + off(ch), len(ch) * x.es);
  }));
  return avg ? hostScale(recv, count, x.dt, n) : mcclSuccess;
}

Ctx makeCtx(mcclComm* c, mcclDataType_t dt, mcclRedOp_t op) {
  Ctx x;
  x.c = c; x.n = c->nRanks; x.r = c->rank; x.es = mcclDataSize(dt); x.dt = dt;
  x.op = (op == mcclAvg) ? mcclSum : op;
  return x;
}

}  // namespace

mcclResult_t cpuAllReduce(mcclComm* c, const void* send, void* recv, size_t count, mcclDataType_t dt, mcclRedOp_t op, int algo) {
  Ctx x = makeCtx(c, dt, op);
  const size_t bytes = count * x.es;
  char* out = static_cast<char*>(recv);
  if (x.n == 1) { if (send != recv) memmove(recv, send, bytes); return mcclSuccess; }
  if (algo == mcclAlgoOneShot) {
    MCCLCHECK(directAllReduce(x, static_cast<const char*>(send), out, count));
  } else {
    if (send != recv) memcpy(recv, send, bytes);
    if (algo == mcclAlgoTree || count < (size_t)x.n) MCCLCHECK(treeAllReduce(x, out, count));
    else MCCLCHECK(ringAllReduce(x, out, count));
  }
  return op == mcclAvg ? hostScale(recv, count, dt, x.n) : mcclSuccess;
}

mcclResult_t cpuAllGather(mcclComm* c, const void* send, void* recv, size_t sendcount, mcclDataType_t dt, int algo) {
  Ctx x = makeCtx(c, dt, mcclSum);
  const size_t slot = sendcount * x.es;
  char* out = static_cast<char*>(recv);
  if (out + (size_t)x.r * slot != send) memmove(out + (size_t)x.r * slot, send, slot);
  if (x.n == 1) return mcclSuccess;
  if (algo == mcclAlgoOneShot) return directAllGather(x, out, slot);
  if (algo == mcclAlgoTree) return treeAllGather(x, out, slot);
  return ringAllGather(x, out, sendcount);
}

mcclResult_t cpuReduceScatter(mcclComm* c, const void* send, void* recv, size_t recvcount, mcclDataType_t dt, mcclRedOp_t op, int algo) {
  Ctx x = makeCtx(c, dt, op);
  const size_t blk = recvcount * x.es;
  const char* in = static_cast<const char*>(send);
  char* out = static_cast<char*>(recv);
  if (x.n == 1) { if (send != recv) memmove(recv, send, blk); return mcclSuccess; }
  // recv == send + rank*block (the in-place form) is safe: every variant writes recv only at the very end.
  // Any other overlap would be overwritten mid-way, so the input is copied first.
  void* copy = nullptr;
  const bool alias = out + blk > in && out < in + blk * x.n && out != in + (size_t)x.r * blk;
  if (alias) {
    MCCLCHECK(mcclPageAlloc(blk * x.n, &copy));
    memcpy(copy, send, blk * x.n);
    in = static_cast<const char*>(copy);
  }
  mcclResult_t rc;
  if (algo == mcclAlgoOneShot) rc = directReduceScatter(x, in, out, recvcount);
  else if (algo == mcclAlgoTree) rc = treeReduceScatter(x, in, out, recvcount);
  else rc = ringReduceScatter(x, in, out, recvcount);
  mcclPageFree(copy);
  MCCLCHECK(rc);
  return op == mcclAvg ? hostScale(recv, recvcount, dt, x.n) : mcclSuccess;
}

mcclResult_t cpuBroadcast(mcclComm* c, const void* send, void* recv, size_t count, mcclDataType_t dt, int root, int algo) {
  Ctx x = makeCtx(c, dt, mcclSum);
  const size_t bytes = count * x.es;
  if (x.r == root && send != recv) memmove(recv, send, bytes);
  if (x.n == 1) return mcclSuccess;
  if (algo == mcclAlgoTree) return treeBroadcast(x, static_cast<char*>(recv), bytes, root);
  return ringBroadcast(x, static_cast<char*>(recv), bytes, root);
}

mcclResult_t cpuReduce(mcclComm* c, const void* send, void* recv, size_t count, mcclDataType_t dt, mcclRedOp_t op, int root, int algo) {
  Ctx x = makeCtx(c, dt, op);
  const bool avg = op == mcclAvg;
  if (x.n == 1) {
    if (send != recv) memmove(recv, send, count * x.es);
    return mcclSuccess;
  }
  const char* in = static_cast<const char*>(send);
  char* out = static_cast<char*>(recv);
  if (algo == mcclAlgoOneShot) return directReduce(x, in, out, count, root, avg);
  if (algo == mcclAlgoTree) return treeReduce(x, in, out, count, root, avg);
  if (count < (size_t)x.n) return directReduce(x, in, out, count, root, avg);
  return ringReduce(x, in, out, count, root, avg);
}

}  // namespace mccl
