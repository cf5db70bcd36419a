// Public collectives: validate, plan, launch.
// All argument checks happen before anything is launched; count == 0 is a successful no-op; a
// single-rank communicator degenerates to a local copy.  The planner's choice (or the forced algorithm)
// is recorded in comm->lastAlgo.  Inside a group the call is recorded and issued by GroupEnd.
// Parity: src/coll/coll.cc:16-106 of the reference.
#include <cstring>
#include <mutex>

#include <cuda_runtime_api.h>
#include <nvtx3/nvToolsExt.h>

#include "../comm/comm.h"
#include "../core/trace.h"

using namespace mccl;

DEFINE_MCCL_PARAM(Nvtx, "NVTX", 1)

namespace {

// An NVTX range around the host side of every collective ("mcclAllReduce", ...), visible to any attached
// profiler; with none attached the header-only NVTX stubs return at once.  MCCL_NVTX=0 removes the calls.
// The header-only NVTX layer installs its entry points on first use without synchronisation; doing that first use
// once, under call_once, keeps concurrent first calls from different threads from racing on its table.
void nvtxWarmUp() {
  static std::once_flag once;
  std::call_once(once, [] { nvtxRangePushA("mcclInit"); nvtxRangePop(); });
}

struct NvtxRange {
  bool on;
  explicit NvtxRange(const char* name) : on(mcclParamNvtx() != 0) { if (on) { nvtxWarmUp(); nvtxRangePushA(name); } }
  ~NvtxRange() { if (on) nvtxRangePop(); }
};

mcclResult_t checkCommon(mcclComm_t comm, mcclDataType_t dt) {
  if (comm == nullptr) return mcclInvalidArgument;
  if (mcclDataSize(dt) == 0) return mcclInvalidArgument;
  if (comm->aborted.load()) return mcclInvalidUsage;
  return mcclSuccess;
}

// `what`, `bytes`, `stream` feed the optional trace (MCCL_TRACE); the span covers the launch on the
// caller's stream (cuda) or the whole blocking call (tcp).
mcclResult_t issue(mcclComm_t comm, const char* what, size_t bytes, mcclStream_t stream, std::function<mcclResult_t()> fn,
                   const CollCall& call = CollCall()) {
  auto traced = [=]() -> mcclResult_t {
    NvtxRange range(what);
    if (!traceEnabled()) {
      const mcclResult_t rc = fn();
      MCCL_TRACE("%s %zu bytes on %s rank %d/%d: algo %s -> %s", what, bytes, comm->transport.c_str(), comm->rank, comm->nRanks,
                 mcclAlgoStr(comm->lastAlgo.load()), mcclResultStr(rc));
      return rc;
    }
    TraceSpan span = traceBegin(comm, what, bytes, comm->lastAlgo.load(), stream);
    const mcclResult_t rc = fn();
    traceEnd(comm, span, stream);
    return rc;
  };
  if (groupActive()) {
    CollCall c = call;
    c.stream = stream;
    return groupRecordColl(comm, [=]() { return commLaunch(comm, traced); }, c);
  }
  return commLaunch(comm, traced);
}

}  // namespace

extern "C" {

mcclResult_t mcclAllReduce(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count, mcclDataType_t dt,
                           mcclRedOp_t op, mcclStream_t stream) {
  MCCLCHECK(checkCommon(comm, dt));
  if ((unsigned)op >= (unsigned)mcclNumOps) MCCLFAIL(mcclInvalidArgument);
  if (count == 0) return mcclSuccess;
  if (sendbuff == nullptr || recvbuff == nullptr) MCCLFAIL(mcclInvalidArgument);
  const int algo = commPickAlgo(comm, mcclCollAllReduce, count * mcclDataSize(dt), dt, op);
  return issue(comm, "AllReduce", count * mcclDataSize(dt), stream, [=]() -> mcclResult_t {
    comm->lastAlgo.store(algo);
    if (comm->cuda) return cudaCollective(comm, mcclCollAllReduce, sendbuff, recvbuff, count, dt, op, 0, algo, stream);
    return cpuAllReduce(comm, sendbuff, recvbuff, count, dt, op, algo);
  }, [&] { CollCall c; c.coll = mcclCollAllReduce; c.send = sendbuff; c.recv = recvbuff; c.count = count; c.dt = dt; c.op = op; c.algo = algo; return c; }());
}

mcclResult_t mcclAllGather(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t sendcount, mcclDataType_t dt,
                           mcclStream_t stream) {
  MCCLCHECK(checkCommon(comm, dt));
  if (sendcount == 0) return mcclSuccess;
  if (sendbuff == nullptr || recvbuff == nullptr) MCCLFAIL(mcclInvalidArgument);
  const int algo = commPickAlgo(comm, mcclCollAllGather, sendcount * mcclDataSize(dt) * comm->nRanks, dt, mcclSum);
  return issue(comm, "AllGather", sendcount * mcclDataSize(dt) * comm->nRanks, stream, [=]() -> mcclResult_t {
    comm->lastAlgo.store(algo);
    if (comm->cuda) return cudaCollective(comm, mcclCollAllGather, sendbuff, recvbuff, sendcount, dt, mcclSum, 0, algo, stream);
    return cpuAllGather(comm, sendbuff, recvbuff, sendcount, dt, algo);
  });
}

mcclResult_t mcclReduceScatter(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t recvcount, mcclDataType_t dt,
                               mcclRedOp_t op, mcclStream_t stream) {
  MCCLCHECK(checkCommon(comm, dt));
  if ((unsigned)op >= (unsigned)mcclNumOps) MCCLFAIL(mcclInvalidArgument);
  if (recvcount == 0) return mcclSuccess;
  if (sendbuff == nullptr || recvbuff == nullptr) MCCLFAIL(mcclInvalidArgument);
  const int algo = commPickAlgo(comm, mcclCollReduceScatter, recvcount * mcclDataSize(dt) * comm->nRanks, dt, op);
  return issue(comm, "ReduceScatter", recvcount * mcclDataSize(dt) * comm->nRanks, stream, [=]() -> mcclResult_t {
    comm->lastAlgo.store(algo);
    if (comm->cuda) return cudaCollective(comm, mcclCollReduceScatter, sendbuff, recvbuff, recvcount, dt, op, 0, algo, stream);
    return cpuReduceScatter(comm, sendbuff, recvbuff, recvcount, dt, op, algo);
  });
}

mcclResult_t mcclBroadcast(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count, mcclDataType_t dt, int root,
                           mcclStream_t stream) {
  MCCLCHECK(checkCommon(comm, dt));
  if (root < 0 || root >= comm->nRanks) MCCLFAIL(mcclInvalidArgument);
  if (count == 0) return mcclSuccess;
  // Only the root reads sendbuff; everyone writes recvbuff.
  if (recvbuff == nullptr || (comm->rank == root && sendbuff == nullptr)) MCCLFAIL(mcclInvalidArgument);
  const int algo = commPickAlgo(comm, mcclCollBroadcast, count * mcclDataSize(dt), dt, mcclSum);
  return issue(comm, "Broadcast", count * mcclDataSize(dt), stream, [=]() -> mcclResult_t {
    comm->lastAlgo.store(algo);
    if (comm->cuda) return cudaCollective(comm, mcclCollBroadcast, sendbuff, recvbuff, count, dt, mcclSum, root, algo, stream);
    return cpuBroadcast(comm, sendbuff, recvbuff, count, dt, root, algo);
  });
}

mcclResult_t mcclReduce(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count, mcclDataType_t dt, mcclRedOp_t op,
                        int root, mcclStream_t stream) {
  MCCLCHECK(checkCommon(comm, dt));
  if ((unsigned)op >= (unsigned)mcclNumOps) MCCLFAIL(mcclInvalidArgument);
  if (root < 0 || root >= comm->nRanks) MCCLFAIL(mcclInvalidArgument);
  if (count == 0) return mcclSuccess;
  // Everyone reads sendbuff; only the root writes recvbuff.
  if (sendbuff == nullptr || (comm->rank == root && recvbuff == nullptr)) MCCLFAIL(mcclInvalidArgument);
  const int algo = commPickAlgo(comm, mcclCollReduce, count * mcclDataSize(dt), dt, op);
  return issue(comm, "Reduce", count * mcclDataSize(dt), stream, [=]() -> mcclResult_t {
    comm->lastAlgo.store(algo);
    if (comm->cuda) return cudaCollective(comm, mcclCollReduce, sendbuff, recvbuff, count, dt, op, root, algo, stream);
    return cpuReduce(comm, sendbuff, recvbuff, count, dt, op, root, algo);
  });
}

// count = elements per peer block: block p of sendbuff goes to rank p, block q of recvbuff comes from rank q.
mcclResult_t mcclAllToAll(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count, mcclDataType_t dt,
                          mcclStream_t stream) {
  MCCLCHECK(checkCommon(comm, dt));
  if (count == 0) return mcclSuccess;
  if (sendbuff == nullptr || recvbuff == nullptr) MCCLFAIL(mcclInvalidArgument);
  if (sendbuff == recvbuff && comm->nRanks > 1) MCCLFAIL(mcclInvalidUsage);   // blocks would overwrite each other
  const size_t blk = count * mcclDataSize(dt);
  if (comm->cuda) {
    return issue(comm, "AllToAll", blk * comm->nRanks, stream, [=]() -> mcclResult_t {
      comm->lastAlgo.store(mcclAlgoOneShot);
      return cudaCollective(comm, mcclCollAllToAll, sendbuff, recvbuff, count, dt, mcclSum, 0, mcclAlgoOneShot, stream);
    });
  }
  // tcp: self copy + one grouped Send/Recv pair per peer.
  MCCLCHECK(mcclGroupStart());
  for (int p = 0; p < comm->nRanks; ++p) {
    mcclSend(comm, static_cast<const char*>(sendbuff) + (size_t)p * blk, count, dt, p, stream);
    mcclRecv(comm, static_cast<char*>(recvbuff) + (size_t)p * blk, count, dt, p, stream);
  }
  return mcclGroupEnd();
}

// ---- compositions of grouped Send / Recv (no counterpart in the reference; NCCL has the same three) ---------------
static mcclResult_t localCopy(mcclComm_t comm, const void* src, void* dst, size_t bytes, mcclStream_t stream) {
  if (bytes == 0 || src == dst) return mcclSuccess;
  if (!comm->cuda) { memmove(dst, src, bytes); return mcclSuccess; }
  return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess
             ? mcclSuccess : mcclSystemError;
}

// Segment j of sendbuff (sendcounts[j] elements at element offset sdispls[j]) goes to rank j; segment i of recvbuff
// receives recvcounts[i] elements from rank i.  Counts and displacements are host arrays of nRanks entries.
mcclResult_t mcclAllToAllv(mcclComm_t comm, const void* sendbuff, const size_t* sendcounts, const size_t* sdispls, void* recvbuff,
                           const size_t* recvcounts, const size_t* rdispls, mcclDataType_t dt, mcclStream_t stream) {
  MCCLCHECK(checkCommon(comm, dt));
  if (sendcounts == nullptr || sdispls == nullptr || recvcounts == nullptr || rdispls == nullptr) MCCLFAIL(mcclInvalidArgument);
  const size_t es = mcclDataSize(dt);
  const int n = comm->nRanks, r = comm->rank;
  if (sendcounts[r] != recvcounts[r]) MCCLFAIL(mcclInvalidArgument);
  for (int p = 0; p < n; ++p)
    if ((sendcounts[p] && sendbuff == nullptr) || (recvcounts[p] && recvbuff == nullptr)) MCCLFAIL(mcclInvalidArgument);
  MCCLCHECK(localCopy(comm, static_cast<const char*>(sendbuff) + sdispls[r] * es, static_cast<char*>(recvbuff) + rdispls[r] * es,
                      sendcounts[r] * es, stream));
  MCCLCHECK(mcclGroupStart());
  for (int i = 1; i < n; ++i) {
    const int dst = (r + i) % n, src = (r - i + n) % n;
    if (sendcounts[dst]) mcclSend(comm, static_cast<const char*>(sendbuff) + sdispls[dst] * es, sendcounts[dst], dt, dst, stream);
    if (recvcounts[src]) mcclRecv(comm, static_cast<char*>(recvbuff) + rdispls[src] * es, recvcounts[src], dt, src, stream);
  }
  return mcclGroupEnd();
}

// recvbuff at the root = the ranks' sendbuff (count elements each) in rank order; recvbuff is ignored elsewhere.
mcclResult_t mcclGather(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count, mcclDataType_t dt, int root,
                        mcclStream_t stream) {
  MCCLCHECK(checkCommon(comm, dt));
  if (root < 0 || root >= comm->nRanks) MCCLFAIL(mcclInvalidArgument);
  if (count == 0) return mcclSuccess;
  if (sendbuff == nullptr || (comm->rank == root && recvbuff == nullptr)) MCCLFAIL(mcclInvalidArgument);
  const size_t blk = count * mcclDataSize(dt);
  if (comm->rank != root) return mcclSend(comm, sendbuff, count, dt, root, stream);
  MCCLCHECK(localCopy(comm, sendbuff, static_cast<char*>(recvbuff) + (size_t)root * blk, blk, stream));
  MCCLCHECK(mcclGroupStart());
  for (int p = 0; p < comm->nRanks; ++p)
    if (p != root) mcclRecv(comm, static_cast<char*>(recvbuff) + (size_t)p * blk, count, dt, p, stream);
  return mcclGroupEnd();
}

// recvbuff on rank p = block p (count elements) of the root's sendbuff; sendbuff is ignored elsewhere.
mcclResult_t mcclScatter(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count, mcclDataType_t dt, int root,
                         mcclStream_t stream) {
  MCCLCHECK(checkCommon(comm, dt));
  if (root < 0 || root >= comm->nRanks) MCCLFAIL(mcclInvalidArgument);
  if (count == 0) return mcclSuccess;
  if (recvbuff == nullptr || (comm->rank == root && sendbuff == nullptr)) MCCLFAIL(mcclInvalidArgument);
  const size_t blk = count * mcclDataSize(dt);
  if (comm->rank != root) return mcclRecv(comm, recvbuff, count, dt, root, stream);
  MCCLCHECK(localCopy(comm, static_cast<const char*>(sendbuff) + (size_t)root * blk, recvbuff, blk, stream));
  MCCLCHECK(mcclGroupStart());
  for (int p = 0; p < comm->nRanks; ++p)
    if (p != root) mcclSend(comm, static_cast<const char*>(sendbuff) + (size_t)p * blk, count, dt, p, stream);
  return mcclGroupEnd();
}

}  // extern "C"
