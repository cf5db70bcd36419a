// Communicator state and the internal entry points shared by the runtime files.
// Parity: mcclComm (src/include/comm.h:31-68), launch policy (src/include/comm.h:106-121), worker queue
// (src/enqueue.cc:17-106), arenas (src/comm.cc:209-232) of the reference.
#pragma once

#include <atomic>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../bootstrap/bootstrap.h"
#include "../core/core.h"
#include "../graph/graph.h"
#include "../transport/tcp.h"

namespace mccl {
struct WorkQueue;
struct CudaState;
}

struct mcclComm {
  int rank = 0;
  int nRanks = 1;
  int device = -1;
  bool cuda = false;                 // transport: true = NVLink kernels on device pointers, false = TCP on host pointers
  int blocking = 1;
  std::string transport;
  std::atomic<int>  asyncState{(int)mcclSuccess};   // sticky fatal error (system/internal/remote)
  std::atomic<bool> aborted{false};
  mccl::BootstrapId id;
  mccl::Bootstrap* bs = nullptr;
  std::vector<mccl::RankInfo> infos;
  mccl::TopoSystem system;
  mccl::TopoGraph  graphs[mcclNumAlgos];
  mccl::Channel    chan;
  mccl::TunerModel tuner;
  int enabled[mcclNumAlgos] = {1, 1, 1, 1, 1};
  // tcp transport
  mccl::TcpEndpoint* ep = nullptr;
  void*  staging = nullptr;  size_t stagingBytes = 0;   // receive staging for the primitives
  void*  scratch = nullptr;  size_t scratchBytes = 0;   // work buffers of the algorithms (disjoint from staging)
  mccl::WorkQueue* work = nullptr;
  // cuda transport
  mccl::CudaState* cu = nullptr;
  // bookkeeping
  std::atomic<int> lastAlgo{-1};
  std::atomic<uint64_t> launches{0};
  int maxCtas = 0;
  int forcedCtas = 0;                // exact CTA count for every collective kernel (tuning aid), 0 = planner's choice
  uint32_t splitSeq = 0;
};

namespace mccl {

// ---- launch policy -------------------------------------------------------------------------------
// Blocking communicators (and single-rank ones) run `op` on the caller and latch fatal results;
// non-blocking ones queue it for the worker and return mcclInProgress... as success to the caller.
mcclResult_t commLaunch(mcclComm* comm, std::function<mcclResult_t()> op);
mcclResult_t workerStart(mcclComm* comm);
void         workerStop(mcclComm* comm);      // drains, then joins
mcclResult_t workerSync(mcclComm* comm);      // wait until the queue is empty; returns the latched error
mcclResult_t workerAsyncError(mcclComm* comm, mcclResult_t* out);

mcclResult_t commReserveStaging(mcclComm* comm, size_t bytes, void** out);
mcclResult_t commReserveScratch(mcclComm* comm, size_t bytes, void** out);
mcclResult_t commPeerConn(mcclComm* comm, int peer, uint32_t kind, TcpConn** out);
int          commPickAlgo(mcclComm* comm, int coll, size_t bytes, int dt, int op);
int          forcedAlgo();                    // thread-local override set by mcclSetForcedAlgo

// ---- CPU (tcp transport) collectives: cpu_coll.cc ---------------------------------------------------
mcclResult_t cpuAllReduce(mcclComm* c, const void* send, void* recv, size_t count, mcclDataType_t dt, mcclRedOp_t op, int algo);
mcclResult_t cpuAllGather(mcclComm* c, const void* send, void* recv, size_t sendcount, mcclDataType_t dt, int algo);
mcclResult_t cpuReduceScatter(mcclComm* c, const void* send, void* recv, size_t recvcount, mcclDataType_t dt, mcclRedOp_t op, int algo);
mcclResult_t cpuBroadcast(mcclComm* c, const void* send, void* recv, size_t count, mcclDataType_t dt, int root, int algo);
mcclResult_t cpuReduce(mcclComm* c, const void* send, void* recv, size_t count, mcclDataType_t dt, mcclRedOp_t op, int root, int algo);

// ---- point to point on the tcp transport: p2p.cc ---------------------------------------------------
struct P2pOp { mcclComm* comm; bool isSend; int peer; void* buf; size_t bytes; mcclStream_t stream; };
mcclResult_t cpuRunP2pBatch(mcclComm* c, const std::vector<P2pOp>& ops);
mcclResult_t cpuRecvAny(mcclComm* c, void* buf, size_t bytes, int* src);
bool         groupActive();
mcclResult_t groupRecord(const P2pOp& op);                         // queue a Send/Recv inside a group
// What a recorded collective was called with; lets GroupEnd fuse the all-reduce calls of a group into one launch.
struct CollCall {
  int coll = -1;
  const void* send = nullptr;
  void* recv = nullptr;
  size_t count = 0;
  mcclDataType_t dt = mcclFloat32;
  mcclRedOp_t op = mcclSum;
  int algo = -1;
  mcclStream_t stream = nullptr;
};
mcclResult_t groupRecordColl(mcclComm* comm, std::function<mcclResult_t()> launch, const CollCall& call);   // queue a collective

// ---- cuda transport: implemented in the .cu files ----------------------------------------------------
mcclResult_t cudaCommInit(mcclComm* c);                            // heap, control block, peer mappings, NVLS
void         cudaCommAbort(mcclComm* c);
void         cudaCommDestroy(mcclComm* c);
mcclResult_t cudaCommAsyncError(mcclComm* c, mcclResult_t* out);
mcclResult_t cudaCollective(mcclComm* c, int coll, const void* send, void* recv, size_t count, mcclDataType_t dt,
                            mcclRedOp_t op, int root, int algo, mcclStream_t stream);
// Launch the all-reduce calls among `calls` that can share one kernel (symmetric, 16-byte aligned buffers of at
// least 16 bytes per rank) and set done[i] for them; the others are left to their own launches.
mcclResult_t cudaGroupAllReduce(mcclComm* c, const std::vector<CollCall>& calls, std::vector<char>* done);
mcclResult_t cudaP2pBatch(mcclComm* c, const std::vector<P2pOp>& ops, mcclStream_t stream);
mcclResult_t cudaRecvAny(mcclComm* c, void* buf, size_t bytes, int* src, mcclStream_t stream);
mcclResult_t cudaBarrier(mcclComm* c, mcclStream_t stream);
mcclResult_t cudaMemAllocSym(mcclComm* c, size_t bytes, void** ptr);
mcclResult_t cudaMemFreeSym(mcclComm* c, void* ptr);
mcclResult_t cudaRegister(mcclComm* c, void* ptr, size_t bytes, void** handle);
mcclResult_t cudaDeregister(mcclComm* c, void* handle);
mcclResult_t cudaPeerPointer(mcclComm* c, const void* local, int peer, void** out);
mcclResult_t cudaMcPointer(mcclComm* c, const void* local, void** out);
bool         cudaNvlsEnabled(mcclComm* c);
mcclResult_t cudaCheckGuards(mcclComm* c, int* intact);
mcclResult_t cudaCalibrate(mcclComm* c);                           // measure links, refine the tuner
mcclResult_t cudaFillRankInfo(int device, RankInfo* ri);           // device facts + peer masks

}  // namespace mccl
