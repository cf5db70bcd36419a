/*
 * mccl-b200 public C API.
 *
 * A collective communication library for one NVSwitch box of B200 GPUs (one process per GPU), with a
 * TCP/CPU path for hosts without a GPU.  The API surface follows Lazarus-931/mccl
 * (src/include/mccl.h:5-15, src/include/coll.h:12-25, src/include/comm.h:80-131,
 * src/definitions.h.in:7-45): same enum names and values, same call names, same argument order, with a
 * trailing CUDA stream on every data call.  Everything is `extern "C"`, returns mcclResult_t, and reports
 * through out-parameters; no exception crosses this boundary.
 *
 * Buffers: with the "cuda" transport every sendbuff/recvbuff is a device pointer and the call is
 * enqueued on `stream`; with the "tcp" transport they are host pointers and `stream` is ignored.
 * Device buffers obtained from mcclMemAlloc (symmetric, peer-mapped, multicast-bound) are used in
 * place; any other device pointer is staged through the communicator's symmetric scratch.
 *
 * Symmetric buffers, the contract: a rank decides from its own pointer whether a buffer is symmetric, and
 * derives the peers' addresses from it.  So an argument that lies in symmetric memory on one rank must be the
 * same part (same allocation, same offset) of that allocation on EVERY rank of the call, and an argument that
 * is an ordinary pointer on one rank must be ordinary on all.  The in-place forms count as the same part:
 * all-gather with sendbuff = recvbuff + rank * sendcount, reduce-scatter with recvbuff = sendbuff + rank *
 * recvcount.  A call that breaks the rule returns wrong data or runs into the device time limit; nothing
 * detects it by default.  With MCCL_CHECK_SYMMETRY=1 every collective is preceded by a small kernel in which
 * the ranks compare (allocation, offset, count, root); a mismatch is reported as mcclInvalidUsage by the next
 * call and by mcclCommGetAsyncError.
 *
 * Groups: the calls between mcclGroupStart and mcclGroupEnd are independent of one another (none may consume
 * another's result).  Per communicator GroupEnd issues first the all-reduce calls on symmetric buffers, as one
 * kernel launch, then the other collectives in program order, then all Send/Recv as one launch.  On the cuda
 * transport all calls of a group on one communicator must name the same stream (mcclInvalidUsage otherwise).
 */
#ifndef MCCL_H_
#define MCCL_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MCCL_MAJOR 0
#define MCCL_MINOR 1
#define MCCL_PATCH 0
#define MCCL_VERSION_CODE (MCCL_MAJOR * 10000 + MCCL_MINOR * 100 + MCCL_PATCH)

typedef enum {
  mcclSuccess         = 0,
  mcclError           = 1,
  mcclSystemError     = 2,
  mcclInternalError   = 3,
  mcclInvalidArgument = 4,
  mcclInvalidUsage    = 5,
  mcclRemoteError     = 6,
  mcclInProgress      = 7,
  mcclNumResults      = 8
} mcclResult_t;

typedef enum {
  mcclInt8     = 0,
  mcclUint8    = 1,
  mcclInt32    = 2,
  mcclUint32   = 3,
  mcclInt64    = 4,
  mcclUint64   = 5,
  mcclFloat16  = 6,
  mcclBfloat16 = 7,
  mcclFloat32  = 8,
  mcclFloat64  = 9,
  mcclNumTypes = 10
} mcclDataType_t;

typedef enum {
  mcclSum    = 0,
  mcclProd   = 1,
  mcclMax    = 2,
  mcclMin    = 3,
  mcclAvg    = 4,
  mcclNumOps = 5
} mcclRedOp_t;

/* Collective algorithms the planner can choose between (MCCL_ALGO accepts the lower-case names). */
typedef enum {
  mcclAlgoRing    = 0,
  mcclAlgoTree    = 1,
  mcclAlgoOneShot = 2,
  mcclAlgoTwoShot = 3,
  mcclAlgoNvls    = 4,
  mcclNumAlgos    = 5,
  mcclAlgoAuto    = -1
} mcclAlgo_t;

typedef enum {
  mcclCollAllReduce     = 0,
  mcclCollAllGather     = 1,
  mcclCollReduceScatter = 2,
  mcclCollBroadcast     = 3,
  mcclCollReduce        = 4,
  mcclCollAllToAll      = 5,
  mcclNumColls          = 6
} mcclColl_t;

typedef struct mcclComm* mcclComm_t;
typedef struct CUstream_st* mcclStream_t; /* same object as cudaStream_t / CUstream */

typedef struct { char internal[128]; } mcclUniqueId;

typedef struct {
  int         blocking;  /* 1: a call returns when the work is done (tcp) or enqueued on the stream (cuda);
                            0: tcp work runs on the communicator's worker thread */
  const char* transport; /* "tcp" | "cuda" | NULL (= MCCL_TRANSPORT, else cuda when a GPU is present, else tcp) */
} mcclConfig_t;
#define MCCL_CONFIG_INITIALIZER { 1, NULL }

#define MCCL_SPLIT_NOCOLOR (-1)

/* ---- library / type helpers ------------------------------------------------------------------ */
mcclResult_t mcclGetVersion(int* version);
const char*  mcclGetErrorString(mcclResult_t r);
const char*  mcclResultStr(mcclResult_t r);
const char*  mcclDataTypeStr(mcclDataType_t t);
const char*  mcclRedOpStr(mcclRedOp_t op);
const char*  mcclAlgoStr(int algo);
const char*  mcclCollStr(int coll);
size_t       mcclDataSize(mcclDataType_t t);
mcclResult_t mcclGetLastError(mcclComm_t comm);   /* thread-local last non-success result */
mcclResult_t mcclSetLastError(mcclResult_t r);
/* 1 for the results that latch on a communicator (system, internal and remote errors), 0 for the rest. */
int          mcclResultFatal(mcclResult_t r);

/* ---- communicator lifecycle ------------------------------------------------------------------ */
mcclResult_t mcclGetUniqueId(mcclUniqueId* id);
mcclResult_t mcclCommInitRank(mcclComm_t* comm, int nRanks, mcclUniqueId id, int rank);
mcclResult_t mcclCommInitRankConfig(mcclComm_t* comm, int nRanks, mcclUniqueId id, int rank,
                                    const mcclConfig_t* config);
mcclResult_t mcclCommSplit(mcclComm_t comm, int color, int key, mcclComm_t* newcomm,
                           const mcclConfig_t* config);
mcclResult_t mcclCommFinalize(mcclComm_t comm);
mcclResult_t mcclCommDestroy(mcclComm_t comm);
mcclResult_t mcclCommAbort(mcclComm_t comm);
mcclResult_t mcclCommCount(mcclComm_t comm, int* count);
mcclResult_t mcclCommUserRank(mcclComm_t comm, int* rank);
mcclResult_t mcclCommDevice(mcclComm_t comm, int* device);
mcclResult_t mcclCommGetAsyncError(mcclComm_t comm, mcclResult_t* asyncErr);
mcclResult_t mcclCommSynchronize(mcclComm_t comm);
/* Host-side all-gather over the communicator's control plane (bootstrap); collective. */
mcclResult_t mcclCommHostAllGather(mcclComm_t comm, const void* send, void* recv, size_t bytesPerRank);
mcclResult_t mcclCommHostBarrier(mcclComm_t comm);
/* "tcp" or "cuda". */
const char*  mcclCommTransport(mcclComm_t comm);
/* Whether NVLS multicast is mapped for this communicator. */
mcclResult_t mcclCommNvlsEnabled(mcclComm_t comm, int* enabled);

/* ---- collectives ----------------------------------------------------------------------------- */
mcclResult_t mcclAllReduce(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count,
                           mcclDataType_t dt, mcclRedOp_t op, mcclStream_t stream);
mcclResult_t mcclAllGather(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t sendcount,
                           mcclDataType_t dt, mcclStream_t stream);
mcclResult_t mcclReduceScatter(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t recvcount,
                               mcclDataType_t dt, mcclRedOp_t op, mcclStream_t stream);
mcclResult_t mcclBroadcast(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count,
                           mcclDataType_t dt, int root, mcclStream_t stream);
mcclResult_t mcclReduce(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count,
                        mcclDataType_t dt, mcclRedOp_t op, int root, mcclStream_t stream);
mcclResult_t mcclAllToAll(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count,
                          mcclDataType_t dt, mcclStream_t stream);

/* Compositions of grouped Send / Recv (not in the reference).  Counts and displacements are in elements, host arrays
 * of one entry per rank. */
mcclResult_t mcclAllToAllv(mcclComm_t comm, const void* sendbuff, const size_t* sendcounts, const size_t* sdispls,
                           void* recvbuff, const size_t* recvcounts, const size_t* rdispls, mcclDataType_t dt,
                           mcclStream_t stream);
mcclResult_t mcclGather(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count, mcclDataType_t dt, int root,
                        mcclStream_t stream);
mcclResult_t mcclScatter(mcclComm_t comm, const void* sendbuff, void* recvbuff, size_t count, mcclDataType_t dt, int root,
                         mcclStream_t stream);

/* ---- point to point and grouping ------------------------------------------------------------- */
mcclResult_t mcclSend(mcclComm_t comm, const void* sendbuff, size_t count, mcclDataType_t dt, int peer,
                      mcclStream_t stream);
mcclResult_t mcclRecv(mcclComm_t comm, void* recvbuff, size_t count, mcclDataType_t dt, int peer,
                      mcclStream_t stream);
mcclResult_t mcclRecvAny(mcclComm_t comm, void* recvbuff, size_t count, mcclDataType_t dt, int* srcRank,
                         mcclStream_t stream);
mcclResult_t mcclGroupStart(void);
mcclResult_t mcclGroupEnd(void);
mcclResult_t mcclGroupAbort(void);

/* ---- memory ---------------------------------------------------------------------------------- */
/* Symmetric device allocation: collective over `comm`, every rank passes the same size.  The memory is
 * mapped into every peer (and bound to the NVLS multicast object when there is one), so collectives use
 * it in place. */
mcclResult_t mcclMemAlloc(mcclComm_t comm, size_t bytes, void** ptr);
mcclResult_t mcclMemFree(mcclComm_t comm, void* ptr);
/* A pool over ONE symmetric allocation: Create and Destroy are collective (they are mcclMemAlloc / mcclMemFree),
 * Alloc and Free are local bookkeeping (first fit, 256-byte granularity, neighbours merged on free).  Every rank
 * must make the same sequence of Alloc / Free calls, so that a sub-allocation is the same part of the allocation
 * on every rank.  Alloc returns mcclSystemError (and NULL) when no free range is large enough. */
typedef struct mcclSymPool* mcclSymPool_t;
mcclResult_t mcclSymPoolCreate(mcclComm_t comm, size_t bytes, mcclSymPool_t* pool);
mcclResult_t mcclSymPoolAlloc(mcclSymPool_t pool, size_t bytes, void** ptr);
mcclResult_t mcclSymPoolFree(mcclSymPool_t pool, void* ptr);
mcclResult_t mcclSymPoolStats(mcclSymPool_t pool, size_t* total, size_t* inUse, size_t* largestFree);
mcclResult_t mcclSymPoolDestroy(mcclSymPool_t pool);
/* Collective registration of an existing cudaMalloc'ed range (CUDA IPC); after it the range is used in
 * place by the peer-to-peer algorithms. */
mcclResult_t mcclCommRegister(mcclComm_t comm, void* ptr, size_t bytes, void** handle);
mcclResult_t mcclCommDeregister(mcclComm_t comm, void* handle);
/* Device pointer through which this rank reaches `peer`'s copy of symmetric address `localPtr`
 * (NULL if `localPtr` is not symmetric). */
mcclResult_t mcclMemPeerPointer(mcclComm_t comm, const void* localPtr, int peer, void** peerPtr);
/* Multicast (NVLS) alias of a symmetric address, NULL when the range has none. */
mcclResult_t mcclMemMulticastPointer(mcclComm_t comm, const void* localPtr, void** mcPtr);

/* Host-side fixed-size buffer pool (page aligned; pinned when a GPU is present). */
typedef struct mcclMemPool* mcclMemPool_t;
typedef struct { void* host; size_t size; } mcclBuf;
mcclResult_t mcclPageAlloc(size_t bytes, void** out);
void         mcclPageFree(void* ptr);
mcclResult_t mcclMemPoolCreate(size_t buffSize, int count, mcclMemPool_t* out);
mcclResult_t mcclMemPoolAlloc(mcclMemPool_t p, mcclBuf* out);
mcclResult_t mcclMemPoolFree(mcclMemPool_t p, const mcclBuf* buf);
mcclResult_t mcclMemPoolStats(mcclMemPool_t p, int* total, int* free_);
mcclResult_t mcclMemPoolDestroy(mcclMemPool_t p);

/* ---- planner introspection and control ------------------------------------------------------- */
/* Algorithm the tuner would use for (coll, bytes) on this communicator. */
mcclResult_t mcclCommPickAlgo(mcclComm_t comm, int coll, size_t bytes, int dt, int op, int* algo);
/* Force one algorithm for the following calls on this thread (mcclAlgoAuto restores the tuner). */
mcclResult_t mcclSetForcedAlgo(int algo);
/* Algorithm used by the most recent collective issued on this communicator. */
mcclResult_t mcclCommLastAlgo(mcclComm_t comm, int* algo);
/* Number of device kernels this communicator has launched so far. */
mcclResult_t mcclCommLaunchCount(mcclComm_t comm, uint64_t* launches);
/* Limit the CTAs per collective kernel (0 = tuner default); used to leave SMs to overlapped compute. */
mcclResult_t mcclCommSetMaxCtas(mcclComm_t comm, int maxCtas);
/* Use exactly `ctas` CTAs for every collective kernel (0 = planner's choice); a tuning aid. */
mcclResult_t mcclCommSetCtas(mcclComm_t comm, int ctas);
/* Debug aid: verifies the guard word behind the device-side flag arrays of the cuda transport (a kernel that
 * indexed past them would have overwritten it).  *intact = 1 when fine or when there is nothing to check. */
mcclResult_t mcclCommCheckGuards(mcclComm_t comm, int* intact);
/* Topology of the communicator as XML (caller frees with mcclFreeString). */
mcclResult_t mcclCommTopoXml(mcclComm_t comm, char** xml);
void         mcclFreeString(char* s);

#ifdef __cplusplus
}
#endif
#endif /* MCCL_H_ */
