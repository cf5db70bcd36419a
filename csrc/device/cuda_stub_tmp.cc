#include "../comm/comm.h"
namespace mccl {
mcclResult_t cudaCommInit(mcclComm*) { return mcclInternalError; }
void cudaCommAbort(mcclComm*) {}
void cudaCommDestroy(mcclComm*) {}
mcclResult_t cudaCommAsyncError(mcclComm*, mcclResult_t* o) { *o = mcclSuccess; return mcclSuccess; }
mcclResult_t cudaCollective(mcclComm*, int, const void*, void*, size_t, mcclDataType_t, mcclRedOp_t, int, int, mcclStream_t) { return mcclInternalError; }
mcclResult_t cudaP2pBatch(mcclComm*, const std::vector<P2pOp>&, mcclStream_t) { return mcclInternalError; }
mcclResult_t cudaRecvAny(mcclComm*, void*, size_t, int*, mcclStream_t) { return mcclInternalError; }
mcclResult_t cudaBarrier(mcclComm*, mcclStream_t) { return mcclInternalError; }
mcclResult_t cudaMemAllocSym(mcclComm*, size_t, void**) { return mcclInternalError; }
mcclResult_t cudaMemFreeSym(mcclComm*, void*) { return mcclInternalError; }
mcclResult_t cudaRegister(mcclComm*, void*, size_t, void**) { return mcclInternalError; }
mcclResult_t cudaDeregister(mcclComm*, void*) { return mcclInternalError; }
mcclResult_t cudaPeerPointer(mcclComm*, const void*, int, void**) { return mcclInternalError; }
mcclResult_t cudaMcPointer(mcclComm*, const void*, void**) { return mcclInternalError; }
bool cudaNvlsEnabled(mcclComm*) { return false; }
mcclResult_t cudaCalibrate(mcclComm*) { return mcclSuccess; }
mcclResult_t cudaFillRankInfo(int, RankInfo*) { return mcclInternalError; }
}
