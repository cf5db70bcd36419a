// Bring-up and teardown of the cuda transport for one communicator: device facts for discovery, the
// AF_UNIX endpoint for descriptor passing, the control segment (flags, one-shot slots, Send/Recv FIFOs,
// staging area) mapped from every peer, the pinned status word, and symmetric user allocations.
// Role parity: the connection and arena set-up part of mcclCommInitRankConfig in the reference
// (src/comm.cc:139-232); sockets become peer mappings, the two host arenas become one device segment.
#include <cstring>
#include <cuda_runtime.h>

#include "../os/socket.h"
#include "../transport/cuda_mem.h"
#include "comm.h"

namespace mccl {

DEFINE_MCCL_PARAM(DeviceTimeoutMs, "DEVICE_TIMEOUT_MS", 10000);
DEFINE_MCCL_PARAM(StageMb, "STAGE_MB", 256);
DEFINE_MCCL_PARAM(OneShotSlotKb, "ONESHOT_SLOT_KB", 1024);
DEFINE_MCCL_PARAM(P2pSlotKb, "P2P_SLOT_KB", 0);      // 0: MCCL_P2P_DEPTH chunks of 512 KB per channel
DEFINE_MCCL_PARAM(NvlsEnable, "NVLS_ENABLE", 1);

mcclResult_t cudaFillRankInfo(int device, RankInfo* ri) {
  GpuInfo g;
  MCCLCHECK(discoverGpu(device, &g));
  if (!gpuSupported(g) && envInt("MCCL_ALLOW_ANY_GPU", 0) == 0) {
    MCCL_WARN("the cuda transport needs a compute-capability 10.x GPU, found %s", gpuDescribe(g).c_str());
    return mcclInvalidUsage;
  }
  ri->device = g.device;
  ri->smCount = g.smCount;
  ri->cc = g.ccMajor * 10 + g.ccMinor;
  ri->multicast = g.multicast;
  ri->vmm = g.vmm;
  ri->hbmBytes = g.hbmBytes;
  memcpy(ri->busId, g.busId, sizeof(ri->busId));
  int nDev = cudaDeviceCountSafe();
  ri->peerMask = 0;
  ri->atomicMask = 0;
  for (int d = 0; d < nDev && d < 32; ++d) {
    if (d == g.device) { ri->peerMask |= 1u << d; ri->atomicMask |= 1u << d; continue; }
    int can = 0, atom = 0;
    if (cudaDeviceCanAccessPeer(&can, g.device, d) == cudaSuccess && can) ri->peerMask |= 1u << d;
    if (cudaDeviceGetP2PAttribute(&atom, cudaDevP2PAttrNativeAtomicSupported, g.device, d) == cudaSuccess && atom) ri->atomicMask |= 1u << d;
  }
  cudaGetLastError();
  return mcclSuccess;
}

static size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

mcclResult_t cudaCommInit(mcclComm* c) {
  if (c->nRanks > MCCL_MAX_RANKS) {
    MCCL_WARN("the cuda transport addresses at most %d ranks", MCCL_MAX_RANKS);
    return mcclInvalidUsage;
  }
  MCCLCHECK(cuInitApi());
  CudaState* st = new CudaState();
  c->cu = st;
  st->device = c->device;
  CUDACHECK(cudaSetDevice(c->device));
  CUDACHECK(cudaFree(nullptr));   // make sure the primary context exists

  bool vmm = envInt("MCCL_HEAP_MODE_IPC", 0) == 0;
  bool mc = mcclParamNvlsEnable() != 0 && c->system.nvls && c->nRanks > 1;
  for (const RankInfo& ri : c->infos) vmm = vmm && ri.vmm;
  st->vmm = vmm;
  st->nvls = vmm && mc;

  // Descriptor-passing endpoint; names are derived from the communicator id so every rank can address every peer.
  if (st->vmm && c->nRanks > 1) {
    char name[96];
    for (int r = 0; r < c->nRanks; ++r) {
      snprintf(name, sizeof(name), "mccl-%016llx-%u-%d", (unsigned long long)c->id.nonce, (unsigned)c->id.port, r);
      st->udsNames.push_back(name);
    }
    MCCLCHECK(udsBind(st->udsNames[c->rank].c_str(), &st->udsFd));
    MCCLCHECK(bootstrapBarrier(c->bs));   // every endpoint is bound before anyone sends
  }

  // Status word in pinned, device-mapped host memory: the host can poll it while kernels run.
  CUDACHECK(cudaHostAlloc((void**)&st->statusHost, sizeof(DevStatus), cudaHostAllocMapped | cudaHostAllocPortable));
  memset((void*)st->statusHost, 0, sizeof(DevStatus));
  CUDACHECK(cudaHostGetDevicePointer((void**)&st->statusDev, (void*)st->statusHost, 0));
  CUDACHECK(cudaHostAlloc(&st->probeHost, 64, cudaHostAllocMapped | cudaHostAllocPortable));
  memset(st->probeHost, 0, 64);
  cudaStream_t s;
  CUDACHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  st->internalStream = s;
  {
    cudaStream_t cs;
    int lo = 0, hi = 0;
    CUDACHECK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    CUDACHECK(cudaStreamCreateWithPriority(&cs, cudaStreamNonBlocking, hi));
    st->copyStream = cs;
    cudaEvent_t e;
    CUDACHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming)); st->evStart = e;
    for (int i = 0; i < 2; ++i) {
      CUDACHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming)); st->evCopied[i] = e;
      CUDACHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming)); st->evFree[i] = e;
    }
  }

  CtrlLayout& L = st->layout;
  L.flagsOff = 0;
  L.oneShotSlotBytes = (uint64_t)mcclParamOneShotSlotKb() * 1024;
  L.oneShotOff = alignUp(sizeof(CtrlFlags), 4096);
  L.p2pSlotBytes = mcclParamP2pSlotKb() > 0 ? (uint64_t)mcclParamP2pSlotKb() * 1024 : (uint64_t)p2pChannels(c->nRanks) * MCCL_P2P_DEPTH * (512u << 10);
  L.p2pOff = L.oneShotOff + 2 * (uint64_t)c->nRanks * L.oneShotSlotBytes;
  L.stageOff = alignUp(L.p2pOff + (uint64_t)c->nRanks * L.p2pSlotBytes, 1u << 21);
  L.stageBytes = (uint64_t)mcclParamStageMb() << 20;
  L.totalBytes = L.stageOff + L.stageBytes;
  if (c->nRanks == 1) {   // nothing to exchange: only the flags page is ever touched
    L.p2pOff = L.oneShotOff; L.stageOff = L.oneShotOff; L.stageBytes = 0; L.totalBytes = L.oneShotOff + 4096;
  }
  MCCLCHECK(segmentCreate(c, L.totalBytes, true, &st->ctrl));
  const uint64_t canary = kCanary;
  CUDACHECK(cudaMemcpy(st->ctrl->local + L.flagsOff + offsetof(CtrlFlags, canary), &canary, sizeof(canary), cudaMemcpyHostToDevice));

  DevPeers& P = st->peers;
  memset(&P, 0, sizeof(P));
  P.rank = c->rank;
  P.n = c->nRanks;
  for (int r = 0; r < c->nRanks; ++r) P.ctrl[r] = st->ctrl->peer[r];
  P.ctrlMc = st->ctrl->mc;
  P.layout = L;
  P.status = st->statusDev;
  P.timeoutNs = (uint64_t)mcclParamDeviceTimeoutMs() * 1000000ull;
  // What the tuner may choose depends on what got mapped.
  c->tuner.viable[mcclAlgoNvls] = c->tuner.viable[mcclAlgoNvls] && st->nvls;
  c->graphs[mcclAlgoNvls].viable = c->tuner.viable[mcclAlgoNvls];
  c->tuner.oneShotMaxBytes = std::min<size_t>(c->tuner.oneShotMaxBytes, (size_t)L.oneShotSlotBytes);
  MCCLCHECK(bootstrapBarrier(c->bs));
  return mcclSuccess;
}

void cudaCommAbort(mcclComm* c) {
  if (c->cu && c->cu->statusHost) c->cu->statusHost->abort = 1;   // every device wait gives up at once
}

void cudaCommDestroy(mcclComm* c) {
  CudaState* st = c->cu;
  if (st == nullptr) return;
  cudaSetDevice(st->device);
  cudaDeviceSynchronize();
  // Peers may still be reading this rank's memory: leave together when the control plane still works.
  if (!c->aborted.load() && c->bs && !resultFatal((mcclResult_t)c->asyncState.load())) bootstrapBarrier(c->bs);
  while (!st->segments.empty()) segmentDestroy(c, st->segments.back());
  if (st->statusHost) cudaFreeHost((void*)st->statusHost);
  if (st->probeHost) cudaFreeHost(st->probeHost);
  if (st->internalStream) cudaStreamDestroy((cudaStream_t)st->internalStream);
  if (st->copyStream) cudaStreamDestroy((cudaStream_t)st->copyStream);
  if (st->evStart) cudaEventDestroy((cudaEvent_t)st->evStart);
  for (int i = 0; i < 2; ++i) {
    if (st->evCopied[i]) cudaEventDestroy((cudaEvent_t)st->evCopied[i]);
    if (st->evFree[i]) cudaEventDestroy((cudaEvent_t)st->evFree[i]);
  }
  if (st->udsFd >= 0) sockClose(st->udsFd);
  cudaGetLastError();
  delete st;
  c->cu = nullptr;
}

mcclResult_t cudaCommAsyncError(mcclComm* c, mcclResult_t* out) {
  CudaState* st = c->cu;
  const uint32_t code = st->statusHost->code;
  if (code != 0) {
    const mcclResult_t e = (code == 3 || code == 4) ? mcclInvalidUsage : mcclRemoteError;
    if (code != 3 && code != 4) c->asyncState.store((int)e);
    if (logLevel() >= LOG_WARN) {
      if (code == 4)
        MCCL_WARN("rank %u passed different buffers to a collective than this rank (allocation, offset, count or root): "
                  "a buffer in symmetric memory must be the same part of the same allocation on every rank", st->statusHost->peer);
      else
        MCCL_WARN("device wait gave up: code %u peer %u cta %u step %u", code, st->statusHost->peer, st->statusHost->cta, st->statusHost->step);
    }
    *out = e;
    return mcclSuccess;
  }
  *out = (mcclResult_t)c->asyncState.load();
  return mcclSuccess;
}

mcclResult_t cudaMemAllocSym(mcclComm* c, size_t bytes, void** ptr) {
  CUDACHECK(cudaSetDevice(c->device));
  Segment* s = nullptr;
  MCCLCHECK(segmentCreate(c, bytes, false, &s));
  *ptr = s->local;
  return mcclSuccess;
}

mcclResult_t cudaMemFreeSym(mcclComm* c, void* ptr) {
  CudaState* st = c->cu;
  for (Segment* s : st->segments) {
    if (s->internal || s->registered || s->local != ptr) continue;
    CUDACHECK(cudaSetDevice(c->device));
    CUDACHECK(cudaDeviceSynchronize());
    MCCLCHECK(bootstrapBarrier(c->bs));    // no peer may still be inside a kernel that reads this memory
    segmentDestroy(c, s);
    return mcclSuccess;
  }
  MCCLFAIL(mcclInvalidArgument);
}

mcclResult_t cudaRegister(mcclComm* c, void* ptr, size_t bytes, void** handle) {
  CUDACHECK(cudaSetDevice(c->device));
  Segment* s = nullptr;
  MCCLCHECK(segmentRegister(c, ptr, bytes, &s));
  *handle = s;
  return mcclSuccess;
}

mcclResult_t cudaDeregister(mcclComm* c, void* handle) {
  CudaState* st = c->cu;
  for (Segment* s : st->segments) {
    if (s != handle || !s->registered) continue;
    CUDACHECK(cudaDeviceSynchronize());
    MCCLCHECK(bootstrapBarrier(c->bs));
    segmentDestroy(c, s);
    return mcclSuccess;
  }
  MCCLFAIL(mcclInvalidArgument);
}

mcclResult_t cudaPeerPointer(mcclComm* c, const void* local, int peer, void** out) {
  Segment* s = segmentFind(c->cu, local, 1);
  *out = s ? s->peer[peer] + (static_cast<const char*>(local) - s->local) : nullptr;
  return mcclSuccess;
}

mcclResult_t cudaMcPointer(mcclComm* c, const void* local, void** out) {
  Segment* s = segmentFind(c->cu, local, 1);
  *out = (s && s->mc) ? s->mc + (static_cast<const char*>(local) - s->local) : nullptr;
  return mcclSuccess;
}

mcclResult_t cudaCheckGuards(mcclComm* c, int* intact) {
  CudaState* st = c->cu;
  uint64_t v = 0;
  CUDACHECK(cudaSetDevice(c->device));
  CUDACHECK(cudaDeviceSynchronize());
  CUDACHECK(cudaMemcpy(&v, st->ctrl->local + st->layout.flagsOff + offsetof(CtrlFlags, canary), sizeof(v), cudaMemcpyDeviceToHost));
  *intact = v == kCanary ? 1 : 0;
  return mcclSuccess;
}

bool cudaNvlsEnabled(mcclComm* c) { return c->cu && c->cu->nvls && c->cu->ctrl && c->cu->ctrl->mc != nullptr; }

}  // namespace mccl
