#include "cuda_mem.h"

#include <cstring>
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include "../os/socket.h"

namespace mccl {

namespace {

// ---- driver API table -----------------------------------------------------------------------------------
struct CuApi {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*GetErrorString)(CUresult, const char**);
  CUresult (*MemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr);
  bool ready = false;
};
CuApi cu;

template <typename F> bool resolve(const char* name, F* fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qr;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &qr) != cudaSuccess || p == nullptr) {
    cudaGetLastError();
    return false;
  }
  *fn = reinterpret_cast<F>(p);
  return true;
}

const char* cuErr(CUresult r) {
  const char* s = nullptr;
  if (cu.GetErrorString && cu.GetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "unknown";
}

#define CUCHECK(call)                                                                  \
  do {                                                                                 \
    CUresult r_ = (call);                                                              \
    if (r_ != CUDA_SUCCESS) {                                                          \
      MCCL_WARN("driver error %d (%s) at %s", (int)r_, cuErr(r_), #call);              \
      return ::mccl::noteFailure(mcclSystemError, __FILE__, __LINE__);                 \
    }                                                                                  \
  } while (0)

size_t roundUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

CUmemAllocationProp allocProp(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

mcclResult_t mapWithAccess(CUmemGenericAllocationHandle h, size_t bytes, size_t gran, int device, char** out) {
  CUdeviceptr va = 0;
  CUCHECK(cu.MemAddressReserve(&va, bytes, gran, 0, 0));
  CUresult r = cu.MemMap(va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    cu.MemAddressFree(va, bytes);
    MCCL_WARN("cuMemMap failed: %s", cuErr(r));
    return mcclSystemError;
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = cu.MemSetAccess(va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    cu.MemUnmap(va, bytes);
    cu.MemAddressFree(va, bytes);
    MCCL_WARN("cuMemSetAccess failed: %s", cuErr(r));
    return mcclSystemError;
  }
  *out = reinterpret_cast<char*>(va);
  return mcclSuccess;
}

void unmapVa(char* p, size_t bytes) {
  if (p == nullptr) return;
  cu.MemUnmap((CUdeviceptr)p, bytes);
  cu.MemAddressFree((CUdeviceptr)p, bytes);
}

struct FdMsg { int32_t srcRank; uint32_t serial; uint32_t what; uint32_t pad; };   // what: 0 = memory, 1 = multicast

// All ranks agree: did every rank succeed?
bool allOk(mcclComm* c, bool mine) {
  std::vector<int32_t> v(c->nRanks, 0);
  int32_t m = mine ? 1 : 0;
  if (bootstrapAllGather(c->bs, &m, v.data(), sizeof(int32_t)) != mcclSuccess) return false;
  for (int32_t x : v) if (!x) return false;
  return true;
}

mcclResult_t vmmCreateLocal(mcclComm* c, Segment* s, size_t bytes) {
  CudaState* st = c->cu;
  CUmemAllocationProp prop = allocProp(st->device);
  size_t gran = 0;
  CUCHECK(cu.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  if (st->nvls) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)c->nRanks;
    mp.size = roundUp(bytes, gran);
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    CUCHECK(cu.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
    if (mg > gran) gran = mg;
  }
  s->bytes = roundUp(bytes, gran);
  CUmemGenericAllocationHandle h = 0;
  CUCHECK(cu.MemCreate(&h, s->bytes, &prop, 0));
  s->handle = h;
  MCCLCHECK(mapWithAccess(h, s->bytes, gran, st->device, &s->local));
  s->peer[c->rank] = s->local;
  return mcclSuccess;
}

// Send my descriptor to every peer, receive theirs, map them.
mcclResult_t vmmExchange(mcclComm* c, Segment* s, uint32_t serial) {
  CudaState* st = c->cu;
  int myFd = -1;
  CUCHECK(cu.MemExportToShareableHandle(&myFd, (CUmemGenericAllocationHandle)s->handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  mcclResult_t rc = mcclSuccess;
  FdMsg msg = {c->rank, serial, 0, 0};
  for (int p = 0; p < c->nRanks && rc == mcclSuccess; ++p)
    if (p != c->rank) rc = udsSendFd(st->udsFd, st->udsNames[p].c_str(), myFd, &msg, sizeof(msg));
  close(myFd);
  MCCLCHECK(rc);
  CUmemAllocationProp prop = allocProp(st->device);
  size_t gran = 0;
  CUCHECK(cu.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  for (int k = 0; k < c->nRanks - 1; ++k) {
    FdMsg in;
    int fd = -1;
    rc = udsRecvFd(st->udsFd, 30000, &fd, &in, sizeof(in));
    if (rc != mcclSuccess || fd < 0 || in.serial != serial || in.what != 0 || in.srcRank < 0 || in.srcRank >= c->nRanks) {
      if (fd >= 0) close(fd);
      MCCL_WARN("fd exchange failed (rc %d, serial %u vs %u)", (int)rc, in.serial, serial);
      return mcclSystemError;
    }
    CUmemGenericAllocationHandle hp = 0;
    CUresult r = cu.MemImportFromShareableHandle(&hp, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    if (r != CUDA_SUCCESS) {
      MCCL_WARN("cuMemImportFromShareableHandle failed: %s", cuErr(r));
      return mcclSystemError;
    }
    s->peerHandle[in.srcRank] = hp;
    MCCLCHECK(mapWithAccess(hp, s->bytes, gran, st->device, &s->peer[in.srcRank]));
  }
  return mcclSuccess;
}

mcclResult_t nvlsAttach(mcclComm* c, Segment* s, uint32_t serial) {
  CudaState* st = c->cu;
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = (unsigned)c->nRanks;
  mp.size = s->bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle mch = 0;
  if (c->rank == 0) {
    CUCHECK(cu.MulticastCreate(&mch, &mp));
    int fd = -1;
    CUCHECK(cu.MemExportToShareableHandle(&fd, mch, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    FdMsg msg = {0, serial, 1, 0};
    mcclResult_t rc = mcclSuccess;
    for (int p = 1; p < c->nRanks && rc == mcclSuccess; ++p) rc = udsSendFd(st->udsFd, st->udsNames[p].c_str(), fd, &msg, sizeof(msg));
    close(fd);
    MCCLCHECK(rc);
  } else {
    FdMsg in;
    int fd = -1;
    mcclResult_t rc = udsRecvFd(st->udsFd, 30000, &fd, &in, sizeof(in));
    if (rc != mcclSuccess || fd < 0 || in.serial != serial || in.what != 1) {
      if (fd >= 0) close(fd);
      return mcclSystemError;
    }
    CUresult r = cu.MemImportFromShareableHandle(&mch, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    if (r != CUDA_SUCCESS) { MCCL_WARN("multicast import failed: %s", cuErr(r)); return mcclSystemError; }
  }
  s->mcHandle = mch;
  CUCHECK(cu.MulticastAddDevice(mch, (CUdevice)st->device));
  return mcclSuccess;
}

mcclResult_t nvlsBind(mcclComm* c, Segment* s) {
  CudaState* st = c->cu;
  CUCHECK(cu.MulticastBindMem((CUmemGenericAllocationHandle)s->mcHandle, 0, (CUmemGenericAllocationHandle)s->handle, 0, s->bytes, 0));
  s->mcBound = true;
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = (unsigned)c->nRanks;
  mp.size = s->bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t mg = 0;
  CUCHECK(cu.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
  MCCLCHECK(mapWithAccess((CUmemGenericAllocationHandle)s->mcHandle, s->bytes, mg, st->device, &s->mc));
  return mcclSuccess;
}

void vmmTeardown(mcclComm* c, Segment* s) {
  CudaState* st = c->cu;
  if (s->mc) { unmapVa(s->mc, s->bytes); s->mc = nullptr; }
  if (s->mcBound) { cu.MulticastUnbind((CUmemGenericAllocationHandle)s->mcHandle, (CUdevice)st->device, 0, s->bytes); s->mcBound = false; }
  if (s->mcHandle) { cu.MemRelease((CUmemGenericAllocationHandle)s->mcHandle); s->mcHandle = 0; }
  for (int p = 0; p < c->nRanks; ++p) {
    if (p == c->rank) continue;
    if (s->peer[p]) unmapVa(s->peer[p], s->bytes);
    if (s->peerHandle[p]) cu.MemRelease((CUmemGenericAllocationHandle)s->peerHandle[p]);
    s->peer[p] = nullptr;
    s->peerHandle[p] = 0;
  }
  if (s->local) unmapVa(s->local, s->bytes);
  if (s->handle) cu.MemRelease((CUmemGenericAllocationHandle)s->handle);
  s->local = nullptr;
  s->handle = 0;
}

mcclResult_t ipcShare(mcclComm* c, Segment* s, void* base, size_t offsetInAlloc) {
  struct Msg { cudaIpcMemHandle_t h; uint64_t off; uint64_t pid; };
  Msg mine;
  memset(&mine, 0, sizeof(mine));
  CUDACHECK(cudaIpcGetMemHandle(&mine.h, base));
  mine.off = offsetInAlloc;
  mine.pid = (uint64_t)getpid();
  std::vector<Msg> all(c->nRanks);
  MCCLCHECK(bootstrapAllGather(c->bs, &mine, all.data(), sizeof(Msg)));
  for (int p = 0; p < c->nRanks; ++p) {
    if (p == c->rank) { s->peer[p] = s->local; continue; }
    void* mapped = nullptr;
    CUDACHECK(cudaIpcOpenMemHandle(&mapped, all[p].h, cudaIpcMemLazyEnablePeerAccess));
    s->peerHandle[p] = (unsigned long long)(uintptr_t)mapped;        // what cudaIpcCloseMemHandle wants
    s->peer[p] = static_cast<char*>(mapped) + all[p].off;
  }
  return mcclSuccess;
}

}  // namespace

mcclResult_t cuInitApi() {
  if (cu.ready) return mcclSuccess;
  bool ok = true;
  ok = resolve("cuMemCreate", &cu.MemCreate) && ok;
  ok = resolve("cuMemRelease", &cu.MemRelease) && ok;
  ok = resolve("cuMemExportToShareableHandle", &cu.MemExportToShareableHandle) && ok;
  ok = resolve("cuMemImportFromShareableHandle", &cu.MemImportFromShareableHandle) && ok;
  ok = resolve("cuMemAddressReserve", &cu.MemAddressReserve) && ok;
  ok = resolve("cuMemAddressFree", &cu.MemAddressFree) && ok;
  ok = resolve("cuMemMap", &cu.MemMap) && ok;
  ok = resolve("cuMemUnmap", &cu.MemUnmap) && ok;
  ok = resolve("cuMemSetAccess", &cu.MemSetAccess) && ok;
  ok = resolve("cuMemGetAllocationGranularity", &cu.MemGetAllocationGranularity) && ok;
  ok = resolve("cuGetErrorString", &cu.GetErrorString) && ok;
  ok = resolve("cuMemGetAddressRange", &cu.MemGetAddressRange) && ok;
  // Multicast entry points exist from CUDA 12.1 on; their absence only disables NVLS.
  bool mc = resolve("cuMulticastCreate", &cu.MulticastCreate);
  mc = resolve("cuMulticastAddDevice", &cu.MulticastAddDevice) && mc;
  mc = resolve("cuMulticastBindMem", &cu.MulticastBindMem) && mc;
  mc = resolve("cuMulticastUnbind", &cu.MulticastUnbind) && mc;
  mc = resolve("cuMulticastGetGranularity", &cu.MulticastGetGranularity) && mc;
  if (!mc) cu.MulticastCreate = nullptr;
  if (!ok) MCCLFAIL(mcclSystemError);
  cu.ready = true;
  return mcclSuccess;
}

mcclResult_t segmentCreate(mcclComm* c, size_t bytes, bool internal, Segment** out) {
  CudaState* st = c->cu;
  Segment* s = new Segment();
  s->userBytes = bytes;
  s->internal = internal;
  const uint32_t serial = ++st->segSerial;
  s->serial = serial;
  bool ok = true;
  if (st->vmm) {
    s->mode = SEG_VMM;
    ok = vmmCreateLocal(c, s, bytes) == mcclSuccess;
    // The descriptor exchange only starts once every rank holds its allocation; a rank that failed must
    // not leave the others parked in a receive.
    ok = allOk(c, ok);
    if (ok) ok = allOk(c, vmmExchange(c, s, serial) == mcclSuccess);
    if (ok && st->nvls) {
      bool mcOk = allOk(c, nvlsAttach(c, s, serial) == mcclSuccess);      // every device added before any bind
      if (mcOk) mcOk = allOk(c, nvlsBind(c, s) == mcclSuccess);
      if (!mcOk) {
        MCCL_WARN("NVLS setup failed; continuing without multicast");
        if (s->mc) { unmapVa(s->mc, s->bytes); s->mc = nullptr; }
        if (s->mcBound) { cu.MulticastUnbind((CUmemGenericAllocationHandle)s->mcHandle, (CUdevice)st->device, 0, s->bytes); s->mcBound = false; }
        if (s->mcHandle) { cu.MemRelease((CUmemGenericAllocationHandle)s->mcHandle); s->mcHandle = 0; }
        st->nvls = false;
      }
    }
    if (!ok) {
      MCCL_WARN("VMM segment setup failed; falling back to CUDA IPC for this communicator");
      vmmTeardown(c, s);
      st->vmm = false;
      st->nvls = false;
    }
  }
  if (!st->vmm) {
    s->mode = SEG_IPC;
    s->bytes = roundUp(bytes, 2u << 20);
    void* p = nullptr;
    bool allocOk = cudaMalloc(&p, s->bytes) == cudaSuccess;
    if (!allocOk) cudaGetLastError();
    s->local = static_cast<char*>(p);
    if (!allOk(c, allocOk)) {
      if (p) cudaFree(p);
      delete s;
      MCCLFAIL(mcclSystemError);
    }
    mcclResult_t rc = ipcShare(c, s, p, 0);
    if (!allOk(c, rc == mcclSuccess)) {
      segmentDestroy(c, s);
      MCCLFAIL(mcclSystemError);
    }
  }
  if (cudaMemset(s->local, 0, s->bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    segmentDestroy(c, s);
    MCCLFAIL(mcclSystemError);
  }
  MCCLCHECK(bootstrapBarrier(c->bs));      // nobody touches a peer window before every rank has zeroed its own
  st->segments.push_back(s);
  *out = s;
  MCCL_INFO("segment %u: %zu bytes mode %s mc %p", serial, s->bytes, s->mode == SEG_VMM ? "vmm" : "ipc", (void*)s->mc);
  return mcclSuccess;
}

mcclResult_t segmentRegister(mcclComm* c, void* ptr, size_t bytes, Segment** out) {
  CudaState* st = c->cu;
  Segment* s = new Segment();
  s->mode = SEG_IPC;
  s->registered = true;
  s->serial = ++st->segSerial;
  s->bytes = s->userBytes = bytes;
  s->local = static_cast<char*>(ptr);
  CUdeviceptr base = 0;
  size_t range = 0;
  bool ok = cu.MemGetAddressRange(&base, &range, (CUdeviceptr)ptr) == CUDA_SUCCESS;
  mcclResult_t rc = ok ? ipcShare(c, s, reinterpret_cast<void*>(base), (size_t)((CUdeviceptr)ptr - base)) : mcclSystemError;
  if (!allOk(c, rc == mcclSuccess)) {
    segmentDestroy(c, s);
    MCCLFAIL(mcclSystemError);
  }
  st->segments.push_back(s);
  *out = s;
  return mcclSuccess;
}

void segmentDestroy(mcclComm* c, Segment* s) {
  if (s == nullptr) return;
  CudaState* st = c->cu;
  for (size_t i = 0; i < st->segments.size(); ++i)
    if (st->segments[i] == s) { st->segments.erase(st->segments.begin() + i); break; }
  if (s->mode == SEG_VMM) {
    vmmTeardown(c, s);
  } else {
    for (int p = 0; p < c->nRanks; ++p)
      if (p != c->rank && s->peerHandle[p]) cudaIpcCloseMemHandle(reinterpret_cast<void*>((uintptr_t)s->peerHandle[p]));
    if (!s->registered && s->local) cudaFree(s->local);
    cudaGetLastError();
  }
  delete s;
}

Segment* segmentFind(const CudaState* cu_, const void* ptr, size_t bytes) {
  const char* p = static_cast<const char*>(ptr);
  for (Segment* s : cu_->segments) {
    if (s->internal) continue;
    if (p >= s->local && p + bytes <= s->local + s->bytes) return s;
  }
  return nullptr;
}

}  // namespace mccl
