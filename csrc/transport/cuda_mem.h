// Symmetric device memory of the cuda transport.
//
// A *segment* is one allocation of equal size on every rank that every rank maps from every peer:
// rank r holds peer[0..n-1], peer[r] being its own copy.  Segments are created collectively.
//   * VMM mode (default): cuMemCreate with a POSIX-fd shareable handle; the descriptors travel to the
//     peers over an AF_UNIX datagram socket (SCM_RIGHTS); cuMemImportFromShareableHandle + cuMemMap +
//     cuMemSetAccess give the peer windows.  When every GPU supports multicast, the segment is also bound
//     to an NVLS multicast object and mapped a second time (`mc`), which is what multimem.* addresses.
//   * IPC mode (fallback, and the only way to register memory somebody else allocated with cudaMalloc):
//     cudaIpcGetMemHandle / cudaIpcOpenMemHandle; no multicast.
// Role parity: mcclPageAlloc / mcclMemPool of the reference (src/allocator.cc:11-77) hand out buffers every
// engine can use without a copy; here "every engine" is every GPU of the box.
#pragma once

#include <cstddef>
#include <cstdint>
#include <vector>

#include "../comm/comm.h"
#include "../device/devcomm.h"

namespace mccl {

enum SegMode { SEG_VMM = 0, SEG_IPC = 1 };

struct Segment {
  int mode = SEG_VMM;
  size_t bytes = 0;          // mapped size
  size_t userBytes = 0;      // size the caller asked for
  char* local = nullptr;
  char* peer[MCCL_MAX_RANKS] = {nullptr};
  char* mc = nullptr;        // multicast alias (null without NVLS)
  bool registered = false;   // wraps caller-owned memory (mcclCommRegister)
  bool internal = false;     // control block / staging, not returned by lookups of user pointers
  uint32_t serial = 0;       // creation number: equal on every rank, because segments are created collectively
  // VMM bookkeeping
  unsigned long long handle = 0;
  unsigned long long peerHandle[MCCL_MAX_RANKS] = {0};
  unsigned long long mcHandle = 0;
  bool mcBound = false;
};

struct CudaState {
  int device = 0;
  bool vmm = false;          // segments are created in VMM mode
  bool nvls = false;         // multicast objects are created for new segments
  int udsFd = -1;            // AF_UNIX endpoint for fd passing
  std::vector<std::string> udsNames;
  uint32_t segSerial = 0;
  std::vector<Segment*> segments;
  Segment* ctrl = nullptr;
  CtrlLayout layout;
  DevStatus* statusHost = nullptr;
  DevStatus* statusDev = nullptr;
  DevPeers peers;            // template copied into every kernel's arguments
  void* internalStream = nullptr;   // for library-internal work (finalize barrier, calibration)
  // Staging of ordinary (non-symmetric) buffers: the copy into one half of the stage runs on its own stream
  // while the collective works on the other half.
  void* copyStream = nullptr;
  void* evStart = nullptr;
  void* evCopied[2] = {nullptr, nullptr};
  void* evFree[2] = {nullptr, nullptr};
  void* probeHost = nullptr;        // pinned int for RecvAny
  uint64_t p2pSent[MCCL_MAX_RANKS] = {0};    // host mirrors of the FIFO counters are not needed: device keeps them
};

// Driver entry points (resolved through the runtime, so the library has no link-time libcuda dependency).
mcclResult_t cuInitApi();

mcclResult_t segmentCreate(mcclComm* c, size_t bytes, bool internal, Segment** out);   // collective
mcclResult_t segmentRegister(mcclComm* c, void* ptr, size_t bytes, Segment** out);    // collective, IPC
void         segmentDestroy(mcclComm* c, Segment* s);
// Segment that fully contains [ptr, ptr+bytes), or null.
Segment*     segmentFind(const CudaState* cu, const void* ptr, size_t bytes);

#define CUDACHECK(call)                                                                   \
  do {                                                                                    \
    cudaError_t e_ = (call);                                                              \
    if (e_ != cudaSuccess) {                                                              \
      MCCL_WARN("CUDA error %s at %s", cudaGetErrorString(e_), #call);                    \
      cudaGetLastError();                                                                 \
      return ::mccl::noteFailure(mcclSystemError, __FILE__, __LINE__);                    \
    }                                                                                     \
  } while (0)

}  // namespace mccl
