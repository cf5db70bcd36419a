// Single-GPU emulation of multi-rank all-reduce launches: n buffers of one device stand for n ranks and one
// cooperative launch runs all ranks' CTAs through the production kernel bodies.  For tests on a one-GPU
// machine and for profiling the collective kernels (a profiler cannot wrap a multi-rank job).  NVLS cannot be
// emulated: it needs a multicast object across devices.
#include <cstring>
#include <cuda_runtime.h>
#include <vector>

#include "../core/core.h"
#include "../graph/graph.h"
#include "../transport/cuda_mem.h"
#include "kernels.cuh"

namespace mccl {
namespace {

struct EmuWorld {
  int n = 0;
  int device = -1;
  char* ctrl[MCCL_MAX_RANKS] = {nullptr};
  DevStatus* statusHost = nullptr;
  DevStatus* statusDev = nullptr;
  void* argsDev = nullptr;
  CtrlLayout layout;
};
EmuWorld gEmu;

void emuDestroy() {
  for (int r = 0; r < MCCL_MAX_RANKS; ++r) { if (gEmu.ctrl[r]) cudaFree(gEmu.ctrl[r]); gEmu.ctrl[r] = nullptr; }
  if (gEmu.statusHost) cudaFreeHost((void*)gEmu.statusHost);
  if (gEmu.argsDev) cudaFree(gEmu.argsDev);
  gEmu = EmuWorld();
  cudaGetLastError();
}

mcclResult_t emuEnsure(int n) {
  int dev = 0;
  CUDACHECK(cudaGetDevice(&dev));
  if (gEmu.n == n && gEmu.device == dev) return mcclSuccess;
  emuDestroy();
  CtrlLayout& L = gEmu.layout;
  L.flagsOff = 0;
  L.oneShotSlotBytes = 256u << 10;
  L.oneShotOff = (sizeof(CtrlFlags) + 4095) / 4096 * 4096;
  L.p2pOff = L.stageOff = L.oneShotOff + 2ull * n * L.oneShotSlotBytes;
  L.p2pSlotBytes = 0; L.stageBytes = 0;
  L.totalBytes = L.p2pOff;
  for (int r = 0; r < n; ++r) {
    CUDACHECK(cudaMalloc((void**)&gEmu.ctrl[r], L.totalBytes));
    CUDACHECK(cudaMemset(gEmu.ctrl[r], 0, L.totalBytes));
  }
  CUDACHECK(cudaHostAlloc((void**)&gEmu.statusHost, sizeof(DevStatus), cudaHostAllocMapped));
  memset((void*)gEmu.statusHost, 0, sizeof(DevStatus));
  CUDACHECK(cudaHostGetDevicePointer((void**)&gEmu.statusDev, (void*)gEmu.statusHost, 0));
  CUDACHECK(cudaMalloc(&gEmu.argsDev, MCCL_MAX_RANKS * sizeof(PullArgs)));
  gEmu.n = n;
  gEmu.device = dev;
  return mcclSuccess;
}

DevPeers emuPeers(int r) {
  DevPeers P;
  memset(&P, 0, sizeof(P));
  P.rank = r;
  P.n = gEmu.n;
  for (int p = 0; p < gEmu.n; ++p) P.ctrl[p] = gEmu.ctrl[p];
  P.layout = gEmu.layout;
  P.status = gEmu.statusDev;
  P.timeoutNs = 2000000000ull;
  return P;
}

template <typename Args>
mcclResult_t emuLaunch(const void* kernel, const std::vector<Args>& args, int ctas, cudaStream_t s) {
  CUDACHECK(cudaMemcpyAsync(gEmu.argsDev, args.data(), args.size() * sizeof(Args), cudaMemcpyHostToDevice, s));
  void* devArgs = gEmu.argsDev;
  void* params[] = {&devArgs};
  // Cooperative launch: the runtime refuses grids that cannot be resident at once, which is exactly the
  // guarantee CTAs that wait on one another need.
  CUDACHECK(cudaLaunchCooperativeKernel(kernel, dim3(ctas, (unsigned)args.size()), dim3(kThreads), params, 0, s));
  return mcclSuccess;
}

#define EMU_KERNEL(dt, NAME)                                                                             \
  ((dt) == mcclFloat32 ? (const void*)NAME<float> : (dt) == mcclBfloat16 ? (const void*)NAME<__nv_bfloat16>   \
   : (dt) == mcclFloat16 ? (const void*)NAME<__half> : (dt) == mcclInt32 ? (const void*)NAME<int32_t> : (const void*)nullptr)

}  // namespace
}  // namespace mccl

// In-place all-reduce over `nRanks` buffers of this device, one per emulated rank.  algo: two-shot, one-shot,
// ring or tree.  Returns mcclRemoteError if a device wait gave up.
// `phases` / `shift`: the ring kernel's reduce (1) and gather (2) steps or the tree kernel's up (1) and down (2)
// phases on their own, as the reduce-scatter / all-gather / reduce / broadcast launchers use them (0 = both).
extern "C" mcclResult_t mcclEmuPhases(int nRanks, void* const* bufs, uint64_t count, int dt, int op, int algo, int phases,
                                      int shift, int ctas, mcclStream_t stream) {
  using namespace mccl;
  if (nRanks < 2 || nRanks > MCCL_MAX_RANKS || bufs == nullptr || count == 0 || (unsigned)op >= (unsigned)mcclNumOps) return mcclInvalidArgument;
  const size_t es = mcclDataSize((mcclDataType_t)dt);
  if (es == 0 || EMU_KERNEL(dt, pullKernelEmu) == nullptr) return mcclInvalidArgument;
  MCCLCHECK(emuEnsure(nRanks));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const uint64_t bytes = count * es;
  const int n = nRanks, divisor = op == mcclAvg ? n : 1, redOp = op == mcclAvg ? mcclSum : op;
  if (ctas <= 0) ctas = 8;
  if (ctas * n > 148) ctas = 148 / n;
  mcclResult_t rc;
  if (algo == mcclAlgoTwoShot) {
    std::vector<PullArgs> args(n);
    for (int r = 0; r < n; ++r) {
      PullArgs& a = args[r];
      memset(&a, 0, sizeof(a));
      a.peers = emuPeers(r); a.nCtas = ctas; a.op = redOp; a.divisor = divisor; a.midBarrier = 1;
      const uint64_t o0 = shardOff(bytes, n, r), o1 = shardEnd(bytes, n, r);
      a.nSrcA = n;
      for (int p = 0; p < n; ++p) a.srcA[p] = static_cast<char*>(bufs[p]) + o0;
      a.dstA = static_cast<char*>(bufs[r]) + o0;
      a.aBytes = o1 - o0;
      for (int i = 1; i < n; ++i) {
        const int p = (r + i) % n;
        const uint64_t q0 = shardOff(bytes, n, p), q1 = shardEnd(bytes, n, p);
        a.jobs[a.nJobs++] = CopyJob{static_cast<char*>(bufs[p]) + q0, static_cast<char*>(bufs[r]) + q0, q1 - q0};
      }
    }
    rc = emuLaunch(EMU_KERNEL(dt, pullKernelEmu), args, ctas, s);
  } else if (algo == mcclAlgoOneShot) {
    if (bytes % 16 || bytes > gEmu.layout.oneShotSlotBytes) return mcclInvalidArgument;
    std::vector<OneShotArgs> args(n);
    for (int r = 0; r < n; ++r) {
      OneShotArgs& a = args[r];
      memset(&a, 0, sizeof(a));
      a.peers = emuPeers(r); a.nCtas = ctas; a.op = redOp; a.divisor = divisor;
      a.send = static_cast<const char*>(bufs[r]); a.recv = static_cast<char*>(bufs[r]); a.bytes = bytes;
    }
    if (ctas > MCCL_ONESHOT_MAX_CTAS) ctas = MCCL_ONESHOT_MAX_CTAS;
    for (OneShotArgs& a : args) a.nCtas = ctas;
    rc = emuLaunch(EMU_KERNEL(dt, oneShotKernelEmu), args, ctas, s);
  } else if (algo == mcclAlgoRing) {
    if (bytes % 16 || bytes / 16 < (uint64_t)2 * n) return mcclInvalidArgument;
    std::vector<RingArgs> args(n);
    for (int r = 0; r < n; ++r) {
      RingArgs& a = args[r];
      memset(&a, 0, sizeof(a));
      a.peers = emuPeers(r); a.nCtas = ctas; a.op = redOp; a.divisor = divisor;
      a.prev = (r + n - 1) % n; a.next = (r + 1) % n; a.bytes = bytes; a.phases = phases; a.shift = shift;
      for (int p = 0; p < n; ++p) a.buf[p] = static_cast<char*>(bufs[p]);
    }
    rc = emuLaunch(EMU_KERNEL(dt, ringKernelEmu), args, ctas, s);
  } else if (algo == mcclAlgoTree) {
    if (bytes % 16 || bytes / 16 < (uint64_t)2 * n) return mcclInvalidArgument;
    std::vector<TreeArgs> args(n);
    for (int r = 0; r < n; ++r) {
      TreeArgs& a = args[r];
      memset(&a, 0, sizeof(a));
      a.peers = emuPeers(r); a.nCtas = ctas; a.op = redOp; a.divisor = divisor; a.bytes = bytes; a.phases = phases;
      getDtree(n, r, &a.up[0], &a.down[0][0], &a.down[0][1], &a.up[1], &a.down[1][0], &a.down[1][1]);
      for (int p = 0; p < n; ++p) a.buf[p] = static_cast<char*>(bufs[p]);
    }
    rc = emuLaunch(EMU_KERNEL(dt, treeKernelEmu), args, ctas, s);
  } else {
    return mcclInvalidArgument;
  }
  MCCLCHECK(rc);
  CUDACHECK(cudaStreamSynchronize(s));
  return gEmu.statusHost->code == 0 ? mcclSuccess : mcclRemoteError;
}

extern "C" mcclResult_t mcclEmuAllReduce(int nRanks, void* const* bufs, uint64_t count, int dt, int op, int algo, int ctas,
                                         mcclStream_t stream) {
  return mcclEmuPhases(nRanks, bufs, count, dt, op, algo, 0, 0, ctas, stream);
}

extern "C" void mcclEmuDestroy(void) { mccl::emuDestroy(); }

// The one-shot call counters of emulated rank `rank` (the first `cap` CTAs), for tests of their lockstep.
extern "C" mcclResult_t mcclEmuOneShotCounters(int rank, uint64_t* out, int cap) {
  using namespace mccl;
  if (rank < 0 || rank >= gEmu.n || out == nullptr || cap < 1 || cap > MCCL_MAX_CTAS) return mcclInvalidArgument;
  const CtrlFlags* f = reinterpret_cast<const CtrlFlags*>(gEmu.ctrl[rank] + gEmu.layout.flagsOff);
  CUDACHECK(cudaMemcpy(out, f->oneShotCalls, (size_t)cap * sizeof(uint64_t), cudaMemcpyDeviceToHost));
  return mcclSuccess;
}

// ---- index-arithmetic probes (host only): the work splits the kernels rely on, for exhaustive CPU tests ----------------

// Tiles CTA `cta` of `G` takes out of V units: writes up to `cap` (lo, hi) pairs, returns how many there are.
extern "C" int mcclDbgWorkSplit(uint64_t V, int G, int cta, uint64_t* lo, uint64_t* hi, int cap) {
  const uint64_t tile = mccl::tileUnits(V, G);
  int k = 0;
  for (uint64_t a = (uint64_t)cta * tile; a < V; a += (uint64_t)G * tile, ++k)
    if (k < cap) { lo[k] = a; hi[k] = a + tile < V ? a + tile : V; }
  return k;
}

extern "C" void mcclDbgShard(uint64_t bytes, int n, int r, uint64_t* off, uint64_t* end) {
  *off = mccl::shardOff(bytes, n, r);
  *end = mccl::shardEnd(bytes, n, r);
}
