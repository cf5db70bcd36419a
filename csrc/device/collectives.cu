// Host side of the collective kernels: resolves buffers to symmetric segments, stages what is not
// symmetric, fills the kernel arguments for the chosen algorithm and launches on the caller's stream.
// Role parity: the per-collective algorithm entry points of the reference (src/device/all_reduce.h,
// all_gather.h, reduce_scatter.h, broadcast.h, reduce.h) and its launch step (src/coll/coll.cc:33-43).
#include <algorithm>
#include <cstring>
#include <cuda_runtime.h>

#include "../transport/cuda_mem.h"
#include "kernels.cuh"

namespace mccl {

DEFINE_MCCL_PARAM(NChannels, "NCHANNELS", 0);

namespace {

struct View {
  Segment* seg = nullptr;
  size_t off = 0;
  bool sym() const { return seg != nullptr; }
  char* peer(int p) const { return seg->peer[p] + off; }
  char* mc() const { return seg->mc ? seg->mc + off : nullptr; }
};

View viewOf(const CudaState* st, const void* ptr, size_t bytes) {
  View v;
  if (ptr == nullptr) return v;
  v.seg = segmentFind(st, ptr, bytes);
  if (v.seg) v.off = (size_t)(static_cast<const char*>(ptr) - v.seg->local);
  return v;
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// CTAs for a kernel that moves `bytes` per rank.
int pickCtas(const mcclComm* c, size_t bytes, int algo) {
  int g;
  // From sweeps on 8 B200: NVLS saturates with 16-32 CTAs at every size; the load/store algorithms keep
  // gaining up to 64.
  if (bytes <= (64u << 10)) g = 2;
  else if (bytes <= (512u << 10)) g = 8;
  else if (bytes <= (1u << 20)) g = 16;
  else if (bytes <= (8u << 20) || algo == mcclAlgoNvls) g = 32;
  else g = 64;
  if (algo == mcclAlgoOneShot) g = std::min(g, 8);
  const int limit = c->graphs[algo >= 0 && algo < mcclNumAlgos ? algo : mcclAlgoTwoShot].nChannels;
  if (limit > 0) g = std::min(g, std::max(limit, 1));
  if (mcclParamNChannels() > 0) g = (int)mcclParamNChannels();
  if (c->forcedCtas > 0) g = c->forcedCtas;
  if (c->maxCtas > 0) g = std::min(g, c->maxCtas);
  return std::max(1, std::min(g, MCCL_MAX_CTAS));
}

mcclResult_t launched(mcclComm* c, const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    MCCL_WARN("launch of %s failed: %s", what, cudaGetErrorString(e));
    return mcclSystemError;
  }
  c->launches.fetch_add(1);
  return mcclSuccess;
}

// `maxBlocks`: 592 (four blocks per SM) fills every thread slot of the GPU, which is right for a copy that runs
// alone; a copy meant to run BESIDE a collective takes half of the SMs, or the collective's CTAs would find no room
// until the copy has ended (one copy block and one block of the NVLS kernel do not fit the register file of one SM
// together: with a copy block on every SM, a 1 GB all-reduce ran at 0.78 of the symmetric path, with 74 at 0.89).
mcclResult_t launchCopy(mcclComm* c, const void* src, void* dst, uint64_t rows, uint64_t rowBytes, uint64_t srcPitch,
                        uint64_t dstPitch, cudaStream_t s, int maxBlocks = 592) {
  if (rows == 0 || rowBytes == 0 || (src == dst && srcPitch == dstPitch)) return mcclSuccess;
  const uint64_t total = rows * rowBytes;
  int blocks = (int)std::min<uint64_t>((total / 16 + kThreads - 1) / kThreads + 1, (uint64_t)maxBlocks);
  copyKernel<<<blocks, kThreads, 0, s>>>(static_cast<const char*>(src), static_cast<char*>(dst), rows, rowBytes, srcPitch, dstPitch);
  return launched(c, "copyKernel");
}

template <typename T>
mcclResult_t launchPullT(mcclComm* c, const PullArgs& a, cudaStream_t s, bool fast) {
  const int n = a.nSrcA;
  if (fast && n == 2) pullKernel<T, 2><<<a.nCtas, kThreads, 0, s>>>(a);
  else if (fast && n == 4) pullKernel<T, 4><<<a.nCtas, kThreads, 0, s>>>(a);
  else if (fast && n == 8) pullKernel<T, 8><<<a.nCtas, kThreads, 0, s>>>(a);
  else pullKernel<T, 0><<<a.nCtas, kThreads, 0, s>>>(a);
  return launched(c, "pullKernel");
}

mcclResult_t launchPull(mcclComm* c, const PullArgs& a, mcclDataType_t dt, cudaStream_t s) {
  switch (dt) {
    case mcclFloat32:  return launchPullT<float>(c, a, s, true);
    case mcclFloat16:  return launchPullT<__half>(c, a, s, true);
    case mcclBfloat16: return launchPullT<__nv_bfloat16>(c, a, s, true);
    case mcclInt32:    return launchPullT<int32_t>(c, a, s, true);
    case mcclUint32:   return launchPullT<uint32_t>(c, a, s, false);
    case mcclInt64:    return launchPullT<int64_t>(c, a, s, false);
    case mcclUint64:   return launchPullT<uint64_t>(c, a, s, false);
    case mcclFloat64:  return launchPullT<double>(c, a, s, false);
    case mcclInt8:     return launchPullT<int8_t>(c, a, s, false);
    case mcclUint8:    return launchPullT<uint8_t>(c, a, s, false);
    default: return mcclInvalidArgument;
  }
}

#define DISPATCH_ALL_TYPES(dt, KERNEL, grid, stream, args)                                   \
  switch (dt) {                                                                              \
    case mcclFloat32:  KERNEL<float><<<grid, kThreads, 0, stream>>>(args); break;             \
    case mcclFloat16:  KERNEL<__half><<<grid, kThreads, 0, stream>>>(args); break;            \
    case mcclBfloat16: KERNEL<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(args); break;     \
    case mcclInt32:    KERNEL<int32_t><<<grid, kThreads, 0, stream>>>(args); break;           \
    case mcclUint32:   KERNEL<uint32_t><<<grid, kThreads, 0, stream>>>(args); break;          \
    case mcclInt64:    KERNEL<int64_t><<<grid, kThreads, 0, stream>>>(args); break;           \
    case mcclUint64:   KERNEL<uint64_t><<<grid, kThreads, 0, stream>>>(args); break;          \
    case mcclFloat64:  KERNEL<double><<<grid, kThreads, 0, stream>>>(args); break;            \
    case mcclInt8:     KERNEL<int8_t><<<grid, kThreads, 0, stream>>>(args); break;            \
    case mcclUint8:    KERNEL<uint8_t><<<grid, kThreads, 0, stream>>>(args); break;           \
    default: return mcclInvalidArgument;                                                     \
  }

struct Call {
  mcclComm* c;
  CudaState* st;
  int n, r;
  mcclDataType_t dt;
  size_t es;
  mcclRedOp_t op;
  int divisor;
  cudaStream_t s;
  char* stageLocal() const { return st->ctrl->local + st->layout.stageOff; }
  char* stagePeer(int p) const { return st->ctrl->peer[p] + st->layout.stageOff; }
  char* stageMc() const { return st->ctrl->mc ? st->ctrl->mc + st->layout.stageOff : nullptr; }
  size_t stageBytes() const { return (size_t)st->layout.stageBytes; }
};

PullArgs basePull(const Call& k, size_t bytesForCtas, int algo) {
  PullArgs a;
  memset(&a, 0, sizeof(a));
  a.peers = k.st->peers;
  a.nCtas = pickCtas(k.c, bytesForCtas, algo);
  a.op = (k.op == mcclAvg) ? mcclSum : k.op;
  a.divisor = k.divisor;
  return a;
}

// Defined further down (they need the ring / tree launcher).
mcclResult_t agRingFwd(const Call& k, const void* send, void* recv, size_t slot);
mcclResult_t rsRingFwd(const Call& k, const void* send, void* recv, size_t blk);
mcclResult_t bcastTreeFwd(const Call& k, const void* send, void* recv, size_t bytes, int root);
mcclResult_t reduceTreeFwd(const Call& k, const void* send, void* recv, size_t bytes, int root);
mcclResult_t bcastRingFwd(const Call& k, const void* send, void* recv, size_t bytes, int root);
mcclResult_t reduceRingFwd(const Call& k, const void* send, void* recv, size_t bytes, int root);
mcclResult_t agTreeFwd(const Call& k, const void* send, void* recv, size_t slot);
mcclResult_t rsTreeFwd(const Call& k, const void* send, void* recv, size_t blk);

}  // namespace

namespace {

// ---- two-shot core: fold my shard from everyone's input, then collect the other shards -----------------------
// in[p]  : rank p's input (as mapped here)      red[p] : rank p's peer-visible result area
// out    : this rank's final destination (may equal red[r]); `collect` = run phase B on this rank
mcclResult_t twoShot(const Call& k, char* const in[], char* const red[], char* out, size_t bytes, bool collect, int algoForCtas) {
  PullArgs a = basePull(k, bytes, algoForCtas);
  const int n = k.n, r = k.r;
  const uint64_t o0 = shardOff(bytes, n, r), o1 = shardEnd(bytes, n, r);
  a.nSrcA = n;
  for (int p = 0; p < n; ++p) a.srcA[p] = in[p] + o0;
  a.dstA = red[r] + o0;
  a.dstA2 = (out != nullptr && out != red[r]) ? out + o0 : nullptr;
  a.aBytes = o1 - o0;
  a.nJobs = 0;
  a.midBarrier = 1;
  if (collect) {
    char* dst = out ? out : red[r];
    // Rank r starts with peer r+1: at any moment every peer is being read by a different rank, instead
    // of all ranks draining peer 0 first, then peer 1, ...
    for (int i = 1; i < n; ++i) {
      const int p = (r + i) % n;
      const uint64_t q0 = shardOff(bytes, n, p), q1 = shardEnd(bytes, n, p);
      a.jobs[a.nJobs++] = CopyJob{red[p] + q0, dst + q0, q1 - q0};
    }
  }
  return launchPull(k.c, a, k.dt, k.s);
}

size_t stageChunk(const Call& k, size_t rows) {
  size_t per = k.stageBytes() / std::max<size_t>(rows, 1);
  per = per / 256 * 256;
  return per;
}

// Staged all-reduce of an ordinary buffer, two halves of the stage in flight: while the collective kernel works on
// one half (on the caller's stream), the communicator's copy stream brings the next chunk into the other half and,
// where the result lands in the stage (`copyBack`), takes the previous chunk's result out to `recv`.  Order on the
// copy stream: in(0), in(1), out(0), in(2), out(1), ... so a copy-in never waits for the collective before it.
// `run(half offset in the stage, offset in the message, length)` launches the collective for one chunk on the
// caller's stream.  Messages that fit one half take the plain path (copy, collective, copy, one stream).
template <typename Run>
mcclResult_t stagedPipeline(const Call& k, const void* send, void* recv, bool copyBack, size_t bytes, size_t align, Run&& run) {
  CudaState* st = k.st;
  size_t half = k.stageBytes() / 2 / 256 * 256;
  if (align > 1) half = half / align * align;
  if (half == 0) return mcclInternalError;
  const char* src = static_cast<const char*>(send);
  char* dst = static_cast<char*>(recv);
  if (bytes <= half || st->copyStream == nullptr) {
    const size_t whole = align > 1 ? k.stageBytes() / 256 * 256 / align * align : k.stageBytes() / 256 * 256;
    for (size_t off = 0; off < bytes; off += whole) {
      const size_t len = std::min(whole, bytes - off);
      MCCLCHECK(launchCopy(k.c, src + off, k.stageLocal(), 1, len, len, len, k.s));
      MCCLCHECK(run((size_t)0, off, len));
      if (copyBack) MCCLCHECK(launchCopy(k.c, k.stageLocal(), dst + off, 1, len, len, len, k.s));
    }
    return mcclSuccess;
  }
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(st->copyStream);
  static const int besideBlocks = std::max(1, (int)envInt("MCCL_STAGE_COPY_CTAS", 74));
  cudaEvent_t evStart = reinterpret_cast<cudaEvent_t>(st->evStart);
  auto copied = [&](int c) { return reinterpret_cast<cudaEvent_t>(st->evCopied[c & 1]); };
  auto freed = [&](int c) { return reinterpret_cast<cudaEvent_t>(st->evFree[c & 1]); };
  const int chunks = (int)((bytes + half - 1) / half);
  auto copyIn = [&](int c) -> mcclResult_t {
    const size_t off = (size_t)c * half, len = std::min(half, bytes - off);
    if (c >= 2 && !copyBack) CUDACHECK(cudaStreamWaitEvent(cs, freed(c), 0));    // the collective that read this half is done
    MCCLCHECK(launchCopy(k.c, src + off, k.stageLocal() + (size_t)(c & 1) * half, 1, len, len, len, cs, c == 0 ? 592 : besideBlocks));
    CUDACHECK(cudaEventRecord(copied(c), cs));
    return mcclSuccess;
  };
  CUDACHECK(cudaEventRecord(evStart, k.s));               // whatever produced `send` on the caller's stream comes first
  CUDACHECK(cudaStreamWaitEvent(cs, evStart, 0));
  MCCLCHECK(copyIn(0));
  for (int c = 0; c < chunks; ++c) {
    const size_t off = (size_t)c * half, len = std::min(half, bytes - off);
    CUDACHECK(cudaStreamWaitEvent(k.s, copied(c), 0));
    if (c + 1 < chunks) MCCLCHECK(copyIn(c + 1));
    MCCLCHECK(run((size_t)(c & 1) * half, off, len));
    CUDACHECK(cudaEventRecord(freed(c), k.s));
    if (copyBack) {
      CUDACHECK(cudaStreamWaitEvent(cs, freed(c), 0));
      MCCLCHECK(launchCopy(k.c, k.stageLocal() + (size_t)(c & 1) * half, dst + off, 1, len, len, len, cs, c + 1 == chunks ? 592 : besideBlocks));
    }
  }
  if (copyBack) {                                         // the caller's stream continues once the last result is out
    CUDACHECK(cudaEventRecord(evStart, cs));
    CUDACHECK(cudaStreamWaitEvent(k.s, evStart, 0));
  }
  return mcclSuccess;
}

mcclResult_t arTwoShot(const Call& k, const void* send, void* recv, size_t bytes) {
  const View sv = viewOf(k.st, send, bytes), rv = viewOf(k.st, recv, bytes);
  char* in[MCCL_MAX_RANKS];
  char* red[MCCL_MAX_RANKS];
  if (sv.sym() && rv.sym()) {
    for (int p = 0; p < k.n; ++p) { in[p] = sv.peer(p); red[p] = rv.peer(p); }
    return twoShot(k, in, red, static_cast<char*>(recv), bytes, true, mcclAlgoTwoShot);
  }
  // Phase A writes the folded shard to the stage (for the peers) and to `recv`; phase B pulls the other shards from
  // the peers' stages straight into `recv`: no copy back.
  return stagedPipeline(k, send, recv, false, bytes, k.es, [&](size_t stageOff, size_t off, size_t len) -> mcclResult_t {
    for (int p = 0; p < k.n; ++p) in[p] = red[p] = k.stagePeer(p) + stageOff;
    return twoShot(k, in, red, static_cast<char*>(recv) + off, len, true, mcclAlgoTwoShot);
  });
}

mcclResult_t arOneShot(const Call& k, const void* send, void* recv, size_t bytes) {
  OneShotArgs a;
  memset(&a, 0, sizeof(a));
  a.peers = k.st->peers;
  a.nCtas = std::min(pickCtas(k.c, bytes, mcclAlgoOneShot), MCCL_ONESHOT_MAX_CTAS);
  a.op = (k.op == mcclAvg) ? mcclSum : k.op;
  a.divisor = k.divisor;
  a.send = static_cast<const char*>(send);
  a.recv = static_cast<char*>(recv);
  a.bytes = bytes;
  DISPATCH_ALL_TYPES(k.dt, oneShotKernel, a.nCtas, k.s, a);
  return launched(k.c, "oneShotKernel");
}

bool nvlsType(mcclDataType_t dt, mcclRedOp_t op, int n) {
  if (!nvlsAvgExact(dt, op, n)) return false;
  if (dt == mcclFloat32) return op == mcclSum || op == mcclAvg;
  if (dt == mcclFloat16 || dt == mcclBfloat16) return op == mcclSum || op == mcclAvg || op == mcclMin || op == mcclMax;
  return false;
}

template <int U>
mcclResult_t launchNvlsU(const Call& k, const NvlsArgs& a, bool reducing) {
  if (!reducing) { nvlsKernel<float, U><<<a.nCtas, kThreads, 0, k.s>>>(a); return launched(k.c, "nvlsKernel"); }
  switch (k.dt) {
    case mcclFloat32:  nvlsKernel<float, U><<<a.nCtas, kThreads, 0, k.s>>>(a); break;
    case mcclFloat16:  nvlsKernel<__half, U><<<a.nCtas, kThreads, 0, k.s>>>(a); break;
    case mcclBfloat16: nvlsKernel<__nv_bfloat16, U><<<a.nCtas, kThreads, 0, k.s>>>(a); break;
    default: return mcclInvalidArgument;
  }
  return launched(k.c, "nvlsKernel");
}

mcclResult_t launchNvls(const Call& k, const NvlsArgs& a, bool reducing, bool rootOnly = false) {
  // One rank moving the whole message needs about 8 MB in flight to fill its port (the round trip through
  // the switch is several microseconds): 128 CTAs x 512 threads x 8 vectors.
  if (rootOnly) return launchNvlsU<8>(k, a, reducing);
  static const int unroll = (int)envInt("MCCL_NVLS_UNROLL", 4);
  if (unroll >= 8) return launchNvlsU<8>(k, a, reducing);
  if (unroll <= 2) return launchNvlsU<2>(k, a, reducing);
  return launchNvlsU<4>(k, a, reducing);
}

// `rootOnly`: one rank moves the whole message (broadcast, reduce), so it needs the CTAs that an
// all-reduce spreads over all ranks.
NvlsArgs baseNvls(const Call& k, size_t bytes, bool rootOnly = false) {
  NvlsArgs a;
  memset(&a, 0, sizeof(a));
  a.peers = k.st->peers;
  a.nCtas = pickCtas(k.c, bytes, rootOnly ? mcclAlgoTwoShot : mcclAlgoNvls);
  if (rootOnly && bytes > (32u << 20) && k.c->forcedCtas == 0 && mcclParamNChannels() == 0)
    a.nCtas = k.c->maxCtas > 0 ? std::min(128, k.c->maxCtas) : 128;
  a.op = (k.op == mcclAvg) ? mcclSum : k.op;
  a.divisor = 1;
  a.active = 1;
  return a;
}

// Rooted collectives with one shard per rank (NvlsRootedArgs) or with the root moving the whole message.  Measured
// on 4 B200 (us, NCCL / root only / spread): broadcast 64 MB 143 / 161 / 159, 1 GB 1635 / 2125 / 2042; reduce 64 MB
// 145 / 162 / 162, 256 MB 452 / 618 / 511, 1 GB 1656 / 2385 / 1936; below 64 MB the root-only form is the faster
// one (16 MB: 59 against 63 - 67).  So: spread from 64 MB up.  MCCL_NVLS_SPREAD=0 never, =1 at every size.
bool nvlsSpread(size_t bytes) {
  static const int mode = (int)envInt("MCCL_NVLS_SPREAD", -1);
  if (mode >= 0) return mode != 0;
  return bytes >= ((size_t)64 << 20);
}

mcclResult_t launchNvlsRooted(const Call& k, const NvlsRootedArgs& a) {
  static const int unroll = (int)envInt("MCCL_NVLS_UNROLL", 4);
  const mcclDataType_t dt = a.reducing ? k.dt : mcclFloat32;      // a broadcast moves bits
#define ROOTED(T)                                                                        \
  do {                                                                                   \
    if (unroll >= 8) nvlsRootedKernel<T, 8><<<a.nCtas, kThreads, 0, k.s>>>(a);           \
    else nvlsRootedKernel<T, 4><<<a.nCtas, kThreads, 0, k.s>>>(a);                       \
  } while (0)
  switch (dt) {
    case mcclFloat32:  ROOTED(float); break;
    case mcclFloat16:  ROOTED(__half); break;
    case mcclBfloat16: ROOTED(__nv_bfloat16); break;
    default: return mcclInvalidArgument;
  }
#undef ROOTED
  return launched(k.c, "nvlsRootedKernel");
}

// NVLS all-reduce on multicast-mapped memory: the switch adds my shard across ranks and replicates the result.
mcclResult_t arNvlsOn(const Call& k, char* mcIn, char* mcOut, size_t bytes) {
  NvlsArgs a = baseNvls(k, bytes);
  const uint64_t o0 = shardOff(bytes, k.n, k.r), o1 = shardEnd(bytes, k.n, k.r);
  a.loadReduce = 1;
  a.mcStore = 1;
  a.mcSrc = mcIn + o0;
  a.mcDst = mcOut + o0;
  a.bytes = o1 - o0;
  a.divisor = k.divisor;
  return launchNvls(k, a, true);
}

mcclResult_t arNvls(const Call& k, const void* send, void* recv, size_t bytes) {
  const View sv = viewOf(k.st, send, bytes), rv = viewOf(k.st, recv, bytes);
  if (sv.sym() && rv.sym() && sv.mc() && rv.mc() && al16(send) && al16(recv))
    return arNvlsOn(k, sv.mc(), rv.mc(), bytes);
  // Chunks are multiples of 16 x n bytes so that every chunk but the last splits into whole vectors per rank.
  return stagedPipeline(k, send, recv, true, bytes, (size_t)16 * k.n, [&](size_t stageOff, size_t off, size_t len) -> mcclResult_t {
    if (len % 16 || len / 16 < (size_t)k.n) {              // a ragged tail: the peer-load kernel takes any length
      char* in[MCCL_MAX_RANKS];
      for (int p = 0; p < k.n; ++p) in[p] = k.stagePeer(p) + stageOff;
      return twoShot(k, in, in, nullptr, len, true, mcclAlgoTwoShot);      // the result stays in the stage, like the NVLS chunks'
    }
    return arNvlsOn(k, k.stageMc() + stageOff, k.stageMc() + stageOff, len);
  });
}

mcclResult_t ringTreeOn(const Call& k, char* const buf[], size_t bytes, int algo, int phases = 0, int shift = 0) {
  const Channel& ch = k.c->chan;
  if (algo == mcclAlgoRing) {
    RingArgs a;
    memset(&a, 0, sizeof(a));
    a.peers = k.st->peers;
    a.nCtas = pickCtas(k.c, bytes, algo);
    a.op = (k.op == mcclAvg) ? mcclSum : k.op;
    a.divisor = k.divisor;
    a.prev = ch.ring.prev;
    a.next = ch.ring.next;
    a.bytes = bytes;
    a.phases = phases;
    a.shift = shift;
    for (int p = 0; p < k.n; ++p) a.buf[p] = buf[p];
    DISPATCH_ALL_TYPES(k.dt, ringKernel, a.nCtas, k.s, a);
    return launched(k.c, "ringKernel");
  }
  TreeArgs a;
  memset(&a, 0, sizeof(a));
  a.peers = k.st->peers;
  a.nCtas = pickCtas(k.c, bytes, algo);
  a.op = (k.op == mcclAvg) ? mcclSum : k.op;
  a.divisor = k.divisor;
  a.bytes = bytes;
  a.phases = phases;
  const TreeView* tv[2] = {&ch.tree, ch.dtree ? &ch.treeB : &ch.tree};
  for (int t = 0; t < 2; ++t) {
    a.up[t] = tv[t]->up;
    a.down[t][0] = tv[t]->down.size() > 0 ? tv[t]->down[0] : -1;
    a.down[t][1] = tv[t]->down.size() > 1 ? tv[t]->down[1] : -1;
  }
  for (int p = 0; p < k.n; ++p) a.buf[p] = buf[p];
  DISPATCH_ALL_TYPES(k.dt, treeKernel, a.nCtas, k.s, a);
  return launched(k.c, "treeKernel");
}

// Roots of the two trees the tree kernel walks (the second equals the first without a double-binary tree).
void treeRoots(const mcclComm* c, int* rootA, int* rootB) {
  *rootA = *rootB = 0;
  for (int r = 0; r < c->nRanks; ++r) if (c->chan.treeParent[r] < 0) *rootA = r;
  *rootB = *rootA;
  if (c->chan.dtree) for (int r = 0; r < c->nRanks; ++r) if (c->chan.treeParentB[r] < 0) *rootB = r;
}

mcclResult_t arRingTree(const Call& k, const void* send, void* recv, size_t bytes, int algo) {
  const View rv = viewOf(k.st, recv, bytes);
  char* buf[MCCL_MAX_RANKS];
  if (rv.sym() && al16(recv)) {
    MCCLCHECK(launchCopy(k.c, send, recv, 1, bytes, bytes, bytes, k.s));
    for (int p = 0; p < k.n; ++p) buf[p] = rv.peer(p);
    return ringTreeOn(k, buf, bytes, algo);
  }
  // Chunks keep the 16-byte and n-way divisibility the kernels rely on.
  size_t chunk = stageChunk(k, 1);
  chunk = chunk / (16 * (size_t)k.n) * (16 * (size_t)k.n);
  for (int p = 0; p < k.n; ++p) buf[p] = k.stagePeer(p);
  for (size_t off = 0; off < bytes; off += chunk) {
    const size_t len = std::min(chunk, bytes - off);
    MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), 1, len, len, len, k.s));
    if (len % 16 == 0 && len / 16 >= (size_t)2 * k.n) {
      MCCLCHECK(ringTreeOn(k, buf, len, algo));
    } else {
      char* in[MCCL_MAX_RANKS];
      for (int p = 0; p < k.n; ++p) in[p] = k.stagePeer(p);
      MCCLCHECK(twoShot(k, in, in, nullptr, len, true, mcclAlgoTwoShot));
    }
    MCCLCHECK(launchCopy(k.c, k.stageLocal(), static_cast<char*>(recv) + off, 1, len, len, len, k.s));
  }
  return mcclSuccess;
}

mcclResult_t allReduce(const Call& k, const void* send, void* recv, size_t count, int algo) {
  const size_t bytes = count * k.es;
  const bool vecOk = bytes % 16 == 0 && al16(send) && al16(recv);
  if (algo == mcclAlgoOneShot && vecOk && bytes <= k.st->layout.oneShotSlotBytes) return arOneShot(k, send, recv, bytes);
  if (algo == mcclAlgoNvls && k.st->nvls && nvlsType(k.dt, k.op, k.n) && bytes % 16 == 0 && bytes / 16 >= (size_t)k.n)
    return arNvls(k, send, recv, bytes);
  if ((algo == mcclAlgoRing || algo == mcclAlgoTree) && bytes % 16 == 0 && bytes / 16 >= (size_t)2 * k.n)
    return arRingTree(k, send, recv, bytes, algo);
  k.c->lastAlgo.store(mcclAlgoTwoShot);
  return arTwoShot(k, send, recv, bytes);
}

}  // namespace

namespace {

// Type used to move opaque bytes through the fold path (single source, no arithmetic).
mcclDataType_t carrierType(size_t bytes) { return bytes % 4 == 0 ? mcclInt32 : mcclUint8; }

// ---- all-gather ----------------------------------------------------------------------------------------------
mcclResult_t allGather(const Call& k, const void* send, void* recv, size_t sendcount, int algo) {
  const size_t slot = sendcount * k.es;
  char* out = static_cast<char*>(recv);
  const bool inPlace = send == out + (size_t)k.r * slot;
  const View rv = viewOf(k.st, recv, slot * k.n), sv = viewOf(k.st, send, slot);
  if (algo == mcclAlgoNvls && k.st->nvls && rv.sym() && rv.mc() && slot % 16 == 0 && al16(send) && al16(recv)) {
    NvlsArgs a = baseNvls(k, slot);
    a.loadReduce = 0;
    a.mcStore = 1;
    a.src = static_cast<const char*>(send);
    a.mcDst = rv.mc() + (size_t)k.r * slot;
    a.bytes = slot;
    return launchNvls(k, a, false);
  }
  if (algo == mcclAlgoRing && slot % 16 == 0 && slot >= 16 && al16(send) && al16(recv)) return agRingFwd(k, send, recv, slot);
  if (algo == mcclAlgoTree && slot % 16 == 0 && slot * k.n >= 64 && al16(send) && al16(recv)) return agTreeFwd(k, send, recv, slot);
  k.c->lastAlgo.store(mcclAlgoOneShot);
  if ((inPlace && rv.sym()) || sv.sym()) {
    PullArgs a = basePull(k, slot * k.n, mcclAlgoTwoShot);
    for (int i = 0; i < k.n; ++i) {
      const int p = (k.r + i) % k.n;          // rotated start, see twoShot
      const char* src = (inPlace && rv.sym()) ? rv.peer(p) + (size_t)p * slot : sv.peer(p);
      if (p == k.r) { if (!inPlace) a.jobs[a.nJobs++] = CopyJob{static_cast<const char*>(send), out + (size_t)p * slot, slot}; continue; }
      a.jobs[a.nJobs++] = CopyJob{src, out + (size_t)p * slot, slot};
    }
    return launchPull(k.c, a, carrierType(slot), k.s);
  }
  const size_t chunk = stageChunk(k, 1);
  for (size_t off = 0; off < slot; off += chunk) {
    const size_t len = std::min(chunk, slot - off);
    MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), 1, len, len, len, k.s));
    PullArgs a = basePull(k, len * k.n, mcclAlgoTwoShot);
    for (int i = 0; i < k.n; ++i) {
      const int p = (k.r + i) % k.n;
      if (p == k.r) { if (!inPlace) a.jobs[a.nJobs++] = CopyJob{static_cast<const char*>(send) + off, out + (size_t)p * slot + off, len}; continue; }
      a.jobs[a.nJobs++] = CopyJob{k.stagePeer(p), out + (size_t)p * slot + off, len};
    }
    MCCLCHECK(launchPull(k.c, a, carrierType(len), k.s));
  }
  return mcclSuccess;
}

// ---- reduce-scatter ------------------------------------------------------------------------------------------
mcclResult_t reduceScatter(const Call& k, const void* send, void* recv, size_t recvcount, int algo) {
  const size_t blk = recvcount * k.es;
  const View sv = viewOf(k.st, send, blk * k.n);
  if (algo == mcclAlgoNvls && k.st->nvls && sv.sym() && sv.mc() && nvlsType(k.dt, k.op, k.n) && blk % 16 == 0 && al16(send) && al16(recv)) {
    NvlsArgs a = baseNvls(k, blk);
    a.loadReduce = 1;
    a.mcStore = 0;
    a.mcSrc = sv.mc() + (size_t)k.r * blk;
    a.dst = static_cast<char*>(recv);
    a.bytes = blk;
    a.divisor = k.divisor;
    return launchNvls(k, a, true);
  }
  if (algo == mcclAlgoRing && blk % 16 == 0 && blk >= 16 && al16(send) && al16(recv)) return rsRingFwd(k, send, recv, blk);
  if (algo == mcclAlgoTree && blk % 16 == 0 && blk * k.n >= 64 && al16(send) && al16(recv)) return rsTreeFwd(k, send, recv, blk);
  k.c->lastAlgo.store(mcclAlgoOneShot);
  if (sv.sym()) {
    PullArgs a = basePull(k, blk * k.n, mcclAlgoTwoShot);
    a.nSrcA = k.n;
    for (int p = 0; p < k.n; ++p) a.srcA[p] = sv.peer(p) + (size_t)k.r * blk;
    a.dstA = static_cast<char*>(recv);
    a.aBytes = blk;
    return launchPull(k.c, a, k.dt, k.s);
  }
  size_t chunk = stageChunk(k, k.n);
  chunk = std::max<size_t>(chunk / k.es * k.es, k.es);
  for (size_t off = 0; off < blk; off += chunk) {
    const size_t len = std::min(chunk, blk - off);
    MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), k.n, len, blk, len, k.s));
    PullArgs a = basePull(k, len * k.n, mcclAlgoTwoShot);
    a.nSrcA = k.n;
    for (int p = 0; p < k.n; ++p) a.srcA[p] = k.stagePeer(p) + (size_t)k.r * len;
    a.dstA = static_cast<char*>(recv) + off;
    a.aBytes = len;
    MCCLCHECK(launchPull(k.c, a, k.dt, k.s));
  }
  return mcclSuccess;
}

// ---- broadcast -------------------------------------------------------------------------------------------------
// Scatter + all-gather ("two-shot"): rank r fetches shard r from the root, then the shards are exchanged, so
// the root's outbound traffic is one copy of the message instead of n-1.  `direct` makes every rank fetch
// the whole message from the root (lowest latency for small messages).
mcclResult_t bcastOn(const Call& k, char* const work[], char* out, size_t bytes, int root, bool direct) {
  Call kk = k;
  kk.op = mcclSum;
  kk.divisor = 1;
  PullArgs a = basePull(kk, bytes, mcclAlgoTwoShot);
  const int r = k.r, n = k.n;
  a.midBarrier = direct ? 0 : 1;
  if (r != root) {
    char* dst = out ? out : work[r];
    if (direct) {
      a.jobs[a.nJobs++] = CopyJob{work[root], dst, bytes};
    } else {
      const uint64_t o0 = shardOff(bytes, n, r), o1 = shardEnd(bytes, n, r);
      a.nSrcA = 1;
      a.srcA[0] = work[root] + o0;
      a.dstA = work[r] + o0;
      a.dstA2 = (out && out != work[r]) ? out + o0 : nullptr;
      a.aBytes = o1 - o0;
      for (int i = 1; i < n; ++i) {
        const int p = (r + i) % n;
        const uint64_t q0 = shardOff(bytes, n, p), q1 = shardEnd(bytes, n, p);
        a.jobs[a.nJobs++] = CopyJob{work[p] + q0, dst + q0, q1 - q0};   // the root's own copy is complete too
      }
    }
  }
  return launchPull(k.c, a, carrierType(bytes), k.s);
}

mcclResult_t broadcast(const Call& k, const void* send, void* recv, size_t count, int root, int algo) {
  const size_t bytes = count * k.es;
  const View rv = viewOf(k.st, recv, bytes);
  const bool direct = algo == mcclAlgoOneShot;
  if (algo == mcclAlgoNvls && k.st->nvls && rv.sym() && rv.mc() && bytes % 16 == 0 && al16(recv) && (k.r != root || al16(send))) {
    if (nvlsSpread(bytes) && bytes >= (size_t)k.n * 16) {
      // The peers read the root's destination buffer, so an out-of-place root copies there first.
      if (k.r == root) MCCLCHECK(launchCopy(k.c, send, recv, 1, bytes, bytes, bytes, k.s));
      NvlsRootedArgs a;
      memset(&a, 0, sizeof(a));
      a.peers = k.st->peers;
      a.nCtas = pickCtas(k.c, bytes, mcclAlgoNvls);
      a.root = root;
      a.reducing = 0;
      a.rootBuf = k.r == root ? static_cast<const char*>(recv) : rv.peer(root);
      a.mcDst = rv.mc();
      a.bytes = bytes;
      a.divisor = 1;
      return launchNvlsRooted(k, a);
    }
    NvlsArgs a = baseNvls(k, bytes, true);
    a.loadReduce = 0;
    a.mcStore = 1;
    a.active = k.r == root;
    a.src = static_cast<const char*>(send);
    a.mcDst = rv.mc();
    a.bytes = bytes;
    return launchNvls(k, a, false, true);
  }
  if (algo == mcclAlgoTree && bytes % 16 == 0 && bytes >= 64 && al16(recv) && (k.r != root || al16(send)))
    return bcastTreeFwd(k, send, recv, bytes, root);
  if (algo == mcclAlgoRing && bytes % 16 == 0 && bytes / 16 >= (size_t)k.n && al16(recv) && (k.r != root || al16(send)))
    return bcastRingFwd(k, send, recv, bytes, root);
  k.c->lastAlgo.store(direct ? mcclAlgoOneShot : mcclAlgoTwoShot);
  char* work[MCCL_MAX_RANKS];
  if (rv.sym()) {
    if (k.r == root) MCCLCHECK(launchCopy(k.c, send, recv, 1, bytes, bytes, bytes, k.s));
    for (int p = 0; p < k.n; ++p) work[p] = rv.peer(p);
    return bcastOn(k, work, static_cast<char*>(recv), bytes, root, direct);
  }
  const size_t chunk = stageChunk(k, 1);
  for (int p = 0; p < k.n; ++p) work[p] = k.stagePeer(p);
  for (size_t off = 0; off < bytes; off += chunk) {
    const size_t len = std::min(chunk, bytes - off);
    if (k.r == root) {
      MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), 1, len, len, len, k.s));
      MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, static_cast<char*>(recv) + off, 1, len, len, len, k.s));
    }
    MCCLCHECK(bcastOn(k, work, static_cast<char*>(recv) + off, len, root, direct));
  }
  return mcclSuccess;
}

// ---- reduce ----------------------------------------------------------------------------------------------------
// Two-shot: every rank folds its shard, the root collects the shards.  Direct: the root folds everything.
mcclResult_t reduceOn(const Call& k, char* const in[], char* const red[], char* recvAt, size_t bytes, int root, bool direct) {
  const int n = k.n, r = k.r;
  if (direct) {
    PullArgs a = basePull(k, bytes, mcclAlgoTwoShot);
    if (r == root) {
      a.nSrcA = n;
      for (int p = 0; p < n; ++p) a.srcA[p] = in[p];
      a.dstA = recvAt;
      a.aBytes = bytes;
    }
    return launchPull(k.c, a, k.dt, k.s);
  }
  return twoShot(k, in, red, r == root ? recvAt : nullptr, bytes, r == root, mcclAlgoTwoShot);
}

mcclResult_t reduce(const Call& k, const void* send, void* recv, size_t count, int root, int algo) {
  const size_t bytes = count * k.es;
  const View sv = viewOf(k.st, send, bytes);
  const bool direct = algo == mcclAlgoOneShot;
  if (algo == mcclAlgoNvls && k.st->nvls && sv.sym() && sv.mc() && nvlsType(k.dt, k.op, k.n) && bytes % 16 == 0 && al16(send) &&
      (k.r != root || al16(recv))) {
    if (nvlsSpread(bytes) && bytes >= (size_t)k.n * 16) {
      NvlsRootedArgs a;
      memset(&a, 0, sizeof(a));
      a.peers = k.st->peers;
      a.nCtas = baseNvls(k, bytes, true).nCtas;      // enough CTAs for the root to work alone if it has to
      a.op = (k.op == mcclAvg) ? mcclSum : k.op;
      a.root = root;
      a.reducing = 1;
      a.rootBuf = sv.peer(root);
      a.mcSrc = sv.mc();
      a.bytes = bytes;
      a.divisor = k.divisor;
      if (k.r == root) {
        // The peers can reach the destination only through their mapping of the root's source allocation.
        const View rv = viewOf(k.st, recv, bytes);
        a.local = static_cast<char*>(recv);
        a.note = kNoteAlone;
        if (rv.sym() && rv.seg == sv.seg) {
          const int64_t delta = (int64_t)rv.off - (int64_t)sv.off;
          if (delta == 0 || (uint64_t)(delta < 0 ? -delta : delta) >= bytes) a.note = (uint64_t)delta;
        }
      }
      return launchNvlsRooted(k, a);
    }
    NvlsArgs a = baseNvls(k, bytes, true);
    a.loadReduce = 1;
    a.mcStore = 0;
    a.active = k.r == root;
    a.mcSrc = sv.mc();
    a.dst = static_cast<char*>(recv);
    a.bytes = bytes;
    a.divisor = k.divisor;
    return launchNvls(k, a, true, true);
  }
  if (algo == mcclAlgoTree && bytes % 16 == 0 && bytes >= 64 && al16(send) && (k.r != root || al16(recv)))
    return reduceTreeFwd(k, send, recv, bytes, root);
  if (algo == mcclAlgoRing && bytes % 16 == 0 && bytes / 16 >= (size_t)2 * k.n && al16(send) && (k.r != root || al16(recv)))
    return reduceRingFwd(k, send, recv, bytes, root);
  k.c->lastAlgo.store(direct ? mcclAlgoOneShot : mcclAlgoTwoShot);
  // The stage is cut in two: inputs that are not symmetric go to the first half, folded shards to the second.
  size_t half = k.stageBytes() / 2 / 256 * 256;
  half = std::max<size_t>(half / k.es * k.es, k.es);
  char* in[MCCL_MAX_RANKS];
  char* red[MCCL_MAX_RANKS];
  for (size_t off = 0; off < bytes; off += half) {
    const size_t len = std::min(half, bytes - off);
    if (sv.sym()) {
      for (int p = 0; p < k.n; ++p) in[p] = sv.peer(p) + off;
    } else {
      MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), 1, len, len, len, k.s));
      for (int p = 0; p < k.n; ++p) in[p] = k.stagePeer(p);
    }
    for (int p = 0; p < k.n; ++p) red[p] = k.stagePeer(p) + half;
    MCCLCHECK(reduceOn(k, in, red, k.r == root ? static_cast<char*>(recv) + off : nullptr, len, root, direct));
  }
  return mcclSuccess;
}

// ---- all-to-all --------------------------------------------------------------------------------------------------
mcclResult_t allToAll(const Call& k, const void* send, void* recv, size_t count) {
  const size_t blk = count * k.es;
  const View sv = viewOf(k.st, send, blk * k.n);
  char* out = static_cast<char*>(recv);
  if (sv.sym()) {
    PullArgs a = basePull(k, blk * k.n, mcclAlgoTwoShot);
    for (int i = 0; i < k.n; ++i) {
      const int p = (k.r + i) % k.n;
      a.jobs[a.nJobs++] = CopyJob{sv.peer(p) + (size_t)k.r * blk, out + (size_t)p * blk, blk};
    }
    return launchPull(k.c, a, carrierType(blk), k.s);
  }
  const size_t chunk = stageChunk(k, k.n);
  for (size_t off = 0; off < blk; off += chunk) {
    const size_t len = std::min(chunk, blk - off);
    MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), k.n, len, blk, len, k.s));
    PullArgs a = basePull(k, len * k.n, mcclAlgoTwoShot);
    for (int i = 0; i < k.n; ++i) {
      const int p = (k.r + i) % k.n;
      a.jobs[a.nJobs++] = CopyJob{k.stagePeer(p) + (size_t)k.r * len, out + (size_t)p * blk + off, len};
    }
    MCCLCHECK(launchPull(k.c, a, carrierType(len), k.s));
  }
  return mcclSuccess;
}

}  // namespace

namespace {

// Ring all-gather: the gather steps of the ring kernel on a buffer of n slots; with shift 1 a rank starts
// out holding its own slot.
mcclResult_t agRing(const Call& k, const void* send, void* recv, size_t slot) {
  char* out = static_cast<char*>(recv);
  const View rv = viewOf(k.st, recv, slot * k.n);
  Call kk = k; kk.op = mcclSum; kk.divisor = 1; kk.dt = carrierType(slot); kk.es = mcclDataSize(kk.dt);
  char* buf[MCCL_MAX_RANKS];
  if (rv.sym() && al16(recv)) {
    MCCLCHECK(launchCopy(k.c, send, out + (size_t)k.r * slot, 1, slot, slot, slot, k.s));
    for (int p = 0; p < k.n; ++p) buf[p] = rv.peer(p);
    return ringTreeOn(kk, buf, slot * k.n, mcclAlgoRing, 2, 1);
  }
  size_t chunk = stageChunk(k, k.n) / 16 * 16;
  for (int p = 0; p < k.n; ++p) buf[p] = k.stagePeer(p);
  for (size_t off = 0; off < slot; off += chunk) {
    const size_t len = std::min(chunk, slot - off);
    MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal() + (size_t)k.r * len, 1, len, len, len, k.s));
    MCCLCHECK(ringTreeOn(kk, buf, len * k.n, mcclAlgoRing, 2, 1));
    MCCLCHECK(launchCopy(k.c, k.stageLocal(), out + off, k.n, len, len, slot, k.s));
  }
  return mcclSuccess;
}

// Ring reduce-scatter: the reduce steps of the ring kernel on a staged copy of the input (they fold in
// place); with shift 1 rank r ends up owning block r.
mcclResult_t rsRing(const Call& k, const void* send, void* recv, size_t blk) {
  size_t chunk = stageChunk(k, k.n) / 16 * 16;
  char* buf[MCCL_MAX_RANKS];
  for (int p = 0; p < k.n; ++p) buf[p] = k.stagePeer(p);
  for (size_t off = 0; off < blk; off += chunk) {
    const size_t len = std::min(chunk, blk - off);
    MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), k.n, len, blk, len, k.s));
    MCCLCHECK(ringTreeOn(k, buf, len * k.n, mcclAlgoRing, 1, 1));
    MCCLCHECK(launchCopy(k.c, k.stageLocal() + (size_t)k.r * len, static_cast<char*>(recv) + off, 1, len, len, len, k.s));
  }
  return mcclSuccess;
}

// The two halves the tree kernel works on, as byte ranges.
void treeHalves(size_t bytes, size_t* h0, size_t* h1) {
  const size_t V = bytes / 16;
  *h0 = (V / 2) * 16;
  *h1 = bytes - *h0;
}

// Tree broadcast: the tree roots fetch their halves from the broadcast root, then the down phase of the tree
// kernel carries them to everyone.
mcclResult_t bcastTreeOn(const Call& k, char* const work[], size_t bytes, int root) {
  int rootA, rootB;
  treeRoots(k.c, &rootA, &rootB);
  size_t h0, h1;
  treeHalves(bytes, &h0, &h1);
  Call kk = k; kk.op = mcclSum; kk.divisor = 1; kk.dt = carrierType(bytes); kk.es = mcclDataSize(kk.dt);
  PullArgs a = basePull(kk, bytes, mcclAlgoTwoShot);
  if (k.r == rootA && k.r != root && h0 > 0) a.jobs[a.nJobs++] = CopyJob{work[root], work[k.r], h0};
  if (k.r == rootB && k.r != root && h1 > 0) a.jobs[a.nJobs++] = CopyJob{work[root] + h0, work[k.r] + h0, h1};
  MCCLCHECK(launchPull(k.c, a, kk.dt, k.s));
  return ringTreeOn(kk, work, bytes, mcclAlgoTree, 2, 0);
}

mcclResult_t bcastTree(const Call& k, const void* send, void* recv, size_t bytes, int root) {
  const View rv = viewOf(k.st, recv, bytes);
  char* work[MCCL_MAX_RANKS];
  if (rv.sym() && al16(recv)) {
    if (k.r == root) MCCLCHECK(launchCopy(k.c, send, recv, 1, bytes, bytes, bytes, k.s));
    for (int p = 0; p < k.n; ++p) work[p] = rv.peer(p);
    return bcastTreeOn(k, work, bytes, root);
  }
  const size_t chunk = stageChunk(k, 1) / 16 * 16;
  for (int p = 0; p < k.n; ++p) work[p] = k.stagePeer(p);
  for (size_t off = 0; off < bytes; off += chunk) {
    const size_t len = std::min(chunk, bytes - off);
    if (k.r == root) MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), 1, len, len, len, k.s));
    MCCLCHECK(bcastTreeOn(k, work, len, root));
    MCCLCHECK(launchCopy(k.c, k.stageLocal(), static_cast<char*>(recv) + off, 1, len, len, len, k.s));
  }
  return mcclSuccess;
}

// Tree reduce: the up phase of the tree kernel on a staged copy of the input leaves each half reduced at its
// tree's root; the reduce root then fetches the two halves.
mcclResult_t reduceTree(const Call& k, const void* send, void* recv, size_t bytes, int root) {
  int rootA, rootB;
  treeRoots(k.c, &rootA, &rootB);
  const size_t chunk = stageChunk(k, 1) / 16 * 16;
  char* work[MCCL_MAX_RANKS];
  for (int p = 0; p < k.n; ++p) work[p] = k.stagePeer(p);
  for (size_t off = 0; off < bytes; off += chunk) {
    const size_t len = std::min(chunk, bytes - off);
    MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), 1, len, len, len, k.s));
    MCCLCHECK(ringTreeOn(k, work, len, mcclAlgoTree, 1, 0));
    size_t h0, h1;
    treeHalves(len, &h0, &h1);
    Call kk = k; kk.op = mcclSum; kk.divisor = 1;
    PullArgs a = basePull(kk, len, mcclAlgoTwoShot);
    if (k.r == root) {
      char* dst = static_cast<char*>(recv) + off;
      if (h0 > 0) a.jobs[a.nJobs++] = CopyJob{work[rootA], dst, h0};
      if (h1 > 0) a.jobs[a.nJobs++] = CopyJob{work[rootB] + h0, dst + h0, h1};
    }
    MCCLCHECK(launchPull(k.c, a, carrierType(len), k.s));
  }
  return mcclSuccess;
}

// Ring broadcast: every rank fetches its own part from the root, then the gather steps of the ring kernel pass
// the parts around (the root's outbound traffic is one copy of the message).
mcclResult_t bcastRingOn(const Call& k, char* const work[], size_t bytes, int root) {
  Call kk = k; kk.op = mcclSum; kk.divisor = 1; kk.dt = carrierType(bytes); kk.es = mcclDataSize(kk.dt);
  PullArgs a = basePull(kk, bytes, mcclAlgoTwoShot);
  const uint64_t o0 = shardOff(bytes, k.n, k.r), o1 = shardEnd(bytes, k.n, k.r);
  if (k.r != root && o1 > o0) a.jobs[a.nJobs++] = CopyJob{work[root] + o0, work[k.r] + o0, o1 - o0};
  MCCLCHECK(launchPull(k.c, a, kk.dt, k.s));
  return ringTreeOn(kk, work, bytes, mcclAlgoRing, 2, 1);
}

mcclResult_t bcastRing(const Call& k, const void* send, void* recv, size_t bytes, int root) {
  const View rv = viewOf(k.st, recv, bytes);
  char* work[MCCL_MAX_RANKS];
  if (rv.sym()) {
    if (k.r == root) MCCLCHECK(launchCopy(k.c, send, recv, 1, bytes, bytes, bytes, k.s));
    for (int p = 0; p < k.n; ++p) work[p] = rv.peer(p);
    return bcastRingOn(k, work, bytes, root);
  }
  const size_t chunk = stageChunk(k, 1) / (16 * (size_t)k.n) * (16 * (size_t)k.n);
  if (chunk == 0) return mcclInternalError;
  for (int p = 0; p < k.n; ++p) work[p] = k.stagePeer(p);
  for (size_t off = 0; off < bytes; off += chunk) {
    const size_t len = std::min(chunk, bytes - off);
    if (k.r == root) MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), 1, len, len, len, k.s));
    if (len / 16 >= (size_t)k.n) MCCLCHECK(bcastRingOn(k, work, len, root));
    else MCCLCHECK(bcastOn(k, work, nullptr, len, root, true));          // a tail shorter than one vector per rank
    MCCLCHECK(launchCopy(k.c, k.stageLocal(), static_cast<char*>(recv) + off, 1, len, len, len, k.s));
  }
  return mcclSuccess;
}

// Ring reduce: the reduce steps of the ring kernel on a staged copy of the input leave part p reduced at rank
// p; the root then fetches every part from its owner (src/device/reduce.h:104-173 of the reference).
mcclResult_t reduceRing(const Call& k, const void* send, void* recv, size_t bytes, int root) {
  const size_t chunk = stageChunk(k, 1) / (16 * (size_t)k.n) * (16 * (size_t)k.n);
  if (chunk == 0) return mcclInternalError;
  char* work[MCCL_MAX_RANKS];
  for (int p = 0; p < k.n; ++p) work[p] = k.stagePeer(p);
  for (size_t off = 0; off < bytes; off += chunk) {
    const size_t len = std::min(chunk, bytes - off);
    MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), 1, len, len, len, k.s));
    if (len / 16 < (size_t)2 * k.n) {                                     // a tail too short for the ring
      MCCLCHECK(reduceOn(k, work, work, k.r == root ? static_cast<char*>(recv) + off : nullptr, len, root, true));
      continue;
    }
    MCCLCHECK(ringTreeOn(k, work, len, mcclAlgoRing, 1, 1));
    Call kk = k; kk.op = mcclSum; kk.divisor = 1;
    PullArgs a = basePull(kk, len, mcclAlgoTwoShot);
    if (k.r == root) {
      for (int i = 0; i < k.n; ++i) {
        const int p = (k.r + i) % k.n;
        const uint64_t q0 = shardOff(len, k.n, p), q1 = shardEnd(len, k.n, p);
        if (q1 > q0) a.jobs[a.nJobs++] = CopyJob{work[p] + q0, static_cast<char*>(recv) + off + q0, q1 - q0};
      }
    }
    MCCLCHECK(launchPull(k.c, a, carrierType(len), k.s));
  }
  return mcclSuccess;
}

// Tree all-gather: every rank puts its slot into a zeroed buffer of n slots and the tree kernel adds the
// buffers as integers (x + 0 + ... + 0 = x bit for bit), the masked-sum form the reference uses for its deep
// tree broadcast (src/device/broadcast.h:85-88).
mcclResult_t agTree(const Call& k, const void* send, void* recv, size_t slot) {
  char* out = static_cast<char*>(recv);
  const View rv = viewOf(k.st, recv, slot * k.n);
  Call kk = k; kk.op = mcclSum; kk.divisor = 1; kk.dt = mcclUint32; kk.es = 4;
  char* buf[MCCL_MAX_RANKS];
  if (rv.sym()) {
    char* mine = out + (size_t)k.r * slot;
    if (send != mine) MCCLCHECK(launchCopy(k.c, send, mine, 1, slot, slot, slot, k.s));
    if (k.r > 0 && cudaMemsetAsync(out, 0, (size_t)k.r * slot, k.s) != cudaSuccess) return mcclSystemError;
    if (k.r < k.n - 1 && cudaMemsetAsync(mine + slot, 0, (size_t)(k.n - 1 - k.r) * slot, k.s) != cudaSuccess) return mcclSystemError;
    for (int p = 0; p < k.n; ++p) buf[p] = rv.peer(p);
    return ringTreeOn(kk, buf, slot * k.n, mcclAlgoTree);
  }
  const size_t chunk = stageChunk(k, k.n) / 16 * 16;
  if (chunk == 0) return mcclInternalError;
  for (int p = 0; p < k.n; ++p) buf[p] = k.stagePeer(p);
  for (size_t off = 0; off < slot; off += chunk) {
    const size_t len = std::min(chunk, slot - off);
    if (cudaMemsetAsync(k.stageLocal(), 0, len * k.n, k.s) != cudaSuccess) return mcclSystemError;
    MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal() + (size_t)k.r * len, 1, len, len, len, k.s));
    if (len * k.n >= 64) MCCLCHECK(ringTreeOn(kk, buf, len * k.n, mcclAlgoTree));
    else MCCLCHECK(twoShot(kk, buf, buf, nullptr, len * k.n, true, mcclAlgoTwoShot));
    MCCLCHECK(launchCopy(k.c, k.stageLocal(), out + off, k.n, len, len, slot, k.s));
  }
  return mcclSuccess;
}

// Tree reduce-scatter: the up phase of the tree kernel on a staged copy of the n blocks leaves each half of it
// reduced at its tree's root; rank r then fetches block r, which may straddle the two halves.
mcclResult_t rsTree(const Call& k, const void* send, void* recv, size_t blk) {
  int rootA, rootB;
  treeRoots(k.c, &rootA, &rootB);
  const size_t chunk = stageChunk(k, k.n) / 16 * 16;
  if (chunk == 0) return mcclInternalError;
  char* work[MCCL_MAX_RANKS];
  for (int p = 0; p < k.n; ++p) work[p] = k.stagePeer(p);
  for (size_t off = 0; off < blk; off += chunk) {
    const size_t len = std::min(chunk, blk - off), total = len * k.n;
    MCCLCHECK(launchCopy(k.c, static_cast<const char*>(send) + off, k.stageLocal(), k.n, len, blk, len, k.s));
    char* dst = static_cast<char*>(recv) + off;
    if (total < 64) {                                                      // too short for two halves
      PullArgs a = basePull(k, total, mcclAlgoTwoShot);
      a.nSrcA = k.n;
      for (int p = 0; p < k.n; ++p) a.srcA[p] = work[p] + (size_t)k.r * len;
      a.dstA = dst;
      a.aBytes = len;
      MCCLCHECK(launchPull(k.c, a, k.dt, k.s));
      continue;
    }
    MCCLCHECK(ringTreeOn(k, work, total, mcclAlgoTree, 1, 0));
    size_t h0, h1;
    treeHalves(total, &h0, &h1);
    Call kk = k; kk.op = mcclSum; kk.divisor = 1;
    PullArgs a = basePull(kk, total, mcclAlgoTwoShot);
    const size_t b0 = (size_t)k.r * len, b1 = b0 + len;
    if (b0 < h0) a.jobs[a.nJobs++] = CopyJob{work[rootA] + b0, dst, std::min(b1, h0) - b0};
    if (b1 > h0) { const size_t s0 = std::max(b0, h0); a.jobs[a.nJobs++] = CopyJob{work[rootB] + s0, dst + (s0 - b0), b1 - s0}; }
    MCCLCHECK(launchPull(k.c, a, carrierType(len), k.s));
  }
  return mcclSuccess;
}

}  // namespace

namespace {
mcclResult_t bcastRingFwd(const Call& k, const void* send, void* recv, size_t bytes, int root) { return bcastRing(k, send, recv, bytes, root); }
mcclResult_t reduceRingFwd(const Call& k, const void* send, void* recv, size_t bytes, int root) { return reduceRing(k, send, recv, bytes, root); }
mcclResult_t agTreeFwd(const Call& k, const void* send, void* recv, size_t slot) { return agTree(k, send, recv, slot); }
mcclResult_t rsTreeFwd(const Call& k, const void* send, void* recv, size_t blk) { return rsTree(k, send, recv, blk); }
mcclResult_t agRingFwd(const Call& k, const void* send, void* recv, size_t slot) { return agRing(k, send, recv, slot); }
mcclResult_t rsRingFwd(const Call& k, const void* send, void* recv, size_t blk) { return rsRing(k, send, recv, blk); }
mcclResult_t bcastTreeFwd(const Call& k, const void* send, void* recv, size_t bytes, int root) { return bcastTree(k, send, recv, bytes, root); }
mcclResult_t reduceTreeFwd(const Call& k, const void* send, void* recv, size_t bytes, int root) { return reduceTree(k, send, recv, bytes, root); }
}  // namespace

// ---- entry points used by the runtime ------------------------------------------------------------------------------
static mcclResult_t latchedError(mcclComm* c) {
  const uint32_t code = c->cu->statusHost->code;
  if (code == 0) return mcclSuccess;
  return (code == 3 || code == 4) ? mcclInvalidUsage : mcclRemoteError;
}

// The kernels take a buffer that lies in symmetric memory on this rank to lie at the same offset of the same
// allocation on every rank (the peers' addresses are derived from the local one).  With MCCL_CHECK_SYMMETRY=1
// every collective is preceded by a small kernel in which the ranks compare what they passed.
static mcclResult_t checkSymmetry(mcclComm* c, CudaState* st, int coll, const void* send, void* recv, size_t count, size_t es,
                                  int root, cudaStream_t s) {
  static const bool on = envInt("MCCL_CHECK_SYMMETRY", 0) != 0;
  if (!on || c->nRanks < 2) return mcclSuccess;
  const size_t n = (size_t)c->nRanks, r = (size_t)c->rank;
  size_t sendBytes = count * es, recvBytes = count * es;
  if (coll == mcclCollAllGather) recvBytes *= n;
  if (coll == mcclCollReduceScatter || coll == mcclCollAllToAll) sendBytes *= n;
  if (coll == mcclCollAllToAll) recvBytes *= n;
  View sv = viewOf(st, send, sendBytes), rv = viewOf(st, recv, recvBytes);
  uint64_t sig[4] = {0, 0, 0, 0};
  // Rooted calls: only the root's send (broadcast) or receive (reduce) buffer is used, so it is not compared.
  if (sv.sym() && coll != mcclCollBroadcast) {
    uint64_t off = sv.off;
    if (coll == mcclCollAllGather && rv.sym() && rv.seg == sv.seg && sv.off == rv.off + r * sendBytes) off -= r * sendBytes;   // in place
    sig[0] = sv.seg->serial; sig[1] = off;
  }
  if (rv.sym() && coll != mcclCollReduce) {
    uint64_t off = rv.off;
    if (coll == mcclCollReduceScatter && sv.sym() && rv.seg == sv.seg && rv.off == sv.off + r * recvBytes) off -= r * recvBytes;   // in place
    sig[2] = rv.seg->serial; sig[3] = off;
  }
  sig[0] |= (uint64_t)(coll + 1) << 56;
  sig[2] |= (uint64_t)(root + 1) << 56;
  sig[1] ^= (uint64_t)count << 40;
  symCheckKernel<<<1, kThreads, 0, s>>>(st->peers, sig[0], sig[1], sig[2], sig[3]);
  return launched(c, "symCheckKernel");
}

mcclResult_t cudaCollective(mcclComm* c, int coll, const void* send, void* recv, size_t count, mcclDataType_t dt,
                            mcclRedOp_t op, int root, int algo, mcclStream_t stream) {
  CudaState* st = c->cu;
  if (st == nullptr) MCCLFAIL(mcclInternalError);
  // A wait that gave up earlier leaves the flags of this communicator desynchronised: refuse further work.
  MCCLCHECK(latchedError(c));
  int dev = -1;
  CUDACHECK(cudaGetDevice(&dev));
  if (dev != c->device) CUDACHECK(cudaSetDevice(c->device));
  Call k;
  k.c = c; k.st = st; k.n = c->nRanks; k.r = c->rank; k.dt = dt; k.es = mcclDataSize(dt); k.op = op;
  k.divisor = (op == mcclAvg) ? c->nRanks : 1;
  k.s = reinterpret_cast<cudaStream_t>(stream);
  mcclResult_t rc = mcclSuccess;
  if (c->nRanks == 1) {
    // Single rank: every collective is a local copy (avg over one rank is the identity).
    if (recv != nullptr && send != nullptr) rc = launchCopy(c, send, recv, 1, count * k.es, count * k.es, count * k.es, k.s);
  } else {
    rc = checkSymmetry(c, st, coll, send, recv, count, k.es, root, k.s);
    if (rc == mcclSuccess) switch (coll) {
      case mcclCollAllReduce:     rc = allReduce(k, send, recv, count, algo); break;
      case mcclCollAllGather:     rc = allGather(k, send, recv, count, algo); break;
      case mcclCollReduceScatter: rc = reduceScatter(k, send, recv, count, algo); break;
      case mcclCollBroadcast:     rc = broadcast(k, send, recv, count, root, algo); break;
      case mcclCollReduce:        rc = reduce(k, send, recv, count, root, algo); break;
      case mcclCollAllToAll:      rc = allToAll(k, send, recv, count); break;
      default: rc = mcclInvalidArgument;
    }
  }
  if (dev != c->device) cudaSetDevice(dev);
  return rc;
}

mcclResult_t cudaGroupAllReduce(mcclComm* c, const std::vector<CollCall>& calls, std::vector<char>* done) {
  CudaState* st = c->cu;
  done->assign(calls.size(), 0);
  if (st == nullptr || c->nRanks < 2) return mcclSuccess;
  MCCLCHECK(latchedError(c));
  int dev = -1;
  CUDACHECK(cudaGetDevice(&dev));
  if (dev != c->device) CUDACHECK(cudaSetDevice(c->device));
  const int n = c->nRanks;
  GroupArgs a;
  size_t total = 0;
  int fusedNow = 0;
  cudaStream_t s = nullptr;
  auto reset = [&]() { memset(&a, 0, sizeof(a)); a.peers = st->peers; total = 0; };
  auto flush = [&]() -> mcclResult_t {
    if (a.nJobs == 0) return mcclSuccess;
    bool allNvls = !a.anyTwoShot;
    a.nCtas = pickCtas(c, total, allNvls ? mcclAlgoNvls : mcclAlgoTwoShot);
    groupAllReduceKernel<<<a.nCtas, kThreads, 0, s>>>(a);
    c->lastAlgo.store(allNvls ? mcclAlgoNvls : mcclAlgoTwoShot);
    MCCL_TRACE("group of %d all-reduce calls, %zu bytes, one launch of %d CTAs", a.nJobs, total, a.nCtas);
    mcclResult_t rc = launched(c, "groupAllReduceKernel");
    reset();
    return rc;
  };
  reset();
  // A single fusable call gains nothing from this kernel: count them first.
  std::vector<char> can(calls.size(), 0);
  int fusable = 0;
  for (size_t i = 0; i < calls.size(); ++i) {
    const CollCall& k = calls[i];
    const size_t bytes = k.count * mcclDataSize(k.dt);
    if (k.coll != mcclCollAllReduce || bytes % 16 || bytes / 16 < (size_t)n || !al16(k.send) || !al16(k.recv)) continue;
    if (!viewOf(st, k.send, bytes).sym() || !viewOf(st, k.recv, bytes).sym()) continue;
    can[i] = 1;
    ++fusable;
  }
  if (fusable < 2) { if (dev != c->device) cudaSetDevice(dev); return mcclSuccess; }
  mcclResult_t rc = mcclSuccess;
  for (size_t i = 0; i < calls.size() && rc == mcclSuccess; ++i) {
    if (!can[i]) continue;
    const CollCall& k = calls[i];
    const size_t bytes = k.count * mcclDataSize(k.dt);
    const View sv = viewOf(st, k.send, bytes), rv = viewOf(st, k.recv, bytes);
    s = reinterpret_cast<cudaStream_t>(k.stream);
    GroupJob& j = a.jobs[a.nJobs++];
    j.bytes = bytes;
    j.dt = k.dt;
    j.op = (k.op == mcclAvg) ? mcclSum : k.op;
    j.divisor = (k.op == mcclAvg) ? n : 1;
    j.nvls = k.algo == mcclAlgoNvls && st->nvls && nvlsType(k.dt, k.op, n) && sv.mc() && rv.mc();
    if (j.nvls) { j.mcIn = sv.mc(); j.mcOut = rv.mc(); }
    else a.anyTwoShot = 1;
    for (int p = 0; p < n; ++p) { j.in[p] = sv.peer(p); j.red[p] = rv.peer(p); }
    j.out = static_cast<char*>(k.recv);
    total += bytes;
    (*done)[i] = 1;
    ++fusedNow;
    if (a.nJobs == MCCL_MAX_GROUP_JOBS) rc = flush();
  }
  if (rc == mcclSuccess) rc = flush();
  (void)fusedNow;
  if (dev != c->device) cudaSetDevice(dev);
  return rc;
}

mcclResult_t cudaBarrier(mcclComm* c, mcclStream_t stream) {
  CudaState* st = c->cu;
  MCCLCHECK(latchedError(c));
  CUDACHECK(cudaSetDevice(c->device));
  cudaStream_t s = stream ? reinterpret_cast<cudaStream_t>(stream) : reinterpret_cast<cudaStream_t>(st->internalStream);
  // Whatever the caller queued on any stream of this device comes first.
  if (!stream) CUDACHECK(cudaDeviceSynchronize());
  barrierKernel<<<1, kThreads, 0, s>>>(st->peers);
  MCCLCHECK(launched(c, "barrierKernel"));
  CUDACHECK(cudaStreamSynchronize(s));
  return latchedError(c);
}

mcclResult_t cudaP2pBatch(mcclComm* c, const std::vector<P2pOp>& ops, mcclStream_t stream) {
  CudaState* st = c->cu;
  MCCLCHECK(latchedError(c));
  CUDACHECK(cudaSetDevice(c->device));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // Sends to self pair with receives from self, in order.
  std::vector<const P2pOp*> selfS, selfR;
  for (const P2pOp& op : ops) if (op.peer == c->rank) (op.isSend ? selfS : selfR).push_back(&op);
  if (selfS.size() != selfR.size()) MCCLFAIL(mcclInvalidUsage);
  for (size_t i = 0; i < selfS.size(); ++i) {
    if (selfS[i]->bytes != selfR[i]->bytes) MCCLFAIL(mcclInvalidUsage);
    MCCLCHECK(launchCopy(c, selfS[i]->buf, selfR[i]->buf, 1, selfS[i]->bytes, selfS[i]->bytes, selfS[i]->bytes, s));
  }
  // One row of MCCL_P2P_CHANNELS CTAs per (peer, direction) flow, all flows of the batch in ONE launch (two launches in a row could wait for
  // each other across ranks).  The descriptors travel as kernel arguments; a batch longer than that holds goes
  // through stream-ordered device memory.
  std::vector<P2pDesc> descs;
  int flowOf[MCCL_MAX_RANKS][2];
  for (auto& f : flowOf) f[0] = f[1] = -1;
  int flows = 0;
  for (const P2pOp& op : ops) {
    if (op.peer == c->rank || op.bytes == 0) continue;
    int& f = flowOf[op.peer][op.isSend ? 1 : 0];
    if (f < 0) f = flows++;
    P2pDesc d;
    d.isSend = (f << 1) | (op.isSend ? 1 : 0);
    d.peer = op.peer;
    d.buf = static_cast<char*>(op.buf);
    d.bytes = op.bytes;
    descs.push_back(d);
  }
  if (descs.empty()) return mcclSuccess;
  P2pArgs a;
  memset(&a, 0, sizeof(a));
  a.peers = st->peers;
  a.nOps = (int)descs.size();
  void* devDescs = nullptr;
  if (descs.size() <= MCCL_MAX_P2P_OPS) {
    memcpy(a.ops, descs.data(), descs.size() * sizeof(P2pDesc));
  } else {
    CUDACHECK(cudaMallocAsync(&devDescs, descs.size() * sizeof(P2pDesc), s));
    CUDACHECK(cudaMemcpyAsync(devDescs, descs.data(), descs.size() * sizeof(P2pDesc), cudaMemcpyHostToDevice, s));
    a.more = static_cast<const P2pDesc*>(devDescs);
  }
  p2pKernel<<<dim3(flows, p2pChannels(c->nRanks)), kThreads, 0, s>>>(a);
  mcclResult_t rc = launched(c, "p2pKernel");
  if (devDescs) {
    CUDACHECK(cudaFreeAsync(devDescs, s));
    CUDACHECK(cudaStreamSynchronize(s));       // `descs` is pageable memory the copy may still be reading
  }
  return rc;
}

mcclResult_t cudaRecvAny(mcclComm* c, void* buf, size_t bytes, int* src, mcclStream_t stream) {
  CudaState* st = c->cu;
  MCCLCHECK(latchedError(c));
  CUDACHECK(cudaSetDevice(c->device));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int* host = static_cast<int*>(st->probeHost);
  int* dev = nullptr;
  CUDACHECK(cudaHostGetDevicePointer((void**)&dev, host, 0));
  *host = -2;
  recvAnyProbeKernel<<<1, 32, 0, s>>>(st->peers, dev);
  MCCLCHECK(launched(c, "recvAnyProbeKernel"));
  CUDACHECK(cudaStreamSynchronize(s));
  if (*host < 0) {
    MCCL_WARN("RecvAny: no sender within the device time budget");
    return c->aborted.load() ? mcclInvalidUsage : mcclRemoteError;
  }
  *src = *host;
  std::vector<P2pOp> one{P2pOp{c, false, *src, buf, bytes, stream}};
  return cudaP2pBatch(c, one, stream);
}

// Measure what the cost model assumes: per-pair pull bandwidth and the latency of an empty collective,
// then refine the tuner's constants (maximum over ranks, so every rank ends with the same table).
// Role parity: mcclCalibrateTbLinks (src/init.cc:164-204) of the reference, with a timed pull kernel in
// place of a one-second TCP stream.
mcclResult_t cudaCalibrate(mcclComm* c) {
  CudaState* st = c->cu;
  if (c->nRanks < 2 || st->layout.stageBytes < (8u << 20)) return mcclSuccess;
  CUDACHECK(cudaSetDevice(c->device));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(st->internalStream);
  cudaEvent_t e0, e1;
  CUDACHECK(cudaEventCreate(&e0));
  CUDACHECK(cudaEventCreate(&e1));
  Call k;
  k.c = c; k.st = st; k.n = c->nRanks; k.r = c->rank; k.dt = mcclFloat32; k.es = 4; k.op = mcclSum; k.divisor = 1; k.s = s;
  std::vector<float> bw(c->nRanks, 0.f);
  const size_t probe = std::min<size_t>(st->layout.stageBytes / 2, 32u << 20);
  char* scratch = k.stageLocal() + st->layout.stageBytes / 2;
  float latencyUs = 0.f;
  // Latency: empty pull kernels (three barriers each); bandwidth: pull `probe` bytes from one peer at a time.
  for (int round = -1; round < c->nRanks; ++round) {
    const int peer = round;
    if (peer == c->rank) continue;
    const int iters = peer < 0 ? 20 : 4;
    for (int it = -1; it < iters; ++it) {     // first pass warms up
      if (it == 0) CUDACHECK(cudaEventRecord(e0, s));
      PullArgs a = basePull(k, probe, mcclAlgoTwoShot);
      if (peer >= 0) a.jobs[a.nJobs++] = CopyJob{k.stagePeer(peer), scratch, probe};
      MCCLCHECK(launchPull(c, a, mcclInt32, s));
    }
    CUDACHECK(cudaEventRecord(e1, s));
    CUDACHECK(cudaStreamSynchronize(s));
    float ms = 0.f;
    CUDACHECK(cudaEventElapsedTime(&ms, e0, e1));
    if (peer < 0) latencyUs = ms * 1000.f / iters;
    else bw[peer] = (float)((double)probe * iters / (ms * 1e-3) / 1e9);
    MCCLCHECK(latchedError(c));
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  struct Row { float bw[MCCL_MAX_RANKS]; float lat; };
  Row mine;
  memset(&mine, 0, sizeof(mine));
  for (int p = 0; p < c->nRanks; ++p) mine.bw[p] = bw[p];
  mine.lat = latencyUs;
  std::vector<Row> all(c->nRanks);
  MCCLCHECK(bootstrapAllGather(c->bs, &mine, all.data(), sizeof(Row)));
  float minBw = 1e9f, maxLat = 0.f;
  for (int a = 0; a < c->nRanks; ++a) {
    maxLat = std::max(maxLat, all[a].lat);
    for (TopoLink& l : c->system.nodes[a].links) {
      l.measured = all[a].bw[l.remote];
      l.latencyUs = all[a].lat / 3.f;
      if (l.measured > 0.f) { l.bw = l.measured; minBw = std::min(minBw, l.measured); }
    }
  }
  // Per algorithm a two-point fit of the model's alpha and bandwidth: the all-reduce on the stage at a small and a
  // large size (fp32 sum, best of three timings of a few back-to-back calls), the slowest rank's figures for all.
  // One peer at a time cannot saturate the port, so the per-pair numbers above describe links (and reveal a dead
  // one), while these fits describe what each kernel makes of all links together.
  {
    cudaEvent_t f0, f1;
    CUDACHECK(cudaEventCreate(&f0));
    CUDACHECK(cudaEventCreate(&f1));
    const size_t big = std::min<size_t>(st->layout.stageBytes / 2, 32u << 20) / (16 * (size_t)k.n) * (16 * (size_t)k.n);
    const size_t slot = (size_t)st->layout.oneShotSlotBytes / 16 * 16;
    struct Point { int algo; size_t small, large; };
    const Point points[3] = {{mcclAlgoOneShot, 4096, std::min<size_t>(slot, 1u << 20)}, {mcclAlgoTwoShot, 65536, big}, {mcclAlgoNvls, 65536, big}};
    float us[3][2] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
    char* in[MCCL_MAX_RANKS];
    for (int p = 0; p < k.n; ++p) in[p] = k.stagePeer(p);
    for (int a = 0; a < 3; ++a) {
      const int algo = points[a].algo;
      if (!c->tuner.viable[algo] || (algo == mcclAlgoNvls && !st->nvls)) continue;
      for (int pt = 0; pt < 2; ++pt) {
        const size_t bytes = pt == 0 ? points[a].small : points[a].large;
        const int iters = pt == 0 ? 8 : 3;
        float best = 1e30f;
        for (int rep = -1; rep < 3; ++rep) {          // rep -1 warms up
          CUDACHECK(cudaEventRecord(f0, s));
          for (int it = 0; it < iters; ++it) {
            if (algo == mcclAlgoOneShot) MCCLCHECK(arOneShot(k, k.stageLocal(), k.stageLocal() + st->layout.stageBytes / 2, bytes));
            else if (algo == mcclAlgoTwoShot) MCCLCHECK(twoShot(k, in, in, nullptr, bytes, true, mcclAlgoTwoShot));
            else MCCLCHECK(arNvlsOn(k, k.stageMc(), k.stageMc(), bytes));
          }
          CUDACHECK(cudaEventRecord(f1, s));
          CUDACHECK(cudaStreamSynchronize(s));
          float ms = 0.f;
          CUDACHECK(cudaEventElapsedTime(&ms, f0, f1));
          if (rep >= 0) best = std::min(best, ms * 1000.f / iters);
          MCCLCHECK(latchedError(c));
        }
        us[a][pt] = best;
      }
    }
    cudaEventDestroy(f0);
    cudaEventDestroy(f1);
    std::vector<float> allUs((size_t)c->nRanks * 6);
    MCCLCHECK(bootstrapAllGather(c->bs, &us[0][0], allUs.data(), sizeof(us)));
    for (int a = 0; a < 3; ++a) {
      float t[2] = {0.f, 0.f};
      for (int r = 0; r < c->nRanks; ++r) for (int pt = 0; pt < 2; ++pt) t[pt] = std::max(t[pt], allUs[(size_t)r * 6 + a * 2 + pt]);
      const int algo = points[a].algo;
      if (t[0] <= 0.f || t[1] <= t[0]) continue;
      const double f = algoTraffic(algo, mcclCollAllReduce, c->nRanks);
      const float bwFit = (float)((double)(points[a].large - points[a].small) * f / (1000.0 * (t[1] - t[0])));
      const float alphaFit = std::max(1.f, t[0] - (float)((double)points[a].small * f / (1000.0 * bwFit)));
      // A fit far from the built-in constants means a disturbed measurement (a busy GPU): keep the constants then.
      if (bwFit < 0.25f * c->tuner.bw[algo] || bwFit > 4.f * c->tuner.bw[algo]) {
        MCCL_WARN("calibration of %s looks disturbed (%.1f GB/s against %.1f assumed): keeping the built-in constants", mcclAlgoStr(algo), bwFit, c->tuner.bw[algo]);
        continue;
      }
      MCCL_INFO("calibration: %-8s alpha %.1f us (was %.1f), bandwidth %.1f GB/s (was %.1f)", mcclAlgoStr(algo), alphaFit,
                c->tuner.alphaUs[algo], bwFit, c->tuner.bw[algo]);
      c->tuner.alphaUs[algo] = alphaFit;
      c->tuner.stepUs[algo] = 0.f;
      c->tuner.bw[algo] = bwFit;
    }
    c->tuner.measured = true;
  }
  if (minBw < 1e9f && minBw < 1.f) MCCL_WARN("calibration: a peer link moved less than 1 GB/s");
  MCCL_INFO("calibration: empty collective %.1f us, slowest pair %.1f GB/s", maxLat, minBw);
  return mcclSuccess;
}

}  // namespace mccl
