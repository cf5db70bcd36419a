// Communicator lifecycle: unique id, init, split, finalize, abort, destroy, queries, arenas.
// Parity: src/comm.cc:50-356 of the reference.  Differences: the unique id is backed by a listener that
// the creating process opens (the environment pair MCCL_BOOTSTRAP_IP/PORT remains as the shared-by-
// convention form); an unknown transport name is refused instead of silently meaning TCP; a split child
// rendezvouses on a fresh listener of its leader instead of a port derived from the parent's.
#include "comm.h"

#include <arpa/inet.h>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <unistd.h>

#include "../os/pool.h"
#include "../os/socket.h"
#include "../core/trace.h"

using namespace mccl;

namespace mccl {

static uint64_t fnv1a(const void* data, size_t n, uint64_t h = 1469598103934665603ull) {
  const unsigned char* p = static_cast<const unsigned char*>(data);
  for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
  return h;
}

static uint64_t hostHash() {
  char name[256] = {0};
  gethostname(name, sizeof(name) - 1);
  uint64_t h = fnv1a(name, strlen(name));
  // Containers can share a hostname; the boot id separates machines.
  FILE* f = fopen("/proc/sys/kernel/random/boot_id", "r");
  if (f) {
    char id[64] = {0};
    if (fgets(id, sizeof(id), f)) h = fnv1a(id, strlen(id), h);
    fclose(f);
  }
  const char* extra = envStr("MCCL_HOSTID");
  if (extra) h = fnv1a(extra, strlen(extra), h);
  return h;
}

static mcclResult_t resolveTransport(const mcclConfig_t* cfg, bool* cuda, std::string* name) {
  const char* t = (cfg && cfg->transport && *cfg->transport) ? cfg->transport : envStr("MCCL_TRANSPORT");
  if (t == nullptr) {
    *cuda = cudaDeviceCountSafe() > 0;
  } else if (!strcasecmp(t, "tcp") || !strcasecmp(t, "cpu")) {
    *cuda = false;
  } else if (!strcasecmp(t, "cuda") || !strcasecmp(t, "nvlink") || !strcasecmp(t, "gpu")) {
    *cuda = true;
    if (cudaDeviceCountSafe() <= 0) {
      MCCL_WARN("transport '%s' requested but no CUDA device is visible", t);
      return mcclInvalidUsage;
    }
  } else {
    MCCL_WARN("unknown transport '%s' (tcp | cuda)", t);
    return mcclInvalidArgument;
  }
  *name = *cuda ? "cuda" : "tcp";
  return mcclSuccess;
}

mcclResult_t commReserveStaging(mcclComm* comm, size_t bytes, void** out) {
  if (bytes > comm->stagingBytes) {
    mcclPageFree(comm->staging);
    comm->staging = nullptr;
    comm->stagingBytes = 0;
    size_t want = std::max(bytes, (size_t)(1u << 20));
    MCCLCHECK(mcclPageAlloc(want, &comm->staging));
    comm->stagingBytes = want;
  }
  *out = comm->staging;
  return mcclSuccess;
}

mcclResult_t commReserveScratch(mcclComm* comm, size_t bytes, void** out) {
  if (bytes > comm->scratchBytes) {
    mcclPageFree(comm->scratch);
    comm->scratch = nullptr;
    comm->scratchBytes = 0;
    size_t want = std::max(bytes, (size_t)(1u << 20));
    MCCLCHECK(mcclPageAlloc(want, &comm->scratch));
    comm->scratchBytes = want;
  }
  *out = comm->scratch;
  return mcclSuccess;
}

mcclResult_t commPeerConn(mcclComm* comm, int peer, uint32_t kind, TcpConn** out) {
  if (comm->ep == nullptr) MCCLFAIL(mcclInternalError);
  if (comm->aborted.load()) MCCLFAIL(mcclInvalidUsage);
  struct in_addr a;
  a.s_addr = htonl(comm->infos[peer].ip);
  char ip[64];
  inet_ntop(AF_INET, &a, ip, sizeof(ip));
  return tcpConnectPair(comm->ep, peer, kind, ip, comm->infos[peer].dataPort, out);
}

static thread_local int tlsForcedAlgo = mcclAlgoAuto;
int forcedAlgo() { return tlsForcedAlgo; }

int commPickAlgo(mcclComm* comm, int coll, size_t bytes, int dt, int op) {
  int algo = mcclAlgoRing;
  const int f = forcedAlgo();
  if (f >= 0 && f < mcclNumAlgos && comm->tuner.viable[f] && algoSupports(f, coll, dt, op, comm->cuda)) return f;
  if (tunerPick(comm->tuner, coll, comm->nRanks, bytes, dt, op, comm->enabled, comm->cuda, &algo) != mcclSuccess)
    algo = mcclAlgoRing;
  return algo;
}

static mcclResult_t buildPlan(mcclComm* c) {
  MCCLCHECK(topoGetSystem(c->infos.data(), c->nRanks, c->cuda, &c->system));
  MCCLCHECK(topoComputePaths(&c->system));
  for (int a = 0; a < mcclNumAlgos; ++a) MCCLCHECK(topoCompute(c->system, a, &c->graphs[a]));
  MCCLCHECK(topoConnect(c->system, c->graphs[mcclAlgoRing], c->graphs[mcclAlgoTree], c->rank, &c->chan));
  MCCLCHECK(tunerInit(c->system, c->graphs, c->cuda, &c->tuner));
  MCCLCHECK(getEnabledAlgos(c->enabled));
  return mcclSuccess;
}

static void freeComm(mcclComm* c) {
  if (c == nullptr) return;
  if (c->work) workerStop(c);
  traceFlush(c);
  if (c->cu) cudaCommDestroy(c);
  if (c->ep) tcpEndpointClose(c->ep);
  if (c->bs) bootstrapClose(c->bs);
  mcclPageFree(c->staging);
  mcclPageFree(c->scratch);
  delete c;
}

}  // namespace mccl

extern "C" {

mcclResult_t mcclGetUniqueId(mcclUniqueId* id) {
  if (id == nullptr) MCCLFAIL(mcclInvalidArgument);
  static_assert(sizeof(BootstrapId) <= sizeof(mcclUniqueId), "id layout");
  memset(id, 0, sizeof(*id));
  BootstrapId b;
  MCCLCHECK(bootstrapCreateId(&b));
  memcpy(id->internal, &b, sizeof(b));
  return mcclSuccess;
}

mcclResult_t mcclCommInitRank(mcclComm_t* comm, int nRanks, mcclUniqueId id, int rank) {
  return mcclCommInitRankConfig(comm, nRanks, id, rank, nullptr);
}

mcclResult_t mcclCommInitRankConfig(mcclComm_t* out, int nRanks, mcclUniqueId id, int rank, const mcclConfig_t* config) {
  if (out == nullptr || nRanks < 1 || rank < 0 || rank >= nRanks) MCCLFAIL(mcclInvalidArgument);
  *out = nullptr;
  bool cuda = false;
  std::string tname;
  // Decide the transport before any rendezvous so that a host that cannot run it fails with everyone else.
  MCCLCHECK(resolveTransport(config, &cuda, &tname));
  mcclComm* c = new mcclComm();
  c->rank = rank;
  c->nRanks = nRanks;
  c->cuda = cuda;
  c->transport = tname;
  c->blocking = config ? config->blocking : 1;
  memcpy(&c->id, id.internal, sizeof(BootstrapId));
  c->id.ip[sizeof(c->id.ip) - 1] = '\0';
  logSetRank(rank);
  mcclResult_t rc = mcclSuccess;
  RankInfo mine;
  memset(&mine, 0, sizeof(mine));

  MCCLCHECKGOTO(bootstrapInit(c->id, rank, nRanks, &c->bs), rc, fail);
  mine.hostHash = hostHash();
  mine.pidHash = ((uint64_t)getpid() << 32) ^ (uint64_t)(uintptr_t)c;
  mine.device = -1;
  {
    const char* ipEnv = envStr("MCCL_SOCKET_IP");
    uint32_t ip = 0;
    struct in_addr a;
    if (ipEnv && inet_pton(AF_INET, ipEnv, &a) == 1) ip = ntohl(a.s_addr);
    if (ip == 0) ip = bootstrapLocalIp(c->bs);
    if (ip == 0 && inet_pton(AF_INET, c->id.ip, &a) == 1) ip = ntohl(a.s_addr);
    mine.ip = ip;
  }
  if (!cuda) {
    MCCLCHECKGOTO(tcpEndpointStart(rank, c->id.nonce ^ 0x5bd1e995u, &c->ep), rc, fail);
    mine.dataPort = c->ep->port;
  } else {
    MCCLCHECKGOTO(cudaFillRankInfo(-1, &mine), rc, fail);
    c->device = mine.device;
  }
  c->infos.resize(nRanks);
  MCCLCHECKGOTO(bootstrapAllGather(c->bs, &mine, c->infos.data(), sizeof(RankInfo)), rc, fail);
  for (int r = 0; r < nRanks; ++r) {
    if ((c->infos[r].device >= 0) != cuda) {
      MCCL_WARN("rank %d uses a different transport than rank %d", r, rank);
      rc = mcclInvalidUsage;
      goto fail;
    }
  }
  if (cuda) {
    // One GPU per rank: the kernels of different ranks wait for one another, and nothing makes two kernels of
    // different processes run at the same time on one GPU.
    for (int a = 0; a < nRanks; ++a)
      for (int b = a + 1; b < nRanks; ++b)
        if (c->infos[a].hostHash == c->infos[b].hostHash && !strncmp(c->infos[a].busId, c->infos[b].busId, sizeof(c->infos[a].busId))) {
          MCCL_WARN("ranks %d and %d of this communicator use the same GPU (%s): set one device per rank before creating it", a, b,
                    c->infos[a].busId);
          rc = mcclInvalidUsage;
          goto fail;
        }
  }
  MCCLCHECKGOTO(buildPlan(c), rc, fail);
  if (cuda) {
    MCCLCHECKGOTO(cudaCommInit(c), rc, fail);
    // The tuner's constants for this machine: loaded from the cache of an earlier calibration when there is one,
    // else measured now (a few tens of milliseconds) and cached.  MCCL_CALIBRATE=1 measures afresh, =0 keeps the
    // built-in constants.  Rank 0 decides, so every rank takes the same path.
    if (nRanks > 1) {
      const int mode = (int)envInt("MCCL_CALIBRATE", -1);
      char gpuTag[48];
      snprintf(gpuTag, sizeof(gpuTag), "cc%d-sm%d", (int)c->infos[0].cc, (int)c->infos[0].smCount);
      const std::string path = tunerCachePath(nRanks, gpuTag);
      int have = 0;
      if (rank == 0 && mode < 0) { FILE* f = fopen(path.c_str(), "r"); if (f) { have = 1; fclose(f); } }
      std::vector<int> haves(nRanks, 0);
      MCCLCHECKGOTO(bootstrapAllGather(c->bs, &have, haves.data(), sizeof(int)), rc, fail);
      if (haves[0]) {
        MCCLCHECKGOTO(tunerLoadCache(&c->tuner, path.c_str()), rc, fail);
      } else if (mode != 0) {
        MCCLCHECKGOTO(cudaCalibrate(c), rc, fail);
        if (rank == 0 && c->tuner.measured) tunerSaveCache(c->tuner, path.c_str());
      }
    }
  }
  if (rank == 0) {
    const char* dump = envStr("MCCL_TOPO_DUMP_FILE");
    if (dump) topoDumpXmlToFile(c->system, c->graphs, mcclNumAlgos, &c->tuner, dump);
  }
  if (logLevel() >= LOG_INFO && rank == 0) {
    MCCL_INFO("comm %p: %d ranks, transport %s, nvls %d", (void*)c, nRanks, c->transport.c_str(), (int)c->system.nvls);
    for (int a = 0; a < mcclNumAlgos; ++a)
      MCCL_INFO("  algo %-8s viable %d bw %.1f GB/s alpha %.1f us step %.2f us channels %d (%s)", mcclAlgoStr(a),
                (int)c->graphs[a].viable, c->tuner.bw[a], c->tuner.alphaUs[a], c->tuner.stepUs[a], c->graphs[a].nChannels,
                c->tuner.measured && (a == mcclAlgoOneShot || a == mcclAlgoTwoShot || a == mcclAlgoNvls) ? "measured" : "built in");
  }
  if (!cuda && c->blocking == 0 && nRanks > 1) MCCLCHECKGOTO(workerStart(c), rc, fail);
  *out = c;
  return mcclSuccess;
fail:
  freeComm(c);
  return rc;
}

mcclResult_t mcclCommSplit(mcclComm_t comm, int color, int key, mcclComm_t* newcomm, const mcclConfig_t* config) {
  if (comm == nullptr || newcomm == nullptr) MCCLFAIL(mcclInvalidArgument);
  if (color < 0 && color != MCCL_SPLIT_NOCOLOR) MCCLFAIL(mcclInvalidArgument);
  if (comm->aborted.load()) MCCLFAIL(mcclInvalidUsage);
  *newcomm = nullptr;
  // Outstanding work must not interleave with the control-plane rounds below.
  MCCLCHECK(mcclCommSynchronize(comm));
  struct SplitInfo { int32_t color, key; };
  std::vector<SplitInfo> all(comm->nRanks);
  SplitInfo mine = {color, key};
  MCCLCHECK(bootstrapAllGather(comm->bs, &mine, all.data(), sizeof(SplitInfo)));

  // My group: ranks with my color ordered by (key, parent rank).
  std::vector<int> group;
  for (int r = 0; r < comm->nRanks; ++r)
    if (color != MCCL_SPLIT_NOCOLOR && all[r].color == color) group.push_back(r);
  std::stable_sort(group.begin(), group.end(), [&](int a, int b) {
    return all[a].key != all[b].key ? all[a].key < all[b].key : a < b;
  });
  int newRank = -1;
  for (size_t i = 0; i < group.size(); ++i) if (group[i] == comm->rank) newRank = (int)i;

  // Each group's leader opens a fresh listener; the ids travel through the parent's control plane, so
  // successive splits never meet on a derived port.
  std::vector<BootstrapId> ids(comm->nRanks);
  BootstrapId myId;
  memset(&myId, 0, sizeof(myId));
  if (newRank == 0) {
    struct in_addr a;
    a.s_addr = htonl(comm->infos[comm->rank].ip);
    char ip[64];
    inet_ntop(AF_INET, &a, ip, sizeof(ip));
    MCCLCHECK(bootstrapCreateId(&myId, ip, true));
  }
  MCCLCHECK(bootstrapAllGather(comm->bs, &myId, ids.data(), sizeof(BootstrapId)));
  if (color == MCCL_SPLIT_NOCOLOR) return mcclSuccess;

  mcclUniqueId uid;
  memset(&uid, 0, sizeof(uid));
  memcpy(uid.internal, &ids[group[0]], sizeof(BootstrapId));
  mcclConfig_t inherited = {comm->blocking, comm->transport.c_str()};
  return mcclCommInitRankConfig(newcomm, (int)group.size(), uid, newRank, config ? config : &inherited);
}

mcclResult_t mcclCommSynchronize(mcclComm_t comm) {
  if (comm == nullptr) MCCLFAIL(mcclInvalidArgument);
  if (comm->work) return workerSync(comm);
  const mcclResult_t st = (mcclResult_t)comm->asyncState.load();
  return resultFatal(st) ? st : mcclSuccess;
}

mcclResult_t mcclCommFinalize(mcclComm_t comm) {
  if (comm == nullptr) MCCLFAIL(mcclInvalidArgument);
  if (comm->aborted.load()) MCCLFAIL(mcclInvalidUsage);
  mcclResult_t rc = mcclCommSynchronize(comm);
  if (rc != mcclSuccess) return rc;
  if (comm->nRanks > 1) {
    if (comm->cuda) {
      MCCLCHECK(cudaBarrier(comm, nullptr));
    } else {
      // Barrier: a one-element sum all-reduce, as in the reference (src/comm.cc:280-281).
      int32_t one = 1, sum = 0;
      MCCLCHECK(mcclAllReduce(comm, &one, &sum, 1, mcclInt32, mcclSum, nullptr));
      MCCLCHECK(mcclCommSynchronize(comm));
      if (sum != comm->nRanks) MCCLFAIL(mcclInternalError);
    }
  }
  return mcclSuccess;
}

mcclResult_t mcclCommDestroy(mcclComm_t comm) {
  if (comm == nullptr) return mcclSuccess;
  freeComm(comm);
  return mcclSuccess;
}

// Abort unblocks every thread parked in this communicator's sockets or device waits and frees nothing:
// those threads still hold pointers into the communicator (src/comm.cc:288-305 of the reference).
mcclResult_t mcclCommAbort(mcclComm_t comm) {
  if (comm == nullptr) MCCLFAIL(mcclInvalidArgument);
  comm->aborted.store(true);
  if (comm->ep) tcpEndpointShutdown(comm->ep);
  if (comm->bs) bootstrapAbort(comm->bs);
  if (comm->cu) cudaCommAbort(comm);
  if (comm->work) workerStop(comm);
  return mcclSuccess;
}

mcclResult_t mcclCommCount(mcclComm_t comm, int* count) {
  if (comm == nullptr || count == nullptr) MCCLFAIL(mcclInvalidArgument);
  *count = comm->nRanks;
  return mcclSuccess;
}
mcclResult_t mcclCommUserRank(mcclComm_t comm, int* rank) {
  if (comm == nullptr || rank == nullptr) MCCLFAIL(mcclInvalidArgument);
  *rank = comm->rank;
  return mcclSuccess;
}
mcclResult_t mcclCommDevice(mcclComm_t comm, int* device) {
  if (comm == nullptr || device == nullptr) MCCLFAIL(mcclInvalidArgument);
  *device = comm->device;
  return mcclSuccess;
}
const char* mcclCommTransport(mcclComm_t comm) { return comm ? comm->transport.c_str() : "none"; }

mcclResult_t mcclCommNvlsEnabled(mcclComm_t comm, int* enabled) {
  if (comm == nullptr || enabled == nullptr) MCCLFAIL(mcclInvalidArgument);
  *enabled = (comm->cuda && comm->cu && cudaNvlsEnabled(comm)) ? 1 : 0;
  return mcclSuccess;
}

mcclResult_t mcclCommGetAsyncError(mcclComm_t comm, mcclResult_t* asyncErr) {
  if (comm == nullptr || asyncErr == nullptr) MCCLFAIL(mcclInvalidArgument);
  if (comm->aborted.load()) { *asyncErr = mcclInvalidUsage; return mcclSuccess; }
  if (comm->work) return workerAsyncError(comm, asyncErr);
  if (comm->cu) return cudaCommAsyncError(comm, asyncErr);
  *asyncErr = (mcclResult_t)comm->asyncState.load();
  return mcclSuccess;
}

mcclResult_t mcclCommHostAllGather(mcclComm_t comm, const void* send, void* recv, size_t bytes) {
  if (comm == nullptr || send == nullptr || recv == nullptr) MCCLFAIL(mcclInvalidArgument);
  return bootstrapAllGather(comm->bs, send, recv, bytes);
}
mcclResult_t mcclCommHostBarrier(mcclComm_t comm) {
  if (comm == nullptr) MCCLFAIL(mcclInvalidArgument);
  return bootstrapBarrier(comm->bs);
}

mcclResult_t mcclCommPickAlgo(mcclComm_t comm, int coll, size_t bytes, int dt, int op, int* algo) {
  if (comm == nullptr || algo == nullptr || (unsigned)coll >= (unsigned)mcclNumColls) MCCLFAIL(mcclInvalidArgument);
  *algo = commPickAlgo(comm, coll, bytes, dt, op);
  return mcclSuccess;
}
mcclResult_t mcclSetForcedAlgo(int algo) {
  if (algo != mcclAlgoAuto && (unsigned)algo >= (unsigned)mcclNumAlgos) MCCLFAIL(mcclInvalidArgument);
  tlsForcedAlgo = algo;
  return mcclSuccess;
}
mcclResult_t mcclCommLastAlgo(mcclComm_t comm, int* algo) {
  if (comm == nullptr || algo == nullptr) MCCLFAIL(mcclInvalidArgument);
  *algo = comm->lastAlgo.load();
  return mcclSuccess;
}
mcclResult_t mcclCommLaunchCount(mcclComm_t comm, uint64_t* launches) {
  if (comm == nullptr || launches == nullptr) MCCLFAIL(mcclInvalidArgument);
  *launches = comm->launches.load();
  return mcclSuccess;
}
mcclResult_t mcclCommSetMaxCtas(mcclComm_t comm, int maxCtas) {
  if (comm == nullptr || maxCtas < 0) MCCLFAIL(mcclInvalidArgument);
  comm->maxCtas = maxCtas;
  return mcclSuccess;
}
mcclResult_t mcclCommSetCtas(mcclComm_t comm, int ctas) {
  if (comm == nullptr || ctas < 0) MCCLFAIL(mcclInvalidArgument);
  comm->forcedCtas = ctas;
  return mcclSuccess;
}
mcclResult_t mcclCommCheckGuards(mcclComm_t comm, int* intact) {
  if (comm == nullptr || intact == nullptr) MCCLFAIL(mcclInvalidArgument);
  *intact = 1;
  if (!comm->cuda || comm->cu == nullptr) return mcclSuccess;
  return cudaCheckGuards(comm, intact);
}
mcclResult_t mcclCommTopoXml(mcclComm_t comm, char** xml) {
  if (comm == nullptr || xml == nullptr) MCCLFAIL(mcclInvalidArgument);
  XmlNode* root = topoToXml(comm->system, comm->graphs, mcclNumAlgos, &comm->tuner);
  std::string s = xmlToString(root);
  delete root;
  *xml = strdup(s.c_str());
  return *xml ? mcclSuccess : mcclSystemError;
}

mcclResult_t mcclMemAlloc(mcclComm_t comm, size_t bytes, void** ptr) {
  if (comm == nullptr || ptr == nullptr || bytes == 0) MCCLFAIL(mcclInvalidArgument);
  if (!comm->cuda) return mcclPageAlloc(bytes, ptr);   // tcp transport: plain page-aligned host memory
  return cudaMemAllocSym(comm, bytes, ptr);
}
mcclResult_t mcclMemFree(mcclComm_t comm, void* ptr) {
  if (comm == nullptr) MCCLFAIL(mcclInvalidArgument);
  if (ptr == nullptr) return mcclSuccess;
  if (!comm->cuda) { mcclPageFree(ptr); return mcclSuccess; }
  return cudaMemFreeSym(comm, ptr);
}
mcclResult_t mcclCommRegister(mcclComm_t comm, void* ptr, size_t bytes, void** handle) {
  if (comm == nullptr || ptr == nullptr || handle == nullptr || bytes == 0) MCCLFAIL(mcclInvalidArgument);
  if (!comm->cuda) { *handle = ptr; return mcclSuccess; }
  return cudaRegister(comm, ptr, bytes, handle);
}
mcclResult_t mcclCommDeregister(mcclComm_t comm, void* handle) {
  if (comm == nullptr) MCCLFAIL(mcclInvalidArgument);
  if (!comm->cuda || handle == nullptr) return mcclSuccess;
  return cudaDeregister(comm, handle);
}
mcclResult_t mcclMemPeerPointer(mcclComm_t comm, const void* localPtr, int peer, void** peerPtr) {
  if (comm == nullptr || peerPtr == nullptr || peer < 0 || peer >= comm->nRanks) MCCLFAIL(mcclInvalidArgument);
  *peerPtr = nullptr;
  if (!comm->cuda) return mcclSuccess;
  return cudaPeerPointer(comm, localPtr, peer, peerPtr);
}
mcclResult_t mcclMemMulticastPointer(mcclComm_t comm, const void* localPtr, void** mcPtr) {
  if (comm == nullptr || mcPtr == nullptr) MCCLFAIL(mcclInvalidArgument);
  *mcPtr = nullptr;
  if (!comm->cuda) return mcclSuccess;
  return cudaMcPointer(comm, localPtr, mcPtr);
}

}  // extern "C"
