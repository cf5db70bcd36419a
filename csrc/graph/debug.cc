// Probe entry points: each exposes one subsystem on synthetic inputs so it can be exercised without a
// network or a GPU, the role the reference's `#ifdef MCCL_*_MAIN` programs play (src/graph/trees.cc:57-81,
// src/graph/connect.cc:98-143, src/graph/xml.cc:158-184, src/allocator.cc:81-115).
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../device/devcomm.h"
#include "../device/host_reduce.h"
#include "graph.h"

using namespace mccl;

namespace {
// n ranks on one host.  cuda: GPU r has peer access to every GPU except pairs listed in `cut`
// (bit a*32+b unused; cutA/cutB name one severed pair, -1 = none).
std::vector<RankInfo> syntheticInfos(int n, bool cuda, bool nvls, int cutA = -1, int cutB = -1) {
  std::vector<RankInfo> v(n);
  for (int r = 0; r < n; ++r) {
    RankInfo& ri = v[r];
    memset(&ri, 0, sizeof(ri));
    ri.hostHash = 0x1234;
    ri.ip = 0x7f000001u;
    ri.dataPort = (uint16_t)(40000 + r);
    ri.device = cuda ? r : -1;
    ri.smCount = cuda ? 148 : 0;
    ri.cc = cuda ? 100 : 0;
    ri.multicast = nvls;
    ri.vmm = cuda;
    ri.hbmBytes = cuda ? (180ull << 30) : 0;
    ri.peerMask = cuda ? 0xffffffffu : 0;
    if (cuda && r == cutA && cutB >= 0) ri.peerMask &= ~(1u << cutB);
    if (cuda && r == cutB && cutA >= 0) ri.peerMask &= ~(1u << cutA);
    snprintf(ri.busId, sizeof(ri.busId), "0000:%02x:00.0", r);
  }
  return v;
}

mcclResult_t syntheticPlan(int n, bool cuda, bool nvls, TopoSystem* sys, TopoGraph graphs[mcclNumAlgos], TunerModel* tuner,
                           int cutA = -1, int cutB = -1) {
  std::vector<RankInfo> infos = syntheticInfos(n, cuda, nvls, cutA, cutB);
  MCCLCHECK(topoGetSystem(infos.data(), n, cuda, sys));
  MCCLCHECK(topoComputePaths(sys));
  for (int a = 0; a < mcclNumAlgos; ++a) MCCLCHECK(topoCompute(*sys, a, &graphs[a]));
  if (tuner) MCCLCHECK(tunerInit(*sys, graphs, cuda, tuner));
  return mcclSuccess;
}
}  // namespace

extern "C" {

void mcclDbgBtree(int n, int rank, int* out3) { getBtree(n, rank, &out3[0], &out3[1], &out3[2]); }
void mcclDbgDtree(int n, int rank, int* out6) {
  getDtree(n, rank, &out6[0], &out6[1], &out6[2], &out6[3], &out6[4], &out6[5]);
}

mcclResult_t mcclDbgSyntheticTopoXml(int n, int cuda, float bw, int nvls, char** xml) {
  TopoSystem sys;
  TopoGraph graphs[mcclNumAlgos];
  TunerModel tuner;
  if (bw > 0.f) setenv(cuda ? "MCCL_NVL_BW" : "MCCL_LAN_BW", std::to_string(bw).c_str(), 1);
  mcclResult_t rc = syntheticPlan(n, cuda != 0, nvls != 0, &sys, graphs, &tuner);
  if (bw > 0.f) unsetenv(cuda ? "MCCL_NVL_BW" : "MCCL_LAN_BW");
  MCCLCHECK(rc);
  XmlNode* root = topoToXml(sys, graphs, mcclNumAlgos, &tuner);
  std::string s = xmlToString(root);
  delete root;
  *xml = strdup(s.c_str());
  return mcclSuccess;
}

// out: [ringPrev, ringNext, flat, dtree, upA, nDownA, downA0, downA1, downA2..(pad to 8), upB, nDownB, downB0.. (pad to 8)]
// Layout: out[0..3] header, out[4]=upA, out[5]=nDownA, out[6..6+cap) children A, then upB, nDownB, children B.
mcclResult_t mcclDbgSyntheticChannel(int n, int rank, int cuda, int forceDtree, int* out, int cap) {
  TopoSystem sys;
  TopoGraph graphs[mcclNumAlgos];
  if (forceDtree) setenv("MCCL_DTREE", "1", 1);
  mcclResult_t rc = syntheticPlan(n, cuda != 0, false, &sys, graphs, nullptr);
  Channel ch;
  if (rc == mcclSuccess) rc = topoConnect(sys, graphs[mcclAlgoRing], graphs[mcclAlgoTree], rank, &ch);
  if (forceDtree) unsetenv("MCCL_DTREE");
  MCCLCHECK(rc);
  const int need = 4 + 2 * (2 + cap);
  for (int i = 0; i < need; ++i) out[i] = -1;
  out[0] = ch.ring.prev; out[1] = ch.ring.next; out[2] = ch.flatTree; out[3] = ch.dtree;
  int* a = out + 4;
  a[0] = ch.tree.up; a[1] = (int)ch.tree.down.size();
  for (int k = 0; k < (int)ch.tree.down.size() && k < cap; ++k) a[2 + k] = ch.tree.down[k];
  int* b = a + 2 + cap;
  b[0] = ch.treeB.up; b[1] = (int)ch.treeB.down.size();
  for (int k = 0; k < (int)ch.treeB.down.size() && k < cap; ++k) b[2 + k] = ch.treeB.down[k];
  return mcclSuccess;
}

mcclResult_t mcclDbgTunerPick(int n, int cuda, int nvls, size_t bytes, int coll, int dtop, const char* algoList, int* algo,
                              float* timesUs) {
  TopoSystem sys;
  TopoGraph graphs[mcclNumAlgos];
  TunerModel tuner;
  MCCLCHECK(syntheticPlan(n, cuda != 0, nvls != 0, &sys, graphs, &tuner));
  static const char* const names[] = {"ring", "tree", "oneshot", "twoshot", "nvls"};
  int enabled[mcclNumAlgos];
  MCCLCHECK(parseList(algoList, names, mcclNumAlgos, enabled));
  const int dt = dtop & 0xff, op = (dtop >> 8) & 0xff;
  if (timesUs) for (int a = 0; a < mcclNumAlgos; ++a) tunerAlgoTime(tuner, a, coll, n, bytes, &timesUs[a]);
  return tunerPick(tuner, coll, n, bytes, dt, op, enabled, cuda != 0, algo);
}

mcclResult_t mcclDbgParseList(const char* s, int* enabled) {
  static const char* const names[] = {"ring", "tree", "oneshot", "twoshot", "nvls"};
  return parseList(s, names, mcclNumAlgos, enabled);
}

mcclResult_t mcclDbgHostReduce(void* dst, const void* src, size_t count, int dt, int op) {
  return hostReduce(dst, src, count, (mcclDataType_t)dt, (mcclRedOp_t)op);
}
mcclResult_t mcclDbgHostScale(void* buf, size_t count, int dt, int n) { return hostScale(buf, count, (mcclDataType_t)dt, n); }

mcclResult_t mcclDbgXmlRoundTrip(const char* text, char** out) {
  XmlNode* root = xmlParse(text);
  if (root == nullptr) return mcclInvalidArgument;
  XmlNode* copy = xmlAddNode(nullptr, root->name.c_str());
  xmlFuse(copy, root);
  std::string s = xmlToString(copy);
  delete root;
  delete copy;
  *out = strdup(s.c_str());
  return mcclSuccess;
}

int64_t mcclDbgParam(const char* env, int64_t deflt) { return loadParam(env, deflt); }

// The cut of a Send/Recv message over channels: out3 = {channels, bytes per channel, bytes per chunk}.
void mcclDbgP2pSplit(uint64_t bytes, uint64_t slotBytes, int n, uint64_t* out3) {
  const P2pSplit sp = p2pSplit(bytes, slotBytes, n);
  out3[0] = (uint64_t)sp.channels; out3[1] = sp.per; out3[2] = sp.half;
}
int mcclDbgP2pChannels(int n) { return p2pChannels(n); }

// Path table of a synthetic cuda system with the (cutA, cutB) NVLink pair severed.
// types[a*n+b] = path type, hops[a*n+b] = hop count.
mcclResult_t mcclDbgPaths(int n, int cutA, int* cutBAndTypes, int* hops) {
  const int cutB = cutBAndTypes[0];
  TopoSystem sys;
  TopoGraph graphs[mcclNumAlgos];
  MCCLCHECK(syntheticPlan(n, true, false, &sys, graphs, nullptr, cutA, cutB));
  for (int a = 0; a < n; ++a)
    for (int b = 0; b < n; ++b) {
      cutBAndTypes[a * n + b] = sys.nodes[a].paths[b].type;
      hops[a * n + b] = sys.nodes[a].paths[b].count;
    }
  return mcclSuccess;
}

}  // extern "C"
