// Topology model, path search, per-algorithm search, trees, channel connect, tuner and XML dump.
//
// A node is one rank: a GPU of the NVSwitch box (cuda transport) or a process reachable over TCP (tcp
// transport).  Links are what discovery found: NVLink through NVSwitch between GPUs with peer access,
// PCIe between GPUs of one host without it, NET between hosts or for the CPU path.  The planner asks five
// questions of it (one per algorithm): is it viable, at what bandwidth, with how many channels.
//
// Parity with the reference: topology model src/graph/topo.h:12-75 / topo.cc:9-158, widest paths
// src/graph/paths.cc:13-60, per-algo search src/graph/search.cc:9-77, double-binary trees
// src/graph/trees.cc:7-53, channel connect src/graph/connect.cc:10-94, cost model
// src/graph/tuning.cc:12-88, XML src/graph/xml.cc:12-154, discovery src/graph/discover.cc:23-174.
#pragma once

#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "../core/core.h"

namespace mccl {

enum LinkType { LINK_LOC = 0, LINK_NVL = 1, LINK_PCI = 2, LINK_NET = 3 };
// Path quality, low = best: same device, one NVLink hop through the switch, relayed over another GPU,
// PCIe, network, unreachable.
enum PathType { PATH_LOC = 0, PATH_NVL = 1, PATH_NVL_HOP = 2, PATH_PCI = 3, PATH_NET = 4, PATH_DIS = 5 };
const char* linkTypeStr(int t);
const char* pathTypeStr(int t);

struct TopoLink {
  int   type = LINK_LOC;
  float bw = 0.f;         // GB/s per direction used by the cost model
  float measured = 0.f;   // GB/s from the calibration probe, 0 if not probed
  float latencyUs = 0.f;  // one-way flag latency from calibration, 0 if not probed
  int   remote = -1;
};

struct TopoPath {
  int   count = 0;        // hops
  float bw = 0.f;         // bottleneck
  int   type = PATH_DIS;
  int   firstHop = -1;
};

struct TopoNode {
  int         rank = -1;
  uint64_t    hostHash = 0;
  int         device = -1;      // cuda ordinal, -1 on the tcp transport
  int         smCount = 0;
  int         cc = 0;           // compute capability * 10 (100 = sm_100)
  uint64_t    hbmGiB = 0;
  int         multicast = 0;
  uint32_t    ip = 0;           // data-plane IPv4 (host order)
  std::string busId;
  std::vector<TopoLink> links;
  std::vector<TopoPath> paths;
};

struct TopoSystem {
  std::vector<TopoNode> nodes;
  bool netAllToAll = false;     // every rank reaches every rank over TCP
  bool nvls = false;            // one multicast group can span every rank
};

// What each rank contributes to discovery (all-gathered over the bootstrap).
struct RankInfo {
  uint64_t hostHash;
  uint32_t ip;
  uint16_t dataPort;
  uint16_t pad;
  int32_t  device;       // -1: no GPU (tcp transport)
  int32_t  smCount;
  int32_t  cc;
  int32_t  multicast;
  int32_t  vmm;
  uint32_t peerMask;     // bit d set: this rank's GPU has peer access to cuda device d of the same host
  uint32_t atomicMask;   // bit d set: native atomics over that peer link
  uint64_t hbmBytes;
  uint64_t pidHash;
  char     busId[32];
};

float nvlinkTableBw();   // GB/s per direction assumed for an unmeasured NVLink 5 port (MCCL_NVL_BW)
float pciTableBw();
float netTableBw();      // MCCL_LAN_BW

// Build the system from every rank's RankInfo.  Links: same host and peer access both ways -> NVL;
// same host without -> PCI; everything else (and every pair on the tcp transport) -> NET.
mcclResult_t topoGetSystem(const RankInfo* infos, int nRanks, bool cudaTransport, TopoSystem* out);
mcclResult_t topoComputePaths(TopoSystem* sys);

float topoMaxBw(const TopoSystem& sys);
float topoMinBw(const TopoSystem& sys);
float topoTotalBw(const TopoSystem& sys);
int   topoDegree(const TopoSystem& sys, int rank);        // number of NVL neighbours
bool  topoDirectLink(const TopoSystem& sys, int a, int b, float* bw, int* type);
bool  topoNvlAllToAll(const TopoSystem& sys);
float topoTreeBottleneckBw(const TopoSystem& sys, int root, std::vector<int>* parentOut);
float nodeScore(const TopoNode& n);

struct TopoGraph {
  int   algo = mcclAlgoRing;
  bool  viable = false;
  std::vector<int> order;   // ring: the cycle; tree: hub first; others: rank order
  float bw = 0.f;           // GB/s per direction available to the algorithm
  float latencyUs = 0.f;    // per-step latency
  int   nChannels = 1;      // CTAs (cuda) or concurrent legs (tcp)
};

mcclResult_t topoCompute(const TopoSystem& sys, int algo, TopoGraph* out);

// Double-binary trees over positions 0..n-1 (-1 = none).  Tree 0 is the lowest-set-bit binary tree;
// tree 1 is its shift (odd n) or mirror (even n), so a rank that is interior in one is a leaf in the other.
void getBtree(int n, int rank, int* up, int* down0, int* down1);
void getDtree(int n, int rank, int* up0, int* d00, int* d01, int* up1, int* d10, int* d11);

struct RingView { int prev = -1, next = -1; std::vector<int> userRanks; };
struct TreeView { int up = -1; std::vector<int> down; };
struct Channel {
  RingView ring;
  TreeView tree, treeB;
  std::vector<int> treeParent;    // tree A's parent of every rank
  std::vector<int> treeParentB;   // tree B's parent of every rank (dtree only)
  bool flatTree = false;          // depth-1 star
  bool dtree = false;             // tree + treeB are a double-binary tree
};
MCCL_PARAM(DtreeMinRanks);

mcclResult_t topoConnect(const TopoSystem& sys, const TopoGraph& ring, const TopoGraph& tree, int rank, Channel* out);

// ---- tuner ------------------------------------------------------------------------------------------
struct TunerModel {
  // time_us = alphaUs[algo] + stepUs[algo] * steps(algo, n) + bytes * trafficFactor(algo, coll, n) / (1000 * bw[algo])
  float alphaUs[mcclNumAlgos];
  float stepUs[mcclNumAlgos];
  float bw[mcclNumAlgos];
  bool  viable[mcclNumAlgos];
  size_t oneShotMaxBytes;   // one-shot scratch slot size (cuda) / MCCL_DIRECT_MAX_BYTES (tcp)
  int    oneShotMaxRanks;
  bool   cuda;              // constants describe the cuda transport's kernels
  bool   measured = false;  // alpha / bandwidth of the switch-era algorithms come from a calibration (now or cached)
};
// Where a calibration is kept between runs: MCCL_TUNER_CACHE, else ~/.cache/mccl_b200/tuner-<ranks>x<gpu>.txt.
std::string tunerCachePath(int nRanks, const char* gpuName);

mcclResult_t tunerInit(const TopoSystem& sys, const TopoGraph graphs[mcclNumAlgos], bool cudaTransport, TunerModel* out);
// Overrides from MCCL_TUNER_CACHE (a file of "algo alpha_us step_us bw_gbs" lines) if set.
mcclResult_t tunerLoadCache(TunerModel* m, const char* path);
mcclResult_t tunerSaveCache(const TunerModel& m, const char* path);
int          algoSteps(int algo, int n);
double       algoTraffic(int algo, int coll, int n);   // bytes on the busiest direction per payload byte
mcclResult_t tunerAlgoTime(const TunerModel& m, int algo, int coll, int n, size_t bytes, float* us);
// Whether `algo` can execute (coll, dt, op) at all on this transport (e.g. NVLS has no prod).
bool         algoSupports(int algo, int coll, int dt, int op, bool cudaTransport);
bool         nvlsAvgExact(int dt, int op, int n);       // NVLS can serve this average without rounding twice
mcclResult_t tunerPick(const TunerModel& m, int coll, int n, size_t bytes, int dt, int op, const int enabled[mcclNumAlgos],
                       bool cudaTransport, int* algo);
// "ring,tree" allow-list or "^ring" deny-list -> mask.
mcclResult_t parseList(const char* str, const char* const names[], int n, int* enabled);
mcclResult_t getEnabledAlgos(int enabled[mcclNumAlgos]);

// ---- XML --------------------------------------------------------------------------------------------
struct XmlNode {
  std::string name;
  std::vector<std::pair<std::string, std::string>> attrs;
  std::vector<XmlNode*> subs;
  ~XmlNode();
};
XmlNode*     xmlAddNode(XmlNode* parent, const char* name);
void         xmlSetAttr(XmlNode* n, const char* key, const std::string& value);
void         xmlSetAttrInt(XmlNode* n, const char* key, long long v);
void         xmlSetAttrFloat(XmlNode* n, const char* key, double v);
const char*  xmlGetAttr(const XmlNode* n, const char* key);
std::string  xmlToString(const XmlNode* root);
// Parse what xmlToString wrote (elements and attributes only).
XmlNode*     xmlParse(const std::string& text);
XmlNode*     topoToXml(const TopoSystem& sys, const TopoGraph* graphs, int nGraphs, const TunerModel* tuner);
mcclResult_t topoDumpXmlToFile(const TopoSystem& sys, const TopoGraph* graphs, int nGraphs, const TunerModel* tuner, const char* path);
// Merge `src` into `dst`: nodes are matched by their "rank"/"peer" attribute, new ones appended.
void         xmlFuse(XmlNode* dst, const XmlNode* src);

}  // namespace mccl
