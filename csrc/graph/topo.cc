// Topology construction, queries and all-pairs widest paths.
#include <algorithm>
#include <cstring>

#include "graph.h"

namespace mccl {

const char* linkTypeStr(int t) {
  static const char* n[] = {"LOC", "NVL", "PCI", "NET"};
  return (t >= 0 && t < 4) ? n[t] : "?";
}
const char* pathTypeStr(int t) {
  static const char* n[] = {"LOC", "NVL", "NVL_HOP", "PCI", "NET", "DIS"};
  return (t >= 0 && t < 6) ? n[t] : "?";
}

float nvlinkTableBw() { return (float)envDouble("MCCL_NVL_BW", 900.0); }   // NVLink 5: 18 links, per direction
float pciTableBw()    { return (float)envDouble("MCCL_PCI_BW", 50.0); }
float netTableBw()    { return (float)envDouble("MCCL_LAN_BW", 1.0); }

float nodeScore(const TopoNode& n) {
  return 1000.f * (float)n.cc + 10.f * (float)n.smCount + (float)n.hbmGiB;
}

mcclResult_t topoGetSystem(const RankInfo* infos, int nRanks, bool cudaTransport, TopoSystem* out) {
  if (infos == nullptr || nRanks < 1 || out == nullptr) MCCLFAIL(mcclInvalidArgument);
  out->nodes.assign(nRanks, TopoNode());
  bool allMc = cudaTransport;
  bool oneHost = true;
  for (int r = 0; r < nRanks; ++r) {
    TopoNode& nd = out->nodes[r];
    const RankInfo& ri = infos[r];
    nd.rank = r;
    nd.hostHash = ri.hostHash;
    nd.device = cudaTransport ? ri.device : -1;
    nd.smCount = ri.smCount;
    nd.cc = ri.cc;
    nd.hbmGiB = ri.hbmBytes >> 30;
    nd.multicast = ri.multicast;
    nd.ip = ri.ip;
    nd.busId = std::string(ri.busId, strnlen(ri.busId, sizeof(ri.busId)));
    allMc = allMc && ri.multicast && ri.vmm;
    oneHost = oneHost && ri.hostHash == infos[0].hostHash;
  }
  for (int a = 0; a < nRanks; ++a) {
    for (int b = 0; b < nRanks; ++b) {
      if (a == b) continue;
      const RankInfo& ia = infos[a];
      const RankInfo& ib = infos[b];
      TopoLink l;
      l.remote = b;
      const bool sameHost = ia.hostHash == ib.hostHash;
      if (cudaTransport && sameHost && ia.device >= 0 && ib.device >= 0) {
        const bool peer = ia.device == ib.device ||
                          (((ia.peerMask >> ib.device) & 1u) && ((ib.peerMask >> ia.device) & 1u));
        l.type = peer ? LINK_NVL : LINK_PCI;
        l.bw = peer ? nvlinkTableBw() : pciTableBw();
      } else {
        l.type = LINK_NET;
        l.bw = netTableBw();
      }
      out->nodes[a].links.push_back(l);
    }
  }
  out->netAllToAll = true;  // the bootstrap reached every rank, so TCP reaches every rank
  out->nvls = allMc && oneHost && nRanks > 1 && topoNvlAllToAll(*out);
  return mcclSuccess;
}

static int linkPathType(int linkType, bool firstHop) {
  switch (linkType) {
    case LINK_NVL: return firstHop ? PATH_NVL : PATH_NVL_HOP;
    case LINK_PCI: return PATH_PCI;
    case LINK_NET: return PATH_NET;
    default:       return PATH_LOC;
  }
}

static bool betterPath(const TopoPath& a, const TopoPath& b) {
  if (a.type != b.type) return a.type < b.type;
  if (a.bw != b.bw) return a.bw > b.bw;
  return a.count < b.count;
}

mcclResult_t topoComputePaths(TopoSystem* sys) {
  const int n = (int)sys->nodes.size();
  for (int s = 0; s < n; ++s) {
    std::vector<TopoPath>& p = sys->nodes[s].paths;
    p.assign(n, TopoPath());
    p[s].count = 0; p[s].bw = 1e9f; p[s].type = PATH_LOC; p[s].firstHop = s;
    // Relaxation over NVL links only (relaying through a GPU makes sense on NVLink, never over PCIe/NET).
    for (int round = 0; round < n; ++round) {
      bool changed = false;
      for (int u = 0; u < n; ++u) {
        if (p[u].type == PATH_DIS) continue;
        for (const TopoLink& l : sys->nodes[u].links) {
          if (l.type != LINK_NVL) continue;
          TopoPath cand;
          cand.count = p[u].count + 1;
          cand.bw = std::min(p[u].bw, l.bw);
          cand.type = std::max(p[u].type, linkPathType(l.type, p[u].count == 0));
          if (cand.count > 1 && cand.type < PATH_NVL_HOP) cand.type = PATH_NVL_HOP;
          cand.firstHop = (u == s) ? l.remote : p[u].firstHop;
          if (betterPath(cand, p[l.remote])) { p[l.remote] = cand; changed = true; }
        }
      }
      if (!changed) break;
    }
    // One-hop PCI / NET candidates.
    for (const TopoLink& l : sys->nodes[s].links) {
      if (l.type == LINK_NVL) continue;
      TopoPath cand;
      cand.count = 1; cand.bw = l.bw; cand.type = linkPathType(l.type, true); cand.firstHop = l.remote;
      if (betterPath(cand, p[l.remote])) p[l.remote] = cand;
    }
  }
  return mcclSuccess;
}

float topoMaxBw(const TopoSystem& sys) {
  float m = 0.f;
  for (auto& nd : sys.nodes) for (auto& l : nd.links) m = std::max(m, l.bw);
  return m;
}
float topoMinBw(const TopoSystem& sys) {
  float m = 0.f; bool any = false;
  for (auto& nd : sys.nodes) for (auto& l : nd.links) { m = any ? std::min(m, l.bw) : l.bw; any = true; }
  return m;
}
float topoTotalBw(const TopoSystem& sys) {
  float t = 0.f;
  for (auto& nd : sys.nodes) for (auto& l : nd.links) t += l.bw;
  return t;
}
int topoDegree(const TopoSystem& sys, int rank) {
  int d = 0;
  for (auto& l : sys.nodes[rank].links) d += l.type == LINK_NVL;
  return d;
}

bool topoDirectLink(const TopoSystem& sys, int a, int b, float* bw, int* type) {
  if (a == b) { if (bw) *bw = 1e9f; if (type) *type = LINK_LOC; return true; }
  const TopoLink* best = nullptr;
  for (const TopoLink& l : sys.nodes[a].links) {
    if (l.remote != b) continue;
    if (best == nullptr || l.type < best->type || (l.type == best->type && l.bw > best->bw)) best = &l;
  }
  if (best == nullptr) return false;
  if (bw) *bw = best->bw;
  if (type) *type = best->type;
  return true;
}

bool topoNvlAllToAll(const TopoSystem& sys) {
  const int n = (int)sys.nodes.size();
  for (int a = 0; a < n; ++a)
    for (int b = 0; b < n; ++b) {
      int t = LINK_NET;
      if (a != b && (!topoDirectLink(sys, a, b, nullptr, &t) || t != LINK_NVL)) return false;
    }
  return n > 1;
}

// Prim's algorithm maximising the bottleneck edge: the spanning tree whose weakest link is strongest.
float topoTreeBottleneckBw(const TopoSystem& sys, int root, std::vector<int>* parentOut) {
  const int n = (int)sys.nodes.size();
  std::vector<float> key(n, -1.f);
  std::vector<int> parent(n, -1);
  std::vector<bool> in(n, false);
  key[root] = 1e9f;
  float bottleneck = 1e9f;
  for (int it = 0; it < n; ++it) {
    int u = -1;
    for (int v = 0; v < n; ++v) if (!in[v] && key[v] >= 0.f && (u < 0 || key[v] > key[u])) u = v;
    if (u < 0) { bottleneck = 0.f; break; }   // disconnected
    in[u] = true;
    if (u != root) bottleneck = std::min(bottleneck, key[u]);
    for (const TopoLink& l : sys.nodes[u].links)
      if (!in[l.remote] && l.bw > key[l.remote]) { key[l.remote] = l.bw; parent[l.remote] = u; }
  }
  if (parentOut) *parentOut = parent;
  return n > 1 ? bottleneck : 1e9f;
}

}  // namespace mccl
