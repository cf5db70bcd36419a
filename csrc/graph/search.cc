// Per-algorithm search: can this algorithm run on the discovered system, at what bandwidth, how wide.
#include <algorithm>
#include <cmath>

#include "graph.h"

namespace mccl {

static float latencyOf(const TopoSystem& sys, int a, int b) {
  for (const TopoLink& l : sys.nodes[a].links)
    if (l.remote == b && l.latencyUs > 0.f) return l.latencyUs;
  int type = LINK_NET;
  topoDirectLink(sys, a, b, nullptr, &type);
  if (type == LINK_NVL) return (float)envDouble("MCCL_NVL_LATENCY_US", 1.2);
  if (type == LINK_PCI) return 3.0f;
  return (float)envDouble("MCCL_HOP_LATENCY_US", 50.0);
}

static void rankOrder(int n, std::vector<int>* order) {
  order->resize(n);
  for (int i = 0; i < n; ++i) (*order)[i] = i;
}

// Ring in rank order; viable when every consecutive pair is one hop.  Bandwidth = weakest link.
static void computeRing(const TopoSystem& sys, TopoGraph* g) {
  const int n = (int)sys.nodes.size();
  rankOrder(n, &g->order);
  g->viable = true;
  g->bw = 1e9f;
  g->latencyUs = 0.f;
  for (int i = 0; i < n && n > 1; ++i) {
    float bw = 0.f;
    const int a = g->order[i], b = g->order[(i + 1) % n];
    if (!topoDirectLink(sys, a, b, &bw, nullptr)) { g->viable = false; g->bw = 0.f; return; }
    g->bw = std::min(g->bw, bw);
    g->latencyUs = std::max(g->latencyUs, latencyOf(sys, a, b));
  }
}

// Tree: hub = best-connected node (NVL degree, then node score); bandwidth = bottleneck of the
// max-bottleneck spanning tree from it.
static void computeTree(const TopoSystem& sys, TopoGraph* g) {
  const int n = (int)sys.nodes.size();
  int hub = 0;
  for (int r = 1; r < n; ++r) {
    const int dr = topoDegree(sys, r), dh = topoDegree(sys, hub);
    if (dr > dh || (dr == dh && nodeScore(sys.nodes[r]) > nodeScore(sys.nodes[hub]))) hub = r;
  }
  g->order.clear();
  g->order.push_back(hub);
  for (int r = 0; r < n; ++r) if (r != hub) g->order.push_back(r);
  g->bw = topoTreeBottleneckBw(sys, hub, nullptr);
  g->viable = n == 1 || g->bw > 0.f;
  g->latencyUs = n > 1 ? latencyOf(sys, hub, g->order[1]) : 0.f;
}

// One-shot / two-shot: every rank talks to every rank directly.  On the cuda transport that needs peer
// access between all pairs; on tcp every pair must be one hop.
static void computeAllPairs(const TopoSystem& sys, TopoGraph* g, bool needNvl) {
  const int n = (int)sys.nodes.size();
  rankOrder(n, &g->order);
  g->viable = true;
  g->bw = 1e9f;
  g->latencyUs = 0.f;
  for (int a = 0; a < n; ++a)
    for (int b = 0; b < n; ++b) {
      if (a == b) continue;
      float bw = 0.f; int type = LINK_NET;
      if (!topoDirectLink(sys, a, b, &bw, &type) || (needNvl && type != LINK_NVL)) { g->viable = false; g->bw = 0.f; return; }
      g->bw = std::min(g->bw, bw);
      g->latencyUs = std::max(g->latencyUs, latencyOf(sys, a, b));
    }
}

mcclResult_t topoCompute(const TopoSystem& sys, int algo, TopoGraph* out) {
  if (out == nullptr || sys.nodes.empty()) MCCLFAIL(mcclInvalidArgument);
  *out = TopoGraph();
  out->algo = algo;
  const bool cuda = sys.nodes[0].device >= 0;
  switch (algo) {
    case mcclAlgoRing:    computeRing(sys, out); break;
    case mcclAlgoTree:    computeTree(sys, out); break;
    case mcclAlgoOneShot: computeAllPairs(sys, out, cuda); break;
    case mcclAlgoTwoShot: computeAllPairs(sys, out, cuda); out->viable = out->viable && cuda; break;
    case mcclAlgoNvls:
      computeAllPairs(sys, out, true);
      out->viable = out->viable && sys.nvls;
      break;
    default: MCCLFAIL(mcclInvalidArgument);
  }
  // Channels = CTAs a collective kernel may use on the cuda transport; concurrent legs on tcp.
  if (cuda) {
    const int sm = sys.nodes[0].smCount > 0 ? sys.nodes[0].smCount : 148;
    switch (algo) {
      case mcclAlgoRing: case mcclAlgoTree: out->nChannels = std::min(32, sm / 4); break;
      case mcclAlgoOneShot: out->nChannels = std::min(32, sm / 4); break;
      default: out->nChannels = std::min(64, sm / 2); break;
    }
  } else {
    out->nChannels = (algo == mcclAlgoRing || algo == mcclAlgoTree) ? 2 : 1;
  }
  if (!out->viable) out->nChannels = 0;
  return mcclSuccess;
}

}  // namespace mccl
