// Turn the ring and tree search results into one rank's channel: ring neighbours, tree parent/children.
// Tree shape: a double-binary tree when every pair has its own NVLink path (always so on the cuda
// transport through NVSwitch), when MCCL_DTREE=1, or above MCCL_DTREE_MIN_RANKS ranks; otherwise the
// max-bottleneck spanning tree from the hub, which on a uniform network is the depth-1 star.
#include <algorithm>

#include "graph.h"

namespace mccl {

DEFINE_MCCL_PARAM(DtreeMinRanks, "DTREE_MIN_RANKS", 8);

mcclResult_t topoConnect(const TopoSystem& sys, const TopoGraph& ring, const TopoGraph& tree, int rank, Channel* out) {
  const int n = (int)sys.nodes.size();
  if (out == nullptr || rank < 0 || rank >= n) MCCLFAIL(mcclInvalidArgument);
  *out = Channel();

  // ---- ring: rotate the cycle so that userRanks[0] is this rank
  if ((int)ring.order.size() == n) {
    int pos = 0;
    for (int i = 0; i < n; ++i) if (ring.order[i] == rank) pos = i;
    out->ring.userRanks.resize(n);
    for (int i = 0; i < n; ++i) out->ring.userRanks[i] = ring.order[(pos + i) % n];
    out->ring.next = ring.order[(pos + 1) % n];
    out->ring.prev = ring.order[(pos + n - 1) % n];
  }
  if (n == 1) { out->treeParent.assign(1, -1); out->flatTree = true; return mcclSuccess; }

  // ---- tree
  if ((int)tree.order.size() != n) MCCLFAIL(mcclInternalError);
  const bool nvlMesh = topoNvlAllToAll(sys);
  const bool wantDtree = n > 2 && (envInt("MCCL_DTREE", 0) != 0 || nvlMesh || n > mcclParamDtreeMinRanks());
  out->treeParent.assign(n, -1);
  if (wantDtree) {
    out->dtree = true;
    out->treeParentB.assign(n, -1);
    // Positions index tree.order (hub first), so the hub is the root of tree A.
    for (int pos = 0; pos < n; ++pos) {
      int u0, a0, b0, u1, a1, b1;
      getDtree(n, pos, &u0, &a0, &b0, &u1, &a1, &b1);
      const int r = tree.order[pos];
      out->treeParent[r] = u0 < 0 ? -1 : tree.order[u0];
      out->treeParentB[r] = u1 < 0 ? -1 : tree.order[u1];
      if (r == rank) {
        out->tree.up = out->treeParent[r];
        out->treeB.up = out->treeParentB[r];
        if (a0 >= 0) out->tree.down.push_back(tree.order[a0]);
        if (b0 >= 0) out->tree.down.push_back(tree.order[b0]);
        if (a1 >= 0) out->treeB.down.push_back(tree.order[a1]);
        if (b1 >= 0) out->treeB.down.push_back(tree.order[b1]);
      }
    }
  } else {
    std::vector<int> parent;
    topoTreeBottleneckBw(sys, tree.order[0], &parent);
    // On a uniform mesh Prim attaches everything to the hub; make that explicit so ties never build chains.
    bool uniform = true;
    const float bw0 = topoMinBw(sys);
    for (auto& nd : sys.nodes) for (auto& l : nd.links) uniform = uniform && l.bw == bw0;
    if (uniform) for (int r = 0; r < n; ++r) parent[r] = (r == tree.order[0]) ? -1 : tree.order[0];
    out->treeParent = parent;
    out->tree.up = parent[rank];
    for (int r = 0; r < n; ++r) if (parent[r] == rank) out->tree.down.push_back(r);
    out->flatTree = true;
    for (int r = 0; r < n; ++r) if (parent[r] >= 0 && parent[r] != tree.order[0]) out->flatTree = false;
  }
  return mcclSuccess;
}

}  // namespace mccl
