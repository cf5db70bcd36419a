// Double-binary trees.  Positions 0..n-1; -1 means "none".
//
// Tree 0: a rank's level is its lowest set bit b.  Its parent is the rank one level up that covers it,
// (rank with bit b cleared) | 2b, or rank - b when that falls beyond n.  Its children sit b/2 below and
// above; the upper child's distance is halved until it lands inside [0, n).  Position 0 has no set bit: it
// is the root, with the highest power of two below n as its only child.
// Tree 1 re-labels tree 0 so that interior ranks become leaves: shift by one for odd n, mirror for even n.
// Parity: src/graph/trees.cc:7-53 of the reference (same construction as NCCL's).
#include "graph.h"

namespace mccl {

void getBtree(int n, int rank, int* up, int* down0, int* down1) {
  *up = *down0 = *down1 = -1;
  if (n <= 1) return;
  int b = 1;
  while (b < n && !(rank & b)) b <<= 1;   // lowest set bit of rank, or the first power of two >= n for rank 0
  if (rank == 0) {
    *down1 = b >> 1;
    return;
  }
  int parent = (rank & ~b) | (b << 1);
  if (parent >= n) parent = rank & ~b;
  *up = parent;
  int step = b >> 1;
  if (step == 0) return;                  // odd ranks are leaves
  *down0 = rank - step;
  int hi = rank + step;
  while (hi >= n) {
    step >>= 1;
    if (step == 0) { hi = -1; break; }
    hi = rank + step;
  }
  *down1 = hi;
}

void getDtree(int n, int rank, int* up0, int* d00, int* d01, int* up1, int* d10, int* d11) {
  getBtree(n, rank, up0, d00, d01);
  if (n % 2 == 1) {
    // shift: tree 1 of rank r is tree 0 of r-1, every answer moved up by one
    const int shifted = (rank - 1 + n) % n;
    int u, a, b;
    getBtree(n, shifted, &u, &a, &b);
    *up1 = u < 0 ? -1 : (u + 1) % n;
    *d10 = a < 0 ? -1 : (a + 1) % n;
    *d11 = b < 0 ? -1 : (b + 1) % n;
  } else {
    // mirror: tree 1 of rank r is tree 0 of n-1-r, every answer reflected (children swap sides)
    int u, a, b;
    getBtree(n, n - 1 - rank, &u, &a, &b);
    *up1 = u < 0 ? -1 : n - 1 - u;
    *d10 = b < 0 ? -1 : n - 1 - b;
    *d11 = a < 0 ? -1 : n - 1 - a;
  }
}

}  // namespace mccl
