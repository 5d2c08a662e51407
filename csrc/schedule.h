// Schedule math shared by kernels, the host simulator, the CPU (gloo) backend
// and the ring visualiser: who sends which chunk to whom at which step.
//
// Everything here is a pure function of (world, nnodes, route, rank, step), so
// the permutation / coverage properties can be enumerated on the CPU.  The
// reference finds its node-aware ring position by walking a successor function
// inside the kernel (csrc/all_reduce_ring_standard.cu:34-81) and replays it in
// extra/ring_visualize.py; here the order is closed-form and tabulated once per
// launch.
//
// "Nodes" are virtual on a single NVSwitch box: nnodes groups of world/nnodes
// consecutive ranks.  They only shape the schedules (double ring, tree,
// node-aware ring) so that the multi-node algorithms keep their semantics.
#pragma once
#include "pk.h"

namespace penny {

constexpr int kMaxRoutes = 8;

// Contiguous split of V items into `parts` pieces of ceil(V/parts) (the last
// ones may be short or empty).
struct Span {
  size_t begin, end;
};
PK_HD Span split_span(size_t V, int parts, int i) {
  size_t per = ceil_div(V, (size_t)parts);
  size_t b = per * (size_t)i;
  size_t e = b + per;
  if (b > V) b = V;
  if (e > V) e = V;
  return Span{b, e};
}

PK_HD int gcd_int(int a, int b) {
  while (b) {
    int t = a % b;
    a = b;
    b = t;
  }
  return a;
}

// Number of distinct stride rings on `world` ranks: strides coprime to world.
PK_HD int num_ring_strides(int world) {
  int n = 0;
  for (int s = 1; s < world; ++s)
    if (gcd_int(s, world) == 1) ++n;
  return n > 0 ? n : 1;
}
// Stride of route q.  Routes alternate direction first (1, world-1, 3, world-3,
// ...) so that two routes already use both directions of every NVLink port.
PK_HD int ring_stride(int world, int route) {
  if (world <= 2) return 1;
  int n = num_ring_strides(world);
  int want = (route % n) / 2;  // want-th unit from below
  bool rev = (route % n) & 1;
  int seen = 0;
  for (int s = 1; s < world; ++s) {
    if (gcd_int(s, world) != 1) continue;
    if (seen == want) return rev ? world - s : s;
    ++seen;
  }
  return 1;
}

// Rank at ring position pos of route `route`.
//   nnodes == 1 : stride ring, pos -> (pos * stride) mod world
//   nnodes  > 1 : node-aware ring.  Ring pair k = route/2 enters every node at
//                 local rank 2k+1, walks the node upwards (wrapping) and leaves
//                 it from local rank 2k, so different pairs cross nodes on
//                 different ranks; odd routes run the same ring backwards.
PK_HD int ring_rank_at(int world, int nnodes, int route, int pos) {
  if (nnodes <= 1) {
    int s = ring_stride(world, route);
    return (int)(((long long)pos * s) % world);
  }
  int gpn = world / nnodes;
  int k = route / 2;
  if (route & 1) pos = (world - pos) % world;
  int node = pos / gpn;
  int j = pos % gpn;
  return node * gpn + (2 * k + 1 + j) % gpn;
}
PK_HD int ring_pos_of(int world, int nnodes, int route, int rank) {
  for (int p = 0; p < world; ++p)
    if (ring_rank_at(world, nnodes, route, p) == rank) return p;
  return -1;
}

// Ring reduce-scatter, step s in [0, n-1): the rank at position p sends chunk
// (p - s) and receives (and reduces into) chunk (p - s - 1).  After n-1 steps
// position p holds the finished chunk (p + 1).
PK_HD int ring_rs_send_chunk(int n, int pos, int s) { return ((pos - s) % n + n) % n; }
PK_HD int ring_rs_recv_chunk(int n, int pos, int s) { return ((pos - s - 1) % n + n) % n; }
// Ring all-gather, step s in [0, n-1): sends chunk (p + 1 - s), receives (p - s).
PK_HD int ring_ag_send_chunk(int n, int pos, int s) { return ((pos + 1 - s) % n + n) % n; }
PK_HD int ring_ag_recv_chunk(int n, int pos, int s) { return ((pos - s) % n + n) % n; }

// Tree (chain-tree) schedule.  One tree per local rank t (root = local rank t),
// odd trees walk the node in the opposite direction.  chain position j:
// 0 = far leaf, gpn-1 = root.
PK_HD int tree_local_at(int gpn, int tree, int j) {
  int dir = (tree & 1) ? -1 : 1;
  int v = tree + dir * (gpn - 1 - j);
  return ((v % gpn) + gpn) % gpn;
}
PK_HD int tree_pos_of(int gpn, int tree, int local) {
  for (int j = 0; j < gpn; ++j)
    if (tree_local_at(gpn, tree, j) == local) return j;
  return -1;
}

// Two-level ("double ring") grouping: column group = same local rank on every
// node (size nnodes), row group = the ranks of one node (size gpn).
PK_HD int column_member(int world, int nnodes, int rank, int i) {
  int gpn = world / nnodes;
  return (rank % gpn) + i * gpn;
}
PK_HD int row_member(int world, int nnodes, int rank, int i) {
  int gpn = world / nnodes;
  return (rank / gpn) * gpn + i;
}

}  // namespace penny
