// Tree all-reduce: one chain-tree per local rank of a (virtual) node.
//
// The data is cut into gpn = world / nnodes parts; part t belongs to tree t,
// whose root is local rank t of every node.  Inside a node the part is reduced
// along a chain that ends at the root (odd trees walk the node the other way
// round), the roots of all nodes exchange their partial sums and add them in
// node order, and the result is broadcast back down the chain.
//
// Same shape as the reference's csrc/all_reduce_tree.cu:26-143, which however is
// only correct for exactly two nodes (its root's send peer is itself when there
// is one node, :49) and is not reachable from Python; here nnodes may be any
// divisor of world, including 1.
//
// grid: gpn * lanes blocks; block -> (tree = bid / lanes, lane = bid % lanes)
// scratch half: up area [V] + down area [V] + root-exchange area [nnodes][V]
#pragma once
#include "coll_args.h"
#include "schedule.h"

namespace penny {

PK_HD size_t tree_scratch_bytes(size_t n, int elem_size, int nnodes) {
  return 2 * (size_t)(2 + nnodes) * vecs_for(n, elem_size) * 16;
}

template <typename T>
struct TreeAllReduce {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const int N = c.world;
    const int nnodes = a.nnodes;
    const int gpn = N / nnodes;
    const int node = rank / gpn;
    const int local = rank % gpn;
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t V = ceil_div(a.n, E);
    const int lanes = b.nblocks / gpn;
    const int tree = b.bid / lanes;
    const int lane = b.bid % lanes;
    const Span part = split_span(V, gpn, tree);
    const size_t len = part.end - part.begin;
    const size_t up_off = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const size_t down_off = up_off + V * 16;
    const size_t x_off = up_off + 2 * V * 16;
    const u64 f_up = flag_value(seq, 1), f_x = flag_value(seq, 2), f_down = flag_value(seq, 3);
    const size_t stride = (size_t)lanes * b.nthreads;
    const size_t first = (size_t)lane * b.nthreads;

    const int j = tree_pos_of(gpn, tree, local);  // 0 = far leaf, gpn-1 = root
    const bool is_root = (j == gpn - 1);
    const int up_peer = is_root ? -1 : node * gpn + tree_local_at(gpn, tree, j + 1);
    const int down_peer = (j == 0) ? -1 : node * gpn + tree_local_at(gpn, tree, j - 1);

    // ---- reduce towards the root ----
    if (j > 0) {
      PK_FOR_THREADS(b, tid) {
        if (tid == 0 && !wait_peer(c, rank, down_peer, CH_DATA, b, f_up, ST_TIMEOUT_DATA))
          s_abort = 1;
      }
      PK_SYNC(b);
    }
    if (!s_abort) {
      PK_FOR_THREADS(b, tid) {
        for (size_t i = first + tid; i < len; i += stride) {
          const size_t v = part.begin + i;
          V16 x = load_user_vec<T>(in, v, a.n);
          if (j > 0) {
            float acc[E];
            unpack_set<T>(ld16(c.heap[rank] + up_off + v * 16), acc);
            unpack_add<T>(x, acc);
            x = pack<T>(acc);
          }
          if (!is_root) {
            st16(c.heap[up_peer] + up_off + v * 16, x);
          } else {
            // node partial: keep a copy in my own exchange row and push it to the other roots
            for (int m = 0; m < nnodes; ++m)
              st16(c.heap[m * gpn + local] + x_off + ((size_t)node * V + v) * 16, x);
          }
        }
      }
      PK_SYNC(b);
      if (!is_root) {
        PK_FOR_THREADS(b, tid) {
          if (tid == 0) signal_peer(c, rank, up_peer, CH_DATA, b, f_up);
        }
      } else {
        // ---- roots exchange and add in node order ----
        PK_FOR_THREADS(b, tid) {
          if (tid < nnodes && tid != node) signal_peer(c, rank, tid * gpn + local, CH_DATA, b, f_x);
        }
        PK_FOR_THREADS(b, tid) {
          if (tid < nnodes && tid != node &&
              !wait_peer(c, rank, tid * gpn + local, CH_DATA, b, f_x, ST_TIMEOUT_DATA))
            s_abort = 1;
        }
        PK_SYNC(b);
        if (!s_abort) {
          PK_FOR_THREADS(b, tid) {
            for (size_t i = first + tid; i < len; i += stride) {
              const size_t v = part.begin + i;
              float acc[E];
#pragma unroll
              for (size_t q = 0; q < E; ++q) acc[q] = 0.f;
              for (int m = 0; m < nnodes; ++m)
                unpack_add<T>(ld16(c.heap[rank] + x_off + ((size_t)m * V + v) * 16), acc);
              const V16 r = pack<T>(acc);
              store_user_vec<T>(out, v, a.n, r);
              if (down_peer >= 0) st16(c.heap[down_peer] + down_off + v * 16, r);
            }
          }
          PK_SYNC(b);
          if (down_peer >= 0) {
            PK_FOR_THREADS(b, tid) {
              if (tid == 0) signal_peer(c, rank, down_peer, CH_DATA, b, f_down);
            }
          }
        }
      }
    }
    // ---- broadcast back down the chain ----
    if (!is_root && !s_abort) {
      PK_FOR_THREADS(b, tid) {
        if (tid == 0 && !wait_peer(c, rank, up_peer, CH_DATA, b, f_down, ST_TIMEOUT_DATA))
          s_abort = 1;
      }
      PK_SYNC(b);
      if (!s_abort) {
        PK_FOR_THREADS(b, tid) {
          for (size_t i = first + tid; i < len; i += stride) {
            const size_t v = part.begin + i;
            const V16 r = ld16(c.heap[rank] + down_off + v * 16);
            store_user_vec<T>(out, v, a.n, r);
            if (down_peer >= 0) st16(c.heap[down_peer] + down_off + v * 16, r);
          }
        }
        PK_SYNC(b);
        if (down_peer >= 0) {
          PK_FOR_THREADS(b, tid) {
            if (tid == 0) signal_peer(c, rank, down_peer, CH_DATA, b, f_down);
          }
        }
      }
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<TreeAllReduce<T>, CollArgs>(c, rank, a, b);
  }
};

}  // namespace penny
