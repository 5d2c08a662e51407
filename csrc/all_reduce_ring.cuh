// Ring all-reduce family: simple ring (chain), standard multi-route ring and
// the two-level "double ring" with credit flow control.
//
// Data moves by direct 16-byte stores into the next rank's heap followed by one
// release store of a step counter (CH_DATA); the receiver waits for the counter
// with a bounded spin.  The reference does the same hops with
// nvshmemx_putmem_signal(_nbi)_block + nvshmem_signal_wait_until:
//   chain        csrc/all_reduce_ring_simple.cu:14-80
//   ring         csrc/all_reduce_ring_standard.cu:13-148
//   double ring  csrc/all_reduce_double_ring.cu:11-143 (credits at :36,42,52)
// Differences that matter: any dtype with fp32 adds, ragged sizes, any world
// size, routes that really are different rings (stride rings on NVSwitch,
// node-aware rings for virtual nodes), and bounded waits.
#pragma once
#include "coll_args.h"
#include "schedule.h"

namespace penny {

// ---------------------------------------------------------------------------
// simple ring: the whole buffer is reduced along 0 -> 1 -> ... -> N-1, then the
// result travels N-1 -> 0 -> 1 -> ... -> N-2.
// scratch half: reduce area [V] + broadcast area [V]
// ---------------------------------------------------------------------------
PK_HD size_t ring_simple_scratch_bytes(size_t n, int elem_size, int) {
  return 4 * vecs_for(n, elem_size) * 16;
}

template <typename T>
struct RingSimple {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const int N = c.world;
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t V = ceil_div(a.n, E);
    const size_t red_off = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const size_t bc_off = red_off + V * 16;
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t first = (size_t)b.bid * b.nthreads;
    const int prev = (rank + N - 1) % N;
    const int next = (rank + 1) % N;
    const u64 f_red = flag_value(seq, 1), f_bc = flag_value(seq, 2);

    // reduce pass
    if (rank > 0) {
      PK_FOR_THREADS(b, tid) {
        if (tid == 0 && !wait_peer(c, rank, prev, CH_DATA, b, f_red, ST_TIMEOUT_DATA)) s_abort = 1;
      }
      PK_SYNC(b);
      if (s_abort) return;
    }
    PK_FOR_THREADS(b, tid) {
      for (size_t v = first + tid; v < V; v += stride) {
        V16 x = load_user_vec<T>(in, v, a.n);
        if (rank > 0) {
          float acc[E];
          unpack_set<T>(ld16(c.heap[rank] + red_off + v * 16), acc);
          unpack_add<T>(x, acc);
          x = pack<T>(acc);
        }
        if (rank < N - 1) {
          st16(c.heap[next] + red_off + v * 16, x);
        } else {
          store_user_vec<T>(out, v, a.n, x);
          st16(c.heap[next] + bc_off + v * 16, x);  // next == rank 0: start of the broadcast
        }
      }
    }
    PK_SYNC(b);
    PK_FOR_THREADS(b, tid) {
      if (tid == 0) signal_peer(c, rank, next, CH_DATA, b, rank < N - 1 ? f_red : f_bc);
    }
    if (rank == N - 1) return;
    // broadcast pass
    PK_FOR_THREADS(b, tid) {
      if (tid == 0 && !wait_peer(c, rank, prev, CH_DATA, b, f_bc, ST_TIMEOUT_DATA)) s_abort = 1;
    }
    PK_SYNC(b);
    if (s_abort) return;
    PK_FOR_THREADS(b, tid) {
      for (size_t v = first + tid; v < V; v += stride) {
        V16 x = ld16(c.heap[rank] + bc_off + v * 16);
        store_user_vec<T>(out, v, a.n, x);
        if (rank < N - 2) st16(c.heap[next] + bc_off + v * 16, x);
      }
    }
    if (rank < N - 2) {
      PK_SYNC(b);
      PK_FOR_THREADS(b, tid) {
        if (tid == 0) signal_peer(c, rank, next, CH_DATA, b, f_bc);
      }
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<RingSimple<T>, CollArgs>(c, rank, a, b);
  }
};

// ---------------------------------------------------------------------------
// one ring all-reduce over an ordered group of ranks; building block of the
// standard ring and of both phases of the double ring
// ---------------------------------------------------------------------------
struct RingGroup {
  int size;               // members
  int pos;                // my position
  int member[kMaxRanks];  // rank at each position
};

struct RingPlan {
  size_t seg_begin;  // first vector of the segment this ring works on
  size_t seg_len;    // vectors in the segment (split into group.size chunks)
  size_t recv_off;   // heap offset of the receive area
  bool single_slot;  // true: one chunk-sized slot guarded by credits
                     // false: RS area + AG area indexed by position in the segment
  int lane;          // this block's index among the blocks working on the segment
  int lanes;         // number of such blocks
  int step0;         // first flag step used by this ring inside the call
};

// Runs RS + AG.  src supplies this rank's contribution (may equal out).  Returns
// false after a timeout.  Uses flag steps step0+1 .. step0+2*(size-1).
template <typename T>
PK_DEV bool ring_allreduce_group(const CommCtx& c, int rank, const RingGroup& g, const RingPlan& p,
                                 const T* src, T* out, size_t n, const Blk& b, u64 seq,
                                 int& s_abort) {
  constexpr size_t E = 16 / sizeof(T);
  const int G = g.size;
  if (G <= 1) {
    if (src != out) {
      PK_FOR_THREADS(b, tid) {
        for (size_t j = (size_t)p.lane * b.nthreads + tid; j < p.seg_len;
             j += (size_t)p.lanes * b.nthreads)
          store_user_vec<T>(out, p.seg_begin + j, n, load_user_vec<T>(src, p.seg_begin + j, n));
      }
      PK_SYNC(b);
    }
    return true;
  }
  const int next = g.member[(g.pos + 1) % G];
  const int prev = g.member[(g.pos + G - 1) % G];
  const size_t stride = (size_t)p.lanes * b.nthreads;
  const size_t first = (size_t)p.lane * b.nthreads;
  const int steps = 2 * (G - 1);

  for (int s = 0; s < steps; ++s) {
    const bool rs = s < G - 1;
    const int ss = rs ? s : s - (G - 1);
    const int send_chunk = rs ? ring_rs_send_chunk(G, g.pos, ss) : ring_ag_send_chunk(G, g.pos, ss);
    const int recv_chunk = rs ? ring_rs_recv_chunk(G, g.pos, ss) : ring_ag_recv_chunk(G, g.pos, ss);
    const Span sc = split_span(p.seg_len, G, send_chunk);
    const Span rc = split_span(p.seg_len, G, recv_chunk);
    // where the data of this step lands in the receiver's heap
    const size_t send_base =
        p.single_slot ? p.recv_off : p.recv_off + ((rs ? 0 : p.seg_len) + sc.begin) * 16;
    const size_t recv_base =
        p.single_slot ? p.recv_off : p.recv_off + ((rs ? 0 : p.seg_len) + rc.begin) * 16;
    const u64 fv = flag_value(seq, p.step0 + s + 1);

    if (p.single_slot && s > 0) {
      // the slot on `next` is free once it consumed the previous step
      PK_FOR_THREADS(b, tid) {
        if (tid == 0 && !wait_peer(c, rank, next, CH_CREDIT, b, flag_value(seq, p.step0 + s),
                                   ST_TIMEOUT_CREDIT))
          s_abort = 1;
      }
      PK_SYNC(b);
      if (s_abort) return false;
    }
    // send: step 0 sends the raw contribution, later steps send what `out` holds
    const T* from = (s == 0) ? src : out;
    PK_FOR_THREADS(b, tid) {
      for (size_t j = first + tid; j < sc.end - sc.begin; j += stride) {
        V16 x = load_user_vec<T>(from, p.seg_begin + sc.begin + j, n);
        st16(c.heap[next] + send_base + j * 16, x);
      }
    }
    PK_SYNC(b);
    PK_FOR_THREADS(b, tid) {
      if (tid == 0) signal_peer(c, rank, next, CH_DATA, b, fv);
    }
    // receive
    PK_FOR_THREADS(b, tid) {
      if (tid == 0 && !wait_peer(c, rank, prev, CH_DATA, b, fv, ST_TIMEOUT_DATA)) s_abort = 1;
    }
    PK_SYNC(b);
    if (s_abort) return false;
    PK_FOR_THREADS(b, tid) {
      for (size_t j = first + tid; j < rc.end - rc.begin; j += stride) {
        V16 x = ld16(c.heap[rank] + recv_base + j * 16);
        const size_t v = p.seg_begin + rc.begin + j;
        if (rs) {
          float acc[E];
          unpack_set<T>(load_user_vec<T>(src, v, n), acc);
          unpack_add<T>(x, acc);
          x = pack<T>(acc);
        }
        store_user_vec<T>(out, v, n, x);
      }
    }
    PK_SYNC(b);
    if (p.single_slot && s + 1 < steps) {
      PK_FOR_THREADS(b, tid) {
        if (tid == 0) signal_peer(c, rank, prev, CH_CREDIT, b, flag_value(seq, p.step0 + s + 1));
      }
    }
  }
  return true;
}

// ---------------------------------------------------------------------------
// standard ring with `routes` concurrent rings
// grid: routes * lanes blocks; block -> (route = bid / lanes, lane = bid % lanes)
// scratch half: per route segment, RS area + AG area back to back
// ---------------------------------------------------------------------------
PK_HD size_t ring_standard_scratch_bytes(size_t n, int elem_size, int) {
  return 4 * vecs_for(n, elem_size) * 16;
}

template <typename T>
struct RingStandard {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const int N = c.world;
    const size_t V = ceil_div(a.n, E);
    const int routes = a.routes;
    const int lanes = b.nblocks / routes;
    const int route = b.bid / lanes;

    RingGroup g;
    g.size = N;
    g.pos = 0;
    for (int i = 0; i < N; ++i) {
      g.member[i] = ring_rank_at(N, a.nnodes, route, i);
      if (g.member[i] == rank) g.pos = i;
    }
    const Span seg = split_span(V, routes, route);
    RingPlan p;
    p.seg_begin = seg.begin;
    p.seg_len = seg.end - seg.begin;
    p.recv_off = scratch_half(a.scratch_off, a.scratch_bytes, seq) + seg.begin * 2 * 16;
    p.single_slot = false;
    p.lane = b.bid % lanes;
    p.lanes = lanes;
    p.step0 = 0;
    ring_allreduce_group<T>(c, rank, g, p, reinterpret_cast<const T*>(a.in),
                            reinterpret_cast<T*>(a.out), a.n, b, seq, s_abort);
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<RingStandard<T>, CollArgs>(c, rank, a, b);
  }
};

// ---------------------------------------------------------------------------
// double ring: ring all-reduce inside each column group (same local rank on
// every virtual node), then ring all-reduce inside each node.  One chunk-sized
// receive slot per block and phase; a sender may refill the slot only after the
// receiver returned a credit for the previous step.
// scratch half: [2 phases][nblocks][slot_vecs]
// ---------------------------------------------------------------------------
PK_HD size_t double_ring_slot_vecs(size_t V, int nblocks, int world, int nnodes) {
  size_t per_block = ceil_div(V, (size_t)nblocks);
  int gpn = world / nnodes;
  int gmin = nnodes < gpn ? nnodes : gpn;
  if (gmin < 2) gmin = (nnodes > gpn ? nnodes : gpn);
  if (gmin < 1) gmin = 1;
  return ceil_div(per_block, (size_t)gmin) + 1;
}
PK_HD size_t double_ring_scratch_bytes(size_t n, int elem_size, int world, int nnodes,
                                       int nblocks) {
  return 4 * (size_t)nblocks *
         double_ring_slot_vecs(vecs_for(n, elem_size), nblocks, world, nnodes) * 16;
}

template <typename T>
struct DoubleRing {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const int N = c.world;
    const int nnodes = a.nnodes;
    const int gpn = N / nnodes;
    const size_t V = ceil_div(a.n, E);
    const size_t half = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    // sized from the call's shape, NOT from scratch_bytes: every call sharing a
    // scratch region must cut it into the same two halves
    const size_t slot_vecs = double_ring_slot_vecs(V, b.nblocks, N, nnodes);
    const Span seg = split_span(V, b.nblocks, b.bid);  // this block's contiguous piece

    RingPlan p;
    p.seg_begin = seg.begin;
    p.seg_len = seg.end - seg.begin;
    p.single_slot = true;
    p.lane = 0;
    p.lanes = 1;

    RingGroup col;
    col.size = nnodes;
    col.pos = rank / gpn;
    for (int i = 0; i < nnodes; ++i) col.member[i] = column_member(N, nnodes, rank, i);
    p.recv_off = half + ((size_t)0 * b.nblocks + b.bid) * slot_vecs * 16;
    p.step0 = 0;
    if (!ring_allreduce_group<T>(c, rank, col, p, reinterpret_cast<const T*>(a.in),
                                 reinterpret_cast<T*>(a.out), a.n, b, seq, s_abort))
      return;
    RingGroup row;
    row.size = gpn;
    row.pos = rank % gpn;
    for (int i = 0; i < gpn; ++i) row.member[i] = row_member(N, nnodes, rank, i);
    p.recv_off = half + ((size_t)1 * b.nblocks + b.bid) * slot_vecs * 16;
    p.step0 = 2 * (nnodes - 1);
    // phase 2 reduces what phase 1 left in `out`
    ring_allreduce_group<T>(c, rank, row, p, reinterpret_cast<const T*>(a.out),
                            reinterpret_cast<T*>(a.out), a.n, b, seq, s_abort);
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<DoubleRing<T>, CollArgs>(c, rank, a, b);
  }
};

}  // namespace penny
