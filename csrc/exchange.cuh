// Exchange: pairwise buffer swap and the N-way all-to-all built on the same
// push + flag step.
//
//   ExchangePair – every rank swaps its buffer, in place, with rank a.peer
//     (the peer must name this rank back).  Same contract as the reference's
//     penny_cpp.exchange (csrc/exchange.cu:11-64), but the receive slot is
//     persistent heap scratch: no allocation, no host barrier and no stream
//     synchronise per call.
//   AllToAll – out[s*n .. (s+1)*n) on rank r = in[r*n .. (r+1)*n) of rank s.
//     The reference has no N-way form; this is what expert-parallel dispatch
//     and combine need.
#pragma once
#include "coll_args.h"

namespace penny {

// one receive slot of [V] (not halved: see ExchangePair)
PK_HD size_t exchange_scratch_bytes(size_t n, int elem_size) {
  return vecs_for(n, elem_size) * 16;
}
// both halves of: [world][chunk vecs]
PK_HD size_t all_to_all_scratch_bytes(size_t chunk_n, int elem_size, int world) {
  return 2 * (size_t)world * vecs_for(chunk_n, elem_size) * 16;
}

template <typename T>
struct ExchangePair {
  // Not every rank depends on every other rank here, so the two-halves rule of
  // the other collectives does not protect the slot, and exchange calls are
  // counted on their own sequence (SEQ_PAIR).  Every rank must take part in
  // every exchange call (with peer == its own rank to sit one out).  The pair
  // first shakes hands ("I am in exchange call seq": my previous exchange,
  // whoever it was with, has completely finished), then pushes, flags, copies.
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    T* buf = reinterpret_cast<T*>(a.out);
    const int peer = a.peer;
    const size_t V = ceil_div(a.n, E);
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t first = (size_t)b.bid * b.nthreads;
    if (peer == rank) return;
    PK_FOR_THREADS(b, tid) {
      if (tid == 0) signal_peer(c, rank, peer, CH_USER, b, flag_value(seq, 1));
    }
    PK_FOR_THREADS(b, tid) {
      if (tid == 0 && !wait_peer(c, rank, peer, CH_USER, b, flag_value(seq, 1), ST_TIMEOUT_DATA))
        s_abort = 1;
    }
    PK_SYNC(b);
    if (s_abort) return;
    PK_FOR_THREADS(b, tid) {
      for (size_t v = first + tid; v < V; v += stride)
        st16(c.heap[peer] + a.scratch_off + v * 16, load_user_vec<T>(buf, v, a.n));
    }
    PK_SYNC(b);
    PK_FOR_THREADS(b, tid) {
      if (tid == 0) signal_peer(c, rank, peer, CH_USER, b, flag_value(seq, 2));
    }
    PK_FOR_THREADS(b, tid) {
      if (tid == 0 && !wait_peer(c, rank, peer, CH_USER, b, flag_value(seq, 2), ST_TIMEOUT_DATA))
        s_abort = 1;
    }
    PK_SYNC(b);
    if (s_abort) return;
    PK_FOR_THREADS(b, tid) {
      for (size_t v = first + tid; v < V; v += stride)
        store_user_vec<T>(buf, v, a.n, ld16(c.heap[rank] + a.scratch_off + v * 16));
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<ExchangePair<T>, CollArgs, SEQ_PAIR>(c, rank, a, b);
  }
};

template <typename T, int NG>
struct AllToAll {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t CV = ceil_div(a.n, E);
    const bool direct = a.out_heap_off != kNotInHeap;
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t first = (size_t)b.bid * b.nthreads;
    if (direct) {
      // the peers' outputs are written in place: wait until every peer is in this call
      PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
      if (s_abort) return;
      PK_FOR_THREADS(b, tid) {
        for (int d = 0; d < NG; ++d) {
          const int p = (rank + d) % NG;
          T* dst = reinterpret_cast<T*>(c.heap[p] + a.out_heap_off) + (size_t)rank * a.n;
          for (size_t j = first + tid; j < CV; j += stride)
            store_user_vec<T>(dst, j, a.n, load_user_vec<T>(in + (size_t)p * a.n, j, a.n));
        }
      }
      PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 2), s_abort);
      return;
    }
    const size_t base = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    PK_FOR_THREADS(b, tid) {
      for (int d = 0; d < NG; ++d) {
        const int p = (rank + d) % NG;
        for (size_t j0 = first + tid; j0 < CV; j0 += kBatch * stride) {
          V16 x[kBatch];
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < CV) x[u] = load_user_vec<T>(in + (size_t)p * a.n, j0 + u * stride, a.n);
#pragma unroll
          for (int u = 0; u < kBatch; ++u) {
            const size_t j = j0 + u * stride;
            if (j >= CV) continue;
            if (p == rank)
              store_user_vec<T>(out + (size_t)rank * a.n, j, a.n, x[u]);
            else
              st16(c.heap[p] + base + ((size_t)rank * CV + j) * 16, x[u]);
          }
        }
      }
    }
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;
    PK_FOR_THREADS(b, tid) {
      for (int d = 1; d < NG; ++d) {
        const int s = (rank + d) % NG;
        for (size_t j = first + tid; j < CV; j += stride)
          store_user_vec<T>(out + (size_t)s * a.n, j, a.n,
                            ld16(c.heap[rank] + base + ((size_t)s * CV + j) * 16));
      }
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<AllToAll<T, NG>, CollArgs>(c, rank, a, b);
  }
};

// All-to-all through scratch with the copy-out overlapped with the pushes: the
// per-peer chunk is cut into up to kA2aMaxChunks pieces; a block pushes its slice
// of piece k to every peer, raises step k + 1 and only then waits for step k and
// copies piece k - 1 from its scratch slots to the output, so one piece is being
// copied out while the next is on the wire (the plain variant pushes everything,
// waits once, then copies everything).  Same scratch layout as AllToAll.
constexpr int kA2aMaxChunks = 16;

template <typename T, int NG>
struct AllToAllPipelined {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t CV = ceil_div(a.n, E);
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t first = (size_t)b.bid * b.nthreads;
    const size_t base = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const size_t per_pass = stride * kBatch;
    const size_t passes = ceil_div(CV, per_pass);
    int chunks = (int)(passes / 4);
    if (chunks < 1) chunks = 1;
    if (chunks > kA2aMaxChunks) chunks = kA2aMaxChunks;
    const size_t CS = ceil_div(passes, (size_t)chunks) * per_pass;  // vectors per piece
    for (int k = 0; k <= chunks; ++k) {
      if (k < chunks) {
        const size_t lo = (size_t)k * CS, hi = (lo + CS < CV) ? lo + CS : CV;
        PK_FOR_THREADS(b, tid) {
          for (int d = 0; d < NG; ++d) {
            const int p = (rank + d) % NG;
            for (size_t j0 = lo + first + tid; j0 < hi; j0 += kBatch * stride) {
              V16 x[kBatch];
#pragma unroll
              for (int u = 0; u < kBatch; ++u)
                if (j0 + u * stride < hi) x[u] = load_user_vec<T>(in + (size_t)p * a.n, j0 + u * stride, a.n);
#pragma unroll
              for (int u = 0; u < kBatch; ++u) {
                const size_t j = j0 + u * stride;
                if (j >= hi) continue;
                if (p == rank)
                  store_user_vec<T>(out + (size_t)rank * a.n, j, a.n, x[u]);
                else
                  st16(c.heap[p] + base + ((size_t)rank * CV + j) * 16, x[u]);
              }
            }
          }
        }
      }
      PK_SYNC(b);  // the block's stores of piece k are issued before anyone signals
      if (k < chunks) {
        PK_FOR_THREADS(b, _t) {
          if (_t < c.world && _t != rank) signal_peer(c, rank, _t, CH_BARRIER, b, flag_value(seq, k + 1));
        }
      }
      if (k >= 1) {
        PK_FOR_THREADS(b, _t) {
          if (_t < c.world && _t != rank) {
            if (!wait_peer(c, rank, _t, CH_BARRIER, b, flag_value(seq, k), ST_TIMEOUT_BARRIER)) s_abort = 1;
          }
        }
        PK_SYNC(b);
        if (s_abort) return;
        const size_t lo = (size_t)(k - 1) * CS, hi = (lo + CS < CV) ? lo + CS : CV;
        PK_FOR_THREADS(b, tid) {
          for (int d = 1; d < NG; ++d) {
            const int s = (rank + d) % NG;
            for (size_t j0 = lo + first + tid; j0 < hi; j0 += kBatch * stride) {
              V16 x[kBatch];
#pragma unroll
              for (int u = 0; u < kBatch; ++u)
                if (j0 + u * stride < hi) x[u] = ld16(c.heap[rank] + base + ((size_t)s * CV + j0 + u * stride) * 16);
#pragma unroll
              for (int u = 0; u < kBatch; ++u)
                if (j0 + u * stride < hi) store_user_vec<T>(out + (size_t)s * a.n, j0 + u * stride, a.n, x[u]);
            }
          }
        }
      }
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<AllToAllPipelined<T, NG>, CollArgs>(c, rank, a, b);
  }
};

}  // namespace penny
