// Two-shot all-reduce = reduce-scatter + all-gather, both by direct pushes over
// NVLink, plus the two halves as collectives of their own.
//
// Block b of every rank owns the same strided slice of every chunk, so all
// synchronisation is between block b of one rank and block b of its peers: two
// flag barriers per all-reduce, no grid-wide barrier and no atomics on the data
// path (the reference counts arrivals with a self-targeted signal_op ADD,
// csrc/all_reduce_twoshot.cu:67-82, and is fixed to 8 ranks).
//
//   scatter : rank r writes its piece of chunk c into rank c's rs slot [r]
//   reduce  : rank c sums the `world` pieces of chunk c in rank order (fp32)
//   gather  : rank c writes the finished chunk into every peer's ag area (or
//             straight into the peer's output when that lives in the heap)
//   copy-out: ag area -> output (skipped in the direct case)
#pragma once
#include "coll_args.h"
#include "schedule.h"

namespace penny {

// both halves of: rs slots [world][chunk_vecs] + ag area [world * chunk_vecs]
PK_HD size_t twoshot_scratch_bytes(size_t n, int elem_size, int world) {
  size_t cv = ceil_div(vecs_for(n, elem_size), (size_t)world);
  return 4 * (size_t)world * cv * 16;
}
// both halves of: [world][shard_vecs]
PK_HD size_t reduce_scatter_scratch_bytes(size_t n, int elem_size, int world) {
  size_t sv = vecs_for(n / (size_t)world, elem_size);
  return 2 * (size_t)world * sv * 16;
}
// both halves of: [world][shard_vecs]
PK_HD size_t all_gather_scratch_bytes(size_t shard_n, int elem_size, int world) {
  return 2 * (size_t)world * vecs_for(shard_n, elem_size) * 16;
}

template <typename T, int NG>
struct TwoShot {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t V = ceil_div(a.n, E);
    const size_t CV = ceil_div(V, (size_t)NG);
    const size_t rs_off = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const size_t ag_off = rs_off + (size_t)NG * CV * 16;
    const bool direct = a.out_heap_off != kNotInHeap;
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t first = (size_t)b.bid * b.nthreads;

    // scatter
    PK_FOR_THREADS(b, tid) {
      for (int d = 1; d < NG; ++d) {
        const int dst = (rank + d) % NG;  // start with a different peer on every rank
        const Span sp = split_span(V, NG, dst);
        const size_t len = sp.end - sp.begin;
        for (size_t j0 = first + tid; j0 < len; j0 += kBatch * stride) {
          V16 x[kBatch];
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < len) x[u] = load_user_vec<T>(in, sp.begin + j0 + u * stride, a.n);
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < len)
              st16(c.heap[dst] + rs_off + ((size_t)rank * CV + j0 + u * stride) * 16, x[u]);
        }
      }
    }
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;

    // reduce own chunk, gather
    const Span mine = split_span(V, NG, rank);
    PK_FOR_THREADS(b, tid) {
      for (size_t j = first + tid; j < mine.end - mine.begin; j += stride) {
        float acc[E];
#pragma unroll
        for (size_t i = 0; i < E; ++i) acc[i] = 0.f;
#pragma unroll
        for (int s = 0; s < NG; ++s) {
          V16 x = (s == rank) ? load_user_vec<T>(in, mine.begin + j, a.n)
                              : ld16(c.heap[rank] + rs_off + ((size_t)s * CV + j) * 16);
          unpack_add<T>(x, acc);
        }
        const V16 r = pack<T>(acc);
        const size_t v = mine.begin + j;
        store_user_vec<T>(out, v, a.n, r);
#pragma unroll
        for (int d = 1; d < NG; ++d) {
          const int p = (rank + d) % NG;
          if (direct)
            store_user_vec<T>(reinterpret_cast<T*>(c.heap[p] + a.out_heap_off), v, a.n, r);
          else
            st16(c.heap[p] + ag_off + v * 16, r);
        }
      }
    }
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 2), s_abort);
    if (s_abort || direct) return;

    // copy-out
    PK_FOR_THREADS(b, tid) {
      for (int d = 1; d < NG; ++d) {
        const int src = (rank + d) % NG;
        const Span sp = split_span(V, NG, src);
        const size_t len = sp.end - sp.begin;
        for (size_t j0 = first + tid; j0 < len; j0 += kBatch * stride) {
          V16 x[kBatch];
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < len) x[u] = ld16(c.heap[rank] + ag_off + (sp.begin + j0 + u * stride) * 16);
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < len) store_user_vec<T>(out, sp.begin + j0 + u * stride, a.n, x[u]);
        }
      }
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<TwoShot<T, NG>, CollArgs>(c, rank, a, b);
  }
};

// Reduce-scatter.  The input has a.n elements and is cut into `world` equal
// shards of a.n / world elements (a.n must divide); rank r receives the sum of
// shard r.  Shard order = rank order, as in the reference's
// cross_device_reduce_scatter_2stage (csrc/custom_all_reduce.cuh:464-539).
template <typename T, int NG>
struct ReduceScatterPush {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t shard = a.n / NG;  // elements
    const size_t SV = ceil_div(shard, E);
    const size_t base = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t first = (size_t)b.bid * b.nthreads;
    PK_FOR_THREADS(b, tid) {
      for (int d = 1; d < NG; ++d) {
        const int dst = (rank + d) % NG;
        const T* src = in + (size_t)dst * shard;
        for (size_t j0 = first + tid; j0 < SV; j0 += kBatch * stride) {
          V16 x[kBatch];
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < SV) x[u] = load_user_vec<T>(src, j0 + u * stride, shard);
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < SV)
              st16(c.heap[dst] + base + ((size_t)rank * SV + j0 + u * stride) * 16, x[u]);
        }
      }
    }
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;
    PK_FOR_THREADS(b, tid) {
      const T* own = in + (size_t)rank * shard;
      for (size_t j = first + tid; j < SV; j += stride) {
        float acc[E];
#pragma unroll
        for (size_t i = 0; i < E; ++i) acc[i] = 0.f;
#pragma unroll
        for (int s = 0; s < NG; ++s) {
          V16 x = (s == rank) ? load_user_vec<T>(own, j, shard)
                              : ld16(c.heap[rank] + base + ((size_t)s * SV + j) * 16);
          unpack_add<T>(x, acc);
        }
        store_user_vec<T>(out, j, shard, pack<T>(acc));
      }
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<ReduceScatterPush<T, NG>, CollArgs>(c, rank, a, b);
  }
};

// The same reduce-scatter with the owner's reduction overlapped with the pushes:
// the shard is cut into up to kRsMaxChunks chunks; a block pushes its slice of
// chunk k to every peer, raises step k + 1 on its peers' flags and only then
// waits for step k and reduces chunk k - 1, so the local reduction of one chunk
// runs while the stores of the next one are still draining over NVLink (the
// plain variant pays push time + reduce time, which costs it the comparison with
// NCCL above 8 MiB shards).  Same scratch layout, same flag channel: the flag
// value only ever grows inside a call (seq * 64 + step, step <= kRsMaxChunks).
constexpr int kRsMaxChunks = 16;

template <typename T, int NG>
struct ReduceScatterPipelined {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t shard = a.n / NG;  // elements
    const size_t SV = ceil_div(shard, E);
    const size_t base = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t first = (size_t)b.bid * b.nthreads;
    // chunks of whole batches: at least four batches per thread and chunk
    const size_t per_pass = stride * kBatch;
    size_t passes = ceil_div(SV, per_pass);
    int chunks = (int)(passes / 4);
    if (chunks < 1) chunks = 1;
    if (chunks > kRsMaxChunks) chunks = kRsMaxChunks;
    const size_t CS = ceil_div(passes, (size_t)chunks) * per_pass;  // vectors per chunk
    for (int k = 0; k <= chunks; ++k) {
      if (k < chunks) {
        const size_t lo = (size_t)k * CS, hi = (lo + CS < SV) ? lo + CS : SV;
        PK_FOR_THREADS(b, tid) {
          for (int d = 1; d < NG; ++d) {
            const int dst = (rank + d) % NG;
            const T* src = in + (size_t)dst * shard;
            for (size_t j0 = lo + first + tid; j0 < hi; j0 += kBatch * stride) {
              V16 x[kBatch];
#pragma unroll
              for (int u = 0; u < kBatch; ++u)
                if (j0 + u * stride < hi) x[u] = load_user_vec<T>(src, j0 + u * stride, shard);
#pragma unroll
              for (int u = 0; u < kBatch; ++u)
                if (j0 + u * stride < hi)
                  st16(c.heap[dst] + base + ((size_t)rank * SV + j0 + u * stride) * 16, x[u]);
            }
          }
        }
      }
      PK_SYNC(b);  // the block's stores of chunk k are issued before anyone signals
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
        const size_t lo = (size_t)(k - 1) * CS, hi = (lo + CS < SV) ? lo + CS : SV;
        PK_FOR_THREADS(b, tid) {
          const T* own = in + (size_t)rank * shard;
          for (size_t j = lo + first + tid; j < hi; j += stride) {
            float acc[E];
#pragma unroll
            for (size_t i = 0; i < E; ++i) acc[i] = 0.f;
#pragma unroll
            for (int s = 0; s < NG; ++s) {
              V16 x = (s == rank) ? load_user_vec<T>(own, j, shard)
                                  : ld16(c.heap[rank] + base + ((size_t)s * SV + j) * 16);
              unpack_add<T>(x, acc);
            }
            store_user_vec<T>(out, j, shard, pack<T>(acc));
          }
        }
      }
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<ReduceScatterPipelined<T, NG>, CollArgs>(c, rank, a, b);
  }
};

// All-gather.  a.n = elements of one shard; out[r*n .. (r+1)*n) = rank r's input.
//   direct (output in the heap): start barrier (every peer has entered the call,
//     so its output buffer is no longer being read by earlier work), push the
//     shard into every peer's output, end barrier.
//   staged: push into scratch slots, one barrier, copy slots -> output.
template <typename T, int NG>
struct AllGatherPush {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t SV = ceil_div(a.n, E);
    const bool direct = a.out_heap_off != kNotInHeap;
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t first = (size_t)b.bid * b.nthreads;
    if (direct) {
      PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
      if (s_abort) return;
      PK_FOR_THREADS(b, tid) {
        for (size_t j0 = first + tid; j0 < SV; j0 += kBatch * stride) {
          V16 x[kBatch];
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < SV) x[u] = load_user_vec<T>(in, j0 + u * stride, a.n);
#pragma unroll
          for (int d = 0; d < NG; ++d) {
            const int p = (rank + d) % NG;
            T* dst = reinterpret_cast<T*>(c.heap[p] + a.out_heap_off) + (size_t)rank * a.n;
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
              if (j0 + u * stride < SV) store_user_vec<T>(dst, j0 + u * stride, a.n, x[u]);
          }
        }
      }
      PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 2), s_abort);
      return;
    }
    const size_t base = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    PK_FOR_THREADS(b, tid) {
      for (size_t j0 = first + tid; j0 < SV; j0 += kBatch * stride) {
        V16 x[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          if (j0 + u * stride < SV) x[u] = load_user_vec<T>(in, j0 + u * stride, a.n);
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          if (j0 + u * stride < SV) store_user_vec<T>(out + (size_t)rank * a.n, j0 + u * stride, a.n, x[u]);
#pragma unroll
        for (int d = 1; d < NG; ++d) {
          const int p = (rank + d) % NG;
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < SV) st16(c.heap[p] + base + ((size_t)rank * SV + j0 + u * stride) * 16, x[u]);
        }
      }
    }
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;
    PK_FOR_THREADS(b, tid) {
      for (int d = 1; d < NG; ++d) {
        const int s = (rank + d) % NG;
        for (size_t j0 = first + tid; j0 < SV; j0 += kBatch * stride) {
          V16 x[kBatch];
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < SV) x[u] = ld16(c.heap[rank] + base + ((size_t)s * SV + j0 + u * stride) * 16);
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (j0 + u * stride < SV) store_user_vec<T>(out + (size_t)s * a.n, j0 + u * stride, a.n, x[u]);
        }
      }
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<AllGatherPush<T, NG>, CollArgs>(c, rank, a, b);
  }
};

}  // namespace penny
