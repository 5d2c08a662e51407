// One-shot all-reduce: every rank pushes its whole input into a slot of every
// peer's heap, then each rank sums the `world` copies locally in fp32, always in
// rank order 0..world-1, so that every rank produces bit-identical output.
//
// Two wire protocols:
//   OneShotFlag – 16-byte stores, then one release flag per (block, peer).
//   OneShotLL   – low latency: every 8 payload bytes travel with their own
//                 4-byte call number ({d0, e, d1, e} lines), so there is no
//                 fence, no separate flag and no block-wide barrier on the
//                 critical path.
// The slots live in the scratch half of the current call, so no end-of-call
// barrier is needed (see scratch_half in pk.h).
//
// Because the input is only ever read by its owner, it needs no registration
// and no staging copy – unlike the pull design of the reference's
// cross_device_reduce_1stage (csrc/custom_all_reduce.cuh:310-367) – and unlike
// csrc/all_reduce_oneshot.cu:13-63 it is not tied to 8 ranks, accumulates in
// fp32 and handles ragged element counts.
#pragma once
#include "coll_args.h"

namespace penny {

// both halves of: [src world][V] vectors
PK_HD size_t oneshot_flag_scratch_bytes(size_t n, int elem_size, int world) {
  return 2 * (size_t)world * vecs_for(n, elem_size) * 16;
}
// both halves of: [src world][V rounded up to 32] pairs of 16-byte lines
PK_HD size_t oneshot_ll_scratch_bytes(size_t n, int elem_size, int world) {
  return 4 * (size_t)world * ((vecs_for(n, elem_size) + 31) / 32 * 32) * 16;
}
// Byte offset of line j (0 or 1) of vector v sent by rank s.  32 consecutive vectors share two
// 512-byte rows (all their lines 0, then all their lines 1), so the store instruction of a warp
// whose lanes hold consecutive vectors writes 512 contiguous bytes - four whole 128-byte lines on
// the wire instead of 32 half-written sectors.
PK_HD size_t ll_line_off(size_t vpad, int s, size_t v, int j) {
  return (((size_t)s * vpad + (v & ~(size_t)31)) * 2 + (size_t)j * 32 + (v & 31)) * 16;
}

template <typename T, int NG>
struct OneShotFlag {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t V = ceil_div(a.n, E);
    const size_t base = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const size_t stride = (size_t)b.nblocks * b.nthreads;

    PK_FOR_THREADS(b, tid) {
      for (size_t v0 = (size_t)b.bid * b.nthreads + tid; v0 < V; v0 += kBatch * stride) {
        V16 x[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          if (v0 + u * stride < V) x[u] = load_user_vec<T>(in, v0 + u * stride, a.n);
#pragma unroll
        for (int d = 1; d < NG; ++d) {
          const int p = (rank + d) % NG;
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (v0 + u * stride < V)
              st16(c.heap[p] + base + ((size_t)rank * V + v0 + u * stride) * 16, x[u]);
        }
      }
    }
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;

    PK_FOR_THREADS(b, tid) {
      for (size_t v = (size_t)b.bid * b.nthreads + tid; v < V; v += stride) {
        float acc[E];
#pragma unroll
        for (size_t i = 0; i < E; ++i) acc[i] = 0.f;
#pragma unroll
        for (int s = 0; s < NG; ++s) {
          V16 x = (s == rank) ? load_user_vec<T>(in, v, a.n)
                              : ld16(c.heap[rank] + base + ((size_t)s * V + v) * 16);
          unpack_add<T>(x, acc);
        }
        store_user_vec<T>(out, v, a.n, pack<T>(acc));
      }
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<OneShotFlag<T, NG>, CollArgs>(c, rank, a, b);
  }
};

// Wait for one LL line whose two flag words equal e.  Bounded.
PK_DEV bool ll_wait_line(const char* p, uint32_t e, V16& line, const CommCtx& c, int peer,
                         int bid) {
  line = ld16_volatile(p);
  if (line.w[1] == e && line.w[3] == e) return true;
  const uint64_t t0 = now_ns();
  for (uint32_t spin = 1;; ++spin) {
    line = ld16_volatile(p);
    if (line.w[1] == e && line.w[3] == e) return true;
    if ((spin & 31u) == 0u) {
      if (now_ns() - t0 > c.timeout_ns) {
        report_status(c, ST_TIMEOUT_LL, peer, bid, e, line.w[1]);
        return false;
      }
      spin_pause();
    }
  }
}
// `line` already holds one volatile load of *p: done if its stamps match, else keep polling.
// Callers issue the first loads of all the lines they need back to back and only then look at
// them, so lines that have already landed cost one memory latency in total, not one each.
PK_DEV bool ll_finish_line(const char* p, uint32_t e, V16& line, const CommCtx& c, int peer, int bid) {
  if (line.w[1] == e && line.w[3] == e) return true;
  return ll_wait_line(p, e, line, c, peer, bid);
}
// The flag carried by every LL line of call `seq`: never 0 (fresh memory).
PK_HD uint32_t ll_flag(u64 seq) { return (uint32_t)(seq + 1) | 0x80000000u; }

template <typename T, int NG>
struct OneShotLL {
  static PK_DEV void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                          int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t V = ceil_div(a.n, E);
    const size_t vpad = (V + 31) / 32 * 32;
    const size_t base = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const uint32_t e = ll_flag(seq);
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    (void)s_abort;

    PK_FOR_THREADS(b, tid) {
      for (size_t v = (size_t)b.bid * b.nthreads + tid; v < V; v += stride) {
        V16 x = load_user_vec<T>(in, v, a.n);
        V16 l0, l1;
        l0.w[0] = x.w[0]; l0.w[1] = e; l0.w[2] = x.w[1]; l0.w[3] = e;
        l1.w[0] = x.w[2]; l1.w[1] = e; l1.w[2] = x.w[3]; l1.w[3] = e;
#pragma unroll
        for (int d = 1; d < NG; ++d) {
          const int p = (rank + d) % NG;
          st16_volatile(c.heap[p] + base + ll_line_off(vpad, rank, v, 0), l0);
          st16_volatile(c.heap[p] + base + ll_line_off(vpad, rank, v, 1), l1);
        }
      }
    }
    PK_FOR_THREADS(b, tid) {
      for (size_t v = (size_t)b.bid * b.nthreads + tid; v < V; v += stride) {
        float acc[E];
#pragma unroll
        for (size_t i = 0; i < E; ++i) acc[i] = 0.f;
        bool ok = true;
        const char* src = c.heap[rank] + base;
        V16 l0[NG], l1[NG];
#pragma unroll
        for (int s = 0; s < NG; ++s) {
          if (s != rank) {
            l0[s] = ld16_volatile(src + ll_line_off(vpad, s, v, 0));
            l1[s] = ld16_volatile(src + ll_line_off(vpad, s, v, 1));
          }
        }
#pragma unroll
        for (int s = 0; s < NG; ++s) {
          V16 x;
          if (s == rank) {
            x = load_user_vec<T>(in, v, a.n);
          } else {
            ok = ok && ll_finish_line(src + ll_line_off(vpad, s, v, 0), e, l0[s], c, s, b.bid);
            ok = ok && ll_finish_line(src + ll_line_off(vpad, s, v, 1), e, l1[s], c, s, b.bid);
            x.w[0] = l0[s].w[0]; x.w[1] = l0[s].w[2]; x.w[2] = l1[s].w[0]; x.w[3] = l1[s].w[2];
          }
          unpack_add<T>(x, acc);
        }
        if (!ok) break;
        store_user_vec<T>(out, v, a.n, pack<T>(acc));
      }
    }
  }
  static PK_DEV void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<OneShotLL<T, NG>, CollArgs>(c, rank, a, b);
  }
};

}  // namespace penny
