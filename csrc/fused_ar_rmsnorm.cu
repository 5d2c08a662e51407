// All-reduce fused with its tensor-parallel consumer: residual add + RMSNorm.
//
// In a TP transformer layer the row-parallel GEMMs (o_proj, down_proj) leave a
// partial sum [rows, hidden] on every rank; what the next op needs is
//     z   = sum_over_ranks(partial) + residual          (new residual stream)
//     out = z * rsqrt(mean(z^2) + eps) * weight         (input of the next GEMM)
// Done separately that is an all-reduce, a write of the sum, and a second kernel
// that re-reads it.  Here the rows never leave registers between the reduction
// and the normalisation, and there is one launch instead of two or three.
//
// Transports, all one block per row:
//   LL    every rank pushes its partial rows to every peer as flag-in-data
//         lines and polls for the peers' lines: no barrier, lowest latency, 2x
//         wire bytes.  Best for a handful of rows.
//   FLAG  16-byte pushes + one flag barrier per block.
//   NVLS  rows are sharded over the ranks; the owner pulls the switch-reduced
//         row (multimem.ld_reduce), normalises it and multicasts the result
//         (multimem.st).  The residual stream stays sharded: each rank only
//         keeps the residual of the rows it owns.  Least wire traffic.
//   NVLS one-shot  every rank pulls all rows switch-reduced and normalises them
//         itself: half the latency steps, `world` times the wire bytes.
//   LL two-shot  rows sharded over the ranks, flag-in-data lines to the owner and
//         back: two one-way trips, no barrier, 1 / world of the one-shot bytes.
// Plus the communication-free kernel (add_rmsnorm) used at world size 1.
//
// The reference stops at the plain all-reduce (penny/custom_all_reduce.py:229-267);
// the norm runs as a separate kernel of the serving framework.
#include "algos.h"
#include "all_reduce_oneshot.cuh"
#include "fused_ops.h"
#include "launch.cuh"
#include "pdl.h"
#include "schedule.h"

namespace penny {

constexpr int kMaxVecPerThread = 4;

__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();  // smem may still be read from the previous row
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? smem[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// z (fp32, K vectors per thread) -> residual_out / out for one row.
template <typename T, int K>
__device__ __forceinline__ void norm_and_store(float (&z)[K][16 / sizeof(T)], int nv, int HV,
                                               const FusedNormArgs& a, size_t row, float* smem) {
  constexpr int E = 16 / sizeof(T);
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    if (k < nv) {
#pragma unroll
      for (int i = 0; i < E; ++i) ss += z[k][i] * z[k][i];
    }
  }
  ss = block_sum(ss, smem);
  const float rstd = rsqrtf(ss / (float)a.hidden + a.eps);
  T* out = reinterpret_cast<T*>(a.out) + row * (size_t)a.hidden;
  T* rout = a.residual_out ? reinterpret_cast<T*>(a.residual_out) + row * (size_t)a.hidden : nullptr;
  const T* w = reinterpret_cast<const T*>(a.weight);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    if (k < nv) {
      const int v = threadIdx.x + k * blockDim.x;
      if (rout) st16(rout + (size_t)v * E, pack<T>(z[k]));
      float wv[E], o[E];
      unpack_set<T>(ld16(w + (size_t)v * E), wv);
#pragma unroll
      for (int i = 0; i < E; ++i) o[i] = z[k][i] * rstd * wv[i];
      st16(out + (size_t)v * E, pack<T>(o));
    }
  }
  (void)HV;
}

// ---------------------------------------------------------------------------
// communication-free: out = rmsnorm(in + residual)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(512) k_add_rmsnorm(const FusedNormArgs a) {
  constexpr int E = 16 / sizeof(T);
  __shared__ float smem[32];
  pdl_launch_dependents();
  const int HV = a.hidden / E;
  pdl_wait();
  for (size_t row = blockIdx.x; row < (size_t)a.rows; row += gridDim.x) {
    float z[kMaxVecPerThread][E];
    int nv = 0;
#pragma unroll
    for (int k = 0; k < kMaxVecPerThread; ++k) {
      const int v = threadIdx.x + k * blockDim.x;
      if (v < HV) {
        nv = k + 1;
        unpack_set<T>(ld16(reinterpret_cast<const T*>(a.in) + row * a.hidden + (size_t)v * E), z[k]);
        if (a.residual)
          unpack_add<T>(ld16(reinterpret_cast<const T*>(a.residual) + row * a.hidden + (size_t)v * E),
                        z[k]);
      }
    }
    norm_and_store<T, kMaxVecPerThread>(z, nv, HV, a, row, smem);
  }
}

// ---------------------------------------------------------------------------
// one-shot (LL or flag) + residual + RMSNorm
// scratch half: LL   [src][rows][HV] pairs of lines
//               FLAG [src][rows][HV] vectors
// ---------------------------------------------------------------------------
template <typename T, int NG, bool LL>
struct FusedOneShotNorm {
  static __device__ void body(const CommCtx& c, int rank, const FusedNormArgs& a, const Blk& b,
                              u64 seq, int& s_abort) {
    constexpr int E = 16 / sizeof(T);
    __shared__ float smem[32];
    const int HV = a.hidden / E;
    const size_t base = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const uint32_t e = ll_flag(seq);
    const T* in = reinterpret_cast<const T*>(a.in);
    constexpr size_t LINE = LL ? 32 : 16;

    // push my partial rows to every peer
    for (size_t row = b.bid; row < (size_t)a.rows; row += b.nblocks) {
      for (int v = threadIdx.x; v < HV; v += blockDim.x) {
        const V16 x = ld16(in + row * a.hidden + (size_t)v * E);
        const size_t off = base + (((size_t)rank * a.rows + row) * HV + v) * LINE;
        if (LL) {
          V16 l0, l1;
          l0.w[0] = x.w[0]; l0.w[1] = e; l0.w[2] = x.w[1]; l0.w[3] = e;
          l1.w[0] = x.w[2]; l1.w[1] = e; l1.w[2] = x.w[3]; l1.w[3] = e;
#pragma unroll
          for (int d = 1; d < NG; ++d) {
            char* dst = c.heap[(rank + d) % NG] + off;
            st16_volatile(dst, l0);
            st16_volatile(dst + 16, l1);
          }
        } else {
#pragma unroll
          for (int d = 1; d < NG; ++d) st16(c.heap[(rank + d) % NG] + off, x);
        }
      }
    }
    if (!LL) {
      PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
      if (s_abort) return;
    }
    // reduce in rank order, add the residual, normalise
    for (size_t row = b.bid; row < (size_t)a.rows; row += b.nblocks) {
      float z[kMaxVecPerThread][E];
      int nv = 0;
      bool ok = true;
#pragma unroll
      for (int k = 0; k < kMaxVecPerThread; ++k) {
        const int v = threadIdx.x + k * blockDim.x;
        if (v < HV) {
          nv = k + 1;
#pragma unroll
          for (int i = 0; i < E; ++i) z[k][i] = 0.f;
          // first loads of every peer's lines back to back; then wait for the late ones
          V16 l0[NG], l1[NG];
          if (LL) {
#pragma unroll
            for (int s = 0; s < NG; ++s) {
              if (s != rank) {
                const char* src = c.heap[rank] + base + (((size_t)s * a.rows + row) * HV + v) * LINE;
                l0[s] = ld16_volatile(src);
                l1[s] = ld16_volatile(src + 16);
              }
            }
          }
#pragma unroll
          for (int s = 0; s < NG; ++s) {
            V16 x;
            if (s == rank) {
              x = ld16(in + row * a.hidden + (size_t)v * E);
            } else {
              const char* src = c.heap[rank] + base + (((size_t)s * a.rows + row) * HV + v) * LINE;
              if (LL) {
                ok = ok && ll_finish_line(src, e, l0[s], c, s, b.bid);
                ok = ok && ll_finish_line(src + 16, e, l1[s], c, s, b.bid);
                x.w[0] = l0[s].w[0]; x.w[1] = l0[s].w[2]; x.w[2] = l1[s].w[0]; x.w[3] = l1[s].w[2];
              } else {
                x = ld16(src);
              }
            }
            unpack_add<T>(x, z[k]);
          }
          if (a.residual)
            unpack_add<T>(
                ld16(reinterpret_cast<const T*>(a.residual) + row * a.hidden + (size_t)v * E), z[k]);
        }
      }
      if (LL) {
        // a timeout anywhere in the block abandons the row for the whole block
        if (__syncthreads_or(ok ? 0 : 1)) return;
      }
      norm_and_store<T, kMaxVecPerThread>(z, nv, HV, a, row, smem);
    }
  }
  static __device__ void run(const CommCtx& c, int rank, const FusedNormArgs& a, const Blk& b) {
    run_collective<FusedOneShotNorm<T, NG, LL>, FusedNormArgs>(c, rank, a, b);
  }
};

// ---------------------------------------------------------------------------
// NVLS: rows sharded over ranks; owner reduces in the switch, normalises,
// multicasts.  in / out live in the heap; residual(_out) hold this rank's rows
// only, indexed by global row (so the buffers are [rows, hidden] everywhere but
// only the owned rows are meaningful).
// ---------------------------------------------------------------------------
__device__ __forceinline__ V16 mm_ld_reduce_bf16(const void* p) {
  V16 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ V16 mm_ld_reduce_f16(const void* p) {
  V16 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ V16 mm_ld_reduce_f32(const void* p) {
  V16 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p)
               : "memory");
  return v;
}
template <typename T>
__device__ __forceinline__ V16 mm_ld_reduce(const void* p) {
  if constexpr (sizeof(T) == 4) return mm_ld_reduce_f32(p);
  else if constexpr (std::is_same<T, __half>::value) return mm_ld_reduce_f16(p);
  else return mm_ld_reduce_bf16(p);
}
__device__ __forceinline__ void mm_st(void* p, const V16& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p),
               "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3])
               : "memory");
}

// ---------------------------------------------------------------------------
// Two-shot with flag-in-data lines in BOTH directions: rows are sharded over the
// ranks; every rank pushes its partial of a row to the row's owner as LL lines,
// the owner adds them in rank order, adds the residual, normalises and sends the
// finished row to every rank, again as LL lines (one multicast store per line
// when the heap is bound to the switch, else one store per peer).  No flag
// barrier and no fence anywhere: the critical path is two one-way trips, and a
// rank moves rows * hidden / world elements per direction instead of rows *
// hidden.  One block handles one row from end to end (its owner's block reduces,
// every other rank's block pushes and then polls for the result), so blocks never
// wait for one another.  The residual stream stays sharded like under NVLS.
// scratch half: [world src][rows per rank][HV] line pairs, then [rows][HV] line pairs
// ---------------------------------------------------------------------------
template <typename T, int NG>
struct FusedTwoShotLLNorm {
  static __device__ void body(const CommCtx& c, int rank, const FusedNormArgs& a, const Blk& b,
                              u64 seq, int& s_abort) {
    constexpr int E = 16 / sizeof(T);
    __shared__ float smem[32];
    const int HV = a.hidden / E;
    const int per = (a.rows + NG - 1) / NG;  // rows per rank, as split_span deals them out
    const size_t base = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const size_t p2 = base + (size_t)NG * per * HV * 32;
    const uint32_t e = ll_flag(seq);
    const T* in = reinterpret_cast<const T*>(a.in);
    const T* w = reinterpret_cast<const T*>(a.weight);
    (void)s_abort;
    auto to_lines = [&](const V16& x, V16& l0, V16& l1) {
      l0.w[0] = x.w[0]; l0.w[1] = e; l0.w[2] = x.w[1]; l0.w[3] = e;
      l1.w[0] = x.w[2]; l1.w[1] = e; l1.w[2] = x.w[3]; l1.w[3] = e;
    };
    for (size_t row = b.bid; row < (size_t)a.rows; row += b.nblocks) {
      const int owner = (int)(row / per), lrow = (int)(row % per);
      bool ok = true;
      if (owner != rank) {
        // my partial of the row -> its owner (unless the GEMM that produced it already did)
        for (int v = threadIdx.x; v < HV && !a.pushed; v += blockDim.x) {
          V16 l0, l1;
          to_lines(ld16(in + row * a.hidden + (size_t)v * E), l0, l1);
          char* dst = c.heap[owner] + base + (((size_t)rank * per + lrow) * HV + v) * 32;
          st16_volatile(dst, l0);
          st16_volatile(dst + 16, l1);
        }
        // the finished row comes back the same way
        T* out = reinterpret_cast<T*>(a.out) + row * (size_t)a.hidden;
        for (int v = threadIdx.x; v < HV && ok; v += blockDim.x) {
          const char* src = c.heap[rank] + p2 + ((size_t)row * HV + v) * 32;
          V16 l0 = ld16_volatile(src), l1 = ld16_volatile(src + 16), x;
          ok = ll_finish_line(src, e, l0, c, owner, b.bid) && ll_finish_line(src + 16, e, l1, c, owner, b.bid);
          x.w[0] = l0.w[0]; x.w[1] = l0.w[2]; x.w[2] = l1.w[0]; x.w[3] = l1.w[2];
          if (ok) st16(out + (size_t)v * E, x);
        }
        if (__syncthreads_or(ok ? 0 : 1)) return;
        continue;
      }
      // owner: the world's partials in rank order + residual
      float z[kMaxVecPerThread][E];
      int nv = 0;
#pragma unroll
      for (int k = 0; k < kMaxVecPerThread; ++k) {
        const int v = threadIdx.x + k * blockDim.x;
        if (v < HV) {
          nv = k + 1;
#pragma unroll
          for (int i = 0; i < E; ++i) z[k][i] = 0.f;
          // first loads of every peer's lines back to back; then wait for the late ones
          V16 l0[NG], l1[NG];
#pragma unroll
          for (int s = 0; s < NG; ++s) {
            if (s != rank) {
              const char* src = c.heap[rank] + base + (((size_t)s * per + lrow) * HV + v) * 32;
              l0[s] = ld16_volatile(src);
              l1[s] = ld16_volatile(src + 16);
            }
          }
#pragma unroll
          for (int s = 0; s < NG; ++s) {
            V16 x;
            if (s == rank) {
              x = ld16(in + row * a.hidden + (size_t)v * E);
            } else {
              const char* src = c.heap[rank] + base + (((size_t)s * per + lrow) * HV + v) * 32;
              ok = ok && ll_finish_line(src, e, l0[s], c, s, b.bid);
              ok = ok && ll_finish_line(src + 16, e, l1[s], c, s, b.bid);
              x.w[0] = l0[s].w[0]; x.w[1] = l0[s].w[2]; x.w[2] = l1[s].w[0]; x.w[3] = l1[s].w[2];
            }
            unpack_add<T>(x, z[k]);
          }
          if (a.residual)
            unpack_add<T>(ld16(reinterpret_cast<const T*>(a.residual) + row * a.hidden + (size_t)v * E), z[k]);
        }
      }
      if (__syncthreads_or(ok ? 0 : 1)) return;
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < kMaxVecPerThread; ++k) {
        if (k < nv) {
#pragma unroll
          for (int i = 0; i < E; ++i) ss += z[k][i] * z[k][i];
        }
      }
      ss = block_sum(ss, smem);
      const float rstd = rsqrtf(ss / (float)a.hidden + a.eps);
      T* out = reinterpret_cast<T*>(a.out) + row * (size_t)a.hidden;
      T* rout = a.residual_out ? reinterpret_cast<T*>(a.residual_out) + row * (size_t)a.hidden : nullptr;
#pragma unroll
      for (int k = 0; k < kMaxVecPerThread; ++k) {
        if (k < nv) {
          const int v = threadIdx.x + k * blockDim.x;
          if (rout) st16(rout + (size_t)v * E, pack<T>(z[k]));
          float wf[E], o[E];
          unpack_set<T>(ld16(w + (size_t)v * E), wf);
#pragma unroll
          for (int i = 0; i < E; ++i) o[i] = z[k][i] * rstd * wf[i];
          const V16 xo = pack<T>(o);
          st16(out + (size_t)v * E, xo);
          V16 l0, l1;
          to_lines(xo, l0, l1);
          const size_t off = p2 + ((size_t)row * HV + v) * 32;
#if !defined(PENNY_HOST_SIM)
          if (c.mc != nullptr) {
            mm_st(c.mc + off, l0);  // one store, every rank's copy
            mm_st(c.mc + off + 16, l1);
            continue;
          }
#endif
#pragma unroll
          for (int d = 1; d < NG; ++d) {
            char* dst = c.heap[(rank + d) % NG] + off;
            st16_volatile(dst, l0);
            st16_volatile(dst + 16, l1);
          }
        }
      }
    }
  }
  static __device__ void run(const CommCtx& c, int rank, const FusedNormArgs& a, const Blk& b) {
    run_collective<FusedTwoShotLLNorm<T, NG>, FusedNormArgs>(c, rank, a, b);
  }
};

// Two transports through the switch:
//   two-shot  rows are sharded over the ranks; the owner pulls the switch-reduced
//             row, normalises it and multicasts the result (multimem.st) into every
//             rank's `out`; a second flag exchange tells the peers that the rows
//             have landed.  The residual stream stays sharded (a rank keeps the
//             residual of the rows it owns).  Least wire traffic.
//   one-shot  every rank pulls ALL rows switch-reduced and normalises them itself:
//             one flag exchange and one round trip instead of two of each, `world`
//             times the wire bytes, no multicast store, `out` is ordinary local
//             memory and the residual stream is replicated.  There is no trailing
//             barrier: a peer may still be reading this rank's `in` when the call
//             returns, so CONSECUTIVE CALLS MUST ALTERNATE BETWEEN TWO INPUT
//             BUFFERS (a rank can be at most one call ahead of any other: it cannot
//             pass the opening barrier of call k + 1 before every rank has finished
//             call k).  For a handful of rows (decode batches up to ~32).
// Launched with programmatic stream serialization: the norm weight (a constant)
// is fetched and the block is resident before the producing GEMM has finished.
template <typename T, bool ONESHOT>
__global__ void __launch_bounds__(512) k_fused_nvls_norm(const CommCtx c, const FusedNormArgs a) {
  constexpr int E = 16 / sizeof(T);
  __shared__ float smem[32];
  __shared__ int s_abort;
  pdl_launch_dependents();
  const int rank = c.rank;
  const Blk b{(int)blockIdx.x, (int)gridDim.x, (int)blockDim.x};
  const int HV = a.hidden / E;
  const T* w = reinterpret_cast<const T*>(a.weight);
  V16 wv[kMaxVecPerThread];
#pragma unroll
  for (int k = 0; k < kMaxVecPerThread; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v < HV) wv[k] = ld16(w + (size_t)v * E);
  }
  if (threadIdx.x == 0) s_abort = 0;
  pdl_wait();  // the partial sums of this rank are complete; the call counter is final
  const u64 seq = begin_call(c, rank, SEQ_ALL);
  PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
  if (!s_abort) {
    Span mine = split_span((size_t)a.rows, c.world, rank);
    if (ONESHOT) {
      mine.begin = 0;
      mine.end = (size_t)a.rows;
    }
    for (size_t row = mine.begin + b.bid; row < mine.end; row += b.nblocks) {
      float z[kMaxVecPerThread][E];
      V16 red[kMaxVecPerThread], res[kMaxVecPerThread];
      int nv = 0;
      // every load of the row is in flight before the first one is used
#pragma unroll
      for (int k = 0; k < kMaxVecPerThread; ++k) {
        const int v = threadIdx.x + k * blockDim.x;
        if (v < HV) {
          nv = k + 1;
          const size_t eoff = (row * a.hidden + (size_t)v * E) * sizeof(T);
          red[k] = mm_ld_reduce<T>(c.mc + a.in_heap_off + eoff);
          if (a.residual) res[k] = ld16(reinterpret_cast<const T*>(a.residual) + row * a.hidden + (size_t)v * E);
        }
      }
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < kMaxVecPerThread; ++k) {
        if (k < nv) {
          unpack_set<T>(red[k], z[k]);
          if (a.residual) unpack_add<T>(res[k], z[k]);
#pragma unroll
          for (int i = 0; i < E; ++i) ss += z[k][i] * z[k][i];
        }
      }
      ss = block_sum(ss, smem);
      const float rstd = rsqrtf(ss / (float)a.hidden + a.eps);
      T* rout = a.residual_out ? reinterpret_cast<T*>(a.residual_out) + row * (size_t)a.hidden : nullptr;
#pragma unroll
      for (int k = 0; k < kMaxVecPerThread; ++k) {
        if (k < nv) {
          const int v = threadIdx.x + k * blockDim.x;
          if (rout) st16(rout + (size_t)v * E, pack<T>(z[k]));
          float wf[E], o[E];
          unpack_set<T>(wv[k], wf);
#pragma unroll
          for (int i = 0; i < E; ++i) o[i] = z[k][i] * rstd * wf[i];
          if (ONESHOT) {
            st16(reinterpret_cast<T*>(a.out) + row * (size_t)a.hidden + (size_t)v * E, pack<T>(o));
          } else {
            const size_t eoff = (row * a.hidden + (size_t)v * E) * sizeof(T);
            mm_st(c.mc + a.out_heap_off + eoff, pack<T>(o));
          }
        }
      }
    }
    if (!ONESHOT) PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 2), s_abort);
  }
  end_call(c, rank, b, seq, SEQ_ALL);
}

static bool shape_ok(int dtype, const FusedNormArgs& a, int threads) {
  const int E = 16 / dtype_size(dtype);
  if (a.hidden % E != 0) return false;
  return a.hidden / E <= kMaxVecPerThread * threads && a.rows >= 1;
}

cudaError_t launch_add_rmsnorm(int dtype, const FusedNormArgs& a, int blocks, int threads,
                               cudaStream_t stream) {
  if (!shape_ok(dtype, a, threads)) return cudaErrorInvalidValue;
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, rc = launch_kernel_ex(k_add_rmsnorm<T>, dim3(blocks), dim3(threads), 0, stream, true, 1, a));
  return rc;
}

cudaError_t launch_fused_ar_rmsnorm(int dtype, int proto, const CommCtx& c, const FusedNormArgs* a,
                                    const LaunchCfg& cfg) {
  if (!shape_ok(dtype, a[0], cfg.threads)) return cudaErrorInvalidValue;
  cudaError_t rc = cudaErrorInvalidValue;
  if (proto == FUSED_PROTO_NVLS || proto == FUSED_PROTO_NVLS_ONESHOT) {
    const bool oneshot = proto == FUSED_PROTO_NVLS_ONESHOT;
    if (c.mc == nullptr || cfg.emu_world > 0 || a[0].in_heap_off == kNotInHeap ||
        (!oneshot && a[0].out_heap_off == kNotInHeap))
      return cudaErrorNotSupported;
    if (cfg.blocks < 1 || cfg.blocks > kMaxBlocks || cfg.threads < 32 || cfg.threads > 512)
      return cudaErrorInvalidConfiguration;
    PENNY_DISPATCH_DTYPE(dtype, T, {
      rc = oneshot ? launch_kernel_ex(k_fused_nvls_norm<T, true>, dim3(cfg.blocks), dim3(cfg.threads), 0, cfg.stream,
                                      true, 1, c, a[0])
                   : launch_kernel_ex(k_fused_nvls_norm<T, false>, dim3(cfg.blocks), dim3(cfg.threads), 0, cfg.stream,
                                      true, 1, c, a[0]);
    });
    return rc;
  }
  if (proto == FUSED_PROTO_LL_TWOSHOT) {
    PENNY_DISPATCH_DTYPE(dtype, T, PENNY_DISPATCH_WORLD(c.world, NG, return cudaErrorInvalidValue, {
      rc = launch_body<FusedTwoShotLLNorm<T, NG>, FusedNormArgs>(c, a, cfg);
    }));
    return rc;
  }
  PENNY_DISPATCH_DTYPE(dtype, T, PENNY_DISPATCH_WORLD(c.world, NG, return cudaErrorInvalidValue, {
    rc = (proto == FUSED_PROTO_LL)
             ? launch_body<FusedOneShotNorm<T, NG, true>, FusedNormArgs>(c, a, cfg)
             : launch_body<FusedOneShotNorm<T, NG, false>, FusedNormArgs>(c, a, cfg);
  }));
  return rc;
}

}  // namespace penny
