// Expert-parallel MoE token exchange over the symmetric heap.
//
//   dispatch  every (token, k) pair whose expert lives on rank d is pushed, as one
//             hidden-sized row, straight into rank d's expert-input buffer at the
//             row the routing tables assign to it (rows of one expert are
//             contiguous and ordered by source rank, so the expert GEMM runs on a
//             dense [rows, hidden] matrix with no padding and no compaction),
//             together with a 4-byte return address (source rank, pair index).
//   combine   each expert output row is pushed back to its source into the slot
//             of its (token, k) pair; after the all-rank barrier the same kernel
//             forms out[t] = sum_k gate[t, k] * y[t, k] in fp32 – the all-to-all
//             and the gate-weighted reduction are one launch.  Pairs whose expert
//             is local are read in place and never travel.
//
// The receive buffers are symmetric heap tensors owned by the caller (expert
// input rows, return addresses, combine slots), so the host knows where the
// expert GEMM finds its input.  Writing into a peer's user-visible buffer needs a
// start barrier ("the peer has entered this call, nothing earlier still reads
// the buffer") and the end barrier is "every block of every peer has flagged",
// since a row may be produced by any block of its source.  Flag values come from
// the communicator's call sequence like everywhere else.  Same all-to-all data movement
// as AllToAll in exchange.cuh but routed row by row.  The reference only has the
// pairwise exchange (csrc/exchange.cu) and no MoE path.
#include "algos.h"
#include "fused_ops.h"
#include "launch.cuh"

namespace penny {

namespace {

// Waits until every block of every OTHER rank has flagged `val` on CH_BARRIER.
// Called by all threads; returns false (uniformly) after a timeout.
__device__ __forceinline__ bool all_blocks_barrier(const CommCtx& c, int rank, const Blk& b, u64 val,
                                                   int& s_abort) {
  __syncthreads();  // this block's pushes are issued
  if ((int)threadIdx.x < c.world && (int)threadIdx.x != rank)
    signal_peer(c, rank, threadIdx.x, CH_BARRIER, b, val);
  for (int idx = threadIdx.x; idx < b.nblocks * c.world; idx += blockDim.x) {
    const int bb = idx / c.world, p = idx % c.world;
    if (p == rank) continue;
    if (!wait_flag_ge(&pad_of(c, rank)->flag[CH_BARRIER][bb][p], val, c, ST_TIMEOUT_BARRIER, p, bb))
      s_abort = 1;
  }
  __syncthreads();
  return s_abort == 0;
}

template <typename T>
struct MoeDispatch {
  // a.recv_off: rows [cap_rows][hidden] T; a.meta_off: [cap_rows] int32 (both symmetric)
  static __device__ void body(const CommCtx& c, int rank, const MoeArgs& a, const Blk& b, u64 seq,
                              int& s_abort) {
    constexpr int E = 16 / sizeof(T);
    const int HV = a.hidden / E;
    const size_t half = a.recv_off;
    const size_t meta_off = a.meta_off;
    PK_BLOCK_BARRIER(c, rank, CH_DATA, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;
    const T* x = reinterpret_cast<const T*>(a.x);
    const int pairs = a.tokens * a.topk;
    const int experts_per_rank = a.experts / c.world;
    // one warp per row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int i = b.bid * nwarps + warp; i < pairs; i += b.nblocks * nwarps) {
      const int pair = a.order[i];
      const int e = a.expert_of_sorted[i];
      const int d = e / experts_per_rank;
      const int dst_row = a.dst_base[e] + (i - a.send_off[e]);
      if (lane == 0) a.dst_row_of_pair[pair] = dst_row;
      if (dst_row >= a.cap_rows) {
        if (lane == 0) report_status(c, ST_BAD_ARGS, d, b.bid, (u64)dst_row, (u64)a.cap_rows);
        continue;
      }
      const T* src = x + (size_t)(pair / a.topk) * a.hidden;
      char* dst = c.heap[d] + half + (size_t)dst_row * a.hidden * sizeof(T);
      for (int v0 = lane; v0 < HV; v0 += kBatch * 32) {
        V16 r[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          if (v0 + u * 32 < HV) r[u] = ld16(src + (size_t)(v0 + u * 32) * E);
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          if (v0 + u * 32 < HV) st16(dst + (size_t)(v0 + u * 32) * 16, r[u]);
      }
      if (lane == 0)
        *reinterpret_cast<int*>(c.heap[d] + meta_off + (size_t)dst_row * 4) = rank * pairs + pair;
    }
    all_blocks_barrier(c, rank, b, flag_value(seq, 2), s_abort);
  }
  static __device__ void run(const CommCtx& c, int rank, const MoeArgs& a, const Blk& b) {
    run_collective<MoeDispatch<T>, MoeArgs>(c, rank, a, b);
  }
};

template <typename T>
struct MoeCombine {
  // a.comb_off: [tokens * topk][hidden] T (symmetric)
  static __device__ void body(const CommCtx& c, int rank, const MoeArgs& a, const Blk& b, u64 seq,
                              int& s_abort) {
    constexpr int E = 16 / sizeof(T);
    const int HV = a.hidden / E;
    const size_t half = a.comb_off;
    PK_BLOCK_BARRIER(c, rank, CH_DATA, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;
    const T* y = reinterpret_cast<const T*>(a.x);  // expert outputs, rows as received
    const int pairs = a.tokens * a.topk;
    const int experts_per_rank = a.experts / c.world;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    // push every remote-sourced row back to its (source, pair) slot
    for (int j = b.bid * nwarps + warp; j < a.recv_rows; j += b.nblocks * nwarps) {
      const int m = a.meta[j];
      const int s = m / pairs, pair = m - s * pairs;
      if (s == rank) continue;  // local pairs are read in place below
      const T* src = y + (size_t)j * a.hidden;
      char* dst = c.heap[s] + half + (size_t)pair * a.hidden * sizeof(T);
      for (int v0 = lane; v0 < HV; v0 += kBatch * 32) {
        V16 r[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          if (v0 + u * 32 < HV) r[u] = ld16(src + (size_t)(v0 + u * 32) * E);
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          if (v0 + u * 32 < HV) st16(dst + (size_t)(v0 + u * 32) * 16, r[u]);
      }
    }
    if (!all_blocks_barrier(c, rank, b, flag_value(seq, 2), s_abort)) return;
    // out[t] = sum_k gate[t, k] * y[t, k]
    T* out = reinterpret_cast<T*>(a.out);
    for (int t = b.bid * nwarps + warp; t < a.tokens; t += b.nblocks * nwarps) {
      for (int v = lane; v < HV; v += 32) {
        float acc[E];
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = 0.f;
        for (int k = 0; k < a.topk; ++k) {
          const int pair = t * a.topk + k;
          const int e = a.topk_ids[pair];
          const float g = a.gates[pair];
          const char* src = (e / experts_per_rank == rank)
                                ? reinterpret_cast<const char*>(y + (size_t)a.dst_row_of_pair[pair] * a.hidden)
                                : c.heap[rank] + half + (size_t)pair * a.hidden * sizeof(T);
          float r[E];
          unpack_set<T>(ld16(src + (size_t)v * 16), r);
#pragma unroll
          for (int i = 0; i < E; ++i) acc[i] += g * r[i];
        }
        st16(out + (size_t)t * a.hidden + (size_t)v * E, pack<T>(acc));
      }
    }
  }
  static __device__ void run(const CommCtx& c, int rank, const MoeArgs& a, const Blk& b) {
    run_collective<MoeCombine<T>, MoeArgs>(c, rank, a, b);
  }
};

}  // namespace

cudaError_t launch_moe_dispatch(int dtype, const CommCtx& c, const MoeArgs* a, const LaunchCfg& cfg) {
  if (a[0].hidden % (16 / dtype_size(dtype)) != 0 || a[0].experts % c.world != 0)
    return cudaErrorInvalidValue;
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, rc = (launch_body<MoeDispatch<T>, MoeArgs>(c, a, cfg)));
  return rc;
}

cudaError_t launch_moe_combine(int dtype, const CommCtx& c, const MoeArgs* a, const LaunchCfg& cfg) {
  if (a[0].hidden % (16 / dtype_size(dtype)) != 0 || a[0].experts % c.world != 0)
    return cudaErrorInvalidValue;
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, rc = (launch_body<MoeCombine<T>, MoeArgs>(c, a, cfg)));
  return rc;
}

}  // namespace penny
