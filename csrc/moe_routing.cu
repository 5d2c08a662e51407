// Expert-parallel MoE routing on the device: everything between the router's logits and the
// dispatch kernel's tables, without a sort, a histogram pass or a host round trip per table.
//
//   k_moe_topk       one thread per token: top-k experts of its logits (ties: lowest expert id, as
//                    torch.topk does on distinct values) and the softmax of the selected logits.
//   k_moe_tables     one block: stable counting sort of the (token, k) pairs by expert.  Pairs are
//                    taken 1024 at a time in their original order; inside a tile a pair's rank among
//                    the pairs of the same expert is (pairs of that expert in lower warps) + (lower
//                    lanes of its own warp that hold the same expert, from __match_any_sync), so the
//                    order of equal keys is the original order.  Outputs: order[P] (pair index by
//                    sorted position), expert_sorted[P], send_off[E + 1], counts[E].
//   k_moe_placement  one block: from every rank's counts (counts_all[W][E]) the row where each
//                    (source rank, expert) block starts at the expert's owner - rows ordered by
//                    local expert, then by source rank - plus rows per rank and per-expert ranges.
//
// The reference has no MoE path (its exchange is a pairwise swap, csrc/exchange.cu); these tables
// are what csrc/moe_dispatch_combine.cu consumes.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "moe_routing.h"

namespace penny {
namespace {

constexpr int kRouteThreads = 1024;
constexpr int kRouteWarps = kRouteThreads / 32;

__global__ void k_moe_topk(const __nv_bfloat16* __restrict__ logits, int tokens, int experts, int topk,
                           int* __restrict__ ids, float* __restrict__ gates) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const __nv_bfloat16* row = logits + (size_t)t * experts;
  float best[kMoeMaxTopk];
  int bi[kMoeMaxTopk];
  for (int k = 0; k < topk; ++k) {
    float bv = -INFINITY;
    int be = 0;
    for (int e = 0; e < experts; ++e) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= (bi[j] == e);
      const float v = __bfloat162float(row[e]);
      if (!taken && v > bv) {
        bv = v;
        be = e;
      }
    }
    best[k] = bv;
    bi[k] = be;
  }
  // softmax over the selected logits
  const float top = best[0];
  float sum = 0.f;
  for (int k = 0; k < topk; ++k) {
    best[k] = __expf(best[k] - top);
    sum += best[k];
  }
  for (int k = 0; k < topk; ++k) {
    ids[(size_t)t * topk + k] = bi[k];
    gates[(size_t)t * topk + k] = best[k] / sum;
  }
}

__global__ void __launch_bounds__(kRouteThreads) k_moe_tables(const int* __restrict__ ids, int pairs, int experts,
                                                              int* __restrict__ order, int* __restrict__ expert_sorted,
                                                              int* __restrict__ send_off, int* __restrict__ counts) {
  extern __shared__ int sm[];
  int* hist = sm;                       // [E] pairs per expert, then the running write position
  int* warp_cnt = sm + experts;         // [warps][E] of the current tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  // ids outside [0, experts) are left out of every table (they would index past the histogram)
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if ((unsigned)e < (unsigned)experts) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      const int c = hist[e];
      counts[e] = c;
      send_off[e] = run;
      hist[e] = run;  // next free sorted position of expert e
      run += c;
    }
    send_off[experts] = run;
  }
  __syncthreads();
  for (int base = 0; base < pairs; base += kRouteThreads) {
    for (int i = threadIdx.x; i < kRouteWarps * experts; i += blockDim.x) warp_cnt[i] = 0;
    __syncthreads();
    const int p = base + threadIdx.x;
    const int id = p < pairs ? ids[p] : -1;
    const bool live = (unsigned)id < (unsigned)experts;
    const int e = live ? id : -1 - lane;  // dead lanes never match anyone
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (live && rank_in_warp == 0) warp_cnt[warp * experts + e] = __popc(same);
    __syncthreads();
    if (live) {
      int before = 0;
      for (int w = 0; w < warp; ++w) before += warp_cnt[w * experts + e];
      const int pos = hist[e] + before + rank_in_warp;
      order[pos] = p;
      expert_sorted[pos] = e;
    }
    __syncthreads();
    // advance the experts' write positions by this tile's totals
    for (int x = threadIdx.x; x < experts; x += blockDim.x) {
      int tot = 0;
      for (int w = 0; w < kRouteWarps; ++w) tot += warp_cnt[w * experts + x];
      hist[x] += tot;
    }
    __syncthreads();
  }
}

__global__ void k_moe_placement(const int* __restrict__ counts_all, int world, int experts, int* __restrict__ dst_base,
                                int* __restrict__ rows_per_rank, int* __restrict__ expert_ranges) {
  // one thread per destination rank: a few hundred additions at most
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= world) return;
  const int epr = experts / world;
  int base = 0;
  for (int le = 0; le < epr; ++le) {
    const int e = d * epr + le;
    expert_ranges[2 * e] = base;
    for (int s = 0; s < world; ++s) {
      dst_base[s * experts + e] = base;
      base += counts_all[s * experts + e];
    }
    expert_ranges[2 * e + 1] = base;
  }
  rows_per_rank[d] = base;
}

}  // namespace

cudaError_t launch_moe_topk(const void* logits, int tokens, int experts, int topk, int* ids, float* gates,
                            cudaStream_t stream) {
  if (tokens <= 0 || experts <= 0 || topk <= 0 || topk > kMoeMaxTopk || topk > experts) return cudaErrorInvalidValue;
  k_moe_topk<<<(tokens + 127) / 128, 128, 0, stream>>>((const __nv_bfloat16*)logits, tokens, experts, topk, ids, gates);
  return cudaGetLastError();
}

cudaError_t launch_moe_tables(const int* ids, int pairs, int experts, int* order, int* expert_sorted, int* send_off,
                              int* counts, cudaStream_t stream) {
  if (pairs <= 0 || experts <= 0 || experts > kMoeMaxExperts) return cudaErrorInvalidValue;
  const size_t smem = (size_t)(1 + kRouteWarps) * experts * sizeof(int);
  k_moe_tables<<<1, kRouteThreads, smem, stream>>>(ids, pairs, experts, order, expert_sorted, send_off, counts);
  return cudaGetLastError();
}

cudaError_t launch_moe_placement(const int* counts_all, int world, int experts, int* dst_base, int* rows_per_rank,
                                 int* expert_ranges, cudaStream_t stream) {
  if (world <= 0 || experts <= 0 || experts % world != 0) return cudaErrorInvalidValue;
  k_moe_placement<<<(world + 31) / 32, 32, 0, stream>>>(counts_all, world, experts, dst_base, rows_per_rank,
                                                         expert_ranges);
  return cudaGetLastError();
}

}  // namespace penny
