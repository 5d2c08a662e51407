// Work split of the decode GEMM (gemm_decode_sm100.cu): plain C++, used by the
// kernel, by its launcher and (through the host simulator library) by the CPU
// tests.
//
//   out[B, N] = x[B, K] W[N, K]^T for a decode batch (one slab of B <= 128 rows; larger batches run
//   their slabs as grid z of the same launch, so the slabs of a weight tile read it from L2 together).
//   * one CTA per (weight tile of 128 rows, K range); the `splits` CTAs of a tile
//     form one thread-block cluster and reduce their fp32 partials through
//     distributed shared memory: no global workspace, no counters, no fix-up pass;
//   * the K steps (64 elements each) are dealt out as `splits` contiguous ranges
//     whose sizes differ by at most one;
//   * after its MMAs a CTA keeps the accumulator columns (= batch rows) of its
//     own slice and sends every other slice to the CTA that owns it: CTA r owns
//     columns [r * slice, min(bt, (r + 1) * slice)) of the bt-wide batch tile.
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define PENNY_PLAN_HD __host__ __device__ inline
#else
#define PENNY_PLAN_HD inline
#endif

namespace penny {
namespace sm100 {

constexpr int kDecodeMaxSplits = 8;  // portable cluster size
constexpr int kDecodeMaxBatch = 1024;  // rows of x per launch

PENNY_PLAN_HD int decode_kb_begin(int num_kb, int splits, int r) {
  return (int)((long long)num_kb * r / splits);
}
// columns of the batch tile owned by one CTA of the cluster
PENNY_PLAN_HD int decode_slice(int bt, int splits) { return (bt + splits - 1) / splits; }
// slot of source CTA `src` in the receive area of CTA `dst` (src != dst): sources in rank order, dst left out
PENNY_PLAN_HD int decode_recv_slot(int src, int dst) { return src - (src > dst ? 1 : 0); }
// fp32 words of the receive area: [splits - 1][slice][128 rows]
PENNY_PLAN_HD size_t decode_recv_floats(int bt, int splits) {
  if (splits <= 1) return 0;
  return (size_t)(splits - 1) * (size_t)decode_slice(bt, splits) * 128;
}

// The cluster size (K ranges per weight tile), from measurements on B200 at batch 64
// (cluster sizes 1-8 timed on every shard shape of a Llama-3-8B layer at TP 1, 2, 4, 8):
//   * what a decode GEMM needs is enough CTAs streaming at once - about two per SM,
//     each with three or four 16 KB weight stages in flight;
//   * all CTAs must be resident together: `capacity[s]` is the number of CTAs the
//     GPU holds at once when they come in clusters of s (the launcher asks the
//     occupancy API; clusters must fit a GPC, so it is a little below 2 x SMs).  A
//     second wave costs far more than a smaller cluster;
//   * a K range shorter than 6 steps (384 elements) is not worth a cluster: the
//     reduction then costs more than the shorter stream saves.
// So: the largest s <= 8 with tiles * s <= capacity[s] and num_kb / s >= 6; 1 when
// nothing larger qualifies (narrow K, or more tiles than fit at once).
PENNY_PLAN_HD int decode_choose_splits(int tiles, int num_kb, const int* capacity) {
  int best = 1;
  for (int s = 2; s <= kDecodeMaxSplits; ++s) {
    if (num_kb / s < 6) break;
    if ((long long)tiles * s <= (long long)capacity[s]) best = s;
  }
  return best;
}

// capacity[] stand-in for a GPU of `sms` SMs in GPCs of `gpc_sms`, two CTAs per SM,
// whole clusters per GPC (used by the CPU tests; the launcher uses the real figure).
PENNY_PLAN_HD void decode_model_capacity(int sms, int gpc_sms, int* capacity) {
  capacity[0] = 0;
  for (int s = 1; s <= kDecodeMaxSplits; ++s) {
    const int gpcs = sms / gpc_sms, rest = sms - gpcs * gpc_sms;
    capacity[s] = (gpcs * ((2 * gpc_sms) / s) + (2 * rest) / s) * s;
  }
}

}  // namespace sm100
}  // namespace penny
