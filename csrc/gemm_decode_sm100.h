// Host API of the decode-batch linear (csrc/gemm_decode_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "decode_gemm_plan.h"

namespace penny {
namespace sm100 {

enum DecodeEpilogue : int {
  DECODE_EPI_PLAIN = 0,
  // W's rows come in blocks of 128 = 64 gate rows followed by the 64 up rows of
  // the same features (N a multiple of 128); out is [B, N / 2] with
  // out[b][blk * 64 + i] = silu(gate) * up.
  DECODE_EPI_SILU_PAIRS = 1,
};

// Epilogue target of a row-parallel linear whose output goes into an all-reduce + RMSNorm of the
// flag-in-data two-shot kind (FUSED_PROTO_LL_TWOSHOT): rows owned by another rank are written
// straight into that rank's receive lines instead of `out`, so the all-reduce kernel has nothing
// to push and starts by polling.  Filled in by Communicator::fused_norm_push_target.
struct DecodePush {
  char* heap[8];                          // every rank's heap as mapped here
  const unsigned long long* call_seq;     // this rank's call counter (device memory)
  size_t scratch_off, scratch_bytes;      // the all-reduce's scratch region (both halves)
  int rank, world;                        // world == 0: unused
  int per;                                // rows per rank = ceil(rows / world)
  int hv;                                 // 16-byte vectors per row = N / 8
};

// out[B, N] = x[B, K] * W[N, K]^T, bf16, row-major with leading dimensions ldx /
// ldw / ldo (elements); 1 <= B <= kDecodeMaxBatch (above 128 rows the batch is cut into slabs of 128, all in this one launch; push: B <= 128); K, ldx, ldw multiples of 8; x, w 16-byte aligned.
//   splits          CTAs per weight tile (cluster size along K), 0 = choose
//   pdl             launch with programmatic stream serialization: the kernel may
//                   start, and load W, while the previous kernel on the stream is
//                   still running.  W must then not be written by that kernel.
//   l2_budget_bytes a whole W no larger than this is prefetched into L2 before the
//                   dependency wait (-1 = default, 0 = only a rolling window)
//   push            null, or where rows owned by other ranks go (see DecodePush); plain epilogue only
//   smem_kb         shared memory the TMA ring may grow to (0 = default: ~106 KB, so
//                   that the next kernel of the step fits on the SM beside this one;
//                   up to 226 for a kernel nothing needs to overlap with)
// Allocates nothing; no workspace; safe to capture.  error_word as in launch_gemm_bf16.
cudaError_t launch_gemm_decode(const void* x, const void* w, void* out, int B, int N, int K, int ldx, int ldw,
                               int ldo, int epi, int splits, bool pdl, long long l2_budget_bytes,
                               int smem_kb, const DecodePush* push, uint32_t* error_word, cudaStream_t stream);

// Diagnostics (PENNY_DEC_STAMPS=1): copies the %globaltimer stamps of the last launch's first CTAs to
// `out` ([ctas][8] nanoseconds: CTA start, prologue done, predecessor complete, last load issued, last
// MMA issued, accumulator complete, peers' partials received, done) and returns the number of CTAs.
int gemm_decode_stamps(unsigned long long* out, int max_ctas);

// CTAs of the decode GEMM the current device holds at once when they come in clusters of `splits`.
int gemm_decode_capacity(int B, int splits);
// The cluster size launch_gemm_decode(splits = 0) uses for this shape on the current device.
int gemm_decode_splits(int B, int N, int K);

}  // namespace sm100
}  // namespace penny
