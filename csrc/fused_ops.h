// Argument blocks and entry points of the fused (collective + consumer) kernels.
#pragma once
#include <cuda_runtime.h>

#include "coll_args.h"

namespace penny {

struct LaunchCfg;

enum FusedProto : int { FUSED_PROTO_LL = 0, FUSED_PROTO_FLAG = 1, FUSED_PROTO_NVLS = 2 };

// all-reduce + residual add + RMSNorm over [rows, hidden]
struct FusedNormArgs {
  const void* in;        // this rank's partial sums
  const void* residual;  // residual stream in, or null
  const void* weight;    // [hidden]
  void* out;             // normalised rows
  void* residual_out;    // sum + residual (may alias `residual`), or null
  int rows;
  int hidden;
  float eps;
  size_t scratch_off;
  size_t scratch_bytes;
  size_t in_heap_off;   // NVLS: offset of `in` in the heap
  size_t out_heap_off;  // NVLS: offset of `out` in the heap
};

// scratch for the one-shot protocols (both halves)
inline size_t fused_norm_scratch_bytes(int proto, int rows, int hidden, int elem_size, int world) {
  size_t v = (size_t)rows * (size_t)(hidden * elem_size / 16);
  return (proto == FUSED_PROTO_LL ? 4 : 2) * (size_t)world * v * 16;
}

cudaError_t launch_add_rmsnorm(int dtype, const FusedNormArgs& a, int blocks, int threads,
                               cudaStream_t stream);
cudaError_t launch_fused_ar_rmsnorm(int dtype, int proto, const CommCtx& c, const FusedNormArgs* a,
                                    const LaunchCfg& cfg);

}  // namespace penny
