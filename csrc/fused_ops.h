// Argument blocks and entry points of the fused (collective + consumer) kernels.
#pragma once
#include <cuda_runtime.h>

#include "coll_args.h"

namespace penny {

struct LaunchCfg;

enum FusedProto : int {
  FUSED_PROTO_LL = 0,
  FUSED_PROTO_FLAG = 1,
  FUSED_PROTO_NVLS = 2,
  FUSED_PROTO_NVLS_ONESHOT = 3,
  FUSED_PROTO_LL_TWOSHOT = 4,
};

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
  int pushed;           // LL two-shot: the producing GEMM already wrote the partial rows of the
                        // other ranks into their receive lines (DecodePush): nothing to push here
};

// scratch for the one-shot protocols (both halves)
inline size_t fused_norm_scratch_bytes(int proto, int rows, int hidden, int elem_size, int world) {
  const size_t hv = (size_t)(hidden * elem_size / 16);
  if (proto == FUSED_PROTO_LL_TWOSHOT) {
    // per half: line pairs of [world][rows per rank][hv] partials and of [rows][hv] finished rows
    const size_t per = (size_t)(rows + world - 1) / world;
    return 2 * ((size_t)world * per + (size_t)rows) * hv * 32;
  }
  size_t v = (size_t)rows * hv;
  return (proto == FUSED_PROTO_LL ? 4 : 2) * (size_t)world * v * 16;
}

// MoE expert-parallel dispatch / combine (csrc/moe_dispatch_combine.cu).
// Routing tables (device int32 arrays of this rank):
//   order[i]            pair index (t * topk + k) of the i-th pair when sorted by expert
//   expert_of_sorted[i] its expert
//   send_off[e]         first sorted position of expert e (prefix sums, [experts + 1])
//   dst_base[e]         row at expert e's owner where this rank's rows of e start
//   dst_row_of_pair[p]  (written by dispatch) row of pair p at its expert's owner
struct MoeArgs {
  const void* x;         // dispatch: tokens [tokens, hidden]; combine: expert outputs [recv_rows, hidden]
  void* out;             // combine: [tokens, hidden]
  const int* order;
  const int* expert_of_sorted;
  const int* send_off;
  const int* dst_base;
  int* dst_row_of_pair;
  const int* topk_ids;   // [tokens * topk]
  const float* gates;    // [tokens * topk]
  const int* meta;       // combine: this rank's copy of the return addresses [recv_rows]
  size_t recv_off;       // heap offset of the symmetric receive rows [cap_rows, hidden]
  size_t meta_off;       // heap offset of the symmetric return addresses [cap_rows] int32
  size_t comb_off;       // heap offset of the symmetric combine slots [tokens * topk, hidden]
  int tokens, topk, hidden, experts, cap_rows, recv_rows;
};
cudaError_t launch_moe_dispatch(int dtype, const CommCtx& c, const MoeArgs* a, const LaunchCfg& cfg);
cudaError_t launch_moe_combine(int dtype, const CommCtx& c, const MoeArgs* a, const LaunchCfg& cfg);

cudaError_t launch_add_rmsnorm(int dtype, const FusedNormArgs& a, int blocks, int threads,
                               cudaStream_t stream);
cudaError_t launch_fused_ar_rmsnorm(int dtype, int proto, const CommCtx& c, const FusedNormArgs* a,
                                    const LaunchCfg& cfg);

}  // namespace penny
