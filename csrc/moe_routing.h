// Device-side routing tables of the expert-parallel MoE layer (csrc/moe_routing.cu).
#pragma once
#include <cuda_runtime.h>

namespace penny {

constexpr int kMoeMaxTopk = 8;
constexpr int kMoeMaxExperts = 256;

// logits [tokens, experts] bf16 -> ids [tokens, topk] int32 (best first), gates [tokens, topk] fp32
// (softmax over the selected logits).
cudaError_t launch_moe_topk(const void* logits, int tokens, int experts, int topk, int* ids, float* gates,
                            cudaStream_t stream);
// ids [pairs] -> stable sort by expert: order[pairs] (pair index at each sorted position),
// expert_sorted[pairs], send_off[experts + 1] (exclusive prefix of counts), counts[experts].
cudaError_t launch_moe_tables(const int* ids, int pairs, int experts, int* order, int* expert_sorted, int* send_off,
                              int* counts, cudaStream_t stream);
// counts_all [world, experts] -> dst_base [world, experts] (row at the expert's owner where the rows of
// (source rank, expert) start; rows ordered by local expert, then source rank), rows_per_rank [world],
// expert_ranges [experts, 2] (start, end at the owner).
cudaError_t launch_moe_placement(const int* counts_all, int world, int experts, int* dst_base, int* rows_per_rank,
                                 int* expert_ranges, cudaStream_t stream);

}  // namespace penny
