// Host API of the fused GEMM + collective kernels (csrc/gemm_fused_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "pk.h"

namespace penny {
namespace sm100 {

// Scratch both kernels need in the symmetric heap (bytes, both halves).
size_t gemm_rs_scratch_bytes(int M, int N, int world);
size_t ag_gemm_scratch_bytes(int M, int K);

// out[M / world, N] (this rank's row shard) = sum over ranks of A_r[M, K_r] * B_r[N, K_r]^T.
// M a multiple of world * 128, N a multiple of 256.  scratch: a region shared
// with the other all-dependent collectives (its halves are cut at scratch_bytes / 2).
cudaError_t launch_gemm_rs(const CommCtx& c, size_t scratch_off, size_t scratch_bytes, const void* a,
                           const void* b, void* out, int M, int N, int K, int lda, int ldb, int ldo,
                           uint32_t* error_word, cudaStream_t stream);

// out[M, N] = gather(A shards)[M, K] * B[N, K]^T, a_shard = this rank's [M / world, K] rows.
// scratch: a region dedicated to this (M, K) of exactly ag_gemm_scratch_bytes(M, K).
// side_ctas: ignored (the pushes are done by copy warps inside every CTA).
cudaError_t launch_ag_gemm(const CommCtx& c, size_t scratch_off, size_t scratch_bytes,
                           const void* a_shard, const void* b, void* out, int M, int N, int K, int lda,
                           int ldb, int ldc, int side_ctas, uint32_t* error_word,
                           cudaStream_t stream);

}  // namespace sm100
}  // namespace penny
