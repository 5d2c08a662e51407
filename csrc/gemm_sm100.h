// Host API of the tcgen05 GEMM family (csrc/gemm_sm100.cu and the fused variants).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace penny {
namespace sm100 {

// TMA descriptor of a row-major [rows, cols] bf16 matrix cut into
// [box_rows x 64] tiles with the 128-byte swizzle.  base must be 16-byte
// aligned and the row stride a multiple of 8 elements.
cudaError_t make_tile_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                          uint64_t row_stride_elems, uint32_t box_rows);

// C[M, N] = A[M, K] * B[N, K]^T, bf16, row-major with leading dimensions lda /
// ldb / ldc (elements).  K, lda, ldb multiples of 8.  block_n: 0 (choose), 128, 192 or
// 256 (one CTA per 128 x block_n tile), or 512 = 256 x 256 tiles computed by CTA
// pairs (cta_group::2).  error_word: device word that receives a GemmError code if a pipeline
// wait runs out (stays 0 otherwise).
cudaError_t launch_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, int lda,
                             int ldb, int ldc, int block_n, uint32_t* error_word,
                             cudaStream_t stream);

// False when PENNY_GEMM_PAIR=0 forces the single-CTA kernels everywhere.
bool pair_kernel_enabled();
// Whether the ragged last wave of the pair kernel is split along K over the idle
// pairs.  Off unless PENNY_GEMM_SPLIT_TAIL=1 or set_split_tail(1); set_split_tail(-1)
// goes back to the environment's choice.
bool split_tail_enabled();
void set_split_tail(int on);
// The block_n that launch_gemm_bf16(block_n = 0) would use (128, 192, 256 or 512 = CTA pairs).
int choose_block_n(int M, int N, int K, int sms, int pairs);

}  // namespace sm100
}  // namespace penny
