// Host API of the weight-streaming decode GEMM (csrc/gemm_skinny_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace penny {
namespace sm100 {

// out[B, N] = x[B, K] * W[N, K]^T, bf16, row-major with leading dimensions ldx /
// ldw / ldo (elements); B <= 128, K, ldx, ldw multiples of 8.
// silu_pairs = 1: W's rows come in blocks of 128 = 64 gate rows followed by the
// 64 up rows of the same features (N a multiple of 128) and
// out[B, N / 2][b][blk * 64 + i] = silu(gate) * up.
// The first call on a device (and the first one that needs a larger one) allocates
// a per-device workspace and must not be made during stream capture; calls must
// be ordered on the device (one stream or one graph).  error_word as in
// launch_gemm_bf16.
cudaError_t launch_gemm_skinny(const void* x, const void* w, void* out, int B, int N, int K, int ldx, int ldw,
                               int ldo, int silu_pairs, uint32_t* error_word, cudaStream_t stream);

}  // namespace sm100
}  // namespace penny
