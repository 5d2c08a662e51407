// Entry points of the decode-step kernels (csrc/decode_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace penny {

// qkv: [B, (Hq + 2*Hkv) * D] bf16; caches: [B, Hkv, max_len, D] bf16; positions: [B] int32.
// Rotates q and k in place (rotate-half RoPE) and stores the new k, v rows at positions[b].
cudaError_t launch_rope_append(void* qkv, void* kcache, void* vcache, const int* positions, int B,
                               int Hq, int Hkv, int D, int max_len, float theta,
                               cudaStream_t stream);

// Prefill form: rotates the q and k heads of every row of qkv [T, (Hq + 2*Hkv) * D] in
// place at position pos0 + row (one sequence of T tokens); v is left alone.
cudaError_t launch_rope_rows(void* qkv, int T, int Hq, int Hkv, int D, int pos0, float theta,
                             cudaStream_t stream);

// Scratch the split-KV attention needs: per (row, head, split) an unnormalised
// fp32 output row plus (max, sum).
size_t decode_attn_workspace_bytes(int B, int Hq, int splits);

// out: [B, Hq * D] bf16.  Attends to cache rows [0, positions[b]] (inclusive).
cudaError_t launch_decode_attention(const void* qkv, const void* kcache, const void* vcache,
                                    const int* positions, void* out, void* workspace, int B, int Hq,
                                    int Hkv, int D, int max_len, int splits, float scale,
                                    cudaStream_t stream);

// One launch for rope + KV append + split-KV attention + merge (csrc/decode_attention_fused.cu).
// qkv holds the UNROTATED projections of the new token; rows [0, positions[b]) of the caches are
// attended to together with the new token, whose rotated k and v are stored at row positions[b].
// workspace: decode_attn_fused_workspace_bytes, zeroed once before the first call (its tail holds
// self-resetting arrival counters).  pdl: launch with programmatic stream serialization.
size_t decode_attn_fused_workspace_bytes(int B, int Hq, int Hkv, int splits);
cudaError_t launch_decode_attention_fused(const void* qkv, void* kcache, void* vcache, const int* positions,
                                          void* out, void* workspace, int B, int Hq, int Hkv, int D, int max_len,
                                          int splits, float scale, float theta, bool pdl, cudaStream_t stream);

// gate_up: [rows, 2F] (gate | up) -> out [rows, F] = silu(gate) * up
cudaError_t launch_silu_mul(const void* gate_up, void* out, int rows, int F, cudaStream_t stream);

// logits: [rows, cols] bf16 -> per-row max value and index (+ index_base).  workspace: zeroed once,
// argmax_workspace_bytes(rows) bytes (nullptr: one block per row); pair: optional [2 * rows] fp32
// (values, then indices).
size_t argmax_workspace_bytes(int rows);
cudaError_t launch_argmax(const void* logits, int rows, int cols, float* out_val, long long* out_idx, float* pair,
                          long long index_base, void* workspace, cudaStream_t stream);
// pairs: [world][2][B] fp32 (values, indices) -> next_tokens[B] = tokens[B] = index of the largest
// value over the ranks; positions[B] += 1.
cudaError_t launch_sample_finish(const float* pairs, int world, int B, long long* next_tokens, long long* tokens,
                                 int* positions, cudaStream_t stream);

}  // namespace penny
