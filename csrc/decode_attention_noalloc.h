// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference.
//
// Who needs it: code that runs where a cudaMalloc is off the table – a plugin
// inside a serving process whose memory pool owns the whole GPU, a latency-
// critical decode loop where an allocation would synchronise the device, a C or
// Rust host that links this library without torch's caching allocator.  The
// regular path (penny_cpp.decode_attention) asks the caller for a workspace
// tensor; here the split-KV partial results live in a fixed array inside the
// library image instead, so the call needs nothing but its inputs and outputs.
//
// Contract
//   * Same math as launch_decode_attention (csrc/decode_kernels.cu): bf16 q/k/v,
//     head_dim 128, grouped-query heads, KV length positions[b] + 1, split over
//     `splits` blocks per (row, KV head) and merged.
//   * Scratch: a file-scope device array of PENNY_NOALLOC_SCRATCH_BYTES (8 MiB).
//     Every GPU that loads the library carries it until the process exits.
//     A call needs B * Hq * splits * (128 + 2) * 4 bytes of it and is REJECTED
//     (return code 2, message in `err`) when that exceeds the array; nothing is
//     launched in that case.
//   * The first call on a device looks up the array's device address (one
//     cudaGetSymbolAddress, with that device current) and raises the kernels'
//     shared-memory limit.  Make that first call outside any stream capture;
//     later calls only launch kernels.
//   * No cudaMalloc, cudaFree or allocating library routine is called, ever.
//   * All calls share the one array and it keeps the previous call's contents.
//     Every slot a call reads is written earlier in the same call, so nothing
//     has to be cleared – but two calls that overlap on the GPU (different
//     streams, or the same stream on different devices is fine: each device has
//     its own copy) would overwrite each other's partials: serialise them.
//
// Returns 0 on success, 1 for bad arguments, 2 for "too large for the built-in
// scratch", 3 for a CUDA error; `err` (may be null) receives a one-line reason.
#pragma once
#include <stddef.h>

#define PENNY_NOALLOC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// qkv:       [B, (Hq + 2*Hkv) * 128] bf16 (q already rotated)
// kcache/vcache: [B, Hkv, max_len, 128] bf16
// positions: [B] int32 (device); out: [B, Hq * 128] bf16
// stream:    a cudaStream_t (0 = the default stream)
int penny_decode_attention_noalloc(const void* qkv, const void* kcache, const void* vcache,
                                   const int* positions, void* out, int B, int Hq, int Hkv,
                                   int max_len, int splits, float scale, void* stream, char* err,
                                   size_t err_len);

#ifdef __cplusplus
}
#endif
