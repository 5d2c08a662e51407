// Decode-step kernels of the tensor-parallel transformer around the fused
// collectives: rotary embedding + KV-cache append, grouped-query decode
// attention (split over the KV length, then merged), SiLU(gate) * up, and a
// per-row arg-max over a vocabulary shard.  bf16 in / out, fp32 math.
//
// All of it is memory-bound work at decode batch sizes, so the goal of each
// kernel is to read its operand once with wide, coalesced loads and keep enough
// bytes in flight per SM.  The reference ships no model code at all; these
// kernels exist so that the TP-decode benchmark runs on this library's own
// kernels end to end (the GEMMs go to cuBLAS).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "decode_kernels.h"

namespace penny {

namespace {

__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }

// ---------------------------------------------------------------------------
// RoPE (rotate-half form) on q and k, then k / v written into the cache.
// qkv: [B, (Hq + 2*Hkv) * D] as produced by the fused QKV GEMM.
// grid = (B, Hq + Hkv), block = D / 2 threads.
// ---------------------------------------------------------------------------
__global__ void k_rope_append(__nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kcache,
                              __nv_bfloat16* __restrict__ vcache, const int* __restrict__ positions,
                              int Hq, int Hkv, int D, int max_len, float theta) {
  const int b = blockIdx.x;
  const int h = blockIdx.y;  // [0, Hq): query heads, [Hq, Hq + Hkv): key heads
  const int i = threadIdx.x;  // pair index, D / 2 of them
  const int pos = positions[b];
  const int half = D / 2;
  const size_t row = (size_t)b * (Hq + 2 * Hkv) * D;
  __nv_bfloat16* x = qkv + row + (size_t)h * D;
  const float inv_freq = __powf(theta, -2.0f * (float)i / (float)D);
  float s, c;
  __sincosf((float)pos * inv_freq, &s, &c);
  const float a = bf2f(x[i]), bb = bf2f(x[i + half]);
  const float ra = a * c - bb * s, rb = bb * c + a * s;
  if (h < Hq) {
    x[i] = __float2bfloat16_rn(ra);
    x[i + half] = __float2bfloat16_rn(rb);
  } else {
    const int kh = h - Hq;
    const size_t coff = (((size_t)b * Hkv + kh) * max_len + pos) * D;
    kcache[coff + i] = __float2bfloat16_rn(ra);
    kcache[coff + i + half] = __float2bfloat16_rn(rb);
    const __nv_bfloat16* v = qkv + row + (size_t)(Hq + Hkv + kh) * D;
    vcache[coff + i] = v[i];
    vcache[coff + i + half] = v[i + half];
  }
}

// ---------------------------------------------------------------------------
// Decode attention, head_dim 128, grouped queries.
//
// One block per (batch row, KV head, split of the KV length).  The G = Hq / Hkv
// query heads that share the KV head are the block's G warps, so K and V are
// read from HBM once for all of them.  KV positions are processed in tiles of
// 32: the tile is brought into shared memory with 16-byte cp.async (double
// buffered), lane l owns dims [4l, 4l+4) of every row, the 32 partial dot
// products of a tile are transposed-and-summed across the warp with 31 shuffles
// (instead of 5 per position), and lane p ends up with the score of position p.
// Each split writes an unnormalised output + (max, sum); k_attn_merge combines.
// ---------------------------------------------------------------------------
constexpr int kD = 128;
constexpr int kTile = 32;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = pred ? 16 : 0;  // zero-fill when out of range
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

template <int G>
__global__ void __launch_bounds__(G * 32) k_decode_attn(
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ positions,
    float* __restrict__ part_o, float* __restrict__ part_ml, int Hq, int Hkv, int max_len,
    int splits, float scale) {
  __shared__ __align__(16) __nv_bfloat16 sk[2][kTile][kD];
  __shared__ __align__(16) __nv_bfloat16 sv[2][kTile][kD];
  const int b = blockIdx.x, kh = blockIdx.y, sp = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = positions[b] + 1;  // the new token was appended at positions[b]
  const int per = ((len + splits - 1) / splits + kTile - 1) / kTile * kTile;
  const int t0 = sp * per;
  const int t1 = min(len, t0 + per);
  const int hq = kh * G + warp;

  // this warp's query head, pre-scaled, 4 dims per lane
  float q[4];
  {
    const __nv_bfloat16* qp = qkv + (size_t)b * (Hq + 2 * Hkv) * kD + (size_t)hq * kD + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(qp);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    q[0] = bf2f(a.x) * scale; q[1] = bf2f(a.y) * scale; q[2] = bf2f(c.x) * scale; q[3] = bf2f(c.y) * scale;
  }
  const __nv_bfloat16* kbase = kcache + ((size_t)b * Hkv + kh) * (size_t)max_len * kD;
  const __nv_bfloat16* vbase = vcache + ((size_t)b * Hkv + kh) * (size_t)max_len * kD;

  auto load_tile = [&](int stage, int start) {
    // 32 rows x 256 B = 512 chunks of 16 B for K, the same for V
    for (int c = threadIdx.x; c < kTile * 16; c += G * 32) {
      const int r = c >> 4, o = (c & 15) * 8;
      const bool ok = start + r < t1;
      const size_t g = (size_t)(ok ? start + r : 0) * kD + o;
      cp_async16(&sk[stage][r][o], kbase + g, ok);
      cp_async16(&sv[stage][r][o], vbase + g, ok);
    }
    cp_async_commit();
  };

  float m = -INFINITY, l = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int ntiles = t1 > t0 ? (t1 - t0 + kTile - 1) / kTile : 0;
  if (ntiles > 0) load_tile(0, t0);
  for (int t = 0; t < ntiles; ++t) {
    const int stage = t & 1;
    if (t + 1 < ntiles) {
      load_tile(stage ^ 1, t0 + (t + 1) * kTile);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // partial dot products of my 4 dims with the 32 rows of the tile
    float p[kTile];
#pragma unroll
    for (int r = 0; r < kTile; ++r) {
      const uint2 raw = *reinterpret_cast<const uint2*>(&sk[stage][r][lane * 4]);
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      p[r] = q[0] * bf2f(a.x) + q[1] * bf2f(a.y) + q[2] * bf2f(c.x) + q[3] * bf2f(c.y);
    }
    // transpose-and-sum: afterwards lane j holds the full score of row j
#pragma unroll
    for (int w = 16; w >= 1; w >>= 1) {
      const bool upper = (lane & w) != 0;
#pragma unroll
      for (int i = 0; i < w; ++i) {
        // keep the half that matches my bit, send the other half
        const float send = upper ? p[i] : p[i + w];
        const float keep = upper ? p[i + w] : p[i];
        p[i] = keep + __shfl_xor_sync(0xffffffffu, send, w);
      }
    }
    // After the last step p[0] is the score of row `lane` with bits taken MSB first:
    // row index = lane (bit w of lane selected the upper half at every step).
    const int row = t0 + t * kTile + lane;
    float s = (row < t1) ? p[0] : -INFINITY;
    float tmax = s;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
    const float mnew = fmaxf(m, tmax);
    const float corr = __expf(m - mnew);
    const float e = (row < t1) ? __expf(s - mnew) : 0.f;
    float tsum = e;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tsum += __shfl_xor_sync(0xffffffffu, tsum, o);
    l = l * corr + tsum;
    m = mnew;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] *= corr;
#pragma unroll
    for (int r = 0; r < kTile; ++r) {
      const float pr = __shfl_sync(0xffffffffu, e, r);
      const uint2 raw = *reinterpret_cast<const uint2*>(&sv[stage][r][lane * 4]);
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      acc[0] += pr * bf2f(a.x); acc[1] += pr * bf2f(a.y); acc[2] += pr * bf2f(c.x); acc[3] += pr * bf2f(c.y);
    }
    __syncthreads();  // the stage is refilled two iterations later
  }
  const size_t slot = ((size_t)b * Hq + hq) * splits + sp;
  float4* po = reinterpret_cast<float4*>(part_o + slot * kD + lane * 4);
  *po = make_float4(acc[0], acc[1], acc[2], acc[3]);
  if (lane == 0) {
    part_ml[slot * 2] = m;
    part_ml[slot * 2 + 1] = l;
  }
}

// out[b, hq, :] = sum_s exp(m_s - M) * o_s / sum_s exp(m_s - M) * l_s
// grid = (B, Hq), block = 32 (4 dims per lane)
__global__ void k_attn_merge(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                             __nv_bfloat16* __restrict__ out, int Hq, int splits) {
  const int b = blockIdx.x, hq = blockIdx.y, lane = threadIdx.x;
  const size_t base = ((size_t)b * Hq + hq) * splits;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  float L = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - M);
    L += w * part_ml[(base + s) * 2 + 1];
    const float4 o = *reinterpret_cast<const float4*>(part_o + (base + s) * kD + lane * 4);
    acc[0] += w * o.x; acc[1] += w * o.y; acc[2] += w * o.z; acc[3] += w * o.w;
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  __nv_bfloat162 r0 = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
  __nv_bfloat162 r1 = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&r0);
  raw.y = *reinterpret_cast<uint32_t*>(&r1);
  *reinterpret_cast<uint2*>(out + ((size_t)b * Hq + hq) * kD + lane * 4) = raw;
}

// out[b, j] = silu(gu[b, j]) * gu[b, F + j]; 8 elements per thread
__global__ void k_silu_mul(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                           int rows, int F) {
  const size_t vec_per_row = (size_t)F / 8;
  const size_t total = (size_t)rows * vec_per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / vec_per_row, c = (i % vec_per_row) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * F + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float g0 = bf2f(gp[k].x), g1 = bf2f(gp[k].y);
      const float s0 = g0 / (1.f + __expf(-g0)), s1 = g1 / (1.f + __expf(-g1));
      op[k] = __floats2bfloat162_rn(s0 * bf2f(up[k].x), s1 * bf2f(up[k].y));
    }
    *reinterpret_cast<uint4*>(out + r * F + c) = o;
  }
}

// Per-row arg-max over a vocabulary shard.  grid = rows, block = 256.
// out_val[row], out_idx[row] (index offset by `index_base`).
__global__ void __launch_bounds__(256) k_argmax(const __nv_bfloat16* __restrict__ logits, int cols,
                                                float* __restrict__ out_val,
                                                long long* __restrict__ out_idx,
                                                long long index_base) {
  __shared__ float sval[8];
  __shared__ int sidx[8];
  const __nv_bfloat16* row = logits + (size_t)blockIdx.x * cols;
  float best = -INFINITY;
  int bi = 0;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    const float v = bf2f(row[i]);
    if (v > best) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sval[warp] = best;
    sidx[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < 8 ? sval[lane] : -INFINITY;
    bi = lane < 8 ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      out_val[blockIdx.x] = best;
      out_idx[blockIdx.x] = index_base + bi;
    }
  }
}

}  // namespace

cudaError_t launch_rope_append(void* qkv, void* kcache, void* vcache, const int* positions, int B,
                               int Hq, int Hkv, int D, int max_len, float theta,
                               cudaStream_t stream) {
  if (D % 2 != 0 || D / 2 > 1024) return cudaErrorInvalidValue;
  dim3 grid(B, Hq + Hkv);
  k_rope_append<<<grid, D / 2, 0, stream>>>((__nv_bfloat16*)qkv, (__nv_bfloat16*)kcache,
                                            (__nv_bfloat16*)vcache, positions, Hq, Hkv, D, max_len,
                                            theta);
  return cudaGetLastError();
}

size_t decode_attn_workspace_bytes(int B, int Hq, int splits) {
  return (size_t)B * Hq * splits * (kD + 2) * sizeof(float);
}

cudaError_t launch_decode_attention(const void* qkv, const void* kcache, const void* vcache,
                                    const int* positions, void* out, void* workspace, int B, int Hq,
                                    int Hkv, int D, int max_len, int splits, float scale,
                                    cudaStream_t stream) {
  if (D != kD || Hkv < 1 || Hq % Hkv != 0 || splits < 1) return cudaErrorInvalidValue;
  const int G = Hq / Hkv;
  float* part_o = reinterpret_cast<float*>(workspace);
  float* part_ml = part_o + (size_t)B * Hq * splits * kD;
  dim3 grid(B, Hkv, splits);
#define PENNY_ATTN(GG)                                                                          \
  k_decode_attn<GG><<<grid, GG * 32, 0, stream>>>(                                              \
      (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache,    \
      positions, part_o, part_ml, Hq, Hkv, max_len, splits, scale)
  switch (G) {
    case 1: PENNY_ATTN(1); break;
    case 2: PENNY_ATTN(2); break;
    case 4: PENNY_ATTN(4); break;
    case 8: PENNY_ATTN(8); break;
    default: return cudaErrorInvalidValue;
  }
#undef PENNY_ATTN
  cudaError_t rc = cudaGetLastError();
  if (rc != cudaSuccess) return rc;
  k_attn_merge<<<dim3(B, Hq), 32, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, Hq, splits);
  return cudaGetLastError();
}

cudaError_t launch_silu_mul(const void* gate_up, void* out, int rows, int F, cudaStream_t stream) {
  if (F % 8 != 0) return cudaErrorInvalidValue;
  const size_t total = (size_t)rows * (F / 8);
  const int blocks = (int)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256);
  k_silu_mul<<<blocks < 1 ? 1 : blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up,
                                                          (__nv_bfloat16*)out, rows, F);
  return cudaGetLastError();
}

cudaError_t launch_argmax(const void* logits, int rows, int cols, float* out_val, long long* out_idx,
                          long long index_base, cudaStream_t stream) {
  k_argmax<<<rows, 256, 0, stream>>>((const __nv_bfloat16*)logits, cols, out_val, out_idx,
                                     index_base);
  return cudaGetLastError();
}

}  // namespace penny
