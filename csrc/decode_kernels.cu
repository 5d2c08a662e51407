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
#include "kernel_setup.h"
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "decode_attn_common.cuh"
#include "decode_kernels.h"

#include <stdio.h>

#include <algorithm>
#include <mutex>

#include "decode_attention_noalloc.h"

namespace penny {

namespace {

using namespace attn;

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

// RoPE for a prefill: row t of qkv is token pos0 + t of one sequence.
// grid = (T, ceil((Hq + Hkv) / 4)), block = (D / 2, 4): four heads per block.
__global__ void k_rope_rows(__nv_bfloat16* __restrict__ qkv, int Hq, int Hkv, int D, int pos0, float theta) {
  const int t = blockIdx.x;
  const int h = blockIdx.y * blockDim.y + threadIdx.y;
  if (h >= Hq + Hkv) return;
  const int i = threadIdx.x;
  const int half = D / 2;
  __nv_bfloat16* x = qkv + (size_t)t * (Hq + 2 * Hkv) * D + (size_t)h * D;
  const float inv_freq = __powf(theta, -2.0f * (float)i / (float)D);
  float s, c;
  __sincosf((float)(pos0 + t) * inv_freq, &s, &c);
  const float a = bf2f(x[i]), bb = bf2f(x[i + half]);
  x[i] = __float2bfloat16_rn(a * c - bb * s);
  x[i + half] = __float2bfloat16_rn(bb * c + a * s);
}

// ---------------------------------------------------------------------------
// Decode attention, head_dim 128, grouped queries, on tensor cores.
//
// One block per (batch row, KV head, split of the KV length), 4 warps.  Each
// warp walks its own tiles of 16 KV positions with a private 3-stage cp.async
// pipeline (no block-wide barrier in the loop) and serves ALL G = Hq / Hkv query
// heads of the KV head at once: the heads are the M rows (padded to 16) of
// mma.sync m16n8k16, so K and V are read from HBM once for the whole group and
// the inner loop is ~30 tensor-core instructions per tile instead of thousands
// of scalar FMAs and shuffles.
//   S = Q K^T : A = Q fragments (registers, pre-scaled by scale * log2 e),
//               B = K rows via ldmatrix from 128-byte-XOR-swizzled shared memory
//   O += P V  : A = P re-packed from the S accumulators, B = V via ldmatrix.trans
// Softmax is online in the log2 domain; the four warps' (max, sum, O) are merged
// through shared memory.  With one split the normalised bf16 output is written
// directly, otherwise an unnormalised fp32 partial + (max, sum) that
// k_attn_merge combines.
// ---------------------------------------------------------------------------
template <int G>
__global__ void __launch_bounds__(kAttnWarps * 32) k_decode_attn(
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ positions,
    __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    int Hq, int Hkv, int max_len, int splits, float scale) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int b = blockIdx.x, kh = blockIdx.y, sp = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int len = positions[b] + 1;  // the new token was appended at positions[b]
  const int per = ((len + splits - 1) / splits + kTile - 1) / kTile * kTile;
  const int t0 = sp * per;
  const int t1 = min(len, t0 + per);
  const int ntiles = t1 > t0 ? (t1 - t0 + kTile - 1) / kTile : 0;
  const uint32_t wbase = smem_u32_local(smem_raw) + warp * (kAttnStages * kStageBytes);

  // Q fragments of this KV head's G query heads: rows g < G, 8 K-chunks of 16 dims
  uint32_t qa[8][2];
  {
    const float qs = scale * kLog2e;
    const __nv_bfloat16* qp = qkv + (size_t)b * (Hq + 2 * Hkv) * kD + (size_t)(kh * G + (g < G ? g : 0)) * kD;
#pragma unroll
    for (int kc = 0; kc < 8; ++kc) {
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(qp + kc * 16 + 2 * t);
      const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(qp + kc * 16 + 8 + 2 * t);
      qa[kc][0] = (g < G) ? pack2(bf2f(lo.x) * qs, bf2f(lo.y) * qs) : 0u;
      qa[kc][1] = (g < G) ? pack2(bf2f(hi.x) * qs, bf2f(hi.y) * qs) : 0u;
    }
  }
  const __nv_bfloat16* kbase = kcache + ((size_t)b * Hkv + kh) * (size_t)max_len * kD;
  const __nv_bfloat16* vbase = vcache + ((size_t)b * Hkv + kh) * (size_t)max_len * kD;

  // tile j of this warp -> positions [t0 + (warp + 4 j) * 16, +16)
  auto issue = [&](int j) {
    const int tile = warp + kAttnWarps * j;
    if (tile < ntiles) {
      const int start = t0 + tile * kTile;
      const uint32_t sb = wbase + (j % kAttnStages) * kStageBytes;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = 2 * i + (lane >> 4), chunk = lane & 15;
        const bool ok = start + row < t1;
        const size_t goff = (size_t)(ok ? start + row : t0) * kD + chunk * 8;
        const uint32_t soff = row * 256 + ((chunk ^ (row & 7)) << 4);
        cp_async16(sb + soff, kbase + goff, ok);
        cp_async16(sb + kTile * 256 + soff, vbase + goff, ok);
      }
    }
    cp_async_commit();  // always: keeps the group count in step with j
  };

  float m = -INFINITY, l = 0.f;  // row g (valid for g < G); l is this thread's share
  float o[16][4];
#pragma unroll
  for (int dc = 0; dc < 16; ++dc) o[dc][0] = o[dc][1] = o[dc][2] = o[dc][3] = 0.f;

  const int my_tiles = ntiles > warp ? (ntiles - warp + kAttnWarps - 1) / kAttnWarps : 0;
  issue(0);
  issue(1);
  for (int j = 0; j < my_tiles; ++j) {
    __syncwarp();  // everyone is done with the stage that tile j + 2 overwrites
    issue(j + 2);
    cp_async_wait<2>();
    __syncwarp();
    const uint32_t sb = wbase + (j % kAttnStages) * kStageBytes;
    const int start = t0 + (warp + kAttnWarps * j) * kTile;
    // ---- S = Q K^T: two N-chunks of 8 positions ----
    float s[2][4];
#pragma unroll
    for (int nc = 0; nc < 2; ++nc) {
      s[nc][0] = s[nc][1] = s[nc][2] = s[nc][3] = 0.f;
      const int row = nc * 8 + (lane & 7);
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {  // pairs of K-chunks
        const int chunk = kp * 4 + (lane >> 3);
        uint32_t kb[4];
        ldmatrix_x4(sb + row * 256 + ((chunk ^ (row & 7)) << 4), kb);
        mma_bf16(s[nc], qa[2 * kp][0], 0u, qa[2 * kp][1], 0u, kb[0], kb[1]);
        mma_bf16(s[nc], qa[2 * kp + 1][0], 0u, qa[2 * kp + 1][1], 0u, kb[2], kb[3]);
      }
    }
    // ---- online softmax on row g: this thread holds positions nc*8 + 2t, +1 ----
    float sv[4];
#pragma unroll
    for (int nc = 0; nc < 2; ++nc) {
      const int p0 = start + nc * 8 + 2 * t;
      sv[nc * 2] = (p0 < t1) ? s[nc][0] : -INFINITY;
      sv[nc * 2 + 1] = (p0 + 1 < t1) ? s[nc][1] : -INFINITY;
    }
    float tmax = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    const float mnew = fmaxf(m, tmax);  // finite: every tile has at least one valid position
    const float corr = exp2f(m - mnew);
    float pv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pv[i] = exp2f(sv[i] - mnew);
    l = l * corr + (pv[0] + pv[1] + pv[2] + pv[3]);
    m = mnew;
    const uint32_t pa0 = pack2(pv[0], pv[1]);  // P[g][2t, 2t+1]
    const uint32_t pa2 = pack2(pv[2], pv[3]);  // P[g][8 + 2t, +1]
    // ---- O = O * corr + P V: 16 N-chunks of 8 dims ----
#pragma unroll
    for (int dp = 0; dp < 8; ++dp) {  // pairs of dim chunks
      const int lj = lane >> 3;
      const int row = (lj & 1) * 8 + (lane & 7);
      const int chunk = dp * 2 + (lj >> 1);
      uint32_t vb[4];
      ldmatrix_x4_trans(sb + kTile * 256 + row * 256 + ((chunk ^ (row & 7)) << 4), vb);
      o[2 * dp][0] *= corr; o[2 * dp][1] *= corr;
      o[2 * dp + 1][0] *= corr; o[2 * dp + 1][1] *= corr;
      mma_bf16(o[2 * dp], pa0, 0u, pa2, 0u, vb[0], vb[1]);
      mma_bf16(o[2 * dp + 1], pa0, 0u, pa2, 0u, vb[2], vb[3]);
    }
  }
  cp_async_wait<0>();
  // this thread's share of the row sum -> whole row
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);

  // ---- merge the four warps through shared memory (reusing the pipeline space) ----
  __syncthreads();
  float* sm_o = reinterpret_cast<float*>(smem_raw);                 // [warps][G][128]
  float* sm_ml = sm_o + kAttnWarps * G * kD;                        // [warps][G][2]
  if (g < G) {
#pragma unroll
    for (int dc = 0; dc < 16; ++dc) {
      float2 v2 = make_float2(o[dc][0], o[dc][1]);
      *reinterpret_cast<float2*>(&sm_o[((size_t)warp * G + g) * kD + dc * 8 + 2 * t]) = v2;
    }
    if (t == 0) {
      sm_ml[(warp * G + g) * 2] = m;
      sm_ml[(warp * G + g) * 2 + 1] = l;
    }
  }
  __syncthreads();
  // thread -> (head hh, 4 dims): G * 32 work items over 128 threads
  for (int item = threadIdx.x; item < G * 32; item += kAttnWarps * 32) {
    const int hh = item >> 5, d4 = (item & 31) * 4;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, sm_ml[(w * G + hh) * 2]);
    float L = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float mw = sm_ml[(w * G + hh) * 2];
      const float wgt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L += wgt * sm_ml[(w * G + hh) * 2 + 1];
      const float4 ov = *reinterpret_cast<const float4*>(&sm_o[((size_t)w * G + hh) * kD + d4]);
      acc[0] += wgt * ov.x; acc[1] += wgt * ov.y; acc[2] += wgt * ov.z; acc[3] += wgt * ov.w;
    }
    const int hq = kh * G + hh;
    if (splits == 1) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      uint2 raw;
      raw.x = pack2(acc[0] * inv, acc[1] * inv);
      raw.y = pack2(acc[2] * inv, acc[3] * inv);
      *reinterpret_cast<uint2*>(out + ((size_t)b * Hq + hq) * kD + d4) = raw;
    } else {
      const size_t slot = ((size_t)b * Hq + hq) * splits + sp;
      *reinterpret_cast<float4*>(part_o + slot * kD + d4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      if (d4 == 0) {
        part_ml[slot * 2] = M;
        part_ml[slot * 2 + 1] = L;
      }
    }
  }
}

// out[b, hq, :] = sum_s 2^(m_s - M) * o_s / sum_s 2^(m_s - M) * l_s  (log2 domain)
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
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    L += w * part_ml[(base + s) * 2 + 1];
    const float4 o = *reinterpret_cast<const float4*>(part_o + (base + s) * kD + lane * 4);
    acc[0] += w * o.x; acc[1] += w * o.y; acc[2] += w * o.z; acc[3] += w * o.w;
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  uint2 raw;
  raw.x = pack2(acc[0] * inv, acc[1] * inv);
  raw.y = pack2(acc[2] * inv, acc[3] * inv);
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

// Per-row arg-max over a vocabulary shard.  grid = (chunks, rows), block = 256: a row is cut into
// `chunks` column ranges so that rows x chunks blocks fill the GPU and every thread streams 16-byte
// vectors; the block that finishes a row last (a counter per row in `workspace`, left at zero again)
// merges the chunk results.  out_val[row], out_idx[row] (index offset by `index_base`); `pair`,
// when given, also receives [rows] values followed by [rows] indices as fp32 (the layout the
// tensor-parallel sampler all-gathers).  Ties: the lowest index.
constexpr int kArgmaxMaxChunks = 32;

__device__ __forceinline__ void argmax_take(float v, int i, float& best, int& bi) {
  if (v > best || (v == best && i < bi)) {
    best = v;
    bi = i;
  }
}

__global__ void __launch_bounds__(256) k_argmax(const __nv_bfloat16* __restrict__ logits, int cols, int per,
                                                float* __restrict__ out_val, long long* __restrict__ out_idx,
                                                float* __restrict__ pair, long long index_base,
                                                unsigned int* __restrict__ workspace) {
  __shared__ float sval[8];
  __shared__ int sidx[8];
  __shared__ bool s_last;
  const int rows = (int)gridDim.y, chunks = (int)gridDim.x, r = (int)blockIdx.y, ch = (int)blockIdx.x;
  const __nv_bfloat16* row = logits + (size_t)r * cols;
  const int c0 = ch * per, c1 = min(cols, c0 + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  if ((reinterpret_cast<uintptr_t>(row + c0) & 15u) == 0) {
    const int nvec = (c1 - c0) / 8;
    const uint4* vp = reinterpret_cast<const uint4*>(row + c0);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 q = vp[i];
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
      for (int k = 0; k < 8; ++k) argmax_take(bf2f(e[k]), c0 + i * 8 + k, best, bi);
    }
    for (int i = c0 + nvec * 8 + threadIdx.x; i < c1; i += blockDim.x) argmax_take(bf2f(row[i]), i, best, bi);
  } else {
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) argmax_take(bf2f(row[i]), i, best, bi);
  }
  auto block_best = [&]() {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      argmax_take(ov, oi, best, bi);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) {
      sval[warp] = best;
      sidx[warp] = bi;
    }
    __syncthreads();
    best = lane < 8 ? sval[lane] : -INFINITY;
    bi = lane < 8 ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      argmax_take(ov, oi, best, bi);
    }
  };
  block_best();  // threads of warp 0 hold the chunk's result
  if (chunks > 1) {  // (a launch without a workspace has one chunk per row)
    unsigned int* counter = workspace + r;
    float* part_val = reinterpret_cast<float*>(workspace + rows) + (size_t)r * kArgmaxMaxChunks;
    int* part_idx =
        reinterpret_cast<int*>(workspace + rows + (size_t)rows * kArgmaxMaxChunks) + (size_t)r * kArgmaxMaxChunks;
    if (threadIdx.x == 0) {
      part_val[ch] = best;
      part_idx[ch] = bi;
      __threadfence();
      s_last = atomicAdd(counter, 1u) == (unsigned)chunks - 1u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    best = -INFINITY;
    bi = 0x7fffffff;
    if (threadIdx.x < chunks) {
      best = __ldcg(part_val + threadIdx.x);
      bi = __ldcg(part_idx + threadIdx.x);
    }
    block_best();
    if (threadIdx.x == 0) *counter = 0;  // ready for the next launch
  }
  if (threadIdx.x == 0) {
    if (bi == 0x7fffffff) bi = 0;  // nothing compared greater than -inf (an all-NaN row)
    out_val[r] = best;
    out_idx[r] = index_base + bi;
    if (pair != nullptr) {
      pair[r] = best;
      pair[rows + r] = (float)(index_base + bi);  // vocabularies stay below 2^24: exact
    }
  }
}

// End of a greedy decode step in one launch: pick, per sequence, the rank whose shard holds the
// largest logit (pairs: [world][2][B] fp32 = values, indices; lowest rank on ties), hand the token
// to the next step and advance the positions.
__global__ void k_sample_finish(const float* __restrict__ pairs, int world, int B, long long* __restrict__ next_tokens,
                                long long* __restrict__ tokens, int* __restrict__ positions) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float best = pairs[b];
  float idx = pairs[B + b];
  for (int w = 1; w < world; ++w) {
    const float v = pairs[(size_t)w * 2 * B + b];
    if (v > best) {
      best = v;
      idx = pairs[(size_t)w * 2 * B + B + b];
    }
  }
  const long long t = (long long)idx;
  next_tokens[b] = t;
  tokens[b] = t;
  positions[b] += 1;
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

cudaError_t launch_rope_rows(void* qkv, int T, int Hq, int Hkv, int D, int pos0, float theta,
                             cudaStream_t stream) {
  if (D % 2 != 0 || D / 2 > 256 || T <= 0) return cudaErrorInvalidValue;
  dim3 grid(T, (Hq + Hkv + 3) / 4), block(D / 2, 4);
  k_rope_rows<<<grid, block, 0, stream>>>((__nv_bfloat16*)qkv, Hq, Hkv, D, pos0, theta);
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
  cudaError_t rc = cudaSuccess;
#define PENNY_ATTN(GG)                                                                            \
  do {                                                                                            \
    rc = kernel_setup(reinterpret_cast<const void*>(k_decode_attn<GG>), kAttnSmem).rc;            \
    if (rc != cudaSuccess) return rc;                                                             \
    k_decode_attn<GG><<<grid, kAttnWarps * 32, kAttnSmem, stream>>>(                              \
        (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache,    \
        positions, (__nv_bfloat16*)out, part_o, part_ml, Hq, Hkv, max_len, splits, scale);        \
  } while (0)
  switch (G) {
    case 1: PENNY_ATTN(1); break;
    case 2: PENNY_ATTN(2); break;
    case 4: PENNY_ATTN(4); break;
    case 8: PENNY_ATTN(8); break;
    default: return cudaErrorInvalidValue;
  }
#undef PENNY_ATTN
  rc = cudaGetLastError();
  if (rc != cudaSuccess || splits == 1) return rc;
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

size_t argmax_workspace_bytes(int rows) {
  return (size_t)rows * 4 + (size_t)rows * kArgmaxMaxChunks * 8;
}

cudaError_t launch_argmax(const void* logits, int rows, int cols, float* out_val, long long* out_idx, float* pair,
                          long long index_base, void* workspace, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || rows > 65535) return cudaErrorInvalidValue;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // enough blocks for two per SM, no chunk below 2048 columns; one chunk when there is no workspace
  int chunks = workspace == nullptr ? 1 : std::min({kArgmaxMaxChunks, (2 * sms + rows - 1) / rows, std::max(1, cols / 2048)});
  chunks = std::max(chunks, 1);
  int per = ((cols + chunks - 1) / chunks + 7) / 8 * 8;
  chunks = (cols + per - 1) / per;
  k_argmax<<<dim3((unsigned)chunks, (unsigned)rows), 256, 0, stream>>>((const __nv_bfloat16*)logits, cols, per, out_val,
                                                                     out_idx, pair, index_base,
                                                                     (unsigned int*)workspace);
  return cudaGetLastError();
}

cudaError_t launch_sample_finish(const float* pairs, int world, int B, long long* next_tokens, long long* tokens,
                                 int* positions, cudaStream_t stream) {
  if (world < 1 || B <= 0) return cudaErrorInvalidValue;
  k_sample_finish<<<(B + 127) / 128, 128, 0, stream>>>(pairs, world, B, next_tokens, tokens, positions);
  return cudaGetLastError();
}

}  // namespace penny

// ---------------------------------------------------------------------------
// Allocation-free decode attention (see decode_attention_noalloc.h).
// ---------------------------------------------------------------------------
namespace {

// Split-KV partials of the allocation-free entry point.  In host code this name
// is only a handle for cudaGetSymbolAddress, never a pointer a kernel may use.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PENNY_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
void* g_noalloc_ptr[kMaxDevices] = {};
bool g_noalloc_attr[kMaxDevices][4] = {};

int noalloc_fail(int code, char* err, size_t err_len, const char* what, const char* detail) {
  if (err != nullptr && err_len > 0) snprintf(err, err_len, "%s%s%s", what, detail ? ": " : "", detail ? detail : "");
  return code;
}

// Raises the kernel's dynamic shared-memory limit on the current device.  Called
// with g_noalloc_mu held (it guards the per-device "done" flags).
cudaError_t noalloc_set_attr(int G) {
  switch (G) {
    case 1: return cudaFuncSetAttribute(penny::k_decode_attn<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, penny::kAttnSmem);
    case 2: return cudaFuncSetAttribute(penny::k_decode_attn<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, penny::kAttnSmem);
    case 4: return cudaFuncSetAttribute(penny::k_decode_attn<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, penny::kAttnSmem);
    default: return cudaFuncSetAttribute(penny::k_decode_attn<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, penny::kAttnSmem);
  }
}

template <int G>
cudaError_t noalloc_launch(const void* qkv, const void* kcache, const void* vcache, const int* positions,
                           void* out, float* part_o, float* part_ml, int B, int Hq, int Hkv, int max_len,
                           int splits, float scale, cudaStream_t stream) {
  dim3 grid(B, Hkv, splits);
  penny::k_decode_attn<G><<<grid, penny::kAttnWarps * 32, penny::kAttnSmem, stream>>>(
      (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, positions,
      (__nv_bfloat16*)out, part_o, part_ml, Hq, Hkv, max_len, splits, scale);
  cudaError_t rc = cudaGetLastError();
  if (rc != cudaSuccess || splits == 1) return rc;
  penny::k_attn_merge<<<dim3(B, Hq), 32, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, Hq, splits);
  return cudaGetLastError();
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int penny_decode_attention_noalloc(
    const void* qkv, const void* kcache, const void* vcache, const int* positions, void* out, int B, int Hq,
    int Hkv, int max_len, int splits, float scale, void* stream, char* err, size_t err_len) {
  if (qkv == nullptr || kcache == nullptr || vcache == nullptr || positions == nullptr || out == nullptr)
    return noalloc_fail(1, err, err_len, "penny_decode_attention_noalloc: null pointer argument", nullptr);
  if (B < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0 || max_len < 1 || splits < 1 || splits > 64)
    return noalloc_fail(1, err, err_len, "penny_decode_attention_noalloc: bad shape (need B, Hq, Hkv, max_len >= 1, "
                        "Hq a multiple of Hkv, 1 <= splits <= 64)", nullptr);
  const int G = Hq / Hkv;
  if (G != 1 && G != 2 && G != 4 && G != 8)
    return noalloc_fail(1, err, err_len, "penny_decode_attention_noalloc: Hq / Hkv must be 1, 2, 4 or 8", nullptr);
  // each factor is bounded on its own first, so that the product below cannot wrap
  constexpr long long kMaxFactor = PENNY_NOALLOC_SCRATCH_BYTES / 520;
  const bool factor_too_large = B > kMaxFactor || Hq > kMaxFactor;
  const size_t need = factor_too_large ? ~(size_t)0 : penny::decode_attn_workspace_bytes(B, Hq, splits);
  if (need > (size_t)PENNY_NOALLOC_SCRATCH_BYTES) {
    char detail[160];
    snprintf(detail, sizeof(detail), "B * Hq * splits * 520 = %zu bytes needed, %u built in; lower `splits` or use "
             "the workspace-taking entry point", need, (unsigned)PENNY_NOALLOC_SCRATCH_BYTES);
    return noalloc_fail(2, err, err_len, "penny_decode_attention_noalloc: too large for the built-in scratch", detail);
  }
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return noalloc_fail(3, err, err_len, "penny_decode_attention_noalloc: cudaGetDevice", cudaGetErrorString(rc));
  void* scratch = nullptr;
  {
    // once per device, with that device current: the device address of the array
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
      void* p = nullptr;
      rc = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (rc != cudaSuccess || p == nullptr) {
        (void)cudaGetLastError();
        return noalloc_fail(3, err, err_len, "penny_decode_attention_noalloc: cudaGetSymbolAddress",
                            cudaGetErrorString(rc));
      }
      g_noalloc_ptr[dev] = p;
    }
    scratch = g_noalloc_ptr[dev];
    bool& attr_done = g_noalloc_attr[dev][G == 1 ? 0 : G == 2 ? 1 : G == 4 ? 2 : 3];
    if (!attr_done) {
      rc = noalloc_set_attr(G);
      if (rc != cudaSuccess) {
        (void)cudaGetLastError();
        return noalloc_fail(3, err, err_len, "penny_decode_attention_noalloc: cudaFuncSetAttribute",
                            cudaGetErrorString(rc));
      }
      attr_done = true;
    }
  }
  float* part_o = reinterpret_cast<float*>(scratch);
  float* part_ml = part_o + (size_t)B * Hq * splits * penny::kD;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (G) {
    case 1: rc = noalloc_launch<1>(qkv, kcache, vcache, positions, out, part_o, part_ml, B, Hq, Hkv, max_len, splits, scale, s); break;
    case 2: rc = noalloc_launch<2>(qkv, kcache, vcache, positions, out, part_o, part_ml, B, Hq, Hkv, max_len, splits, scale, s); break;
    case 4: rc = noalloc_launch<4>(qkv, kcache, vcache, positions, out, part_o, part_ml, B, Hq, Hkv, max_len, splits, scale, s); break;
    default: rc = noalloc_launch<8>(qkv, kcache, vcache, positions, out, part_o, part_ml, B, Hq, Hkv, max_len, splits, scale, s); break;
  }
  if (rc != cudaSuccess) {
    (void)cudaGetLastError();
    return noalloc_fail(3, err, err_len, "penny_decode_attention_noalloc: launch", cudaGetErrorString(rc));
  }
  if (err != nullptr && err_len > 0) err[0] = '\0';
  return 0;
}

