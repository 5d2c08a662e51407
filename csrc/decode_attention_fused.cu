// Decode attention with everything around it folded in: rotary embedding of q and
// k, the KV-cache append of the new token, the split-KV attention itself and the
// merge of the splits - ONE launch where the plain kernels of decode_kernels.cu
// need three (rope + append, attention, merge).
//
//   * grid (batch row, KV head, split), 4 warps, the same tensor-core tile loop
//     as k_decode_attn (decode_attn_common.cuh): G = Hq / Hkv query heads share
//     every K / V tile, each warp runs a private 3-stage cp.async pipeline.
//   * The splits cover the OLD cache rows [0, pos).  The new token never makes a
//     round trip through memory: split 0 rotates k, stores k and v at row pos of
//     the cache (for the next steps) and folds the token into its own running
//     softmax from shared memory.  q is rotated in registers by every CTA.
//   * The last CTA of a (row, KV head) to finish merges the split partials: a
//     self-resetting arrival counter per (row, KV head), no second launch.
//   * Programmatic dependent launch: the kernel may start while the QKV GEMM is
//     still running.  Its first K / V tiles - written by earlier decode steps,
//     never by the kernels just before it - are requested BEFORE the dependency
//     wait; q, k, v of the new token are read after it.
//
// The reference has no attention (it is used inside vLLM / SGLang, README.md:20-33).
#include "decode_attn_common.cuh"
#include "decode_kernels.h"
#include "kernel_setup.h"
#include "pdl.h"

namespace penny {

namespace {
using namespace attn;

template <int G>
__global__ void __launch_bounds__(kAttnWarps * 32) k_decode_attn_fused(
    const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
    const int* __restrict__ positions, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
    float* __restrict__ part_ml, unsigned* __restrict__ counters, int Hq, int Hkv, int max_len, int splits,
    float scale, float theta) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ float s_new[2 * kD];  // rotated k (as stored: bf16-rounded) and v of the new token
  __shared__ int s_last;
  pdl_launch_dependents();
  const int b = blockIdx.x, kh = blockIdx.y, sp = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  // positions[] was advanced at the end of the previous step, long before any kernel
  // that may still be running when this one starts
  const int pos = positions[b];
  const int len = pos;  // old rows; the new token is handled separately
  const int per = ((len + splits - 1) / splits + kTile - 1) / kTile * kTile;
  const int t0 = sp * per;
  const int t1 = min(len, t0 + per);
  const int ntiles = t1 > t0 ? (t1 - t0 + kTile - 1) / kTile : 0;
  const uint32_t wbase = smem_u32_local(smem_raw) + warp * (kAttnStages * kStageBytes);
  const size_t cache_row0 = ((size_t)b * Hkv + kh) * (size_t)max_len;
  const __nv_bfloat16* kbase = kcache + cache_row0 * kD;
  const __nv_bfloat16* vbase = vcache + cache_row0 * kD;

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
  issue(0);
  issue(1);
  pdl_wait();

  const size_t qkv_row = (size_t)b * (Hq + 2 * Hkv) * kD;
  // ---- q of this KV head's G query heads: rotate, scale, pack as MMA A fragments ----
  // dims of this thread: kc * 16 + {2t, 2t + 1, 8 + 2t, 8 + 2t + 1}; the rotation pairs
  // dim d < 64 with d + 64, i.e. chunk kc with chunk kc + 4 at the same offsets
  uint32_t qa[8][2];
  {
    const float qs = scale * kLog2e;
    const __nv_bfloat16* qp = qkv + qkv_row + (size_t)(kh * G + (g < G ? g : 0)) * kD;
#pragma unroll
    for (int kc = 0; kc < 4; ++kc) {
      float ra[4], rb[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int d = kc * 16 + h * 8 + 2 * t;
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(qp + d);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(qp + d + kD / 2);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float inv_freq = __powf(theta, -2.0f * (float)(d + e) / (float)kD);
          float sn, cs;
          __sincosf((float)pos * inv_freq, &sn, &cs);
          const float a = bf2f(e ? lo.y : lo.x), bb = bf2f(e ? hi.y : hi.x);
          ra[h * 2 + e] = (a * cs - bb * sn) * qs;
          rb[h * 2 + e] = (bb * cs + a * sn) * qs;
        }
      }
      qa[kc][0] = (g < G) ? pack2(ra[0], ra[1]) : 0u;
      qa[kc][1] = (g < G) ? pack2(ra[2], ra[3]) : 0u;
      qa[kc + 4][0] = (g < G) ? pack2(rb[0], rb[1]) : 0u;
      qa[kc + 4][1] = (g < G) ? pack2(rb[2], rb[3]) : 0u;
    }
  }
  // ---- the new token: split 0 appends it to the cache and keeps it in shared memory ----
  if (sp == 0) {
    const size_t coff = (cache_row0 + (size_t)pos) * kD;
    const int tid = (int)threadIdx.x;
    if (tid < kD / 2) {
      const __nv_bfloat16* kp = qkv + qkv_row + (size_t)(Hq + kh) * kD;
      const float inv_freq = __powf(theta, -2.0f * (float)tid / (float)kD);
      float sn, cs;
      __sincosf((float)pos * inv_freq, &sn, &cs);
      const float a = bf2f(kp[tid]), bb = bf2f(kp[tid + kD / 2]);
      const __nv_bfloat16 ka = __float2bfloat16_rn(a * cs - bb * sn), kb = __float2bfloat16_rn(bb * cs + a * sn);
      kcache[coff + tid] = ka;
      kcache[coff + tid + kD / 2] = kb;
      s_new[tid] = bf2f(ka);
      s_new[tid + kD / 2] = bf2f(kb);
    } else {
      const __nv_bfloat16* vp = qkv + qkv_row + (size_t)(Hq + Hkv + kh) * kD;
      const int j = (tid - kD / 2) * 2;
      const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(vp + j);
      *reinterpret_cast<__nv_bfloat162*>(vcache + coff + j) = v2;
      s_new[kD + j] = bf2f(v2.x);
      s_new[kD + j + 1] = bf2f(v2.y);
    }
    __syncthreads();
  }

  float m = -INFINITY, l = 0.f;  // row g (valid for g < G); l is this thread's share
  float o[16][4];
#pragma unroll
  for (int dc = 0; dc < 16; ++dc) o[dc][0] = o[dc][1] = o[dc][2] = o[dc][3] = 0.f;

  const int my_tiles = ntiles > warp ? (ntiles - warp + kAttnWarps - 1) / kAttnWarps : 0;
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
  // ---- the new token joins the running softmax of warp 0 of split 0 ----
  if (sp == 0 && warp == 0) {
    float part = 0.f;
#pragma unroll
    for (int kc = 0; kc < 8; ++kc) {
      const __nv_bfloat162 q01 = *reinterpret_cast<const __nv_bfloat162*>(&qa[kc][0]);
      const __nv_bfloat162 q23 = *reinterpret_cast<const __nv_bfloat162*>(&qa[kc][1]);
      const int d = kc * 16 + 2 * t;
      part += bf2f(q01.x) * s_new[d] + bf2f(q01.y) * s_new[d + 1] + bf2f(q23.x) * s_new[d + 8] +
              bf2f(q23.y) * s_new[d + 9];
    }
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    part += __shfl_xor_sync(0xffffffffu, part, 2);
    if (g < G) {
      const float mnew = fmaxf(m, part);
      const float corr = exp2f(m - mnew);
      const float p = exp2f(part - mnew);
      l = l * corr + (t == 0 ? p : 0.f);
      m = mnew;
#pragma unroll
      for (int dc = 0; dc < 16; ++dc) {
        o[dc][0] = o[dc][0] * corr + p * s_new[kD + dc * 8 + 2 * t];
        o[dc][1] = o[dc][1] * corr + p * s_new[kD + dc * 8 + 2 * t + 1];
      }
    }
  }
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
  if (splits == 1) return;
  // ---- the last split of this (row, KV head) to get here merges them all ----
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned* cnt = counters + (size_t)b * Hkv + kh;
    const unsigned old = atomicAdd(cnt, 1u);
    const int last = old == (unsigned)(splits - 1);
    if (last) *cnt = 0u;  // every split has arrived: ready for the next launch
    s_last = last;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int item = threadIdx.x; item < G * 32; item += kAttnWarps * 32) {
    const int hq = kh * G + (item >> 5), d4 = (item & 31) * 4;
    const size_t base = ((size_t)b * Hq + hq) * splits;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, __ldcg(part_ml + (base + s) * 2));
    float L = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < splits; ++s) {
      const float ms = __ldcg(part_ml + (base + s) * 2);
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
      L += w * __ldcg(part_ml + (base + s) * 2 + 1);
      const float4 ov = __ldcg(reinterpret_cast<const float4*>(part_o + (base + s) * kD + d4));
      acc[0] += w * ov.x; acc[1] += w * ov.y; acc[2] += w * ov.z; acc[3] += w * ov.w;
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    uint2 raw;
    raw.x = pack2(acc[0] * inv, acc[1] * inv);
    raw.y = pack2(acc[2] * inv, acc[3] * inv);
    *reinterpret_cast<uint2*>(out + ((size_t)b * Hq + hq) * kD + d4) = raw;
  }
}

}  // namespace

size_t decode_attn_fused_workspace_bytes(int B, int Hq, int Hkv, int splits) {
  // partial rows + (max, sum) per (row, head, split), then one arrival counter per (row, KV head)
  return decode_attn_workspace_bytes(B, Hq, splits) + (size_t)B * Hkv * sizeof(unsigned);
}

cudaError_t launch_decode_attention_fused(const void* qkv, void* kcache, void* vcache, const int* positions,
                                          void* out, void* workspace, int B, int Hq, int Hkv, int D, int max_len,
                                          int splits, float scale, float theta, bool pdl, cudaStream_t stream) {
  if (D != kD || Hkv < 1 || Hq % Hkv != 0 || splits < 1 || B < 1) return cudaErrorInvalidValue;
  const int G = Hq / Hkv;
  float* part_o = reinterpret_cast<float*>(workspace);
  float* part_ml = part_o + (size_t)B * Hq * splits * kD;
  unsigned* counters = reinterpret_cast<unsigned*>(part_ml + (size_t)B * Hq * splits * 2);
  dim3 grid(B, Hkv, splits);
  cudaError_t rc = cudaSuccess;
#define PENNY_ATTN_FUSED(GG)                                                                                  \
  do {                                                                                                        \
    rc = kernel_setup(reinterpret_cast<const void*>(k_decode_attn_fused<GG>), kAttnSmem).rc;                  \
    if (rc != cudaSuccess) return rc;                                                                         \
    rc = launch_kernel_ex(k_decode_attn_fused<GG>, grid, dim3(kAttnWarps * 32), (size_t)kAttnSmem, stream,    \
                          pdl, 1, (const __nv_bfloat16*)qkv, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache,  \
                          positions, (__nv_bfloat16*)out, part_o, part_ml, counters, Hq, Hkv, max_len, splits, \
                          scale, theta);                                                                      \
  } while (0)
  switch (G) {
    case 1: PENNY_ATTN_FUSED(1); break;
    case 2: PENNY_ATTN_FUSED(2); break;
    case 4: PENNY_ATTN_FUSED(4); break;
    case 8: PENNY_ATTN_FUSED(8); break;
    default: return cudaErrorInvalidValue;
  }
#undef PENNY_ATTN_FUSED
  return rc;
}

}  // namespace penny
