// Weight-streaming GEMM for decode batches on sm_100a:
//     out[B, N] = x[B, K] * W[N, K]^T        bf16, fp32 accumulate, B <= 128
// With a handful of rows the operation is a read of W at HBM speed; what
// decides its time is whether all 148 SMs stream weight bytes all the time.
//
//   * Operands are swapped with respect to the large GEMM: the 128 rows of a W
//     tile are the M side of tcgen05.mma (A operand, K-major as stored), the
//     batch rows of x are the N side (B operand, 64 or 128 wide).  The
//     accumulator holds out^T: TMEM lane = output column n, TMEM column = batch row.
//   * Stream-K: the (W tile, K step) units are dealt out as equal contiguous
//     ranges (skinny_order.h), so every CTA loads the same number of bytes for
//     any N and K.  A CTA that has only part of a tile's K steps parks its fp32
//     partial in a workspace slot and bumps the tile's counter; the CTA that
//     arrives last adds the partials in CTA order (the result does not depend on
//     who is last), stores the tile and resets the counter – no spinning, CUDA
//     graph replays keep working.  The workspace is per device: these GEMMs
//     must be ordered on the GPU (one stream or one graph), not concurrent.
//   * warp 0: TMA producer (8-stage ring, 24-32 KB per stage: ~200 KB of weight
//     bytes in flight per SM); warp 1: MMA issuer, two TMEM accumulators;
//     warps 2-5: epilogue.  TMEM lane = n, so for each batch row the 32 lanes of
//     a warp write 32 consecutive bf16 of that output row.
//   * Every wait is bounded (mbar_wait_abortable); TMEM is always freed.
//
// Optional fused epilogue: silu(gate) * up for a gate/up weight whose rows are
// interleaved in blocks of 64 (tile = 64 gate rows followed by the 64 up rows of
// the same features): the two halves meet through shared memory and out gets
// [B, N / 2].
//
// The reference has no GEMM of any kind; cuBLAS picks generic tiles for these
// shapes and leaves SMs idle on the narrow ones (N = 4096: 32 tiles of 128 rows).
#include "gemm_skinny_sm100.h"

#include <cuda.h>

#include <algorithm>
#include <map>
#include <mutex>

#include "gemm_kernel_sm100.cuh"
#include "gemm_sm100.h"
#include "kernel_setup.h"
#include "skinny_order.h"

namespace penny {
namespace sm100 {

namespace {

constexpr int kSkinnyThreads = 192;
constexpr int kXchStride = 65;  // floats per row of the silu exchange buffer (padded: no bank conflicts)

template <int BT>
struct SkinnyCfg {
  static constexpr int kStages = (BT == 64) ? 8 : 6;
  static constexpr int kWBytes = kBlockM * kBlockK * 2;  // 16 KB of weights per stage
  static constexpr int kXBytes = BT * kBlockK * 2;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kTmemCols = 2 * BT;
  static constexpr int kXchBytes = 64 * kXchStride * 4;   // silu exchange: 64 up rows x 64 batch columns
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/ + kXchBytes;
};

struct SkinnyArgs {
  __nv_bfloat16* out;
  int ldo;
  int B, N, K;
  SkinnyPlan plan;
  float* ws;           // [ctas][2 slots][BT columns][128 rows] fp32
  unsigned* counters;  // [tiles], zero between launches
  int silu_pairs;      // 1: rows are 64 gate + 64 up per tile, out[b][tile * 64 + i] = silu(g) * u
};

template <int BT>
__global__ void __launch_bounds__(kSkinnyThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const SkinnyArgs a, uint32_t* error_word) {
  using Cfg = SkinnyCfg<BT>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + kStages * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint64_t* tmem_empty = bars + 2 * kStages + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* s_last = reinterpret_cast<volatile int*>(tmem_holder + 2);
  float* s_xch = reinterpret_cast<float*>(tiles + kStages * Cfg::kStageBytes + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = (int)blockIdx.x;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
  }
  if (warp == 1) tmem_alloc(tmem_holder, Cfg::kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  auto fail = [&](uint32_t code) {
    *s_abort = 1;
    atomicCAS(error_word, 0u, code);
  };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ TMA producer
      int stage = 0;
      uint32_t phase = 0;
      long long cur = skinny_begin(a.plan, cta);
      SkinnySeg sg;
      bool ok = true;
      while (ok && !*s_abort && skinny_next(a.plan, cta, cur, sg)) {
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait_abortable(&empty[stage], phase ^ 1u, s_abort)) {
            ok = false;
            break;
          }
          unsigned char* sw = tiles + stage * Cfg::kStageBytes;
          mbar_expect_tx(&full[stage], Cfg::kStageBytes);
          tma_load_2d(sw, &map_w, &full[stage], kb * kBlockK, sg.tile * kBlockM);
          tma_load_2d(sw + Cfg::kWBytes, &map_x, &full[stage], kb * kBlockK, 0);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) fail(GEMM_ERR_PRODUCER_WAIT);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // -------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc = make_idesc_bf16(kBlockM, BT);
      int stage = 0;
      uint32_t phase = 0;
      long long cur = skinny_begin(a.plan, cta);
      SkinnySeg sg;
      for (int it = 0; !*s_abort && skinny_next(a.plan, cta, cur, sg); ++it) {
        const int ab = it & 1;
        const uint32_t ab_phase = (uint32_t)(it >> 1) & 1u;
        bool ok = mbar_wait_abortable(&tmem_empty[ab], ab_phase ^ 1u, s_abort);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(ab * BT);
        for (int kb = sg.kb0; ok && kb < sg.kb1; ++kb) {
          if (!mbar_wait_abortable(&full[stage], phase, s_abort)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sw = smem_u32(tiles + stage * Cfg::kStageBytes);
          const uint64_t dw = make_smem_desc(sw);
          const uint64_t dx = make_smem_desc(sw + Cfg::kWBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k)
            umma_bf16(d_tmem, advance_desc_k(dw, k), advance_desc_k(dx, k), idesc, (kb != sg.kb0) || k != 0);
          umma_commit(&empty[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) {
          fail(GEMM_ERR_MMA_WAIT);
          break;
        }
        umma_commit(&tmem_full[ab]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;              // TMEM lane quarter of this warp
    const int row = q * 32 + lane;       // weight row inside the tile = output column
    const int etid = (int)threadIdx.x - 64;
    // stores 64 batch columns (registers) of this thread's output column n
    auto store_cols = [&](int tile, int c0, const float (&v)[64]) {
      if (!a.silu_pairs) {
        const int n = tile * kBlockM + row;
        if (n < a.N) {
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (c0 + j < a.B) a.out[(size_t)(c0 + j) * a.ldo + n] = __float2bfloat16_rn(v[j]);
        }
      } else {
        // rows 0-63 of the tile are gate, rows 64-127 the matching up rows: the up
        // half hands its 64 batch columns over through shared memory
        const int n = tile * (kBlockM / 2) + (row & 63);
        if (row >= 64) {
#pragma unroll
          for (int j = 0; j < 64; ++j) s_xch[(row - 64) * kXchStride + j] = v[j];
        }
        named_bar_sync(1, 128);
        if (row < 64 && n < a.N / 2) {
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            if (c0 + j < a.B) {
              const float g = v[j], u = s_xch[row * kXchStride + j];
              a.out[(size_t)(c0 + j) * a.ldo + n] = __float2bfloat16_rn(g / (1.f + __expf(-g)) * u);
            }
          }
        }
        named_bar_sync(1, 128);  // the buffer is free for the next 64 columns
      }
    };
    long long cur = skinny_begin(a.plan, cta);
    SkinnySeg sg;
    for (int it = 0; !*s_abort && skinny_next(a.plan, cta, cur, sg); ++it) {
      const int ab = it & 1;
      const uint32_t ab_phase = (uint32_t)(it >> 1) & 1u;
      if (!mbar_wait_abortable(&tmem_full[ab], ab_phase, s_abort)) {
        if (lane == 0) fail(GEMM_ERR_EPILOGUE_WAIT);
        break;
      }
      tc_fence_after_sync();
      const uint32_t tacc = tmem_base + (uint32_t)(ab * BT) + ((uint32_t)(q * 32) << 16);
      const bool whole = sg.c_lo == sg.c_hi;
      float* my_slot = a.ws + ((size_t)(cta * 2 + sg.slot) * BT) * kBlockM + row;
#pragma unroll 1
      for (int c = 0; c < BT / 64; ++c) {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(tacc + c * 64, r0);
        tmem_ld_32x32(tacc + c * 64 + 32, r1);
        tmem_ld_wait();
        if (whole) {
          float v[64];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __uint_as_float(r0[j]);
            v[32 + j] = __uint_as_float(r1[j]);
          }
          store_cols(sg.tile, c * 64, v);
        } else {
          // partial: [batch column][128 rows] fp32, the 32 lanes of a warp side by side
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            my_slot[(size_t)(c * 64 + j) * kBlockM] = __uint_as_float(r0[j]);
            my_slot[(size_t)(c * 64 + 32 + j) * kBlockM] = __uint_as_float(r1[j]);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[ab]);
      if (whole) continue;
      __threadfence();
      named_bar_sync(2, 128);
      if (etid == 0) {
        const unsigned old = atomicAdd(&a.counters[sg.tile], 1u);
        const int last = old == (unsigned)(sg.c_hi - sg.c_lo);
        if (last) a.counters[sg.tile] = 0u;  // every part has arrived: ready for the next launch
        *s_last = last;
      }
      named_bar_sync(2, 128);
      const bool last = *s_last != 0;
      named_bar_sync(2, 128);  // all have read s_last before a later segment rewrites it
      if (!last) continue;
      __threadfence();
#pragma unroll 1
      for (int c = 0; c < BT / 64; ++c) {
        float v[64];
#pragma unroll
        for (int j = 0; j < 64; ++j) v[j] = 0.f;
        for (int pc = sg.c_lo; pc <= sg.c_hi; ++pc) {  // fixed order
          const float* src = a.ws + ((size_t)(pc * 2 + skinny_slot_of(a.plan, pc, sg.tile)) * BT) * kBlockM + row;
#pragma unroll
          for (int j = 0; j < 64; ++j) v[j] += __ldcg(src + (size_t)(c * 64 + j) * kBlockM);
        }
        store_cols(sg.tile, c * 64, v);
      }
    }
  }
  // ------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

struct SkinnyScratch {
  float* ws = nullptr;
  unsigned* counters = nullptr;
  size_t ws_bytes = 0, counter_words = 0;
};

// One workspace per device, grown on demand (never while the stream is being
// captured: a capture stream is not the stream the warm-up ran on, so the
// workspace cannot be tied to a stream).  Launches are expected to be ordered on
// the device – one stream, or one CUDA graph – as the kernels of a decode step
// are; two of these GEMMs running at the same time on one GPU would share it.
SkinnyScratch* skinny_scratch(cudaStream_t stream, size_t ws_bytes, size_t counter_words) {
  static std::mutex mu;
  static std::map<int, SkinnyScratch> table;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  SkinnyScratch& sc = table[dev];
  if (sc.ws_bytes >= ws_bytes && sc.counter_words >= counter_words) return &sc;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return nullptr;
  }
  cudaDeviceSynchronize();  // nothing in flight still uses the old buffers
  if (sc.ws) cudaFree(sc.ws);
  if (sc.counters) cudaFree(sc.counters);
  sc = SkinnyScratch{};
  ws_bytes = std::max(ws_bytes, (size_t)32 << 20);
  counter_words = std::max(counter_words, (size_t)4096);
  if (cudaMalloc(&sc.ws, ws_bytes) != cudaSuccess || cudaMalloc(&sc.counters, counter_words * 4) != cudaSuccess ||
      cudaMemset(sc.counters, 0, counter_words * 4) != cudaSuccess) {
    (void)cudaGetLastError();
    if (sc.ws) cudaFree(sc.ws);
    if (sc.counters) cudaFree(sc.counters);
    sc = SkinnyScratch{};
    return nullptr;
  }
  sc.ws_bytes = ws_bytes;
  sc.counter_words = counter_words;
  return &sc;
}

template <int BT>
cudaError_t launch_skinny_bt(const void* x, const void* w, void* out, int B, int N, int K, int ldx, int ldw,
                             int ldo, int silu_pairs, int sms, uint32_t* error_word, cudaStream_t stream) {
  using Cfg = SkinnyCfg<BT>;
  CUtensorMap mw, mx;
  cudaError_t rc = make_tile_map(&mw, w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, kBlockM);
  if (rc != cudaSuccess) return rc;
  rc = make_tile_map(&mx, x, (uint64_t)B, (uint64_t)K, (uint64_t)ldx, BT);
  if (rc != cudaSuccess) return rc;
  rc = kernel_setup(reinterpret_cast<const void*>(gemm_skinny_kernel<BT>), Cfg::kSmemBytes).rc;
  if (rc != cudaSuccess) return rc;
  SkinnyArgs a;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.ldo = ldo;
  a.B = B;
  a.N = N;
  a.K = K;
  a.plan.tiles = (N + kBlockM - 1) / kBlockM;
  a.plan.num_kb = (K + kBlockK - 1) / kBlockK;
  a.plan.ctas = (int)std::min<long long>(sms, a.plan.units());
  a.silu_pairs = silu_pairs;
  SkinnyScratch* sc = skinny_scratch(stream, (size_t)a.plan.ctas * 2 * BT * kBlockM * sizeof(float),
                                     (size_t)a.plan.tiles);
  if (sc == nullptr) return cudaErrorMemoryAllocation;
  a.ws = sc->ws;
  a.counters = sc->counters;
  gemm_skinny_kernel<BT><<<a.plan.ctas, kSkinnyThreads, Cfg::kSmemBytes, stream>>>(mw, mx, a, error_word);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemm_skinny(const void* x, const void* w, void* out, int B, int N, int K, int ldx, int ldw,
                               int ldo, int silu_pairs, uint32_t* error_word, cudaStream_t stream) {
  if (B <= 0 || B > 128 || N <= 0 || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0)
    return cudaErrorInvalidValue;
  if (silu_pairs && N % kBlockM != 0) return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (B <= 64)
    return launch_skinny_bt<64>(x, w, out, B, N, K, ldx, ldw, ldo, silu_pairs, sms, error_word, stream);
  return launch_skinny_bt<128>(x, w, out, B, N, K, ldx, ldw, ldo, silu_pairs, sms, error_word, stream);
}

}  // namespace sm100
}  // namespace penny
