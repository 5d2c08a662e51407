// The persistent tcgen05 GEMM kernel, parameterised by a Policy that says
//   * which CTAs do side work instead of GEMM tiles (e.g. pushing A shards to
//     the peers) and what that work is,
//   * what the TMA producer must wait for before it may read the A rows of a
//     tile (nothing, or a "rows have arrived from their owner" flag),
//   * where finished rows go (local C, a peer's heap slot, ...) and what happens
//     when a tile is complete (e.g. raise a cross-GPU flag),
//   * what the epilogue warps do after their last tile (e.g. the reduction of a
//     reduce-scatter) and how the call is closed.
// See gemm_sm100.cu for the role layout.
#pragma once
#include "gemm_sm100.cuh"
#include "gemm_tile_order.h"

namespace penny {
namespace sm100 {

constexpr int kBlockM = 128;
constexpr int kGemmThreads = 320;  // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warps 6-9 copy
constexpr int kCopyThreads = 128;
constexpr int kStageRowBytes = 128;  // epilogue staging: 64 bf16 columns per row and pass

enum GemmError : uint32_t {
  GEMM_OK = 0,
  GEMM_ERR_PRODUCER_WAIT = 101,
  GEMM_ERR_MMA_WAIT = 102,
  GEMM_ERR_EPILOGUE_WAIT = 103,
  GEMM_ERR_GATE_WAIT = 104,
};

// The policy of the plain GEMM; also documents the interface.  A policy may
// replace State (what begin() returns and every hook receives) and any hook.
struct PolicyBase {
  struct State {};
  __device__ __forceinline__ State begin() const { return State{}; }
  // the 128 threads of the copy warps of CTA `cta` (tid in [0, 128)); they run
  // next to the CTA's GEMM roles and may only synchronise among themselves
  // (named barrier 2)
  template <class S>
  __device__ __forceinline__ void side_work(const S&, int /*cta*/, int /*ncta*/, int /*tid*/, uint32_t*) const {}
  // the producer thread, before the first A tile of a row block
  template <class S>
  __device__ __forceinline__ bool wait_rows(const S&, int /*m_blk*/, int /*n_blk*/) const { return true; }
  // rows added to the A tile coordinate (A may live in one of two buffers)
  template <class S>
  __device__ __forceinline__ int a_row_offset(const S&) const { return 0; }
  // the 128 epilogue threads
  template <class S>
  __device__ __forceinline__ void tile_begin(const S&, int, int) const {}
  template <class S>
  __device__ __forceinline__ void tile_end(const S&, int, int) const {}
  template <class S>
  __device__ __forceinline__ void after_tiles(const S&, int /*cta*/, int /*ncta*/, int /*tid*/,
                                              uint32_t*) const {}
  // every thread of every CTA, last thing in the kernel
  template <class S>
  __device__ __forceinline__ void finish(const S&) const {}
};

template <int BN>
struct GemmKernel {
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 192 ? 5 : 6);
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BN * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = (BN == 192) ? 512 : 2 * BN;  // two accumulators, a power of two
  static constexpr int kEpiStageBytes = 4 * 32 * kStageRowBytes;  // 4 warps x 32 rows x 128 B
  static constexpr int kSmemBytes =
      kStages * kStageBytes + kEpiStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

// 8 bf16 (16 bytes) of one C row, bounds-checked.
__device__ __forceinline__ void store16_local(__nv_bfloat16* c, int ldc, int row, int col, const uint4& v,
                                              int M, int N) {
  if (row >= M || col >= N) return;
  __nv_bfloat16* dst = c + (size_t)row * ldc + col;
  if (col + 8 <= N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
    *reinterpret_cast<uint4*>(dst) = v;
  } else {
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
    for (int i = 0; i < 8 && col + i < N; ++i) dst[i] = e[i];
  }
}

__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity,
                                                    volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = gtime_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0u) {
      if (*abort_flag) return false;
      if (gtime_ns() - t0 > kWaitNs) return false;
    }
  }
}

template <int BN, class Policy>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_persistent(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const GemmShape s, const Policy pol, uint32_t* error_word) {
  using Cfg = GemmKernel<BN>;
  const typename Policy::State st = pol.begin();
  const int cta = (int)blockIdx.x;
  const int ncta = (int)gridDim.x;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ unsigned char smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + kStages * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint64_t* tmem_empty = bars + 2 * kStages + 2;
  unsigned char* epi_stage = tiles + kStages * Cfg::kStageBytes + 256;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);  // one arrival per epilogue warp
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) tmem_alloc(tmem_holder, Cfg::kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const int num_kb = (s.K + kBlockK - 1) / kBlockK;

  auto decode = [&](int tile, int& m_blk, int& n_blk) { decode_tile(s, tile, m_blk, n_blk); };
  auto fail = [&](uint32_t code) {
    *s_abort = 1;
    atomicCAS(error_word, 0u, code);
  };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ TMA producer
      int stage = 0;
      uint32_t phase = 0;
      const int a_row0 = pol.a_row_offset(st);
      for (int tile = cta; tile < s.num_tiles && !*s_abort; tile += ncta) {
        int m_blk, n_blk;
        decode(tile, m_blk, n_blk);
        if (!pol.wait_rows(st, m_blk, n_blk)) {
          fail(GEMM_ERR_GATE_WAIT);
          break;
        }
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_abortable(&empty[stage], phase ^ 1u, s_abort)) {
            ok = false;
            break;
          }
          unsigned char* sa = tiles + stage * Cfg::kStageBytes;
          mbar_expect_tx(&full[stage], Cfg::kStageBytes);
          tma_load_2d(sa, &map_a, &full[stage], kb * kBlockK, a_row0 + m_blk * kBlockM);
          tma_load_2d(sa + Cfg::kABytes, &map_b, &full[stage], kb * kBlockK, n_blk * BN);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) {
          fail(GEMM_ERR_PRODUCER_WAIT);
          break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // -------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc = make_idesc_bf16(kBlockM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int tile = cta; tile < s.num_tiles && !*s_abort; tile += ncta, ++it) {
        const int ab = it & 1;
        const uint32_t ab_phase = (uint32_t)(it >> 1) & 1u;
        bool ok = mbar_wait_abortable(&tmem_empty[ab], ab_phase ^ 1u, s_abort);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(ab * BN);
        for (int kb = 0; ok && kb < num_kb; ++kb) {
          if (!mbar_wait_abortable(&full[stage], phase, s_abort)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(tiles + stage * Cfg::kStageBytes);
          const uint64_t da = make_smem_desc(sa);
          const uint64_t db = make_smem_desc(sa + Cfg::kABytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k)
            umma_bf16(d_tmem, advance_desc_k(da, k), advance_desc_k(db, k), idesc, (kb | k) != 0);
          umma_commit(&empty[stage]);  // the slot is free once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) {
          fail(GEMM_ERR_MMA_WAIT);
          break;
        }
        umma_commit(&tmem_full[ab]);  // accumulator complete
      }
    }
  } else if (warp < 6) {
    {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // the TMEM lane quarter this warp may read
    int it = 0;
    // The four epilogue warps share named barriers inside the policy hooks, so
    // they must leave this loop at the same tile: after each bounded wait they
    // vote, and a wait that ran out in ANY of them ends the loop for all.
    bool aborted = false;
    for (int tile = cta; tile < s.num_tiles; tile += ncta, ++it) {
      int m_blk, n_blk;
      decode(tile, m_blk, n_blk);
      const int ab = it & 1;
      const uint32_t ab_phase = (uint32_t)(it >> 1) & 1u;
      const bool ok = !*s_abort && mbar_wait_abortable(&tmem_full[ab], ab_phase, s_abort);
      if (!ok && lane == 0) fail(GEMM_ERR_EPILOGUE_WAIT);
      if (!named_bar_all(3, 128, ok)) {
        aborted = true;
        break;
      }
      tc_fence_after_sync();
      pol.tile_begin(st, m_blk, n_blk);
      // 64 columns per pass: TMEM -> registers (thread = row) -> this warp's
      // swizzled staging rows -> global, 8 lanes writing one contiguous 128-byte
      // row segment (full lines also when the destination is a peer's memory)
      unsigned char* stg = epi_stage + (warp - 2) * (32 * kStageRowBytes);
      const int row0 = m_blk * kBlockM + q * 32;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t r0[32], r1[32];
        const uint32_t taddr = tmem_base + (uint32_t)(ab * BN + c * 64) + ((uint32_t)(q * 32) << 16);
        tmem_ld_32x32(taddr, r0);
        tmem_ld_32x32(taddr + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = pack_bf16x2(r0[8 * j], r0[8 * j + 1]);
          v.y = pack_bf16x2(r0[8 * j + 2], r0[8 * j + 3]);
          v.z = pack_bf16x2(r0[8 * j + 4], r0[8 * j + 5]);
          v.w = pack_bf16x2(r0[8 * j + 6], r0[8 * j + 7]);
          *reinterpret_cast<uint4*>(stg + lane * kStageRowBytes + ((j ^ (lane & 7)) << 4)) = v;
          v.x = pack_bf16x2(r1[8 * j], r1[8 * j + 1]);
          v.y = pack_bf16x2(r1[8 * j + 2], r1[8 * j + 3]);
          v.z = pack_bf16x2(r1[8 * j + 4], r1[8 * j + 5]);
          v.w = pack_bf16x2(r1[8 * j + 6], r1[8 * j + 7]);
          *reinterpret_cast<uint4*>(stg + lane * kStageRowBytes + (((j + 4) ^ (lane & 7)) << 4)) = v;
        }
        __syncwarp();
#pragma unroll
        for (int it2 = 0; it2 < 8; ++it2) {
          const int rr = it2 * 4 + (lane >> 3), j = lane & 7;
          const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * kStageRowBytes + ((j ^ (rr & 7)) << 4));
          pol.store16(st, row0 + rr, n_blk * BN + c * 64 + j * 8, v, s.M, s.N);
        }
        __syncwarp();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[ab]);
      pol.tile_end(st, m_blk, n_blk);
    }
    if (!aborted) pol.after_tiles(st, cta, ncta, (int)threadIdx.x - 64, error_word);
  }
  } else {
    // ---------------------------------------------------------------- copy warps
    pol.side_work(st, cta, ncta, (int)threadIdx.x - 192, error_word);
  }
  // ------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  pol.finish(st);
}

}  // namespace sm100
}  // namespace penny
