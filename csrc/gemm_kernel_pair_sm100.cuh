// The persistent tcgen05 GEMM kernel on CTA pairs (cta_group::2): two CTAs of a
// cluster of size 2, on neighbouring SMs, compute one 256 x 256 tile.
//
//   * CTA r of the pair owns row block m_blk = 2 * pair_row + r.  It stages its
//     own [128 x 64] A tile and its own half of the B tile ([128 x 64], B rows
//     n_blk * 256 + r * 128 ...) per K step: 32 KB per CTA and stage instead of
//     the 48 KB of the single-CTA 128 x 256 tile, i.e. one third less
//     L2 -> shared-memory traffic per FLOP, which is what bounds that kernel.
//   * The leader (r = 0) issues tcgen05.mma.cta_group::2 with M = 256, N = 256:
//     the tensor cores of both SMs read both CTAs' shared memory at the same
//     offsets; rows 0-127 of the result land in the leader's TMEM, rows 128-255
//     in the other CTA's, at the same columns.
//   * All "data has landed" barriers live in the leader: both producers' TMA
//     loads count their bytes there (the leader arms it for both).  "Slot free"
//     and "accumulator ready" are signalled to both CTAs by one multicast
//     tcgen05.commit; "accumulator drained" is counted in the leader from the
//     epilogue warps of both CTAs.
//   * Each CTA drains its own 128 accumulator rows exactly like the single-CTA
//     kernel, through the same Policy hooks, so the fused variants plug in.
//   * Ragged last wave: when GemmShape::split_s > 1 the leftover tiles are cut
//     along K into split_s ranges computed by different pairs at the same time
//     (gemm_tile_order.h: plan_split_tail / pair_work).  Each range's fp32
//     accumulator goes to a workspace; the CTA that arrives last on the tile's
//     counter adds the ranges in order and runs the normal epilogue, then
//     resets the counter for the next launch.
// Every wait is bounded; a failure in one CTA also raises the abort flag of the
// other.  Both CTAs pass a cluster barrier before the pair's TMEM is freed.
#pragma once
#include "gemm_kernel_sm100.cuh"

namespace penny {
namespace sm100 {

struct PairGemmKernel {
  static constexpr int kTileN = 256;
  static constexpr int kStages = 6;
  static constexpr int kABytes = kBlockM * kBlockK * 2;          // this CTA's A rows
  static constexpr int kBBytes = (kTileN / 2) * kBlockK * 2;     // this CTA's half of B
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * kTileN;                   // two accumulators
  static constexpr int kEpiStageBytes = 4 * 32 * kStageRowBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiStageBytes + 1024 + 256;
};

template <class Policy>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_persistent_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const GemmShape s, const Policy pol, uint32_t* error_word) {
  using Cfg = PairGemmKernel;
  constexpr int BN = Cfg::kTileN;
  constexpr int kStages = Cfg::kStages;
  const typename Policy::State st = pol.begin();
  const int cta = (int)blockIdx.x;
  const int ncta = (int)gridDim.x;
  const uint32_t r = cluster_ctarank();
  const int pair = cta >> 1, npairs = ncta >> 1;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + kStages * Cfg::kStageBytes);
  uint64_t* full = bars;                         // used in the leader only
  uint64_t* empty = bars + kStages;              // one in each CTA
  uint64_t* tmem_full = bars + 2 * kStages;      // one in each CTA
  uint64_t* tmem_empty = bars + 2 * kStages + 2; // used in the leader only
  unsigned char* epi_stage = tiles + kStages * Cfg::kStageBytes + 256;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* s_last = reinterpret_cast<volatile int*>(tmem_holder + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full[i], 1);   // the leader's producer arms it for both CTAs' bytes
      mbar_init(&empty[i], 1);  // one multicast commit
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 8);  // four epilogue warps in each CTA
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  __syncwarp();
  if (warp == 1) tmem_alloc_pair(tmem_holder, Cfg::kTmemCols);
  tc_fence_before_sync();
  __syncwarp();
  cluster_sync_all();  // barriers of both CTAs are initialised before either is used
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const int num_kb = (s.K + kBlockK - 1) / kBlockK;

  auto decode = [&](int tile, int& m_blk, int& n_blk) { decode_pair_tile(s, tile, (int)r, m_blk, n_blk); };
  auto fail = [&](uint32_t code) {
    *s_abort = 1;
    st_cluster_u32(map_to_cta(smem_u32(const_cast<int*>(s_abort)), r ^ 1u), 1u);
    atomicCAS(error_word, 0u, code);
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------- TMA producer (in each CTA)
      int stage = 0;
      uint32_t phase = 0;
      const int a_row0 = pol.a_row_offset(st);
      bool ok = true;
      PairWork w;
      for (int it = 0; pair_work(s, num_kb, pair, npairs, it, w) && !*s_abort; ++it) {
        int m_blk, n_blk;
        decode(w.tile, m_blk, n_blk);
        if (m_blk < s.tiles_m && !pol.wait_rows(st, m_blk, n_blk)) {
          fail(GEMM_ERR_GATE_WAIT);
          ok = false;
          break;
        }
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait_abortable(&empty[stage], phase ^ 1u, s_abort)) {
            ok = false;
            break;
          }
          unsigned char* sa = tiles + stage * Cfg::kStageBytes;
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0u);
          if (r == 0) mbar_expect_tx(&full[stage], 2u * Cfg::kStageBytes);
          tma_load_2d_pair(sa, &map_a, bar, kb * kBlockK, a_row0 + m_blk * kBlockM);
          tma_load_2d_pair(sa + Cfg::kABytes, &map_b, bar, kb * kBlockK, n_blk * BN + (int)r * (BN / 2));
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
      // tail: every commit aimed at this CTA's slot barriers has arrived before
      // the CTA may leave
      for (int i = 0; ok && i < kStages && !*s_abort; ++i) {
        if (!mbar_wait_abortable(&empty[stage], phase ^ 1u, s_abort)) break;
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && r == 0) {
      // ------------------------------------------- MMA issuer (leader CTA only)
      constexpr uint32_t idesc = make_idesc_bf16(2 * kBlockM, BN);
      int stage = 0;
      uint32_t phase = 0;
      PairWork w;
      for (int it = 0; pair_work(s, num_kb, pair, npairs, it, w) && !*s_abort; ++it) {
        const int ab = it & 1;
        const uint32_t ab_phase = (uint32_t)(it >> 1) & 1u;
        bool ok = mbar_wait_abortable(&tmem_empty[ab], ab_phase ^ 1u, s_abort);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(ab * BN);
        for (int kb = w.kb0; ok && kb < w.kb1; ++kb) {
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
            umma_bf16_pair(d_tmem, advance_desc_k(da, k), advance_desc_k(db, k), idesc,
                           (kb != w.kb0) || k != 0);
          umma_commit_pair(&empty[stage], (uint16_t)3);  // frees the slot in both CTAs
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) {
          fail(GEMM_ERR_MMA_WAIT);
          break;
        }
        umma_commit_pair(&tmem_full[ab], (uint16_t)3);  // accumulator complete, both halves
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------- epilogue (own 128 rows, in each CTA)
    const int q = warp & 3;
    unsigned char* stg = epi_stage + (warp - 2) * (32 * kStageRowBytes);
    // 64 columns of this warp's 32 rows (fp32 bit patterns, thread = row) ->
    // bf16 -> swizzled staging rows -> 128-byte row segments through the policy
    auto emit = [&](int c, const uint32_t (&r0)[32], const uint32_t (&r1)[32], int row0, int n_blk) {
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
    };
    PairWork w;
    // The four epilogue warps share named barriers (policy hooks, split tiles), so
    // they must leave this loop at the same tile: after each bounded wait they
    // vote, and a wait that ran out in ANY of them ends the loop for all.
    bool aborted = false;
    for (int it = 0; pair_work(s, num_kb, pair, npairs, it, w); ++it) {
      int m_blk, n_blk;
      decode(w.tile, m_blk, n_blk);
      const int ab = it & 1;
      const uint32_t ab_phase = (uint32_t)(it >> 1) & 1u;
      const bool ok = !*s_abort && mbar_wait_abortable(&tmem_full[ab], ab_phase, s_abort);
      if (!ok && lane == 0) fail(GEMM_ERR_EPILOGUE_WAIT);
      if (!named_bar_all(3, 128, ok)) {
        aborted = true;
        break;
      }
      tc_fence_after_sync();
      const bool live = m_blk < s.tiles_m;  // an odd last row block has no partner rows
      const bool split = s.split_s > 1 && w.tile >= s.split_first;
      const int row0 = m_blk * kBlockM + q * 32;
      const uint32_t tacc = tmem_base + (uint32_t)(ab * BN) + ((uint32_t)(q * 32) << 16);
      if (!split) {
        if (live) pol.tile_begin(st, m_blk, n_blk);
#pragma unroll 1
        for (int c = 0; live && c < BN / 64; ++c) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(tacc + c * 64, r0);
          tmem_ld_32x32(tacc + c * 64 + 32, r1);
          tmem_ld_wait();
          emit(c, r0, r1, row0, n_blk);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[ab]), 0u));
        if (live) pol.tile_end(st, m_blk, n_blk);
        continue;
      }
      // ---- one K range of a split tile: park the fp32 partial, the last one in adds them up
      const int tail = w.tile - s.split_first;
      // partial of (range, CTA): [64 vectors of 4 columns][128 rows] float4, so that the
      // 32 rows of a warp are 512 contiguous bytes in every load and store
      const int row_in_cta = q * 32 + lane;
      auto part = [&](int seg) {
        return reinterpret_cast<float4*>(s.split_ws) +
               (size_t)((tail * s.split_s + seg) * 2 + (int)r) * (kBlockM * BN / 4) + row_in_cta;
      };
#pragma unroll 1
      for (int c = 0; live && c < BN / 64; ++c) {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(tacc + c * 64, r0);
        tmem_ld_32x32(tacc + c * 64 + 32, r1);
        tmem_ld_wait();
        float4* dst = part(w.seg) + (size_t)(c * 16) * kBlockM;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dst[(size_t)j * kBlockM] = make_float4(__uint_as_float(r0[4 * j]), __uint_as_float(r0[4 * j + 1]),
                                                 __uint_as_float(r0[4 * j + 2]), __uint_as_float(r0[4 * j + 3]));
          dst[(size_t)(8 + j) * kBlockM] = make_float4(__uint_as_float(r1[4 * j]), __uint_as_float(r1[4 * j + 1]),
                                                       __uint_as_float(r1[4 * j + 2]), __uint_as_float(r1[4 * j + 3]));
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[ab]), 0u));
      if (!live) continue;  // the same for every range of this tile and CTA: no counter traffic
      __threadfence();
      named_bar_sync(1, 128);
      if (threadIdx.x == 64) {
        unsigned* cnt = s.split_counters + tail * 2 + (int)r;
        const unsigned old = atomicAdd(cnt, 1u);
        const int last = old == (unsigned)(s.split_s - 1);
        if (last) *cnt = 0u;  // every range has arrived: ready for the next launch
        *s_last = last;
      }
      named_bar_sync(1, 128);
      if (!*s_last) continue;
      __threadfence();
      pol.tile_begin(st, m_blk, n_blk);
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        float f0[32], f1[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f0[j] = f1[j] = 0.f;
        for (int seg = 0; seg < s.split_s; ++seg) {  // fixed order: the sum does not depend on who is last
          const float4* src = part(seg) + (size_t)(c * 16) * kBlockM;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 x = __ldcg(src + (size_t)j * kBlockM), y = __ldcg(src + (size_t)(8 + j) * kBlockM);
            f0[4 * j] += x.x; f0[4 * j + 1] += x.y; f0[4 * j + 2] += x.z; f0[4 * j + 3] += x.w;
            f1[4 * j] += y.x; f1[4 * j + 1] += y.y; f1[4 * j + 2] += y.z; f1[4 * j + 3] += y.w;
          }
        }
        uint32_t r0[32], r1[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          r0[j] = __float_as_uint(f0[j]);
          r1[j] = __float_as_uint(f1[j]);
        }
        emit(c, r0, r1, row0, n_blk);
      }
      pol.tile_end(st, m_blk, n_blk);
      named_bar_sync(1, 128);  // s_last is rewritten by the next split tile only after all have read it
    }
    if (!aborted) pol.after_tiles(st, cta, ncta, (int)threadIdx.x - 64, error_word);
  } else {
    // ---------------------------------------------------------------- copy warps
    pol.side_work(st, cta, ncta, (int)threadIdx.x - 192, error_word);
  }
  // ------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncwarp();
  cluster_sync_all();  // neither CTA touches the other's shared memory or TMEM after this
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  }
  pol.finish(st);
}

}  // namespace sm100
}  // namespace penny
