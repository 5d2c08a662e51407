// Tensor-parallel GEMMs fused with their collective, one kernel each, over the
// peer-mapped symmetric heap (sequence-parallel transformer layers):
//
//   GEMM -> reduce-scatter   (row-parallel layer: o_proj, down_proj)
//     every rank computes its partial C_r = A_r B_r^T for ALL rows; the epilogue
//     of each 128 x BN tile converts it to bf16 and stores it straight into the
//     heap of the rank that owns those rows (slot [src rank]) and raises a
//     per-tile flag there.  Tiles are visited owner by owner starting with the
//     next rank and ending with the local rows, so the NVLink pushes overlap the
//     remaining MMAs.  After its last tile each CTA reduces a share of the local
//     tiles: wait for the `world` flags of a tile, add the slots in rank order
//     in fp32, write the output shard.
//
//   all-gather -> GEMM       (column-parallel layer: qkv, gate/up)
//     the copy warps of every CTA push the local A shard, 32 rows at a time, into
//     every peer's gathered-A buffer (local memory of the peer) and flag it;
//     the GEMM CTAs walk the row blocks starting with the local shard and their
//     TMA producer waits for a block's flag before loading it – from LOCAL
//     memory: remote tiles are landed first, never fetched by TMA from a peer,
//     and no load uses cluster multicast.
//
// Both run on CTA pairs (cta_group::2, 256 x 256 tiles; gemm_kernel_pair_sm100.cuh)
// when every rank's shard is a whole number of 256-row blocks and there is at
// least one tile per pair, else on the single-CTA 128 x BN kernel; the policies
// are the same for both.
//
// Both use the communicator's call sequence (scratch halves, flag values) like
// every other collective, and every wait is bounded.  The reference has neither
// (it has no GEMM at all); NCCL-based code runs the two steps back to back.
#include <algorithm>

#include "coll_args.h"
#include "gemm_fused_sm100.h"
#include "gemm_kernel_pair_sm100.cuh"
#include "gemm_kernel_sm100.cuh"
#include "gemm_sm100.h"
#include "kernel_setup.h"

namespace penny {
namespace sm100 {

namespace {

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

struct FusedState {
  u64 seq;
  size_t half;  // heap offset of this call's scratch half
};

// ----------------------------------------------------------------------------
// GEMM -> reduce-scatter
// scratch half: [world src][rows_per_shard][N] bf16
// ----------------------------------------------------------------------------
template <int BN>
struct GemmRsPolicy : PolicyBase {
  using State = FusedState;
  CommCtx c;
  size_t scratch_off, scratch_bytes;
  __nv_bfloat16* out;  // [rows_per_shard, N]
  int ldo;
  int N, rows_per_shard, tiles_per_shard, tiles_n, nblocks;

  __device__ __forceinline__ State begin() const {
    State s;
    s.seq = begin_call(c, c.rank, SEQ_ALL);
    s.half = scratch_half(scratch_off, scratch_bytes, s.seq);
    return s;
  }
  __device__ __forceinline__ void store16(const State& st, int row, int col, const uint4& v, int,
                                          int) const {
    const int owner = row / rows_per_shard;
    const int lrow = row - owner * rows_per_shard;
    char* dst = c.heap[owner] + st.half + (((size_t)c.rank * rows_per_shard + lrow) * N + col) * 2;
    V16 x;
    x.w[0] = v.x; x.w[1] = v.y; x.w[2] = v.z; x.w[3] = v.w;
    st16(dst, x);
  }
  __device__ __forceinline__ void tile_end(const State& st, int m_blk, int n_blk) const {
    // all 128 epilogue threads have issued their stores; one of them publishes the tile
    named_bar_sync(1, 128);
    if (threadIdx.x == 64) {
      const int owner = m_blk / tiles_per_shard;
      const int lt = (m_blk - owner * tiles_per_shard) * tiles_n + n_blk;
      st_release_sys(&pad_of(c, owner)->flag[CH_FUSED][lt][c.rank], flag_value(st.seq, 1));
    }
  }
  __device__ __forceinline__ void after_tiles(const State& st, int cta, int ncta, int tid,
                                              uint32_t* error_word) const {
    __shared__ int s_bad;
    const int local_tiles = tiles_per_shard * tiles_n;
    for (int lt = cta; lt < local_tiles; lt += ncta) {
      if (tid == 0) s_bad = 0;
      named_bar_sync(1, 128);
      if (tid < c.world) {
        if (!wait_flag_ge(&pad_of(c, c.rank)->flag[CH_FUSED][lt][tid], flag_value(st.seq, 1), c,
                          ST_TIMEOUT_TILE, tid, lt))
          s_bad = 1;
      }
      named_bar_sync(1, 128);
      if (s_bad) {
        if (tid == 0) atomicCAS(error_word, 0u, (uint32_t)GEMM_ERR_GATE_WAIT);
        return;
      }
      const int lrow0 = (lt / tiles_n) * kBlockM, col0 = (lt % tiles_n) * BN;
      constexpr int kVecPerRow = BN / 8;
      for (int idx = tid; idx < kBlockM * kVecPerRow; idx += 128) {
        const int r = idx / kVecPerRow, cv = idx % kVecPerRow;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        for (int s = 0; s < c.world; ++s) {
          const char* src = c.heap[c.rank] + st.half +
                            (((size_t)s * rows_per_shard + lrow0 + r) * N + col0 + cv * 8) * 2;
          unpack_add<__nv_bfloat16>(ld16(src), acc);
        }
        st16(out + (size_t)(lrow0 + r) * ldo + col0 + cv * 8, pack<__nv_bfloat16>(acc));
      }
    }
  }
  __device__ __forceinline__ void finish(const State& st) const {
    const Blk b{(int)blockIdx.x, nblocks, (int)blockDim.x};
    end_call(c, c.rank, b, st.seq, SEQ_ALL);
  }
};

// ----------------------------------------------------------------------------
// all-gather -> GEMM
// scratch half: gathered A [M, K] bf16 (row block m_blk comes from rank m_blk / tiles_per_shard)
// ----------------------------------------------------------------------------
struct AgGemmPolicy : PolicyBase {
  using State = FusedState;
  CommCtx c;
  size_t scratch_off, scratch_bytes;
  const __nv_bfloat16* a_shard;  // [rows_per_shard, K], row stride lda
  int lda;
  __nv_bfloat16* out;  // [M, N_local]
  int ldc;
  int K, rows_per_shard, tiles_per_shard, nblocks;

  __device__ __forceinline__ State begin() const {
    State s;
    s.seq = begin_call(c, c.rank, SEQ_ALL);
    s.half = scratch_half(scratch_off, scratch_bytes, s.seq);
    return s;
  }
  // unit u = (peer offset d, row block rb, quarter qq of 32 rows): d = 0 (the
  // local copy) first.  Run by the copy warps of every CTA, so the pushes share
  // the SMs with the MMAs instead of taking SMs away from them.
  static constexpr int kSub = 4;
  static constexpr int kDeep = 8;  // 16-byte vectors in flight per thread
  __device__ __forceinline__ void side_work(const State& st, int cta, int ncta, int tid, uint32_t*) const {
    const int units = c.world * tiles_per_shard * kSub;
    const int vec_per_row = K / 8;
    for (int u = cta; u < units; u += ncta) {
      const int d = u / (tiles_per_shard * kSub);
      const int rb = (u / kSub) % tiles_per_shard, qq = u % kSub;
      const int p = (c.rank + d) % c.world;
      const int row0 = rb * kBlockM + qq * (kBlockM / kSub);
      const int rows = max(0, min(kBlockM / kSub, rows_per_shard - row0));
      char* dst = c.heap[p] + st.half + ((size_t)(c.rank * rows_per_shard + row0) * K) * 2;
      const int total = rows * vec_per_row;
      for (int i0 = tid; i0 < total; i0 += kDeep * kCopyThreads) {
        V16 x[kDeep];
#pragma unroll
        for (int k = 0; k < kDeep; ++k) {
          const int i = i0 + k * kCopyThreads;
          if (i < total) {
            const int r = i / vec_per_row, cv = i % vec_per_row;
            x[k] = ld16(a_shard + (size_t)(row0 + r) * lda + cv * 8);
          }
        }
#pragma unroll
        for (int k = 0; k < kDeep; ++k) {
          const int i = i0 + k * kCopyThreads;
          if (i < total) st16(dst + (size_t)i * 16, x[k]);
        }
      }
      named_bar_sync(2, kCopyThreads);
      if (tid == 0) {
        const int m_blk = c.rank * tiles_per_shard + rb;
        st_release_sys(&pad_of(c, p)->flag[CH_FUSED][m_blk * kSub + qq][c.rank], flag_value(st.seq, 1));
      }
    }
  }
  __device__ __forceinline__ bool wait_rows(const State& st, int m_blk, int) const {
    const int owner = m_blk / tiles_per_shard;
    for (int qq = 0; qq < kSub; ++qq)
      if (!wait_flag_ge(&pad_of(c, c.rank)->flag[CH_FUSED][m_blk * kSub + qq][owner], flag_value(st.seq, 1),
                        c, ST_TIMEOUT_TILE, owner, m_blk))
        return false;
    fence_proxy_async();  // the rows were written by another GPU; TMA reads them next
    return true;
  }
  __device__ __forceinline__ int a_row_offset(const State& st) const {
    return (int)(st.seq & 1ull) * (rows_per_shard * c.world);
  }
  __device__ __forceinline__ void store16(const State&, int row, int col, const uint4& v, int M,
                                          int N) const {
    store16_local(out, ldc, row, col, v, M, N);
  }
  __device__ __forceinline__ void finish(const State& st) const {
    const Blk b{(int)blockIdx.x, nblocks, (int)blockDim.x};
    end_call(c, c.rank, b, st.seq, SEQ_ALL);
  }
};

int sm_count() {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace

size_t gemm_rs_scratch_bytes(int M, int N, int world) {
  return 2 * (size_t)M * N * 2;  // both halves of [world][M / world][N] bf16
  (void)world;
}
size_t ag_gemm_scratch_bytes(int M, int K) { return 2 * (size_t)M * K * 2; }

cudaError_t launch_gemm_rs(const CommCtx& c, size_t scratch_off, size_t scratch_bytes, const void* a,
                           const void* b, void* out, int M, int N, int K, int lda, int ldb, int ldo,
                           uint32_t* error_word, cudaStream_t stream) {
  constexpr int BN = 256;
  const int W = c.world;
  if (M % (W * kBlockM) != 0 || N % BN != 0 || K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || ldo % 8 != 0)
    return cudaErrorInvalidValue;
  const int tiles_m = M / kBlockM, tiles_n = N / BN, tps = tiles_m / W;
  if (tps * tiles_n > kMaxBlocks || scratch_bytes < gemm_rs_scratch_bytes(M, N, W))
    return cudaErrorInvalidValue;
  using Policy = GemmRsPolicy<BN>;
  const int sms = sm_count();
  const KernelSetup ks = kernel_setup(reinterpret_cast<const void*>(gemm_persistent_pair<Policy>),
                                      PairGemmKernel::kSmemBytes, kGemmThreads);
  if (ks.rc != cudaSuccess) return ks.rc;
  const int pairs = ks.pairs;
  const bool pair = pair_kernel_enabled() && tps % 2 == 0 && (tiles_m / 2) * tiles_n >= pairs && K >= 1024;
  CUtensorMap ma, mb;
  cudaError_t rc = make_tile_map(&ma, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kBlockM);
  if (rc != cudaSuccess) return rc;
  rc = make_tile_map(&mb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, pair ? BN / 2 : BN);
  if (rc != cudaSuccess) return rc;
  rc = kernel_setup(reinterpret_cast<const void*>(gemm_persistent<BN, Policy>), GemmKernel<BN>::kSmemBytes).rc;
  if (rc != cudaSuccess) return rc;
  const int grid = pair ? 2 * std::min(pairs, (tiles_m / 2) * tiles_n) : std::min(sms, tiles_m * tiles_n);
  Policy pol;
  pol.c = c;
  pol.scratch_off = scratch_off;
  pol.scratch_bytes = scratch_bytes;
  pol.out = reinterpret_cast<__nv_bfloat16*>(out);
  pol.ldo = ldo;
  pol.N = N;
  pol.rows_per_shard = M / W;
  pol.tiles_per_shard = tps;
  pol.tiles_n = tiles_n;
  pol.nblocks = grid;
  // owners in the order rank+1, rank+2, ..., rank: local rows last
  GemmShape shape{M, N, K, tiles_m, tiles_n, ((c.rank + 1) % W) * tps, tiles_m * tiles_n, 0, 0};
  if (pair)
    gemm_persistent_pair<Policy><<<grid, kGemmThreads, PairGemmKernel::kSmemBytes, stream>>>(
        ma, mb, shape, pol, error_word);
  else
    gemm_persistent<BN, Policy><<<grid, kGemmThreads, GemmKernel<BN>::kSmemBytes, stream>>>(
        ma, mb, shape, pol, error_word);
  return cudaGetLastError();
}

cudaError_t launch_ag_gemm(const CommCtx& c, size_t scratch_off, size_t scratch_bytes,
                           const void* a_shard, const void* b, void* out, int M, int N, int K, int lda,
                           int ldb, int ldc, int side_ctas, uint32_t* error_word,
                           cudaStream_t stream) {
  const int W = c.world;
  if (M % (W * kBlockM) != 0 || K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || N <= 0)
    return cudaErrorInvalidValue;
  const int tiles_m = M / kBlockM, tps = tiles_m / W;
  if (tiles_m * AgGemmPolicy::kSub > kMaxBlocks || scratch_bytes != ag_gemm_scratch_bytes(M, K))
    return cudaErrorInvalidValue;
  const int sms = sm_count();
  int BN = (N >= 256) ? 256 : 128;
  if (N >= 192) {
    // 128 x 192 tiles when they fill the SMs better (e.g. N = 768: 128 tiles instead of 96)
    auto waves = [&](int bn) { return (double)((tiles_m * ((N + bn - 1) / bn) + sms - 1) / sms); };
    if (waves(192) * 0.75 * 1.20 < waves(256) * 1.12) BN = 192;
  }
  const int tiles_n = (N + BN - 1) / BN;
  (void)side_ctas;  // kept for API compatibility: the pushes are done by copy warps of every CTA
  const KernelSetup ks = kernel_setup(reinterpret_cast<const void*>(gemm_persistent_pair<AgGemmPolicy>),
                                      PairGemmKernel::kSmemBytes, kGemmThreads);
  if (ks.rc != cudaSuccess) return ks.rc;
  const int pairs = ks.pairs;
  const bool pair = pair_kernel_enabled() && BN == 256 && tps % 2 == 0 && (tiles_m / 2) * tiles_n >= pairs &&
                    K >= 1024;
  const int grid = pair ? 2 * std::min(pairs, (tiles_m / 2) * tiles_n)
                        : std::min(sms, std::max(tiles_m * tiles_n, 1));
  AgGemmPolicy pol;
  pol.c = c;
  pol.scratch_off = scratch_off;
  pol.scratch_bytes = scratch_bytes;
  pol.a_shard = reinterpret_cast<const __nv_bfloat16*>(a_shard);
  pol.lda = lda;
  pol.out = reinterpret_cast<__nv_bfloat16*>(out);
  pol.ldc = ldc;
  pol.K = K;
  pol.rows_per_shard = M / W;
  pol.tiles_per_shard = tps;
  pol.nblocks = grid;
  // Which half holds the gathered A of this call is only known on the device
  // (parity of the call number), so the two halves are described as ONE matrix
  // of 2*M rows and the producer adds M * parity to the row coordinate.  That
  // needs the halves to be exactly M*K elements: the region is dedicated to
  // this (M, K) and scratch_bytes is exactly ag_gemm_scratch_bytes(M, K).
  CUtensorMap ma, mb;
  const char* afull = c.heap[c.rank] + scratch_off;
  cudaError_t rc = make_tile_map(&ma, afull, (uint64_t)2 * M, (uint64_t)K, (uint64_t)K, kBlockM);
  if (rc != cudaSuccess) return rc;
  rc = make_tile_map(&mb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, pair ? 128 : BN);
  if (rc != cudaSuccess) return rc;
  GemmShape shape{M, N, K, tiles_m, tiles_n, c.rank * tps, tiles_m * tiles_n, 0, 0};
  if (pair) {
    gemm_persistent_pair<AgGemmPolicy><<<grid, kGemmThreads, PairGemmKernel::kSmemBytes, stream>>>(
        ma, mb, shape, pol, error_word);
  } else if (BN == 192) {
    rc = kernel_setup(reinterpret_cast<const void*>(gemm_persistent<192, AgGemmPolicy>), GemmKernel<192>::kSmemBytes).rc;
    if (rc != cudaSuccess) return rc;
    gemm_persistent<192, AgGemmPolicy><<<grid, kGemmThreads, GemmKernel<192>::kSmemBytes, stream>>>(
        ma, mb, shape, pol, error_word);
  } else if (BN == 256) {
    rc = kernel_setup(reinterpret_cast<const void*>(gemm_persistent<256, AgGemmPolicy>), GemmKernel<256>::kSmemBytes).rc;
    if (rc != cudaSuccess) return rc;
    gemm_persistent<256, AgGemmPolicy><<<grid, kGemmThreads, GemmKernel<256>::kSmemBytes, stream>>>(
        ma, mb, shape, pol, error_word);
  } else {
    rc = kernel_setup(reinterpret_cast<const void*>(gemm_persistent<128, AgGemmPolicy>), GemmKernel<128>::kSmemBytes).rc;
    if (rc != cudaSuccess) return rc;
    gemm_persistent<128, AgGemmPolicy><<<grid, kGemmThreads, GemmKernel<128>::kSmemBytes, stream>>>(
        ma, mb, shape, pol, error_word);
  }
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace penny
