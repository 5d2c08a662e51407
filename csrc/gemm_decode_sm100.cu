// Decode-batch linear on sm_100a:
//     out[B, N] = x[B, K] * W[N, K]^T        bf16, fp32 accumulate, B <= 128
// With a handful of activation rows the operation is one read of W; at
// tensor-parallel shard sizes that read lasts 1-5 us, so what decides the time
// of a decode step is how early every SM starts streaming and how little
// happens after the last byte has arrived.
//
//   * Operands are swapped with respect to a large GEMM: the 128 rows of a W tile
//     are the M side of tcgen05.mma (K-major as stored), the batch rows of x are
//     the N side (32, 64 or 128 wide).  TMEM lane = output column n, TMEM column =
//     batch row.
//   * One CTA per (W tile, K range).  The K ranges of a tile belong to the CTAs
//     of one thread-block cluster (1-8 CTAs), which add their fp32 partials
//     through distributed shared memory: every CTA owns a slice of the batch
//     columns, receives that slice from its peers (st.shared::cluster + one
//     mbarrier arrival per peer), adds in rank order and stores bf16.  No global
//     workspace, no atomics, no second pass, deterministic.  The cluster size is
//     chosen per shape from a small time model (decode_gemm_plan.h).
//   * Programmatic dependent launch: the kernel may start while its predecessor
//     is still running.  Barrier set-up, TMEM allocation, the cluster handshake,
//     the TMA loads of the first W stages and an L2 prefetch of the rest of this
//     CTA's W range (bounded by a byte budget) all happen BEFORE the dependency
//     wait; only the x tiles wait for the predecessor.  W must therefore not be
//     written by the kernel launched just before (weights never are).
//   * 3-4 stage TMA ring of 24 KB (B <= 64), at most ~106 KB of shared memory, so
//     two of these kernels (or one and the decode attention) are resident per SM:
//     that is what lets the next kernel's prologue overlap this one.
//   * warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue.  Every wait
//     is bounded; TMEM is always freed.
//
// Epilogues: plain store, or silu(gate) * up for a gate/up weight whose rows are
// interleaved in blocks of 64 (tile = 64 gate rows + the 64 up rows of the same
// features; out is [B, N / 2]).
//
// The reference has no GEMM of any kind (it is a collectives library used
// inside vLLM / SGLang, README.md:20-33); this kernel is what lets the TP-decode
// benchmark run without a vendor GEMM between the collectives.
#include "gemm_decode_sm100.h"

#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>

#include "all_reduce_oneshot.cuh"
#include "decode_gemm_plan.h"
#include "gemm_kernel_sm100.cuh"
#include "gemm_sm100.h"
#include "kernel_setup.h"
#include "pdl.h"

namespace penny {

namespace {
std::atomic<int> g_pdl{-1};
}
void set_pdl_enabled(int on) { g_pdl.store(on < 0 ? -1 : (on != 0)); }
bool pdl_enabled() {
  const int v = g_pdl.load();
  if (v >= 0) return v != 0;
  static const bool on = []() {
    const char* e = getenv("PENNY_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

namespace sm100 {

namespace {

constexpr int kDecThreads = 192;
constexpr int kMaxStages = 8;

// Diagnostics: with PENNY_DEC_STAMPS=1 the first 512 CTAs of a launch record
// %globaltimer at eight points (see gemm_decode_stamps in the header).
constexpr int kStampCtas = 512, kStampPoints = 8;
__device__ unsigned long long g_dec_stamps[kStampCtas * kStampPoints];

struct DecodeArgs {
  __nv_bfloat16* out;
  int ldo;
  int B, N, K;
  int num_kb;       // K steps of 64 elements
  int splits;       // CTAs per cluster = K ranges per tile
  int stages;       // depth of the TMA ring
  int l2_prefetch;  // K steps beyond the ring that the producer prefetches into L2 before the dependency wait
  int l2_ahead;     // steady state: W of step i + l2_ahead is prefetched into L2 when step i is loaded
  int k_stagger;    // 1: tiles start their K range at different offsets
  int stamps;       // 1: record timestamps
  int epi;          // DECODE_EPI_*
  int slabs;        // batch slabs of BT rows (1 unless B > 128)
  DecodePush push;  // world == 0: plain store
};

template <int BT>
struct DecodeCfg {
  static constexpr int kWBytes = kBlockM * kBlockK * 2;  // 16 KB of weights per stage
  static constexpr int kXBytes = BT * kBlockK * 2;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kTmemCols = BT < 32 ? 32 : BT;
  // the peers' partials of this CTA's column slice: [splits - 1][slice][128 rows] fp32
  __host__ __device__ static size_t recv_floats(int splits) { return decode_recv_floats(BT, splits); }
  // The ring doubles as the [BT][128] fp32 staging area of the epilogue, so it is never smaller than that.
  __host__ __device__ static int min_stages() { return (BT * kBlockM * 4 + kStageBytes - 1) / kStageBytes; }
  static size_t smem_bytes(int stages, int splits) {
    return (size_t)stages * kStageBytes + recv_floats(splits) * 4 + 1024 /*alignment*/ + 256 /*barriers*/;
  }
};

__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, const float4& v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait for the peers' partials (they were written by other SMs, hence
// the cluster-scope acquire).
__device__ __forceinline__ bool mbar_wait_cluster_abortable(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = gtime_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((i & 255u) == 0u) {
      if (*abort_flag) return false;
      if (gtime_ns() - t0 > kWaitNs) return false;
    }
  }
}
// One [128 x 64] box of W into L2 only (no shared memory, no barrier).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(m), "r"(x), "r"(y) : "memory");
}

template <int BT>
__global__ void __launch_bounds__(kDecThreads)
gemm_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const DecodeArgs a, uint32_t* error_word) {
  using Cfg = DecodeCfg<BT>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
  const int S = a.splits, stages = a.stages;
  float* aux = reinterpret_cast<float*>(tiles + (size_t)stages * Cfg::kStageBytes);
  float* s_recv = aux;  // [S - 1][slice][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(aux + Cfg::recv_floats(S));
  uint64_t* full = bars;
  uint64_t* empty = bars + kMaxStages;
  uint64_t* tmem_full = bars + 2 * kMaxStages;
  uint64_t* recv_bar = bars + 2 * kMaxStages + 1;  // [4]: one per epilogue warp (row quarter)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 5);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_holder + 1);

  pdl_launch_dependents();
  const int cta_lin = (int)(blockIdx.y * gridDim.x + blockIdx.x);
  auto stamp = [&](int point) {
    if (a.stamps && cta_lin < kStampCtas) g_dec_stamps[cta_lin * kStampPoints + point] = gtime_ns();
  };
  if (threadIdx.x == 0) stamp(0);  // CTA start

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = S > 1 ? cluster_ctarank() : 0u;
  // batches above BT rows: grid y = tile * slabs + slab, so the slabs of a weight tile are dispatched
  // next to each other and read the tile from DRAM once
  const int tile = (int)blockIdx.y / a.slabs;
  const int row0 = ((int)blockIdx.y % a.slabs) * BT;
  const int kb0 = decode_kb_begin(a.num_kb, S, (int)crank), kb1 = decode_kb_begin(a.num_kb, S, (int)crank + 1);
  const int nkb = kb1 - kb0;
  const int sl = decode_slice(BT, S);
  // Tiles walk their K range from different starting points (and wrap around), so that at any
  // moment the CTAs of a wave read different column ranges of W rather than the same few
  // hundred bytes of every row.
  const int kshift = a.k_stagger ? (int)(((unsigned)tile * 2654435761u >> 8) % (unsigned)nkb) : 0;
  auto kb_at = [&](int i) {
    int k = i + kshift;
    if (k >= nkb) k -= nkb;
    return kb0 + k;
  };

  const int pre = min(stages, nkb);
  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(tmem_full, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&recv_bar[i], S > 1 ? (uint32_t)(S - 1) : 1u);
    *s_abort = 0;
    mbar_fence_init();
    // The first ring-full of W tiles is requested before anything else happens in
    // the CTA (TMEM allocation, the block and cluster barriers): its HBM latency
    // runs under the rest of the prologue.  W never depends on the predecessor.
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(&full[i], Cfg::kStageBytes);
      tma_load_2d(tiles + (size_t)i * Cfg::kStageBytes, &map_w, &full[i], kb_at(i) * kBlockK, tile * kBlockM);
    }
    tma_prefetch_desc(&map_x);
  }
  if (warp == 1) tmem_alloc(tmem_holder, Cfg::kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // The peers' receive barriers must exist before anyone arrives on them: every thread
  // arrives on the cluster barrier now and waits for it only where it first needs the
  // peers (epilogue warps: before their first remote store; the others: before they leave),
  // so the cluster-wide rendezvous is off the path to the first load and the first MMA.
  if (S > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  auto fail = [&](uint32_t code) {
    *s_abort = 1;
    atomicCAS(error_word, 0u, code);
  };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ TMA producer
      // W of the next K steps goes to L2 ahead of the ring (the whole range when the
      // matrix fits the L2 budget, else a rolling window), still before the
      // dependency wait; the x tiles come after it.
      int pf_next = min(nkb, pre + a.l2_prefetch);
      for (int i = pre; i < pf_next; ++i) tma_prefetch_l2_2d(&map_w, kb_at(i) * kBlockK, tile * kBlockM);
      stamp(1);  // prologue done, about to wait for the predecessor
      pdl_wait();
      stamp(2);  // predecessor complete
      for (int i = 0; i < pre; ++i)
        tma_load_2d(tiles + (size_t)i * Cfg::kStageBytes + Cfg::kWBytes, &map_x, &full[i], kb_at(i) * kBlockK, row0);
      int stage = pre == stages ? 0 : pre;
      uint32_t phase = pre == stages ? 1u : 0u;
      bool ok = true;
      for (int i = pre; i < nkb; ++i) {
        if (!mbar_wait_abortable(&empty[stage], phase ^ 1u, s_abort)) {
          ok = false;
          break;
        }
        unsigned char* sw = tiles + (size_t)stage * Cfg::kStageBytes;
        mbar_expect_tx(&full[stage], Cfg::kStageBytes);
        tma_load_2d(sw, &map_w, &full[stage], kb_at(i) * kBlockK, tile * kBlockM);
        tma_load_2d(sw + Cfg::kWBytes, &map_x, &full[stage], kb_at(i) * kBlockK, row0);
        if (pf_next < nkb && pf_next < i + a.l2_ahead) {
          tma_prefetch_l2_2d(&map_w, kb_at(pf_next) * kBlockK, tile * kBlockM);
          ++pf_next;
        }
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      stamp(3);  // last load issued
      if (!ok) fail(GEMM_ERR_PRODUCER_WAIT);
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // -------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc = make_idesc_bf16(kBlockM, BT);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait_abortable(&full[stage], phase, s_abort)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sw = smem_u32(tiles + (size_t)stage * Cfg::kStageBytes);
        const uint64_t dw = make_smem_desc(sw);
        const uint64_t dx = make_smem_desc(sw + Cfg::kWBytes);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k)
          umma_bf16(tmem_base, advance_desc_k(dw, k), advance_desc_k(dx, k), idesc, (i | k) != 0);
        umma_commit(&empty[stage]);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      stamp(4);  // last MMA issued
      if (ok)
        umma_commit(tmem_full);
      else
        fail(GEMM_ERR_MMA_WAIT);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue
    // Everything after the TMEM read works on shared memory with run-time loops:
    // the code stays small (an unrolled per-column epilogue costs more in
    // instruction-cache misses than the whole GEMM takes).  Each warp owns a
    // quarter of the tile's rows from TMEM to the final store, so the four warps
    // never wait for one another (except for the gate/up pairing).
    const int q = warp & 3;         // TMEM lane quarter of this warp
    const int row = q * 32 + lane;  // weight row inside the tile = output column
    const bool silu = a.epi == DECODE_EPI_SILU_PAIRS;
    bool ok = mbar_wait_abortable(tmem_full, 0u, s_abort);
    if (!ok && lane == 0) fail(GEMM_ERR_EPILOGUE_WAIT);
    ok = __all_sync(0xffffffffu, ok);
    if (q == 0 && lane == 0) stamp(5);  // accumulator complete
    tc_fence_after_sync();
    pdl_wait();  // this thread's stores come after everything the predecessor did
    // accumulator -> shared memory, column-major [BT columns][128 rows] fp32, in the
    // pipeline stages (every MMA that read them has completed)
    float* s_acc = reinterpret_cast<float*>(tiles);
    if (ok) {
      const uint32_t tacc = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BT / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tacc + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) s_acc[(c * 32 + j) * kBlockM + row] = __uint_as_float(r[j]);
      }
    }
    __syncwarp();
    const float4* s_acc4 = reinterpret_cast<const float4*>(s_acc);
    if (S > 1) {
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // the peers' barriers exist
      if (ok) {
        // ---- hand every other CTA the rows of this warp of its column slice: a store
        // instruction covers 4 columns x 128 bytes; then one release-arrive per peer ----
        const uint32_t recv_local = smem_u32(s_recv);
        const int rv = q * 8 + (lane & 7), cl = lane >> 3;  // float4 of my quarter, column within a group of 4
        for (int d = 0; d < S; ++d) {
          if (d == (int)crank) continue;
          const int lo = d * sl, hi = min(BT, lo + sl);
          const uint32_t remote =
              map_to_cta(recv_local, (uint32_t)d) + (uint32_t)(decode_recv_slot((int)crank, d) * sl * kBlockM * 4);
          for (int c = lo + cl; c < hi; c += 4)
            st_cluster_v4(remote + (uint32_t)(((c - lo) * (kBlockM / 4) + rv) * 16), s_acc4[c * (kBlockM / 4) + rv]);
        }
        __syncwarp();
        if (lane == 0) {
          for (int d = 0; d < S; ++d)
            if (d != (int)crank) mbar_arrive_cluster(map_to_cta(smem_u32(&recv_bar[q]), (uint32_t)d));
        }
      }
    }
    if (silu) named_bar_sync(1, 128);  // gate rows meet the up rows another warp staged
    if (ok && S > 1) {
      // my rows of the peers' partials (gate/up pairing: every quarter)
      for (int w = 0; w < 4; ++w) {
        if (!silu && w != q) continue;
        if (!mbar_wait_cluster_abortable(&recv_bar[w], 0u, s_abort)) ok = false;
      }
      if (!ok && lane == 0) fail(GEMM_ERR_EPILOGUE_WAIT);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (q == 0 && lane == 0) stamp(6);  // peers' partials received
    if (ok) {
      // ---- my slice: add the peers' partials in rank order, apply the epilogue, store.
      // A work item is 8 consecutive rows (output columns) of one batch column; a warp takes the
      // items of its own row quarter (gate/up: gate rows 16 q .. 16 q + 15 and their up rows).
      const int lo = (int)crank * sl, hi = min(min(BT, lo + sl), a.B - row0);
      const int groups = silu ? 2 : 4;  // row groups of 8 per column in this warp's share
      const int n_out = silu ? a.N / 2 : a.N;
      const int n_tile0 = tile * (silu ? kBlockM / 2 : kBlockM);
      const bool vec_ok = (a.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.out) & 15u) == 0);
      // push mode: the call number of the all-reduce that follows (final: the predecessor has
      // finished) selects the scratch half and stamps the lines
      unsigned long long push_seq = 0;
      size_t push_base = 0;
      if (a.push.world > 0) {
        push_seq = *reinterpret_cast<const volatile unsigned long long*>(a.push.call_seq);
        push_base = scratch_half(a.push.scratch_off, a.push.scratch_bytes, push_seq);
      }
      for (int idx = lane; idx < (hi - lo) * groups; idx += 32) {
        const int j = lo + idx / groups, g = q * groups + idx % groups;
        // sum over the cluster of rows r0 .. r0 + 7 of column j
        auto sum8 = [&](int r0, float (&acc)[8]) {
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] = 0.f;
          for (int src = 0; src < S; ++src) {
            const float4* p = src == (int)crank
                                  ? s_acc4 + (j * kBlockM + r0) / 4
                                  : reinterpret_cast<const float4*>(s_recv) +
                                        ((decode_recv_slot(src, (int)crank) * sl + (j - lo)) * kBlockM + r0) / 4;
            const float4 v0 = p[0], v1 = p[1];
            acc[0] += v0.x; acc[1] += v0.y; acc[2] += v0.z; acc[3] += v0.w;
            acc[4] += v1.x; acc[5] += v1.y; acc[6] += v1.z; acc[7] += v1.w;
          }
        };
        float v[8];
        sum8(g * 8, v);
        if (silu) {
          // rows 0-63 of the tile are gate, rows 64-127 the matching up rows
          float u[8];
          sum8(64 + g * 8, u);
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] = v[k] / (1.f + __expf(-v[k])) * u[k];
        }
        const int n0 = n_tile0 + g * 8;
        __nv_bfloat16* dst = a.out + (size_t)(row0 + j) * a.ldo + n0;
        if (vec_ok && n0 + 8 <= n_out) {
          uint4 o;
          o.x = pack_bf16x2(__float_as_uint(v[0]), __float_as_uint(v[1]));
          o.y = pack_bf16x2(__float_as_uint(v[2]), __float_as_uint(v[3]));
          o.z = pack_bf16x2(__float_as_uint(v[4]), __float_as_uint(v[5]));
          o.w = pack_bf16x2(__float_as_uint(v[6]), __float_as_uint(v[7]));
          const int owner = a.push.world > 0 ? j / a.push.per : -1;
          if (owner >= 0 && owner != a.push.rank) {
            // a row another rank reduces: straight into that rank's receive lines of the coming
            // all-reduce (flag-in-data: two 16-byte lines carry the 16 bytes and the call's stamp)
            const uint32_t e = ll_flag(push_seq);
            V16 l0, l1;
            l0.w[0] = o.x; l0.w[1] = e; l0.w[2] = o.y; l0.w[3] = e;
            l1.w[0] = o.z; l1.w[1] = e; l1.w[2] = o.w; l1.w[3] = e;
            char* line = a.push.heap[owner] + push_base +
                         (((size_t)a.push.rank * a.push.per + (j - owner * a.push.per)) * a.push.hv + n0 / 8) * 32;
            st16_volatile(line, l0);
            st16_volatile(line + 16, l1);
          } else {
            *reinterpret_cast<uint4*>(dst) = o;
          }
        } else {
          for (int k = 0; k < 8; ++k)
            if (n0 + k < n_out) dst[k] = __float2bfloat16_rn(v[k]);
        }
      }
    }
  }
  // ------------------------------------------------------------------- teardown
  if (S > 1 && warp < 2) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 64) stamp(7);  // done
  pdl_wait();  // no thread leaves before the predecessor has finished
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// CTAs of this kernel the current device holds at once, by cluster size (asked once per device).
template <int BT>
const int* decode_capacity(int sms) {
  struct Table {
    int cap[kDecodeMaxSplits + 1];
  };
  static std::mutex mu;
  static std::map<int, Table> tables;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  auto it = tables.find(dev);
  if (it != tables.end()) return it->second.cap;
  Table t;
  decode_model_capacity(sms, 16, t.cap);  // fallback if a query fails
  const void* fn = reinterpret_cast<const void*>(gemm_decode_kernel<BT>);
  if (kernel_setup(fn, 227 << 10).rc == cudaSuccess) {
    for (int s = 1; s <= kDecodeMaxSplits; ++s) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)s, (unsigned)(2 * sms), 1);
      cfg.blockDim = dim3(kDecThreads, 1, 1);
      cfg.dynamicSmemBytes = DecodeCfg<BT>::smem_bytes(3, s);  // what a split launch typically asks for
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = (unsigned)s;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) == cudaSuccess && n > 0)
        t.cap[s] = n * s;
      else
        (void)cudaGetLastError();
      // The cluster query counts one CTA per SM.  Measured (start stamps of every CTA): with
      // shared memory for two CTAs per SM a second round of clusters becomes resident on
      // the same SMs within 2-3 us, so twice that many CTAs run as ONE wave; beyond it the
      // rest waits for the first CTAs to finish.
      if (cfg.dynamicSmemBytes + 1024 <= ((size_t)228 << 10) / 2) t.cap[s] *= 2;
    }
  }
  tables[dev] = t;
  return tables[dev].cap;
}

template <int BT>
cudaError_t launch_decode_bt(const void* x, const void* w, void* out, int B, int N, int K, int ldx, int ldw, int ldo,
                             int epi, int splits, bool pdl, long long l2_budget, int smem_kb, const DecodePush* push, int sms,
                             uint32_t* error_word,
                             cudaStream_t stream) {
  using Cfg = DecodeCfg<BT>;
  CUtensorMap mw, mx;
  cudaError_t rc = make_tile_map(&mw, w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, kBlockM);
  if (rc != cudaSuccess) return rc;
  rc = make_tile_map(&mx, x, (uint64_t)B, (uint64_t)K, (uint64_t)ldx, BT);
  if (rc != cudaSuccess) return rc;
  DecodeArgs a;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.ldo = ldo;
  a.B = B;
  a.N = N;
  a.K = K;
  a.num_kb = (K + kBlockK - 1) / kBlockK;
  const int tiles = (N + kBlockM - 1) / kBlockM;
  const int slabs = (B + BT - 1) / BT;  // > 1 only with BT = 128
  if ((long long)tiles * slabs > 65535) return cudaErrorInvalidValue;
  a.slabs = slabs;
  if (splits <= 0) splits = decode_choose_splits(tiles * slabs, a.num_kb, decode_capacity<BT>(sms));
  splits = std::max(1, std::min(splits, std::min(kDecodeMaxSplits, a.num_kb)));
  a.splits = splits;
  a.epi = epi;
  if (push != nullptr)
    a.push = *push;
  else
    a.push.world = 0;
  // ring depth: what fits next to the receive area in ~106 KB (two kernels per SM); with a
  // 128-wide batch tile one kernel per SM and as deep as the range needs
  const int kb_per = (a.num_kb + splits - 1) / splits;
  // (measured, whole N = 1 decode step: 106 KB 6.08 ms, 75 KB 6.40, 56 KB 6.72, 150 KB 7.40)
  const size_t budget = smem_kb > 0 ? (size_t)std::min(smem_kb, 226) << 10 : (BT <= 64 ? (size_t)106 << 10 : (size_t)200 << 10);
  int stages = Cfg::min_stages();
  while (stages < kMaxStages && stages < kb_per && Cfg::smem_bytes(stages + 1, splits) <= budget) ++stages;
  a.stages = stages;
  const size_t smem = Cfg::smem_bytes(stages, splits);
  if (smem > ((size_t)227 << 10)) return cudaErrorInvalidValue;
  // L2 prefetch of the rest of the weight range while the predecessor runs: only when
  // the whole matrix fits the budget (a shard of a tensor-parallel layer does; the
  // full-size matrices of a single GPU would just evict one another)
  const long long w_bytes = (long long)tiles * a.num_kb * Cfg::kWBytes;
  static const int env_ahead = getenv("PENNY_DEC_AHEAD") ? atoi(getenv("PENNY_DEC_AHEAD")) : 0;
  static const int env_stagger = getenv("PENNY_DEC_STAGGER") ? atoi(getenv("PENNY_DEC_STAGGER")) : 1;
  a.l2_ahead = env_ahead > 0 ? stages + env_ahead : 0;
  a.l2_prefetch = (w_bytes <= l2_budget) ? kb_per : env_ahead;
  a.k_stagger = env_stagger;
  static const int env_stamps = getenv("PENNY_DEC_STAMPS") ? atoi(getenv("PENNY_DEC_STAMPS")) : 0;
  a.stamps = env_stamps;
  rc = kernel_setup(reinterpret_cast<const void*>(gemm_decode_kernel<BT>), 227 << 10).rc;
  if (rc != cudaSuccess) return rc;
  return launch_kernel_ex(gemm_decode_kernel<BT>, dim3((unsigned)splits, (unsigned)(tiles * slabs), 1), dim3(kDecThreads), smem,
                          stream, pdl, splits, mw, mx, a, error_word);
}

}  // namespace

cudaError_t launch_gemm_decode(const void* x, const void* w, void* out, int B, int N, int K, int ldx, int ldw,
                               int ldo, int epi, int splits, bool pdl, long long l2_budget_bytes,
                               int smem_kb, const DecodePush* push, uint32_t* error_word, cudaStream_t stream) {
  if (B <= 0 || B > kDecodeMaxBatch || N <= 0 || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0)
    return cudaErrorInvalidValue;
  if (push != nullptr && B > 128) return cudaErrorInvalidValue;  // the owners' receive lines cover one slab
  if (epi != DECODE_EPI_PLAIN && epi != DECODE_EPI_SILU_PAIRS) return cudaErrorInvalidValue;
  if (epi == DECODE_EPI_SILU_PAIRS && N % kBlockM != 0) return cudaErrorInvalidValue;
  if ((N + kBlockM - 1) / kBlockM > 65535) return cudaErrorInvalidValue;
  if (push != nullptr && (push->world < 2 || push->world > 8 || epi != DECODE_EPI_PLAIN || N % 8 != 0 || ldo % 8 != 0 ||
                          push->hv * 8 != N || push->per < 1 || (reinterpret_cast<uintptr_t>(out) & 15u) != 0))
    return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (l2_budget_bytes < 0) l2_budget_bytes = (long long)32 << 20;
  if (B <= 32)
    return launch_decode_bt<32>(x, w, out, B, N, K, ldx, ldw, ldo, epi, splits, pdl, l2_budget_bytes, smem_kb, push, sms, error_word, stream);
  if (B <= 64)
    return launch_decode_bt<64>(x, w, out, B, N, K, ldx, ldw, ldo, epi, splits, pdl, l2_budget_bytes, smem_kb, push, sms, error_word, stream);
  return launch_decode_bt<128>(x, w, out, B, N, K, ldx, ldw, ldo, epi, splits, pdl, l2_budget_bytes, smem_kb, push, sms, error_word, stream);
}

int gemm_decode_stamps(unsigned long long* out, int max_ctas) {
  const int n = std::min(max_ctas, kStampCtas);
  if (cudaMemcpyFromSymbol(out, g_dec_stamps, (size_t)n * kStampPoints * sizeof(unsigned long long)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

int gemm_decode_capacity(int B, int splits) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  (void)cudaGetLastError();
  if (splits < 1 || splits > kDecodeMaxSplits) return 0;
  const int* cap = B <= 32 ? decode_capacity<32>(sms) : (B <= 64 ? decode_capacity<64>(sms) : decode_capacity<128>(sms));
  return cap[splits];
}

int gemm_decode_splits(int B, int N, int K) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  (void)cudaGetLastError();
  if (sms <= 0) sms = 148;
  const int num_kb = (K + kBlockK - 1) / kBlockK, tiles = (N + kBlockM - 1) / kBlockM * ((std::max(B, 1) + 127) / 128);
  const int* cap = B <= 32 ? decode_capacity<32>(sms) : (B <= 64 ? decode_capacity<64>(sms) : decode_capacity<128>(sms));
  return decode_choose_splits(tiles, num_kb, cap);
}

}  // namespace sm100
}  // namespace penny
