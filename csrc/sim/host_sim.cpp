// Host protocol simulator: runs the very same collective bodies that the GPU
// kernels run (csrc/*.cuh compiled with -DPENNY_HOST_SIM) with
//   rank   = a "stream" thread issuing calls back to back, never synchronised
//            with the other ranks by anything but the flag protocol itself,
//   block  = a std::thread per call (a call ends when all its blocks joined,
//            like a kernel on a stream),
//   thread = a sequential loop inside the block,
//   heap   = plain host memory, flags = __atomic builtins.
// It exists to find deadlocks, lost flags and buffer-reuse races on the CPU
// (also under -fsanitize=thread) before a kernel ever runs on a shared GPU, and
// to inject failures (a rank that never joins) without touching one.  The
// reference has no such layer: its protocols can only be exercised on real
// multi-GPU hardware (extra/benchmark_allreduce.py:118-134).
//
// Built as a plain shared library (no CUDA, no torch) and driven through ctypes.
#define PENNY_HOST_SIM 1
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

#include "../algos.h"
#include "../gemm_tile_order.h"
#include "../decode_gemm_plan.h"
#include "../all_reduce_oneshot.cuh"
#include "../all_reduce_ring.cuh"
#include "../all_reduce_tree.cuh"
#include "../all_reduce_twoshot.cuh"
#include "../exchange.cuh"

namespace penny {

float host_half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ff;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while ((man & 0x400) == 0);
      man &= 0x3ff;
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t host_float_to_half(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t sign = (u >> 16) & 0x8000u;
  int32_t exp = (int32_t)((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffffu;
  if (((u >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    int shift = 14 - exp;
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1))) ++half_man;
    return (uint16_t)(sign | half_man);
  }
  uint32_t half = sign | ((uint32_t)exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return (uint16_t)half;
}

namespace {

template <typename T>
void run_body(int algo, int world, const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
  switch (algo) {
    case ALGO_RING_STANDARD: RingStandard<T>::run(c, rank, a, b); return;
    case ALGO_RING_SIMPLE: RingSimple<T>::run(c, rank, a, b); return;
    case ALGO_DOUBLE_RING: DoubleRing<T>::run(c, rank, a, b); return;
    case ALGO_TREE: TreeAllReduce<T>::run(c, rank, a, b); return;
    case OP_EXCHANGE: ExchangePair<T>::run(c, rank, a, b); return;
    default: break;
  }
  PENNY_DISPATCH_WORLD(world, NG, return, {
    switch (algo) {
      case ALGO_ONESHOT: OneShotFlag<T, NG>::run(c, rank, a, b); break;
      case ALGO_ONESHOT_LL: OneShotLL<T, NG>::run(c, rank, a, b); break;
      case ALGO_TWOSHOT: TwoShot<T, NG>::run(c, rank, a, b); break;
      case OP_REDUCE_SCATTER: ReduceScatterPush<T, NG>::run(c, rank, a, b); break;
      case OP_REDUCE_SCATTER_PIPELINED: ReduceScatterPipelined<T, NG>::run(c, rank, a, b); break;
      case OP_ALL_GATHER: AllGatherPush<T, NG>::run(c, rank, a, b); break;
      case OP_ALL_TO_ALL: AllToAll<T, NG>::run(c, rank, a, b); break;
      case OP_ALL_TO_ALL_PIPELINED: AllToAllPipelined<T, NG>::run(c, rank, a, b); break;
      default: break;
    }
  });
}

size_t scratch_need(int algo, size_t n, int es, int world, int nnodes, int nblocks) {
  switch (algo) {
    case ALGO_RING_STANDARD: return ring_standard_scratch_bytes(n, es, world);
    case ALGO_RING_SIMPLE: return ring_simple_scratch_bytes(n, es, world);
    case ALGO_ONESHOT: return oneshot_flag_scratch_bytes(n, es, world);
    case ALGO_ONESHOT_LL: return oneshot_ll_scratch_bytes(n, es, world);
    case ALGO_TWOSHOT: return twoshot_scratch_bytes(n, es, world);
    case ALGO_DOUBLE_RING: return double_ring_scratch_bytes(n, es, world, nnodes, nblocks);
    case ALGO_TREE: return tree_scratch_bytes(n, es, nnodes);
    case OP_REDUCE_SCATTER:
    case OP_REDUCE_SCATTER_PIPELINED: return reduce_scatter_scratch_bytes(n, es, world);
    case OP_ALL_GATHER: return all_gather_scratch_bytes(n, es, world);
    case OP_ALL_TO_ALL:
    case OP_ALL_TO_ALL_PIPELINED: return all_to_all_scratch_bytes(n, es, world);
    case OP_EXCHANGE: return exchange_scratch_bytes(n, es);
    default: return 0;
  }
}

// Elements of the per-rank input / output of one call with size parameter n.
void io_elems(int algo, size_t n, int world, size_t* in_n, size_t* out_n) {
  switch (algo) {
    case OP_REDUCE_SCATTER:
    case OP_REDUCE_SCATTER_PIPELINED: *in_n = n; *out_n = n / world; break;
    case OP_ALL_GATHER: *in_n = n; *out_n = n * world; break;
    case OP_ALL_TO_ALL:
    case OP_ALL_TO_ALL_PIPELINED: *in_n = n * world; *out_n = n * world; break;
    default: *in_n = n; *out_n = n; break;
  }
}

template <typename T>
struct Sim {
  int algo, world, nblocks, nthreads, nnodes, routes, iters, stall_rank;
  size_t n;
  bool in_place;
  std::vector<std::vector<char>> heaps;
  std::vector<std::vector<std::vector<T>>> in;   // [iter][rank][elem]
  std::vector<std::vector<std::vector<T>>> out;  // [iter][rank][elem]
  size_t scratch_bytes;
  uint64_t timeout_ns;

  CommCtx ctx_for(int r) {
    CommCtx c;
    memset(&c, 0, sizeof(c));
    for (int i = 0; i < world; ++i) c.heap[i] = heaps[i].data();
    c.mc = nullptr;
    c.rank = r;
    c.world = world;
    c.timeout_ns = timeout_ns;
    c.status = reinterpret_cast<uint32_t*>(heaps[r].data() + kStatusOffset);
    return c;
  }

  void rank_stream(int r) {
    CommCtx c = ctx_for(r);
    for (int it = 0; it < iters; ++it) {
      if (r == stall_rank) return;  // this rank never joins: everyone else must time out
      CollArgs a;
      memset(&a, 0, sizeof(a));
      a.in = in[it][r].data();
      a.out = in_place ? (void*)in[it][r].data() : (void*)out[it][r].data();
      a.n = n;
      a.scratch_off = kHeapReserved;
      a.scratch_bytes = scratch_bytes;
      a.in_heap_off = kNotInHeap;
      a.out_heap_off = kNotInHeap;
      a.nnodes = nnodes;
      a.routes = routes;
      a.peer = (algo == OP_EXCHANGE) ? (r ^ 1) : 0;
      if (a.peer >= world) a.peer = r;
      a.unit_vecs = 0;
      std::vector<std::thread> blocks;
      for (int bi = 0; bi < nblocks; ++bi) {
        blocks.emplace_back([&, bi]() {
          Blk b{bi, nblocks, nthreads};
          run_body<T>(algo, world, c, r, a, b);
        });
      }
      for (auto& t : blocks) t.join();
    }
  }
};

template <typename T>
int sim_run_t(int algo, int world, int nblocks, int nthreads, size_t n, int nnodes, int routes,
              int iters, unsigned seed, int stall_rank, int timeout_ms, int in_place,
              double* max_err, uint32_t* status_out) {
  Sim<T> s;
  s.algo = algo; s.world = world; s.nblocks = nblocks; s.nthreads = nthreads; s.n = n;
  s.nnodes = nnodes; s.routes = routes; s.iters = iters; s.stall_rank = stall_rank;
  s.in_place = in_place != 0 && algo != OP_REDUCE_SCATTER && algo != OP_REDUCE_SCATTER_PIPELINED &&
               algo != OP_ALL_GATHER && algo != OP_ALL_TO_ALL && algo != OP_ALL_TO_ALL_PIPELINED;
  if (algo == OP_EXCHANGE) s.in_place = true;
  s.timeout_ns = (uint64_t)timeout_ms * 1000000ull;
  const int es = (int)sizeof(T);
  s.scratch_bytes = round_up(scratch_need(algo, n, es, world, nnodes, nblocks), 32);
  const size_t heap_bytes = kHeapReserved + s.scratch_bytes + 64;
  s.heaps.assign(world, std::vector<char>(heap_bytes, 0));
  size_t in_n, out_n;
  io_elems(algo, n, world, &in_n, &out_n);
  std::mt19937 rng(seed);
  std::uniform_real_distribution<float> dist(-1.f, 1.f);
  s.in.resize(iters);
  s.out.resize(iters);
  std::vector<std::vector<std::vector<float>>> ref_in(iters);
  for (int it = 0; it < iters; ++it) {
    s.in[it].resize(world);
    s.out[it].resize(world);
    ref_in[it].resize(world);
    for (int r = 0; r < world; ++r) {
      s.in[it][r].resize(in_n);
      s.out[it][r].assign(out_n, T{});
      ref_in[it][r].resize(in_n);
      for (size_t i = 0; i < in_n; ++i) {
        T t;
        from_f32(dist(rng), t);
        s.in[it][r][i] = t;
        ref_in[it][r][i] = to_f32(t);
      }
    }
  }
  std::vector<std::thread> ranks;
  for (int r = 0; r < world; ++r) ranks.emplace_back([&, r]() { s.rank_stream(r); });
  for (auto& t : ranks) t.join();

  // statuses: kStatusWords words per rank
  int failures = 0;
  for (int r = 0; r < world; ++r) {
    const uint32_t* st = reinterpret_cast<const uint32_t*>(s.heaps[r].data() + kStatusOffset);
    if (status_out) memcpy(status_out + (size_t)r * kStatusWords, st, kStatusWords * 4);
    if (st[0] != ST_OK) ++failures;
  }
  double worst = 0.0;
  if (failures == 0 && stall_rank < 0) {
    const double eps = (sizeof(T) == 4) ? 1e-6 : (std::is_same<T, HostBF16>::value ? 8e-3 : 1e-3);
    for (int it = 0; it < iters; ++it) {
      for (int r = 0; r < world; ++r) {
        const std::vector<T>& got = s.in_place ? s.in[it][r] : s.out[it][r];
        for (size_t i = 0; i < out_n; ++i) {
          double want = 0.0, mag = 0.0;
          switch (algo) {
            case OP_REDUCE_SCATTER:
            case OP_REDUCE_SCATTER_PIPELINED:
              for (int q = 0; q < world; ++q) {
                double v = ref_in[it][q][(size_t)r * out_n + i];
                want += v; mag += std::fabs(v);
              }
              break;
            case OP_ALL_GATHER:
              want = ref_in[it][i / n][i % n]; mag = std::fabs(want);
              break;
            case OP_ALL_TO_ALL:
            case OP_ALL_TO_ALL_PIPELINED:
              want = ref_in[it][i / n][(size_t)r * n + i % n]; mag = std::fabs(want);
              break;
            case OP_EXCHANGE: {
              int peer = r ^ 1;
              if (peer >= world) peer = r;
              want = ref_in[it][peer][i]; mag = std::fabs(want);
              break;
            }
            default:
              for (int q = 0; q < world; ++q) {
                double v = ref_in[it][q][i];
                want += v; mag += std::fabs(v);
              }
          }
          // relative to the magnitude that went through the (re-rounded) partial sums
          double err = std::fabs((double)to_f32(got[i]) - want) / (mag * eps * world + 1e-30);
          if (err > worst) worst = err;
        }
      }
    }
  }
  if (max_err) *max_err = worst;  // in units of the allowed error: <= 1 passes
  return failures;
}

}  // namespace
}  // namespace penny

extern "C" {

// Returns the number of ranks that recorded a failure status.  *max_err is the
// worst observed error divided by the allowed error (<= 1.0 is a pass).
// status_out (optional) receives kStatusWords words per rank.
int penny_sim_run(int algo, int dtype, int world, int nblocks, int nthreads, unsigned long long n,
                  int nnodes, int routes, int iters, unsigned seed, int stall_rank,
                  int timeout_ms, int in_place, double* max_err, unsigned* status_out) {
  using namespace penny;
  if (world < 2 || world > kMaxRanks || nblocks < 1 || nblocks > kMaxBlocks) return -1;
  if (nnodes < 1 || world % nnodes != 0) return -1;
  int rc = -1;
  PENNY_DISPATCH_DTYPE(dtype, T,
                       rc = sim_run_t<T>(algo, world, nblocks, nthreads, (size_t)n, nnodes, routes,
                                         iters, seed, stall_rank, timeout_ms, in_place, max_err,
                                         status_out));
  return rc;
}

// Schedule queries for the Python-side schedule tests and the ring visualiser.
int penny_sched_ring_rank_at(int world, int nnodes, int route, int pos) {
  return penny::ring_rank_at(world, nnodes, route, pos);
}
int penny_sched_ring_stride(int world, int route) { return penny::ring_stride(world, route); }
int penny_sched_ring_rs_send_chunk(int n, int pos, int s) { return penny::ring_rs_send_chunk(n, pos, s); }
int penny_sched_ring_rs_recv_chunk(int n, int pos, int s) { return penny::ring_rs_recv_chunk(n, pos, s); }
int penny_sched_ring_ag_send_chunk(int n, int pos, int s) { return penny::ring_ag_send_chunk(n, pos, s); }
int penny_sched_ring_ag_recv_chunk(int n, int pos, int s) { return penny::ring_ag_recv_chunk(n, pos, s); }
int penny_sched_tree_local_at(int gpn, int tree, int j) { return penny::tree_local_at(gpn, tree, j); }
void penny_sched_split_span(unsigned long long V, int parts, int i, unsigned long long* b,
                            unsigned long long* e) {
  penny::Span s = penny::split_span((size_t)V, parts, i);
  *b = s.begin;
  *e = s.end;
}
int penny_status_words() { return penny::kStatusWords; }
// Work split of the decode GEMM (decode_gemm_plan.h): out = {kb0, kb1, slice, recv_floats}
// of CTA `r` of a cluster of `splits` working on a bt-wide batch tile.
void penny_decode_plan(int num_kb, int splits, int r, int bt, long long* out) {
  out[0] = penny::sm100::decode_kb_begin(num_kb, splits, r);
  out[1] = penny::sm100::decode_kb_begin(num_kb, splits, r + 1);
  out[2] = penny::sm100::decode_slice(bt, splits);
  out[3] = (long long)penny::sm100::decode_recv_floats(bt, splits);
}
int penny_decode_recv_slot(int src, int dst) { return penny::sm100::decode_recv_slot(src, dst); }
int penny_decode_choose_splits(int tiles, int num_kb, int sms, int gpc_sms) {
  int cap[penny::sm100::kDecodeMaxSplits + 1];
  penny::sm100::decode_model_capacity(sms, gpc_sms, cap);
  return penny::sm100::decode_choose_splits(tiles, num_kb, cap);
}
// Tile -> (row block, column block) of the persistent GEMM kernels; pair_rank < 0
// selects the single-CTA kernel, 0 / 1 the CTA of a pair.  Returns the number of
// tiles (pair tiles) of the grid.
int penny_gemm_tile_at(int tiles_m, int tiles_n, int m_rot, int m_fastest, int group_m, int pair_rank,
                       int tile, int* m_blk, int* n_blk) {
  penny::sm100::GemmShape s{0, 0, 0, tiles_m, tiles_n, m_rot, tiles_m * tiles_n, m_fastest, group_m};
  if (pair_rank < 0) {
    penny::sm100::decode_tile(s, tile, *m_blk, *n_blk);
    return s.num_tiles;
  }
  penny::sm100::decode_pair_tile(s, tile, pair_rank, *m_blk, *n_blk);
  return penny::sm100::pair_tile_count(s);
}
// The it-th work unit of CTA pair `pair` of `npairs` after planning the split of
// the last wave: out = {tile, kb0, kb1, seg, split_s, split_first}; 0 when the pair
// has no such unit.
int penny_gemm_pair_work(int tiles_m, int tiles_n, int npairs, int num_kb, int max_split, int pair,
                         int it, int* out) {
  penny::sm100::GemmShape s{0, 0, 0, tiles_m, tiles_n, 0, tiles_m * tiles_n, 1, 16};
  penny::sm100::plan_split_tail(s, npairs, num_kb, max_split);
  penny::sm100::PairWork w{0, 0, 0, 0};
  const bool ok = penny::sm100::pair_work(s, num_kb, pair, npairs, it, w);
  out[0] = w.tile; out[1] = w.kb0; out[2] = w.kb1; out[3] = w.seg;
  out[4] = s.split_s; out[5] = s.split_first;
  return ok ? 1 : 0;
}
}
