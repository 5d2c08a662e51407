#include "comm.h"

#include <string.h>

#include <algorithm>
#include <stdexcept>

#include "all_reduce_oneshot.cuh"
#include "all_reduce_ring.cuh"
#include "all_reduce_tree.cuh"
#include "all_reduce_twoshot.cuh"
#include "exchange.cuh"
#include "gemm_fused_sm100.h"
#include "launch.cuh"

namespace penny {

namespace {
void ckrt(cudaError_t r, const char* what) {
  if (r != cudaSuccess) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string("penny: ") + what + ": " + cudaGetErrorString(r));
  }
}
constexpr size_t kScratchCap = (size_t)512 << 20;  // a single call never asks for more
// Switch all-reduce of tensors outside the heap: from this size the staging copies are pipelined
// against the reduction, piece by piece
constexpr size_t kNvlsPipelineBytes = (size_t)256 << 20;  // below, the extra launches and events cost more than the overlap saves (measured)
constexpr int kNvlsPipePieces = 4;
}  // namespace

Communicator::Communicator(const std::string& uid, int rank, int world, const CommOptions& opt)
    : rank_(rank), world_(world), emu_(false) {
  bs_.reset(new Bootstrap(uid, rank, world, opt.bootstrap_timeout_ms));
  heap_.reset(new SymmHeap(bs_.get(), rank, world, opt.heap_bytes, opt.heap_mode, opt.multicast));
  init_ctx(opt);
}

Communicator::Communicator(int emu_world, const CommOptions& opt)
    : rank_(0), world_(emu_world), emu_(true) {
  heap_.reset(new SymmHeap(nullptr, 0, emu_world, opt.heap_bytes, HEAP_EMU, false));
  init_ctx(opt);
}

Communicator::~Communicator() {
  try {
    destroy();
  } catch (...) {
  }
}

void Communicator::init_ctx(const CommOptions& opt) {
  memset(&ctx_, 0, sizeof(ctx_));
  for (int r = 0; r < world_; ++r) ctx_.heap[r] = heap_->base(r);
  ctx_.mc = heap_->mc_base();
  ctx_.rank = rank_;
  ctx_.world = world_;
  ctx_.timeout_ns = (unsigned long long)opt.timeout_ms * 1000000ull;
  ctx_.status = reinterpret_cast<uint32_t*>(heap_->base(rank_) + kStatusOffset);
  if (heap_->bytes() < kHeapReserved + (1u << 20))
    throw std::runtime_error("penny: heap too small");
}

void Communicator::ensure_pipe() {
  if (pipe_in_ != nullptr) return;
  ckrt(cudaStreamCreateWithFlags(&pipe_in_, cudaStreamNonBlocking), "pipeline stream");
  ckrt(cudaStreamCreateWithFlags(&pipe_out_, cudaStreamNonBlocking), "pipeline stream");
  pipe_ev_.resize(2 + 2 * kNvlsPipePieces);
  for (cudaEvent_t& e : pipe_ev_) ckrt(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "pipeline event");
}

void Communicator::destroy() {
  if (destroyed_) return;
  destroyed_ = true;
  for (cudaEvent_t e : pipe_ev_) cudaEventDestroy(e);
  pipe_ev_.clear();
  if (pipe_in_ != nullptr) cudaStreamDestroy(pipe_in_);
  if (pipe_out_ != nullptr) cudaStreamDestroy(pipe_out_);
  pipe_in_ = pipe_out_ = nullptr;
  if (heap_) heap_->destroy();
}

std::string Communicator::describe() const {
  static const char* modes[] = {"auto", "vmm", "ipc", "emu"};
  return std::string("penny communicator rank ") + std::to_string(rank_) + "/" +
         std::to_string(world_) + " heap=" + modes[heap_->mode()] + " " +
         std::to_string(heap_->bytes() >> 20) + " MiB, multicast: " + heap_->multicast_note();
}

void Communicator::set_timeout_ms(int ms) {
  ctx_.timeout_ns = (unsigned long long)ms * 1000000ull;
}

size_t Communicator::alloc(size_t bytes) {
  size_t off = round_up(arena_top_, 256);
  size_t end = off + round_up(bytes, 256);
  if (end > heap_->bytes())
    throw std::runtime_error("penny: symmetric heap exhausted (" + std::to_string(bytes) +
                             " bytes requested, " + std::to_string(heap_->bytes() - arena_top_) +
                             " free); raise heap_bytes / PENNY_HEAP_BYTES");
  arena_top_ = end;
  return off;
}

void* Communicator::local_ptr(size_t off, int view) const {
  return heap_->base(emu_ ? view : rank_) + off;
}

size_t Communicator::heap_offset_of(const void* p, int view) const {
  const char* b = heap_->base(emu_ ? view : rank_);
  const char* c = reinterpret_cast<const char*>(p);
  if (c >= b + kHeapReserved && c < b + heap_->bytes()) return (size_t)(c - b);
  return kNotInHeap;
}

Communicator::Region& Communicator::ensure(Region& r, size_t need, const char* what) {
  need = round_up(need, 512);
  if (r.bytes >= need) return r;
  size_t want = std::max(need, std::min(r.bytes * 2, kScratchCap));
  size_t free_b = heap_free_bytes();
  if (want + 512 > free_b) want = need;
  try {
    r.off = alloc(want);
  } catch (const std::exception& e) {
    throw std::runtime_error(std::string(e.what()) + " [while growing " + what + " scratch]");
  }
  r.bytes = want;
  return r;
}

LaunchCfg Communicator::cfg_for(size_t vecs, const Tuning& t, cudaStream_t s, int max_blocks,
                                int multiple, int vecs_per_thread) const {
  LaunchCfg cfg;
  cfg.threads = t.threads > 0 ? t.threads : 512;
  cfg.stream = s;
  cfg.emu_world = emu_ ? world_ : 0;
  cfg.pdl = true;  // the kernel shell waits for its predecessor before it touches anything
  // emulation: all virtual ranks' blocks must be co-resident (one 512-thread
  // block per SM in the worst case)
  if (emu_) max_blocks = std::max(1, std::min(max_blocks, 128 / world_));
  max_blocks = std::min(max_blocks, kMaxBlocks);
  int blocks = t.blocks;
  if (blocks <= 0) {
    size_t per_block = (size_t)cfg.threads * vecs_per_thread;
    blocks = (int)std::min<size_t>((size_t)max_blocks, std::max<size_t>(1, ceil_div(vecs, per_block)));
  }
  blocks = std::min(blocks, max_blocks);
  if (multiple > 1) {
    blocks = std::max(multiple, blocks / multiple * multiple);
    if (blocks > max_blocks && max_blocks >= multiple) blocks = max_blocks / multiple * multiple;
  }
  cfg.blocks = blocks;
  return cfg;
}

void Communicator::set_tuning(int elem_size, bool symmetric, const std::vector<TuneEntry>& entries) {
  tune_[elem_size == 4 ? 1 : 0][symmetric ? 1 : 0] = entries;
}

int Communicator::pick_algo(int dtype, size_t n, bool symmetric) const {
  const size_t bytes = n * (size_t)dtype_size(dtype);
  if (world_ < 2) return ALGO_ONESHOT;
  const bool even = (world_ == 2 || world_ == 4 || world_ == 6 || world_ == 8);
  if (!even) return ALGO_RING_STANDARD;
  const std::vector<TuneEntry>& table = tune_[dtype_size(dtype) == 4 ? 1 : 0][symmetric ? 1 : 0];
  if (!table.empty()) {
    int algo = table.back().algo;
    for (const TuneEntry& e : table) {
      if (bytes <= e.max_bytes) {
        algo = e.algo;
        break;
      }
    }
    const bool needs_mc = algo == ALGO_NVLS || algo == ALGO_NVLS_ONESHOT;
    if (!needs_mc || has_multicast()) return algo;
    return bytes <= ((size_t)256 << 10) ? ALGO_ONESHOT : ALGO_TWOSHOT;
  }
  // No table installed.  Measured on 8 x B200 (device time per call inside a CUDA
  // graph): the flag-in-data protocol wins up to 32 KiB (9-11 us), the switch
  // reduction from there on (17 us at 256 KiB, 826 GB/s bus bandwidth at 1 GiB);
  // without a multicast mapping the pushes take over (one-shot to 256 KiB, then two-shot).
  if (bytes <= (size_t)32 << 10) return ALGO_ONESHOT_LL;
  if (has_multicast()) return ALGO_NVLS;
  if (bytes <= (size_t)256 << 10) return ALGO_ONESHOT;
  return ALGO_TWOSHOT;
}

void Communicator::all_reduce(int algo, int dtype, const void* const* in, void* const* out,
                              size_t n, const Tuning& t, cudaStream_t stream) {
  if (n == 0) return;
  const int es = dtype_size(dtype);
  if (world_ == 1) {
    if (in[0] != out[0])
      ckrt(cudaMemcpyAsync(out[0], in[0], n * es, cudaMemcpyDeviceToDevice, stream), "memcpy");
    return;
  }
  if (algo == ALGO_AUTO) algo = pick_algo(dtype, n, t.symmetric_in && t.symmetric_out);
  if ((algo == ALGO_NVLS || algo == ALGO_NVLS_ONESHOT) && !has_multicast())
    throw std::runtime_error("penny: NVLS all-reduce requested but the heap has no multicast (" +
                             heap_->multicast_note() + ")");
  // Split so that one launch never needs more scratch than the cap.  Segment
  // boundaries are multiples of 16 bytes so every segment stays vector-aligned.
  size_t per_elem_scratch;  // scratch bytes per element (both halves), upper bound
  switch (algo) {
    case ALGO_ONESHOT: per_elem_scratch = 2 * (size_t)world_ * es; break;
    case ALGO_ONESHOT_LL: per_elem_scratch = 4 * (size_t)world_ * es; break;
    case ALGO_TREE: per_elem_scratch = 2 * (size_t)(2 + t.nnodes) * es; break;
    case ALGO_NVLS: per_elem_scratch = es; break;  // staging at most (the in-kernel variant is small by construction)
    case ALGO_NVLS_ONESHOT: per_elem_scratch = 2 * (size_t)es; break;
    default: per_elem_scratch = 4 * (size_t)es; break;
  }
  size_t budget = std::min(kScratchCap, std::max<size_t>(heap_free_bytes() / 2, (size_t)1 << 20));
  if (algo == ALGO_NVLS) budget = kScratchCap;  // staging regions are sized per call, not from this budget
  size_t seg = std::max<size_t>(budget / per_elem_scratch / 1024 * 1024, 1024);
  if (n <= seg) {
    run_all_reduce_once(algo, dtype, in, out, n, t, stream);
    return;
  }
  std::vector<const void*> in_s(views());
  std::vector<void*> out_s(views());
  for (size_t o = 0; o < n; o += seg) {
    for (int v = 0; v < views(); ++v) {
      in_s[v] = (const char*)in[v] + o * es;
      out_s[v] = (char*)out[v] + o * es;
    }
    run_all_reduce_once(algo, dtype, in_s.data(), out_s.data(), std::min(seg, n - o), t, stream);
  }
}

void Communicator::run_all_reduce_once(int algo, int dtype, const void* const* in,
                                       void* const* out, size_t n, const Tuning& t,
                                       cudaStream_t stream) {
  const int es = dtype_size(dtype);
  const size_t V = vecs_for(n, es);
  const int nv = views();
  int nnodes = t.nnodes > 0 ? t.nnodes : 1;
  if (world_ % nnodes != 0) throw std::runtime_error("penny: nnodes must divide the world size");
  CollArgs a[kMaxRanks];
  memset(a, 0, sizeof(a));
  for (int v = 0; v < nv; ++v) {
    a[v].in = in[v];
    a[v].out = out[v];
    a[v].n = n;
    a[v].in_heap_off = heap_offset_of(in[v], v);
    a[v].out_heap_off = kNotInHeap;
    a[v].nnodes = nnodes;
    a[v].routes = 1;
  }
  auto set_scratch = [&](const Region& r) {
    for (int v = 0; v < nv; ++v) {
      a[v].scratch_off = r.off;
      a[v].scratch_bytes = r.bytes;
    }
  };
  cudaError_t rc = cudaSuccess;
  switch (algo) {
    case ALGO_ONESHOT: {
      set_scratch(ensure(scratch_, oneshot_flag_scratch_bytes(n, es, world_), "one-shot"));
      // latency-bound: one vector per thread while the blocks last
      rc = launch_all_reduce_oneshot(dtype, false, ctx_, a, cfg_for(V, t, stream, 64, 1, 1));
      break;
    }
    case ALGO_ONESHOT_LL: {
      set_scratch(ensure(scratch_ll_, oneshot_ll_scratch_bytes(n, es, world_), "LL"));
      Tuning tt = t;
      if (tt.threads <= 0) tt.threads = 256;
      LaunchCfg cfg = cfg_for(V, tt, stream, 64, 1);
      if (t.blocks <= 0) cfg.blocks = (int)std::min<size_t>(emu_ ? 128 / world_ : 64,
                                                             std::max<size_t>(1, ceil_div(V, cfg.threads)));
      rc = launch_all_reduce_oneshot(dtype, true, ctx_, a, cfg);
      break;
    }
    case ALGO_TWOSHOT: {
      set_scratch(ensure(scratch_, twoshot_scratch_bytes(n, es, world_), "two-shot"));
      // direct gather only if every rank's output sits at the same heap offset
      size_t oo = heap_offset_of(out[0], 0);
      bool same = oo != kNotInHeap && (n * es) % 16 == 0;
      for (int v = 1; v < nv; ++v) same = same && heap_offset_of(out[v], v) == oo;
      if (same && t.symmetric_out)
        for (int v = 0; v < nv; ++v) a[v].out_heap_off = oo;
      rc = launch_all_reduce_twoshot(dtype, ctx_, a, cfg_for(ceil_div(V, world_), t, stream, 128, 1));
      break;
    }
    case ALGO_RING_SIMPLE: {
      set_scratch(ensure(scratch_, ring_simple_scratch_bytes(n, es, world_), "ring"));
      rc = launch_all_reduce_ring_simple(dtype, ctx_, a, cfg_for(V, t, stream, 64, 1));
      break;
    }
    case ALGO_RING_STANDARD: {
      set_scratch(ensure(scratch_, ring_standard_scratch_bytes(n, es, world_), "ring"));
      int routes = t.routes > 0 ? t.routes : (V >= 4096 ? std::min(4, num_ring_strides(world_)) : 1);
      routes = std::min(routes, kMaxRoutes);
      if (nnodes > 1) routes = std::min(routes, std::max(1, world_ / nnodes));
      for (int v = 0; v < nv; ++v) a[v].routes = routes;
      rc = launch_all_reduce_ring_standard(
          dtype, ctx_, a, cfg_for(ceil_div(V, world_), t, stream, 96, routes));
      break;
    }
    case ALGO_DOUBLE_RING: {
      LaunchCfg cfg = cfg_for(V, t, stream, 64, 1);
      set_scratch(ensure(scratch_, double_ring_scratch_bytes(n, es, world_, nnodes, cfg.blocks),
                         "double ring"));
      rc = launch_all_reduce_double_ring(dtype, ctx_, a, cfg);
      break;
    }
    case ALGO_TREE: {
      set_scratch(ensure(scratch_, tree_scratch_bytes(n, es, nnodes), "tree"));
      int gpn = world_ / nnodes;
      rc = launch_all_reduce_tree(dtype, ctx_, a, cfg_for(ceil_div(V, gpn), t, stream, 96, gpn));
      break;
    }
    case ALGO_NVLS_ONESHOT: {
      // stages its input inside the kernel: any memory, in place or not
      set_scratch(ensure(scratch_, nvls_oneshot_scratch(n, es), "NVLS one-shot"));
      rc = launch_all_reduce_nvls(dtype, NVLS_ONESHOT, ctx_, a, cfg_for(V, t, stream, 64, 1, 1));
      break;
    }
    case ALGO_NVLS: {
      const size_t bytes = V * 16;
      const bool in_heap = a[0].in_heap_off != kNotInHeap && t.symmetric_in;
      const size_t out_off = heap_offset_of(out[0], 0);
      const bool out_heap = out_off != kNotInHeap && t.symmetric_out;
      if (in_heap && out_heap) {
        a[0].out_heap_off = out_off;
        rc = launch_all_reduce_nvls(dtype, NVLS_TWOSHOT, ctx_, a, cfg_for(ceil_div(V, world_), t, stream, 64, 1));
        break;
      }
      // tensors outside the heap: one copy in, one copy out (copying inside the kernel was measured
      // slower at 8 ranks: 19.3 vs 16.1 us at 1 KiB, 24.5 vs 17.4 us at 256 KiB, in a graph)
      const size_t in_off0 = in_heap ? a[0].in_heap_off : ensure(stage_in_, bytes, "NVLS input staging").off;
      const size_t out_off0 = out_heap ? out_off : ensure(stage_out_, bytes, "NVLS output staging").off;
      if (bytes < kNvlsPipelineBytes) {
        if (!in_heap)
          ckrt(cudaMemcpyAsync(local_ptr(in_off0), in[0], n * es, cudaMemcpyDeviceToDevice, stream), "stage in");
        a[0].in_heap_off = in_off0;
        a[0].out_heap_off = out_off0;
        rc = launch_all_reduce_nvls(dtype, NVLS_TWOSHOT, ctx_, a, cfg_for(ceil_div(V, world_), t, stream, 64, 1));
        if (rc == cudaSuccess && !out_heap)
          ckrt(cudaMemcpyAsync(out[0], local_ptr(out_off0), n * es, cudaMemcpyDeviceToDevice, stream), "stage out");
        break;
      }
      // Very large: cut into pieces; the copy into the heap of piece i + 1 and the copy out of piece
      // i - 1 run on two side streams under the switch reduction of piece i.  The reductions stay on
      // the caller's stream, in the same order on every rank.  Works under stream capture: the side
      // streams fork from and join back into the caller's stream through events.
      ensure_pipe();
      const size_t piece = round_up(ceil_div(n, (size_t)kNvlsPipePieces), 4096);  // elements; 16-byte multiple
      ckrt(cudaEventRecord(pipe_ev_[0], stream), "pipeline fork");
      if (!in_heap) {
        ckrt(cudaStreamWaitEvent(pipe_in_, pipe_ev_[0], 0), "pipeline fork");
        int i = 0;
        for (size_t o = 0; o < n; o += piece, ++i) {
          const size_t len = std::min(piece, n - o);
          ckrt(cudaMemcpyAsync((char*)local_ptr(in_off0) + o * es, (const char*)in[0] + o * es, len * es,
                               cudaMemcpyDeviceToDevice, pipe_in_), "stage in");
          ckrt(cudaEventRecord(pipe_ev_[1 + i], pipe_in_), "stage in");
        }
      }
      {
        int i = 0;
        for (size_t o = 0; o < n && rc == cudaSuccess; o += piece, ++i) {
          const size_t len = std::min(piece, n - o);
          if (!in_heap) ckrt(cudaStreamWaitEvent(stream, pipe_ev_[1 + i], 0), "stage in");
          a[0].n = len;
          a[0].in = (const char*)in[0] + o * es;
          a[0].out = (char*)out[0] + o * es;
          a[0].in_heap_off = in_off0 + o * es;
          a[0].out_heap_off = out_off0 + o * es;
          rc = launch_all_reduce_nvls(dtype, NVLS_TWOSHOT, ctx_, a,
                                      cfg_for(ceil_div(vecs_for(len, es), world_), t, stream, 64, 1));
          if (rc == cudaSuccess && !out_heap) {
            ckrt(cudaEventRecord(pipe_ev_[1 + kNvlsPipePieces + i], stream), "stage out");
            ckrt(cudaStreamWaitEvent(pipe_out_, pipe_ev_[1 + kNvlsPipePieces + i], 0), "stage out");
            ckrt(cudaMemcpyAsync((char*)out[0] + o * es, (char*)local_ptr(out_off0) + o * es, len * es,
                                 cudaMemcpyDeviceToDevice, pipe_out_), "stage out");
          }
        }
      }
      if (!out_heap) {
        ckrt(cudaEventRecord(pipe_ev_[1 + 2 * kNvlsPipePieces], pipe_out_), "pipeline join");
        ckrt(cudaStreamWaitEvent(stream, pipe_ev_[1 + 2 * kNvlsPipePieces], 0), "pipeline join");
      }
      break;
    }
    default:
      throw std::runtime_error("penny: unknown all-reduce algorithm " + std::to_string(algo));
  }
  ckrt(rc, algo_name(algo));
}

void Communicator::reduce_scatter(int dtype, const void* const* in, void* const* out,
                                  size_t n_total, bool nvls, const Tuning& t,
                                  cudaStream_t stream, bool pipelined) {
  const int es = dtype_size(dtype);
  if (n_total == 0) return;
  if (n_total % world_ != 0)
    throw std::runtime_error("penny: reduce_scatter needs a multiple of the world size");
  if (world_ == 1) {
    if (in[0] != out[0])
      ckrt(cudaMemcpyAsync(out[0], in[0], n_total * es, cudaMemcpyDeviceToDevice, stream), "memcpy");
    return;
  }
  const size_t shard = n_total / world_;
  const int nv = views();
  CollArgs a[kMaxRanks];
  memset(a, 0, sizeof(a));
  for (int v = 0; v < nv; ++v) {
    a[v].in = in[v];
    a[v].out = out[v];
    a[v].n = n_total;
    a[v].in_heap_off = heap_offset_of(in[v], v);
    a[v].out_heap_off = kNotInHeap;
    a[v].nnodes = 1;
    a[v].routes = 1;
  }
  const size_t SV = vecs_for(shard, es);
  if (nvls) {
    if (!has_multicast()) throw std::runtime_error("penny: NVLS reduce-scatter without multicast");
    if ((shard * es) % 16 != 0) throw std::runtime_error("penny: NVLS shards must be 16-byte multiples");
    if (a[0].in_heap_off == kNotInHeap || !t.symmetric_in) {
      ensure(stage_in_, n_total * es, "NVLS input staging");
      ckrt(cudaMemcpyAsync(local_ptr(stage_in_.off), in[0], n_total * es, cudaMemcpyDeviceToDevice,
                           stream), "stage in");
      a[0].in_heap_off = stage_in_.off;
    }
    ckrt(launch_reduce_scatter_nvls(dtype, ctx_, a, cfg_for(SV, t, stream, 64, 1)), "nvls rs");
    return;
  }
  Region& r = ensure(scratch_, reduce_scatter_scratch_bytes(n_total, es, world_), "reduce-scatter");
  for (int v = 0; v < nv; ++v) {
    a[v].scratch_off = r.off;
    a[v].scratch_bytes = r.bytes;
  }
  if (pipelined)
    ckrt(launch_reduce_scatter_pipelined(dtype, ctx_, a, cfg_for(SV, t, stream, 128, 1)), "reduce_scatter (pipelined)");
  else
    ckrt(launch_reduce_scatter(dtype, ctx_, a, cfg_for(SV, t, stream, 128, 1)), "reduce_scatter");
}

void Communicator::all_gather(int dtype, const void* const* in, void* const* out, size_t n_shard,
                              bool nvls, const Tuning& t, cudaStream_t stream) {
  const int es = dtype_size(dtype);
  if (n_shard == 0) return;
  if (world_ == 1) {
    if (in[0] != out[0])
      ckrt(cudaMemcpyAsync(out[0], in[0], n_shard * es, cudaMemcpyDeviceToDevice, stream), "memcpy");
    return;
  }
  const int nv = views();
  CollArgs a[kMaxRanks];
  memset(a, 0, sizeof(a));
  size_t oo = heap_offset_of(out[0], 0);
  bool same = oo != kNotInHeap && (n_shard * es) % 16 == 0;
  for (int v = 1; v < nv; ++v) same = same && heap_offset_of(out[v], v) == oo;
  for (int v = 0; v < nv; ++v) {
    a[v].in = in[v];
    a[v].out = out[v];
    a[v].n = n_shard;
    a[v].in_heap_off = heap_offset_of(in[v], v);
    a[v].out_heap_off = (same && t.symmetric_out) ? oo : kNotInHeap;
    a[v].nnodes = 1;
    a[v].routes = 1;
  }
  const size_t SV = vecs_for(n_shard, es);
  if (nvls) {
    if (!has_multicast()) throw std::runtime_error("penny: NVLS all-gather without multicast");
    if (!same || !t.symmetric_out)
      throw std::runtime_error(
          "penny: NVLS all-gather needs a 16-byte-multiple shard and a symmetric output in the heap");
    a[0].out_heap_off = oo;
    ckrt(launch_all_gather_nvls(dtype, ctx_, a, cfg_for(SV, t, stream, 64, 1)), "nvls ag");
    return;
  }
  if (a[0].out_heap_off == kNotInHeap) {
    Region& r = ensure(scratch_, all_gather_scratch_bytes(n_shard, es, world_), "all-gather");
    for (int v = 0; v < nv; ++v) {
      a[v].scratch_off = r.off;
      a[v].scratch_bytes = r.bytes;
    }
  }
  ckrt(launch_all_gather(dtype, ctx_, a, cfg_for(SV, t, stream, 128, 1)), "all_gather");
}

void Communicator::all_to_all(int dtype, const void* const* in, void* const* out, size_t n_chunk,
                              const Tuning& t, cudaStream_t stream, bool pipelined) {
  const int es = dtype_size(dtype);
  if (n_chunk == 0) return;
  if (world_ == 1) {
    if (in[0] != out[0])
      ckrt(cudaMemcpyAsync(out[0], in[0], n_chunk * es, cudaMemcpyDeviceToDevice, stream), "memcpy");
    return;
  }
  const int nv = views();
  CollArgs a[kMaxRanks];
  memset(a, 0, sizeof(a));
  size_t oo = heap_offset_of(out[0], 0);
  bool same = oo != kNotInHeap && (n_chunk * es) % 16 == 0;
  for (int v = 1; v < nv; ++v) same = same && heap_offset_of(out[v], v) == oo;
  for (int v = 0; v < nv; ++v) {
    a[v].in = in[v];
    a[v].out = out[v];
    a[v].n = n_chunk;
    a[v].in_heap_off = heap_offset_of(in[v], v);
    a[v].out_heap_off = (same && t.symmetric_out) ? oo : kNotInHeap;
    a[v].nnodes = 1;
    a[v].routes = 1;
  }
  if (a[0].out_heap_off == kNotInHeap) {
    Region& r = ensure(scratch_, all_to_all_scratch_bytes(n_chunk, es, world_), "all-to-all");
    for (int v = 0; v < nv; ++v) {
      a[v].scratch_off = r.off;
      a[v].scratch_bytes = r.bytes;
    }
  }
  if (pipelined && a[0].out_heap_off == kNotInHeap)
    ckrt(launch_all_to_all_pipelined(dtype, ctx_, a, cfg_for(vecs_for(n_chunk, es), t, stream, 128, 1)),
         "all_to_all (pipelined)");
  else
    ckrt(launch_all_to_all(dtype, ctx_, a, cfg_for(vecs_for(n_chunk, es), t, stream, 128, 1)),
         "all_to_all");
}

void Communicator::exchange(int dtype, void* const* buf, size_t n, const int* peers,
                            const Tuning& t, cudaStream_t stream) {
  const int es = dtype_size(dtype);
  if (n == 0 || world_ == 1) return;
  const int nv = views();
  Region& r = ensure(scratch_pair_, exchange_scratch_bytes(n, es), "exchange");
  CollArgs a[kMaxRanks];
  memset(a, 0, sizeof(a));
  for (int v = 0; v < nv; ++v) {
    if (peers[v] < 0 || peers[v] >= world_) throw std::runtime_error("penny: bad exchange peer");
    a[v].in = buf[v];
    a[v].out = buf[v];
    a[v].n = n;
    a[v].scratch_off = r.off;
    a[v].scratch_bytes = r.bytes;
    a[v].in_heap_off = kNotInHeap;
    a[v].out_heap_off = kNotInHeap;
    a[v].peer = peers[v];
    a[v].nnodes = 1;
    a[v].routes = 1;
  }
  ckrt(launch_exchange(dtype, ctx_, a, cfg_for(vecs_for(n, es), t, stream, 128, 1)), "exchange");
}

void Communicator::fused_ar_rmsnorm(int dtype, int proto, const void* const* in,
                                    const void* const* residual, const void* weight,
                                    void* const* out, void* const* residual_out, int rows,
                                    int hidden, float eps, const Tuning& t, cudaStream_t stream, bool pushed) {
  const int es = dtype_size(dtype);
  if (pushed && (proto != FUSED_PROTO_LL_TWOSHOT || world_ < 2))
    throw std::runtime_error("penny: pushed inputs are a feature of the LL two-shot fused norm");
  const int nv = views();
  FusedNormArgs a[kMaxRanks];
  memset(a, 0, sizeof(a));
  for (int v = 0; v < nv; ++v) {
    a[v].in = in[v];
    a[v].residual = residual ? residual[v] : nullptr;
    a[v].weight = weight;
    a[v].out = out[v];
    a[v].residual_out = residual_out ? residual_out[v] : nullptr;
    a[v].rows = rows;
    a[v].hidden = hidden;
    a[v].eps = eps;
    a[v].in_heap_off = heap_offset_of(in[v], v);
    a[v].out_heap_off = heap_offset_of(out[v], v);
    a[v].pushed = pushed ? 1 : 0;
  }
  int threads = t.threads > 0 ? t.threads : std::min(512, std::max(32, (hidden * es / 16 + 31) / 32 * 32));
  if (world_ == 1) {
    ckrt(launch_add_rmsnorm(dtype, a[0], std::min(rows, 1024), threads, stream), "add_rmsnorm");
    return;
  }
  LaunchCfg cfg;
  cfg.threads = threads;
  cfg.stream = stream;
  cfg.emu_world = emu_ ? world_ : 0;
  cfg.pdl = true;  // sits between the GEMMs of a decode step: overlap its launch with the producer's tail
  int max_blocks = emu_ ? std::max(1, 128 / world_) : 256;
  if (proto == FUSED_PROTO_NVLS_ONESHOT) {
    if (!has_multicast()) throw std::runtime_error("penny: NVLS fused norm without multicast");
    if (a[0].in_heap_off == kNotInHeap || !t.symmetric_in)
      throw std::runtime_error("penny: one-shot NVLS fused norm needs a symmetric heap tensor for in");
    cfg.blocks = t.blocks > 0 ? t.blocks : std::min(max_blocks, std::max(1, rows));
  } else if (proto == FUSED_PROTO_NVLS) {
    if (!has_multicast()) throw std::runtime_error("penny: NVLS fused norm without multicast");
    if (a[0].in_heap_off == kNotInHeap || a[0].out_heap_off == kNotInHeap || !t.symmetric_in ||
        !t.symmetric_out)
      throw std::runtime_error("penny: NVLS fused norm needs symmetric heap tensors for in and out");
    cfg.blocks = t.blocks > 0 ? t.blocks : std::min(max_blocks, std::max(1, (rows + world_ - 1) / world_));
  } else {
    Region& r = ensure(proto == FUSED_PROTO_LL || proto == FUSED_PROTO_LL_TWOSHOT ? scratch_ll_ : scratch_,
                       fused_norm_scratch_bytes(proto, rows, hidden, es, world_), "fused norm");
    if (pushed && (r.off != push_region_.off || r.bytes != push_region_.bytes))
      throw std::runtime_error("penny: the scratch region changed since fused_norm_push_target; ask for a new target");
    for (int v = 0; v < nv; ++v) {
      a[v].scratch_off = r.off;
      a[v].scratch_bytes = r.bytes;
    }
    cfg.blocks = t.blocks > 0 ? t.blocks : std::min(max_blocks, rows);
  }
  ckrt(launch_fused_ar_rmsnorm(dtype, proto, ctx_, a, cfg), "fused_ar_rmsnorm");
}

sm100::DecodePush Communicator::fused_norm_push_target(int rows, int hidden, int elem_size, int view) {
  if (world_ < 2 || elem_size != 2 || hidden % 8 != 0 || rows < 1)
    throw std::runtime_error("penny: fused_norm_push_target needs >= 2 ranks, bf16 and hidden % 8 == 0");
  Region& r = ensure(scratch_ll_, fused_norm_scratch_bytes(FUSED_PROTO_LL_TWOSHOT, rows, hidden, elem_size, world_),
                     "fused norm");
  push_region_ = r;
  sm100::DecodePush p;
  memset(&p, 0, sizeof(p));
  for (int k = 0; k < world_; ++k) p.heap[k] = heap_->base(k);
  const int me = emu_ ? view : rank_;
  p.call_seq = &reinterpret_cast<const SignalPad*>(heap_->base(me))->call_seq[SEQ_ALL];
  p.scratch_off = r.off;
  p.scratch_bytes = r.bytes;
  p.rank = me;
  p.world = world_;
  p.per = (rows + world_ - 1) / world_;
  p.hv = hidden / 8;
  return p;
}

void Communicator::moe_dispatch(int dtype, const MoeArgs* args, const Tuning& t, cudaStream_t stream) {
  LaunchCfg cfg;
  cfg.threads = t.threads > 0 ? t.threads : 256;
  cfg.stream = stream;
  cfg.emu_world = emu_ ? world_ : 0;
  const int cap = emu_ ? std::max(1, 128 / world_) : 64;  // every block polls blocks * world flags
  cfg.blocks = std::min(cap, t.blocks > 0 ? t.blocks : cap);
  ckrt(launch_moe_dispatch(dtype, ctx_, args, cfg), "moe_dispatch");
}

void Communicator::moe_combine(int dtype, const MoeArgs* args, const Tuning& t, cudaStream_t stream) {
  LaunchCfg cfg;
  cfg.threads = t.threads > 0 ? t.threads : 256;
  cfg.stream = stream;
  cfg.emu_world = emu_ ? world_ : 0;
  const int cap = emu_ ? std::max(1, 128 / world_) : 64;
  cfg.blocks = std::min(cap, t.blocks > 0 ? t.blocks : cap);
  ckrt(launch_moe_combine(dtype, ctx_, args, cfg), "moe_combine");
}

void Communicator::gemm_reduce_scatter(const void* a, const void* b, void* out, int M, int N, int K,
                                       int lda, int ldb, int ldo, uint32_t* error_word,
                                       cudaStream_t stream) {
  if (emu_ && world_ != 1) throw std::runtime_error("penny: fused GEMMs need one process per GPU");
  Region& r = ensure(scratch_, sm100::gemm_rs_scratch_bytes(M, N, world_), "GEMM reduce-scatter");
  ckrt(sm100::launch_gemm_rs(ctx_, r.off, r.bytes, a, b, out, M, N, K, lda, ldb, ldo, error_word, stream),
       "gemm_reduce_scatter (M must be a multiple of 128 * world, N of 256, K and strides of 8)");
}

void Communicator::all_gather_gemm(const void* a_shard, const void* b, void* out, int M, int N, int K,
                                   int lda, int ldb, int ldc, int side_ctas, uint32_t* error_word,
                                   cudaStream_t stream) {
  if (emu_ && world_ != 1) throw std::runtime_error("penny: fused GEMMs need one process per GPU");
  const size_t need = sm100::ag_gemm_scratch_bytes(M, K);
  // A shape gets its own memory (its halves must be exactly M x K) the first time
  // it is seen and the same memory ever after; the call order is the same on
  // every rank, so the table is too.
  Region& ag = ag_regions_[{M, K}];
  if (ag.bytes != need) {
    ag.off = alloc(need);
    ag.bytes = need;
  }
  ckrt(sm100::launch_ag_gemm(ctx_, ag.off, ag.bytes, a_shard, b, out, M, N, K, lda, ldb,
                             ldc, side_ctas, error_word, stream),
       "all_gather_gemm (M must be a multiple of 128 * world, K and strides of 8)");
}

void Communicator::wait_selftest(cudaStream_t stream) {
  LaunchCfg cfg;
  cfg.blocks = 1;
  cfg.threads = 32;
  cfg.stream = stream;
  cfg.emu_world = emu_ ? world_ : 0;
  ckrt(launch_wait_selftest(ctx_, cfg), "wait_selftest");
}

StatusRecord Communicator::read_status(int view, bool clear) {
  uint32_t w[kStatusWords];
  char* p = heap_->base(emu_ ? view : rank_) + kStatusOffset;
  ckrt(cudaDeviceSynchronize(), "synchronize");
  ckrt(cudaMemcpy(w, p, sizeof(w), cudaMemcpyDeviceToHost), "read status");
  if (clear && w[0] != 0) ckrt(cudaMemset(p, 0, sizeof(w)), "clear status");
  StatusRecord s;
  s.code = w[0];
  s.rank = w[1];
  s.peer = w[2];
  s.block = w[3];
  s.want = (unsigned long long)w[4] | ((unsigned long long)w[5] << 32);
  s.seen = (unsigned long long)w[6] | ((unsigned long long)w[7] << 32);
  return s;
}

void Communicator::host_barrier() {
  if (bs_) bs_->barrier();
}

void Communicator::poison_scratch() {
  cudaDeviceSynchronize();
  host_barrier();  // nobody is still reading or writing a peer's scratch
  std::vector<const Region*> regions = {&scratch_, &scratch_ll_, &scratch_pair_, &stage_in_, &stage_out_};
  for (const auto& kv : ag_regions_) regions.push_back(&kv.second);
  for (const Region* r : regions) {
    if (r->bytes == 0) continue;
    for (int v = 0; v < views(); ++v) {
      cudaError_t rc = cudaMemset(local_ptr(r->off, v), 0xFF, r->bytes);
      if (rc != cudaSuccess)
        throw std::runtime_error(std::string("penny: poison_scratch: ") + cudaGetErrorString(rc));
    }
  }
  cudaDeviceSynchronize();
  host_barrier();  // nobody starts the next call before every heap is poisoned
}

}  // namespace penny
