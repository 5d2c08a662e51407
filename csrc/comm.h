// Communicator: owns the bootstrap, the symmetric heap, the scratch regions and
// the launch policy of every collective.  Torch-free; torch_interface.cpp wraps
// it for Python.
//
// It is what the reference spreads over its `AllReduce` base class (symmetric
// scratch + signals + epoch, csrc/common.h:21-59), the per-algorithm subclasses
// (csrc/all_reduce_*.cu constructors) and the NVSHMEM runtime.
//
// Threading / ordering contract: collectives of one communicator are issued
// from one thread onto one stream at a time, in the same order on every rank
// (heap allocations too – they are bump-allocated, so offsets agree).
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "algos.h"
#include "bootstrap.h"
#include "coll_args.h"
#include "fused_ops.h"
#include "gemm_decode_sm100.h"
#include "symm_heap.h"

namespace penny {

struct CommOptions {
  size_t heap_bytes = (size_t)1 << 30;
  int heap_mode = HEAP_AUTO;
  bool multicast = true;
  int timeout_ms = 10000;       // bound of every device-side wait
  int bootstrap_timeout_ms = 120000;
};

struct Tuning {
  int blocks = 0;   // 0 = choose from the message size
  int threads = 0;  // 0 = 512
  int nnodes = 1;   // virtual nodes (double ring / tree / node-aware ring)
  int routes = 0;   // 0 = choose
  // The caller vouches that the tensor sits at the same heap offset on every
  // rank (allocated by the same alloc() call), so peers / the switch may address
  // it directly instead of going through scratch or staging.
  bool symmetric_in = false;
  bool symmetric_out = false;
};

struct StatusRecord {
  uint32_t code, rank, peer, block;
  unsigned long long want, seen;
};

class Communicator {
 public:
  // Real: one process per GPU.  uid from make_unique_id() on one rank.
  Communicator(const std::string& uid, int rank, int world, const CommOptions& opt);
  // Emulated: `world` virtual ranks on the current GPU of this process.
  Communicator(int emu_world, const CommOptions& opt);
  ~Communicator();

  int rank() const { return rank_; }
  int world() const { return world_; }
  bool emulated() const { return emu_; }
  int views() const { return emu_ ? world_ : 1; }  // tensors per call
  bool has_multicast() const { return heap_->has_multicast(); }
  std::string describe() const;
  const CommCtx& ctx() const { return ctx_; }
  SymmHeap& heap() { return *heap_; }
  Bootstrap* bootstrap() { return bs_.get(); }

  // Symmetric allocation (256-byte aligned); returns the heap offset.
  size_t alloc(size_t bytes);
  void* local_ptr(size_t off, int view = 0) const;
  size_t heap_offset_of(const void* p, int view = 0) const;  // kNotInHeap if outside
  size_t heap_free_bytes() const { return heap_->bytes() - arena_top_; }

  // in / out: views() pointers each.  n as documented in CollArgs.
  void all_reduce(int algo, int dtype, const void* const* in, void* const* out, size_t n,
                  const Tuning& t, cudaStream_t stream);
  // pipelined: the push variant that reduces chunk k - 1 while chunk k is on the wire
  void reduce_scatter(int dtype, const void* const* in, void* const* out, size_t n_total, bool nvls,
                      const Tuning& t, cudaStream_t stream, bool pipelined = false);
  void all_gather(int dtype, const void* const* in, void* const* out, size_t n_shard, bool nvls,
                  const Tuning& t, cudaStream_t stream);
  // pipelined (scratch path only): piece k - 1 is copied out while piece k is on the wire
  void all_to_all(int dtype, const void* const* in, void* const* out, size_t n_chunk,
                  const Tuning& t, cudaStream_t stream, bool pipelined = false);
  void exchange(int dtype, void* const* buf, size_t n, const int* peers, const Tuning& t,
                cudaStream_t stream);
  // proto: FusedProto.  Pointer arrays have views() entries.
  void fused_ar_rmsnorm(int dtype, int proto, const void* const* in, const void* const* residual,
                        const void* weight, void* const* out, void* const* residual_out, int rows,
                        int hidden, float eps, const Tuning& t, cudaStream_t stream, bool pushed = false);
  // Where the decode GEMM that feeds fused_ar_rmsnorm(FUSED_PROTO_LL_TWOSHOT, pushed = true) on a
  // [rows, hidden] tensor puts the rows other ranks own (view: the virtual rank when emulated).
  // Reserves the scratch region; the pushed call checks that it is still the same one.
  sm100::DecodePush fused_norm_push_target(int rows, int hidden, int elem_size, int view = 0);

  // MoE expert-parallel row exchange; args: views() entries (see MoeArgs).
  void moe_dispatch(int dtype, const MoeArgs* args, const Tuning& t, cudaStream_t stream);
  void moe_combine(int dtype, const MoeArgs* args, const Tuning& t, cudaStream_t stream);

  // Fused tcgen05 GEMM + collective (bf16; real communicators, or an emulated
  // world of 1).  out = this rank's [M / world, N] shard of sum_r A_r B_r^T.
  void gemm_reduce_scatter(const void* a, const void* b, void* out, int M, int N, int K, int lda,
                           int ldb, int ldo, uint32_t* error_word, cudaStream_t stream);
  // out[M, N] = gather(a_shard)[M, K] * B[N, K]^T.
  void all_gather_gemm(const void* a_shard, const void* b, void* out, int M, int N, int K, int lda,
                       int ldb, int ldc, int side_ctas, uint32_t* error_word, cudaStream_t stream);

  // The all-reduce algorithm `auto` resolves to.  A measured table (set_tuning)
  // for this element size and memory class decides when there is one: the first
  // entry whose byte bound is >= the message size, the last entry beyond.  Without
  // a table a two-threshold rule from 8-GPU measurements is used.  symmetric:
  // both tensors sit at one heap offset on every rank (the switch and the peers
  // can address them directly); otherwise the NVLS algorithms pay staging copies.
  int pick_algo(int dtype, size_t n, bool symmetric = false) const;
  struct TuneEntry {
    size_t max_bytes;  // inclusive upper bound; ~0 for the last entry
    int algo;
  };
  // Installs the all-reduce table of (elem_size 2 or 4, symmetric or not).  Entries sorted by bound.
  void set_tuning(int elem_size, bool symmetric, const std::vector<TuneEntry>& entries);

  // Provokes a device-side timeout on a private flag (nothing else is touched).
  void wait_selftest(cudaStream_t stream);
  // Reads (and optionally clears) the status words; synchronises the device.
  StatusRecord read_status(int view, bool clear);
  void host_barrier();
  // Debug aid: with every rank idle (device synchronised, host barrier on both
  // sides) overwrites every scratch region this communicator has allocated with
  // 0xFF bytes (NaN in every float format, never a valid flag or stamp), so a
  // kernel that reads scratch it was not sent in the current call returns NaNs
  // instead of the previous call's plausible numbers.  Collective: all ranks call it.
  void poison_scratch();
  void set_timeout_ms(int ms);
  void destroy();

 private:
  struct Region {
    size_t off = 0, bytes = 0;
  };
  Region& ensure(Region& r, size_t need, const char* what);
  void init_ctx(const CommOptions& opt);
  LaunchCfg cfg_for(size_t vecs, const Tuning& t, cudaStream_t s, int max_blocks, int multiple,
                    int vecs_per_thread = 4) const;
  void run_all_reduce_once(int algo, int dtype, const void* const* in, void* const* out, size_t n,
                           const Tuning& t, cudaStream_t stream);

  std::unique_ptr<Bootstrap> bs_;
  std::unique_ptr<SymmHeap> heap_;
  CommCtx ctx_;
  int rank_ = 0, world_ = 1;
  bool emu_ = false;
  size_t arena_top_ = kHeapReserved;
  Region scratch_;       // halved, shared by the all-dependent collectives
  Region scratch_ll_;    // halved, LL lines only
  Region scratch_pair_;  // exchange slot
  Region stage_in_, stage_out_;  // NVLS staging for tensors outside the heap
  // side streams + events that overlap the staging copies of a very large switch all-reduce with
  // its reductions (created on first use)
  void ensure_pipe();
  cudaStream_t pipe_in_ = nullptr, pipe_out_ = nullptr;
  std::vector<cudaEvent_t> pipe_ev_;
  // gathered A of all_gather_gemm: one dedicated region per (M, K), kept for the
  // communicator's lifetime and reused, so alternating shapes do not grow the heap
  std::map<std::pair<int, int>, Region> ag_regions_;
  Region push_region_;   // scratch the last fused_norm_push_target was given
  std::vector<TuneEntry> tune_[2][2];  // [elem_size == 4][symmetric]
  bool destroyed_ = false;
};

}  // namespace penny
