// Pull-model collectives on IPC-registered buffers: the engine behind the
// drop-in `CustomAllreduce` class that vLLM / SGLang tensor-parallel workers use.
//
// Capability map to the reference (csrc/custom_all_reduce.cuh):
//   cross_device_reduce_1stage          :310-367  -> pull_reduce_1stage
//   cross_device_reduce_2stage          :374-461  -> pull_reduce_2stage
//   cross_device_reduce_scatter_2stage  :464-539  -> pull_reduce_scatter
//   cross_device_all_gather             :541-595  -> pull_all_gather
//   Signal / RankData / barriers        :60-72, :204-253
//   class CustomAllreduce               :601-1054
// Same contract (every rank reads its peers' registered inputs over NVLink
// between two flag barriers, fp32 accumulation in rank order so all ranks get
// bit-identical results, CUDA-graph capture with late buffer registration), a
// fresh implementation: bounded waits that record a status instead of spinning
// forever, 64-bit indexing, per-block flag counters kept in device memory, a
// block count sized for 148 SMs instead of the 36-block cap tuned on A100-class
// parts (:38-42,759-767), and no NVSHMEM inter-node stage (single box).
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "pk.h"

namespace penny {
namespace pull {

constexpr int kPullMaxBlocks = 128;

// Lives at the start of each rank's meta buffer (the IPC-shared allocation whose
// pointers are handed to init_custom_ar); the 2-stage scratch follows it.
struct alignas(128) PullSignal {
  // flag[phase][block][src]: written by block `block` of rank `src`
  uint32_t flag[3][kPullMaxBlocks][kMaxRanks];
  // per-block call counter, owner only
  uint32_t counter[kPullMaxBlocks];
  // first timeout: {code, rank, peer, block, want, seen}
  uint32_t status[8];
};

struct RankData {
  const void* ptrs[kMaxRanks];
};
struct RankSignals {
  PullSignal* signals[kMaxRanks];
};

enum PullAlgo : int { PULL_AUTO = 0, PULL_1STAGE = 1, PULL_2STAGE = 2 };

class CustomAllreduce {
 public:
  CustomAllreduce(void* const* signals, void* rank_data, size_t rank_data_bytes, int rank,
                  int world, bool fully_connected);
  ~CustomAllreduce();

  int rank() const { return rank_; }
  int world() const { return world_; }

  // ptrs[r] = rank r's buffer as mapped in this process (ptrs[rank] is local).
  void register_buffer(void* const* ptrs);
  // Buffers first seen during graph capture: (concatenated 64-byte IPC handles,
  // offsets inside their allocations).
  std::pair<std::string, std::vector<int64_t>> get_graph_buffer_ipc_meta();
  void register_graph_buffers(const std::vector<std::string>& handles,
                              const std::vector<std::vector<int64_t>>& offsets);

  // input must be registered, or the stream must be capturing.
  void allreduce(int dtype, cudaStream_t stream, const void* input, void* output, size_t n);
  void reduce_scatter(int dtype, cudaStream_t stream, const void* input, void* output, size_t n);
  void all_gather(int dtype, cudaStream_t stream, const void* input, void* output, size_t n_shard);

  // Host-side copy of the status words (synchronises the device).
  void read_status(uint32_t out[8], bool clear);
  void set_timeout_ms(int ms) { timeout_ns_ = (unsigned long long)ms * 1000000ull; }
  void set_max_blocks(int b) { max_blocks_ = b < 1 ? 1 : (b > kPullMaxBlocks ? kPullMaxBlocks : b); }
  void set_algo(int a) { forced_algo_ = a; }

 private:
  const RankData* lookup(cudaStream_t stream, const void* input);
  int blocks_for(size_t vecs) const;

  int rank_, world_;
  bool fully_connected_;
  RankSignals sg_;
  PullSignal* self_sg_;
  RankData* d_rank_data_base_;
  RankData* d_rank_data_end_;
  std::unordered_map<const void*, RankData*> buffers_;
  std::vector<const void*> graph_unreg_buffers_;
  std::map<std::string, char*> ipc_handles_;
  unsigned long long timeout_ns_ = 10000000000ull;
  int max_blocks_ = 64;
  int forced_algo_ = PULL_AUTO;
};

}  // namespace pull
}  // namespace penny
