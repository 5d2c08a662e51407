// Kernels and host class of the pull-model custom all-reduce; see
// custom_all_reduce.cuh for the capability map.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <stdexcept>

#include "algos.h"
#include "custom_all_reduce.cuh"
#include "schedule.h"

namespace penny {
namespace pull {

namespace {

void ckrt(cudaError_t r, const char* what) {
  if (r != cudaSuccess) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string("penny custom_ar: ") + what + ": " + cudaGetErrorString(r));
  }
}

__device__ __forceinline__ void st_flag(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_flag(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct PullCtx {
  RankSignals sg;
  PullSignal* self;
  int rank;
  unsigned long long timeout_ns;
};

// Block-wide barrier with block `blockIdx.x` of every peer.  Threads < NG each
// handle one peer.  Release/acquire at system scope: everything this block wrote
// before the barrier is visible to peers after it, and vice versa.  Returns
// false (uniformly) after a timeout.
template <int NG>
__device__ __forceinline__ bool pull_barrier(const PullCtx& c, int phase, uint32_t flag) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < NG && threadIdx.x != c.rank) {
    const int peer = threadIdx.x;
    st_flag(&c.sg.signals[peer]->flag[phase][blockIdx.x][c.rank], flag);
    const uint32_t* mine = &c.self->flag[phase][blockIdx.x][peer];
    uint32_t seen = ld_flag(mine);
    if ((int32_t)(seen - flag) < 0) {
      const unsigned long long t0 = now_ns();
      for (uint32_t spin = 1;; ++spin) {
        seen = ld_flag(mine);
        if ((int32_t)(seen - flag) >= 0) break;
        if ((spin & 31u) == 0u && now_ns() - t0 > c.timeout_ns) {
          if (atomicCAS(&c.self->status[0], 0u, (uint32_t)ST_TIMEOUT_BARRIER) == 0u) {
            c.self->status[1] = (uint32_t)c.rank;
            c.self->status[2] = (uint32_t)peer;
            c.self->status[3] = blockIdx.x;
            c.self->status[4] = flag;
            c.self->status[5] = seen;
          }
          s_fail = 1;
          break;
        }
      }
    }
  }
  __syncthreads();
  return s_fail == 0;
}

// Each call of a kernel takes the next value of the block's own counter.
__device__ __forceinline__ uint32_t next_flag(const PullCtx& c) {
  __shared__ uint32_t s_flag;
  if (threadIdx.x == 0) {
    s_flag = c.self->counter[blockIdx.x] + 1;
    c.self->counter[blockIdx.x] = s_flag;
  }
  __syncthreads();
  return s_flag;
}

template <typename T, int NG>
__device__ __forceinline__ V16 pull_sum(const RankData& rd, size_t v) {
  constexpr int E = 16 / sizeof(T);
  float acc[E];
#pragma unroll
  for (int i = 0; i < E; ++i) acc[i] = 0.f;
#pragma unroll
  for (int r = 0; r < NG; ++r)
    unpack_add<T>(ld16(reinterpret_cast<const char*>(rd.ptrs[r]) + v * 16), acc);
  return pack<T>(acc);
}

template <typename T, int NG>
__global__ void __launch_bounds__(512) pull_reduce_1stage(PullCtx c, const RankData* rdp, T* out,
                                                          size_t V) {
  const RankData rd = *rdp;
  const uint32_t flag = next_flag(c);
  if (!pull_barrier<NG>(c, 0, flag)) return;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < V;
       v += (size_t)gridDim.x * blockDim.x)
    st16(reinterpret_cast<char*>(out) + v * 16, pull_sum<T, NG>(rd, v));
  pull_barrier<NG>(c, 2, flag);  // nobody overwrites its input while a peer still reads it
}

__device__ __forceinline__ char* tmp_of(PullSignal* s) { return reinterpret_cast<char*>(s + 1); }

template <typename T, int NG>
__global__ void __launch_bounds__(512) pull_reduce_2stage(PullCtx c, const RankData* rdp, T* out,
                                                          size_t V) {
  const RankData rd = *rdp;
  const uint32_t flag = next_flag(c);
  const Span mine = split_span(V, NG, c.rank);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (!pull_barrier<NG>(c, 0, flag)) return;
  // stage 1: reduce my partition into my scratch (it follows my signal block)
  char* my_tmp = tmp_of(c.self);
  for (size_t j = first; j < mine.end - mine.begin; j += stride)
    st16(my_tmp + j * 16, pull_sum<T, NG>(rd, mine.begin + j));
  if (!pull_barrier<NG>(c, 1, flag)) return;
  // stage 2: gather every partition from its owner's scratch.  The thread that
  // reads slot j of a partition is the thread that wrote slot j on the owner.
#pragma unroll
  for (int d = 0; d < NG; ++d) {
    const int r = (c.rank + d) % NG;
    const Span sp = split_span(V, NG, r);
    const char* tmp = tmp_of(c.sg.signals[r]);
    for (size_t j = first; j < sp.end - sp.begin; j += stride)
      st16(reinterpret_cast<char*>(out) + (sp.begin + j) * 16, ld16(tmp + j * 16));
  }
  // No end barrier: a peer's scratch is rewritten only after the start barrier
  // of the next call, which this rank joins after it finished reading.
}

// V = vectors of ONE shard; rank r's shard starts at vector r * V of the input.
template <typename T, int NG>
__global__ void __launch_bounds__(512) pull_reduce_scatter(PullCtx c, const RankData* rdp, T* out,
                                                           size_t V) {
  const RankData rd = *rdp;
  const uint32_t flag = next_flag(c);
  if (!pull_barrier<NG>(c, 0, flag)) return;
  for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < V;
       j += (size_t)gridDim.x * blockDim.x)
    st16(reinterpret_cast<char*>(out) + j * 16, pull_sum<T, NG>(rd, (size_t)c.rank * V + j));
  pull_barrier<NG>(c, 2, flag);
}

template <typename T, int NG>
__global__ void __launch_bounds__(512) pull_all_gather(PullCtx c, const RankData* rdp, T* out,
                                                       size_t V) {
  const RankData rd = *rdp;
  const uint32_t flag = next_flag(c);
  if (!pull_barrier<NG>(c, 0, flag)) return;
#pragma unroll
  for (int d = 0; d < NG; ++d) {
    const int r = (c.rank + d) % NG;
    const char* src = reinterpret_cast<const char*>(rd.ptrs[r]);
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < V;
         j += (size_t)gridDim.x * blockDim.x)
      st16(reinterpret_cast<char*>(out) + ((size_t)r * V + j) * 16, ld16(src + j * 16));
  }
  pull_barrier<NG>(c, 2, flag);
}

}  // namespace

CustomAllreduce::CustomAllreduce(void* const* signals, void* rank_data, size_t rank_data_bytes,
                                 int rank, int world, bool fully_connected)
    : rank_(rank), world_(world), fully_connected_(fully_connected) {
  if (world != 2 && world != 4 && world != 6 && world != 8)
    throw std::runtime_error("penny custom_ar: world size must be 2, 4, 6 or 8");
  if (rank < 0 || rank >= world) throw std::runtime_error("penny custom_ar: bad rank");
  memset(&sg_, 0, sizeof(sg_));
  for (int i = 0; i < world; ++i) sg_.signals[i] = reinterpret_cast<PullSignal*>(signals[i]);
  self_sg_ = sg_.signals[rank];
  d_rank_data_base_ = reinterpret_cast<RankData*>(rank_data);
  d_rank_data_end_ = d_rank_data_base_ + rank_data_bytes / sizeof(RankData);
  if (const char* e = std::getenv("PENNY_TIMEOUT_MS")) set_timeout_ms(std::atoi(e));
  if (const char* e = std::getenv("PENNY_CUSTOM_AR_BLOCKS")) set_max_blocks(std::atoi(e));
  // Same override names as the reference (csrc/custom_all_reduce.cuh:803-818).
  if (const char* e = std::getenv("VLLM_CUSTOM_ALLREDUCE_ALGO")) {
    std::string s(e);
    if (s == "1stage" || s == "oneshot") forced_algo_ = PULL_1STAGE;
    else if (s == "2stage" || s == "twoshot") forced_algo_ = PULL_2STAGE;
    else throw std::runtime_error("penny custom_ar: VLLM_CUSTOM_ALLREDUCE_ALGO must be 1stage|oneshot|2stage|twoshot");
  }
}

CustomAllreduce::~CustomAllreduce() {
  for (auto& kv : ipc_handles_) cudaIpcCloseMemHandle(kv.second);
}

void CustomAllreduce::register_buffer(void* const* ptrs) {
  if (d_rank_data_base_ + 1 > d_rank_data_end_)
    throw std::runtime_error("penny custom_ar: rank data buffer is full");
  RankData data;
  memset(&data, 0, sizeof(data));
  for (int i = 0; i < world_; ++i) data.ptrs[i] = ptrs[i];
  RankData* d = d_rank_data_base_++;
  ckrt(cudaMemcpy(d, &data, sizeof(data), cudaMemcpyHostToDevice), "register_buffer");
  buffers_[ptrs[rank_]] = d;
}

std::pair<std::string, std::vector<int64_t>> CustomAllreduce::get_graph_buffer_ipc_meta() {
  const size_t num = graph_unreg_buffers_.size();
  std::string handles(sizeof(cudaIpcMemHandle_t) * num, '\0');
  std::vector<int64_t> offsets(num);
  // base address of the allocation a pointer belongs to, without linking libcuda
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult st;
  ckrt(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &st), "driver entry");
  auto get_range = reinterpret_cast<CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr)>(fn);
  for (size_t i = 0; i < num; ++i) {
    const void* ptr = graph_unreg_buffers_[i];
    CUdeviceptr base = 0;
    size_t sz = 0;
    if (get_range == nullptr || get_range(&base, &sz, (CUdeviceptr)ptr) != CUDA_SUCCESS)
      throw std::runtime_error("penny custom_ar: cannot find the allocation of a graph buffer");
    ckrt(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(&handles[i * sizeof(cudaIpcMemHandle_t)]),
                             (void*)base), "cudaIpcGetMemHandle");
    offsets[i] = (int64_t)((const char*)ptr - (const char*)base);
  }
  return {handles, offsets};
}

void CustomAllreduce::register_graph_buffers(const std::vector<std::string>& handles,
                                             const std::vector<std::vector<int64_t>>& offsets) {
  const size_t num = graph_unreg_buffers_.size();
  if (d_rank_data_base_ + num > d_rank_data_end_)
    throw std::runtime_error("penny custom_ar: rank data buffer is full");
  std::vector<RankData> rd(num);
  for (size_t i = 0; i < num; ++i) {
    memset(&rd[i], 0, sizeof(RankData));
    for (int j = 0; j < world_; ++j) {
      if (j == rank_) {
        rd[i].ptrs[j] = graph_unreg_buffers_[i];
        continue;
      }
      std::string key = handles[j].substr(i * sizeof(cudaIpcMemHandle_t), sizeof(cudaIpcMemHandle_t));
      auto it = ipc_handles_.find(key);
      if (it == ipc_handles_.end()) {
        void* p = nullptr;
        cudaIpcMemHandle_t h;
        memcpy(&h, key.data(), sizeof(h));
        ckrt(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
        it = ipc_handles_.emplace(key, (char*)p).first;
      }
      rd[i].ptrs[j] = it->second + offsets[j][i];
    }
  }
  if (num)
    ckrt(cudaMemcpy(d_rank_data_base_, rd.data(), sizeof(RankData) * num, cudaMemcpyHostToDevice),
         "register_graph_buffers");
  d_rank_data_base_ += num;
  graph_unreg_buffers_.clear();
}

const RankData* CustomAllreduce::lookup(cudaStream_t stream, const void* input) {
  auto it = buffers_.find(input);
  if (it != buffers_.end()) return it->second;
  cudaStreamCaptureStatus status;
  ckrt(cudaStreamIsCapturing(stream, &status), "cudaStreamIsCapturing");
  if (status != cudaStreamCaptureStatusActive)
    throw std::runtime_error(
        "penny custom_ar: buffer is not registered (register_buffer, or capture a CUDA graph)");
  // slot filled in later by register_graph_buffers; the graph bakes its address
  RankData* slot = d_rank_data_base_ + graph_unreg_buffers_.size();
  if (slot + 1 > d_rank_data_end_) throw std::runtime_error("penny custom_ar: rank data buffer is full");
  graph_unreg_buffers_.push_back(input);
  return slot;
}

int CustomAllreduce::blocks_for(size_t vecs) const {
  size_t b = ceil_div(vecs, (size_t)512);
  if (b < 1) b = 1;
  if (b > (size_t)max_blocks_) b = (size_t)max_blocks_;
  return (int)b;
}

#define PULL_LAUNCH(KERNEL, V)                                                       \
  do {                                                                               \
    PullCtx c;                                                                       \
    c.sg = sg_;                                                                      \
    c.self = self_sg_;                                                               \
    c.rank = rank_;                                                                  \
    c.timeout_ns = timeout_ns_;                                                      \
    const int blocks = blocks_for(V);                                                \
    PENNY_DISPATCH_DTYPE(dtype, T, PENNY_DISPATCH_WORLD(world_, NG, break, {         \
      KERNEL<T, NG><<<blocks, 512, 0, stream>>>(c, rd, reinterpret_cast<T*>(output), V); \
    }));                                                                             \
    ckrt(cudaGetLastError(), #KERNEL);                                               \
  } while (0)

void CustomAllreduce::allreduce(int dtype, cudaStream_t stream, const void* input, void* output,
                                size_t n) {
  const size_t bytes = n * (size_t)dtype_size(dtype);
  if (bytes % 16 != 0)
    throw std::runtime_error("penny custom_ar: all-reduce needs a byte size that is a multiple of 16");
  const RankData* rd = lookup(stream, input);
  const size_t V = bytes / 16;
  // 2 GPUs: always 1-stage; small messages: 1-stage (latency); else 2-stage
  // (bandwidth).  The crossover is far above the reference's 256-512 KiB
  // (csrc/custom_all_reduce.cuh:831-841) because NVSwitch gives every peer the
  // full link rate and B200 has ~4x the SMs' worth of loads in flight.
  int algo = forced_algo_;
  if (algo == PULL_AUTO) {
    if (world_ == 2) algo = PULL_1STAGE;
    else if (fully_connected_ && bytes < (world_ <= 4 ? (size_t)1 << 20 : (size_t)512 << 10)) algo = PULL_1STAGE;
    else algo = PULL_2STAGE;
  }
  if (algo == PULL_1STAGE) PULL_LAUNCH(pull_reduce_1stage, V);
  else PULL_LAUNCH(pull_reduce_2stage, V);
}

void CustomAllreduce::reduce_scatter(int dtype, cudaStream_t stream, const void* input,
                                     void* output, size_t n) {
  const size_t bytes = n * (size_t)dtype_size(dtype);
  if (n % world_ != 0 || (bytes / world_) % 16 != 0)
    throw std::runtime_error("penny custom_ar: reduce-scatter shards must be multiples of 16 bytes");
  const RankData* rd = lookup(stream, input);
  const size_t V = bytes / world_ / 16;
  PULL_LAUNCH(pull_reduce_scatter, V);
}

void CustomAllreduce::all_gather(int dtype, cudaStream_t stream, const void* input, void* output,
                                 size_t n_shard) {
  const size_t bytes = n_shard * (size_t)dtype_size(dtype);
  if (bytes % 16 != 0)
    throw std::runtime_error("penny custom_ar: all-gather shards must be multiples of 16 bytes");
  const RankData* rd = lookup(stream, input);
  const size_t V = bytes / 16;
  PULL_LAUNCH(pull_all_gather, V);
}

void CustomAllreduce::read_status(uint32_t out[8], bool clear) {
  ckrt(cudaDeviceSynchronize(), "synchronize");
  ckrt(cudaMemcpy(out, self_sg_->status, 32, cudaMemcpyDeviceToHost), "read status");
  if (clear && out[0] != 0) ckrt(cudaMemset(self_sg_->status, 0, 32), "clear status");
}

}  // namespace pull
}  // namespace penny
