// Kernel shells around the collective bodies.
//
//   k_real – one rank per GPU: the body runs as rank c.rank.
//   k_emu  – all ranks on ONE GPU in one cooperative launch (gridDim.y = world,
//            virtual rank = blockIdx.y).  Blocks of different virtual ranks
//            wait on one another, so they must all be resident at once; a
//            cooperative launch guarantees that or fails up front.  This is how
//            the multi-rank protocols are tested on a single GPU – separate
//            launches (or processes) that spin on each other may never be
//            scheduled together.
#pragma once
#include <cuda_runtime.h>

#include "coll_args.h"
#include "pdl.h"

namespace penny {

struct LaunchCfg {
  int blocks;
  int threads;
  cudaStream_t stream;
  int emu_world;  // 0: real launch; >0: emulate this many ranks on the current GPU
  // real launches only: programmatic stream serialization, i.e. the kernel may become
  // resident while its predecessor still runs; it waits for it before touching anything
  bool pdl = false;
};

template <class Args>
struct EmuArgs {
  Args a[kMaxRanks];
};

template <class Body, class Args>
__global__ void __launch_bounds__(512) k_real(const CommCtx c, const Args a) {
  pdl_launch_dependents();
  pdl_wait();  // before the call counter is read and anything of the predecessor is touched
  const Blk b{(int)blockIdx.x, (int)gridDim.x, (int)blockDim.x};
  Body::run(c, c.rank, a, b);
}

template <class Body, class Args>
__global__ void __launch_bounds__(512) k_emu(const CommCtx c0, const EmuArgs<Args> ea) {
  CommCtx c = c0;
  c.rank = (int)blockIdx.y;
  c.status = reinterpret_cast<uint32_t*>(c.heap[c.rank] + kStatusOffset);
  const Blk b{(int)blockIdx.x, (int)gridDim.x, (int)blockDim.x};
  Body::run(c, c.rank, ea.a[c.rank], b);
}

// args: one entry (real) or emu_world entries (emulated).
template <class Body, class Args>
cudaError_t launch_body(const CommCtx& c, const Args* args, const LaunchCfg& cfg) {
  if (cfg.blocks < 1 || cfg.blocks > kMaxBlocks || cfg.threads < 32 || cfg.threads > 512)
    return cudaErrorInvalidConfiguration;
  if (cfg.emu_world <= 0) {
    return launch_kernel_ex(k_real<Body, Args>, dim3(cfg.blocks), dim3(cfg.threads), 0, cfg.stream, cfg.pdl, 1, c,
                            args[0]);
  }
  EmuArgs<Args> ea;
  for (int r = 0; r < cfg.emu_world; ++r) ea.a[r] = args[r];
  CommCtx cc = c;
  void* params[2] = {(void*)&cc, (void*)&ea};
  dim3 grid(cfg.blocks, cfg.emu_world, 1);
  return cudaLaunchCooperativeKernel((const void*)k_emu<Body, Args>, grid, dim3(cfg.threads),
                                     params, 0, cfg.stream);
}

// Entry points, one per .cu file of the same name.
cudaError_t launch_all_reduce_oneshot(int dtype, bool ll, const CommCtx& c, const CollArgs* a,
                                      const LaunchCfg& cfg);
cudaError_t launch_all_reduce_twoshot(int dtype, const CommCtx& c, const CollArgs* a,
                                      const LaunchCfg& cfg);
cudaError_t launch_reduce_scatter(int dtype, const CommCtx& c, const CollArgs* a,
                                  const LaunchCfg& cfg);
cudaError_t launch_reduce_scatter_pipelined(int dtype, const CommCtx& c, const CollArgs* a,
                                            const LaunchCfg& cfg);
cudaError_t launch_all_gather(int dtype, const CommCtx& c, const CollArgs* a,
                              const LaunchCfg& cfg);
cudaError_t launch_all_reduce_ring_simple(int dtype, const CommCtx& c, const CollArgs* a,
                                          const LaunchCfg& cfg);
cudaError_t launch_all_reduce_ring_standard(int dtype, const CommCtx& c, const CollArgs* a,
                                            const LaunchCfg& cfg);
cudaError_t launch_all_reduce_double_ring(int dtype, const CommCtx& c, const CollArgs* a,
                                          const LaunchCfg& cfg);
cudaError_t launch_all_reduce_tree(int dtype, const CommCtx& c, const CollArgs* a,
                                   const LaunchCfg& cfg);
cudaError_t launch_exchange(int dtype, const CommCtx& c, const CollArgs* a, const LaunchCfg& cfg);
cudaError_t launch_all_to_all(int dtype, const CommCtx& c, const CollArgs* a,
                              const LaunchCfg& cfg);
cudaError_t launch_all_to_all_pipelined(int dtype, const CommCtx& c, const CollArgs* a,
                                        const LaunchCfg& cfg);
// NVLS (multimem) family: real launches only, c.mc must be set, tensors in the heap.
// kind: which switch all-reduce kernel
enum { NVLS_TWOSHOT = 0, NVLS_ONESHOT = 1 };
size_t nvls_oneshot_scratch(size_t n, int elem_size);  // scratch bytes of NVLS_ONESHOT
cudaError_t launch_all_reduce_nvls(int dtype, int kind, const CommCtx& c, const CollArgs* a,
                                   const LaunchCfg& cfg);
cudaError_t launch_reduce_scatter_nvls(int dtype, const CommCtx& c, const CollArgs* a,
                                       const LaunchCfg& cfg);
cudaError_t launch_all_gather_nvls(int dtype, const CommCtx& c, const CollArgs* a,
                                   const LaunchCfg& cfg);
// A wait on a flag that nobody sets: exercises the bounded-wait / status path.
cudaError_t launch_wait_selftest(const CommCtx& c, const LaunchCfg& cfg);

}  // namespace penny
