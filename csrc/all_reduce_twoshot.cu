// Two-shot all-reduce, reduce-scatter and all-gather kernels; bodies in
// all_reduce_twoshot.cuh.
#include "algos.h"
#include "all_reduce_twoshot.cuh"
#include "launch.cuh"

namespace penny {

cudaError_t launch_all_reduce_twoshot(int dtype, const CommCtx& c, const CollArgs* a,
                                      const LaunchCfg& cfg) {
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, PENNY_DISPATCH_WORLD(c.world, NG, return cudaErrorInvalidValue, {
    rc = launch_body<TwoShot<T, NG>, CollArgs>(c, a, cfg);
  }));
  return rc;
}


cudaError_t launch_reduce_scatter(int dtype, const CommCtx& c, const CollArgs* a,
                                  const LaunchCfg& cfg) {
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, PENNY_DISPATCH_WORLD(c.world, NG, return cudaErrorInvalidValue, {
    rc = launch_body<ReduceScatterPush<T, NG>, CollArgs>(c, a, cfg);
  }));
  return rc;
}

cudaError_t launch_reduce_scatter_pipelined(int dtype, const CommCtx& c, const CollArgs* a,
                                            const LaunchCfg& cfg) {
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, PENNY_DISPATCH_WORLD(c.world, NG, return cudaErrorInvalidValue, {
    rc = launch_body<ReduceScatterPipelined<T, NG>, CollArgs>(c, a, cfg);
  }));
  return rc;
}

cudaError_t launch_all_gather(int dtype, const CommCtx& c, const CollArgs* a,
                              const LaunchCfg& cfg) {
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, PENNY_DISPATCH_WORLD(c.world, NG, return cudaErrorInvalidValue, {
    rc = launch_body<AllGatherPush<T, NG>, CollArgs>(c, a, cfg);
  }));
  return rc;
}

}  // namespace penny
