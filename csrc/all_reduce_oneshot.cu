// One-shot all-reduce kernels (flag and low-latency protocol); body in
// all_reduce_oneshot.cuh.
#include "algos.h"
#include "all_reduce_oneshot.cuh"
#include "launch.cuh"

namespace penny {

cudaError_t launch_all_reduce_oneshot(int dtype, bool ll, const CommCtx& c, const CollArgs* a,
                                      const LaunchCfg& cfg) {
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, PENNY_DISPATCH_WORLD(c.world, NG, return cudaErrorInvalidValue, {
    rc = ll ? launch_body<OneShotLL<T, NG>, CollArgs>(c, a, cfg)
            : launch_body<OneShotFlag<T, NG>, CollArgs>(c, a, cfg);
  }));
  return rc;
}

}  // namespace penny
