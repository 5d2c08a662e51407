// RingSimple all-reduce kernel; body in all_reduce_ring.cuh.
#include "algos.h"
#include "all_reduce_ring.cuh"
#include "launch.cuh"

namespace penny {

cudaError_t launch_all_reduce_ring_simple(int dtype, const CommCtx& c, const CollArgs* a,
                                   const LaunchCfg& cfg) {
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, rc = (launch_body<RingSimple<T>, CollArgs>(c, a, cfg)));
  return rc;
}

}  // namespace penny
