// Tree all-reduce kernel; body in all_reduce_tree.cuh.
#include "algos.h"
#include "all_reduce_tree.cuh"
#include "launch.cuh"

namespace penny {

cudaError_t launch_all_reduce_tree(int dtype, const CommCtx& c, const CollArgs* a,
                                   const LaunchCfg& cfg) {
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, rc = (launch_body<TreeAllReduce<T>, CollArgs>(c, a, cfg)));
  return rc;
}

}  // namespace penny
