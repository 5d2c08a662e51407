// Pairwise exchange and all-to-all kernels; bodies in exchange.cuh.  Also the
// bounded-wait self test.
#include "algos.h"
#include "exchange.cuh"
#include "launch.cuh"

namespace penny {

cudaError_t launch_exchange(int dtype, const CommCtx& c, const CollArgs* a, const LaunchCfg& cfg) {
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, rc = (launch_body<ExchangePair<T>, CollArgs>(c, a, cfg)));
  return rc;
}

cudaError_t launch_all_to_all(int dtype, const CommCtx& c, const CollArgs* a,
                              const LaunchCfg& cfg) {
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, PENNY_DISPATCH_WORLD(c.world, NG, return cudaErrorInvalidValue, {
    rc = launch_body<AllToAll<T, NG>, CollArgs>(c, a, cfg);
  }));
  return rc;
}

cudaError_t launch_all_to_all_pipelined(int dtype, const CommCtx& c, const CollArgs* a,
                                        const LaunchCfg& cfg) {
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, PENNY_DISPATCH_WORLD(c.world, NG, return cudaErrorInvalidValue, {
    rc = launch_body<AllToAllPipelined<T, NG>, CollArgs>(c, a, cfg);
  }));
  return rc;
}

// Waits on a private flag word that nothing ever sets, with the communicator's
// timeout.  The wait must run out, record ST_TIMEOUT_SELFTEST in the status
// words and return: this is the only way a timeout is provoked on a GPU.
struct WaitSelfTest {
  static __device__ void run(const CommCtx& c, int rank, const CollArgs&, const Blk& b) {
    if (threadIdx.x == 0) {
      const u64* p = &pad_of(c, rank)->flag[CH_FUSED][kMaxBlocks - 1][kMaxRanks - 1];
      wait_flag_ge(p, ~0ull, c, ST_TIMEOUT_SELFTEST, rank, b.bid);
    }
  }
};

cudaError_t launch_wait_selftest(const CommCtx& c, const LaunchCfg& cfg) {
  CollArgs a[kMaxRanks];
  memset(a, 0, sizeof(a));
  return launch_body<WaitSelfTest, CollArgs>(c, a, cfg);
}

}  // namespace penny
