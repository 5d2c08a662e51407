// Runs every protocol of the host simulator (csrc/sim/host_sim.cpp: the kernels'
// bodies with ranks and blocks as free-running threads) a few times; built with
// -fsanitize=thread by tests/test_cpu_host_sim.py, so a data race between two
// simulated ranks (a flag read that does not order the data it guards, a scratch
// slot reused too early) is reported by ThreadSanitizer and fails the test.
#include <cstdio>

#include "../../csrc/sim/host_sim.cpp"

int main() {
  // ids as in csrc/algos.h and the simulator's extra collectives
  const int algos[] = {0, 1, 2, 3, 4, 5, 7, 16, 17, 18, 19};
  int bad = 0;
  for (int algo : algos)
    for (int world : {2, 4}) {
      const int nnodes = ((algo == 4 || algo == 5) && world == 4) ? 2 : 1;
      double err = 0.0;
      const int rc = penny_sim_run(algo, /*dtype*/ 0, world, /*nblocks*/ 2, /*nthreads*/ 4, /*n*/ 1536, nnodes,
                                   /*routes*/ 2, /*iters*/ 3, /*seed*/ 7u, /*stall_rank*/ -1,
                                   /*timeout_ms*/ 20000, /*in_place*/ 0, &err, nullptr);
      if (rc != 0 || !(err <= 1.0)) {
        std::fprintf(stderr, "algo %d world %d: rc=%d err=%g\n", algo, world, rc, err);
        ++bad;
      }
    }
  std::printf(bad ? "sim_tsan failed\n" : "sim_tsan ok\n");
  return bad ? 1 : 0;
}
