// Runs every protocol of the host simulator (csrc/sim/host_sim.cpp: the kernels'
// bodies with ranks and blocks as free-running threads) on a few sizes and dtypes.
// tests/test_cpu_host_sim.py builds it twice:
//   -fsanitize=thread              a data race between two simulated ranks (a flag read
//                                  that does not order the data it guards, a scratch slot
//                                  reused too early) is reported by ThreadSanitizer;
//   -fsanitize=address,undefined   the simulated heaps are exactly as large as the
//                                  scratch the launchers ask for, so an index that runs
//                                  past a slot, a ragged tail read as a full vector or a
//                                  misaligned vector access is reported.
#include <cstdio>

#include "../../csrc/sim/host_sim.cpp"

int main() {
  // ids as in csrc/algos.h and the simulator's extra collectives
  const int algos[] = {0, 1, 2, 3, 4, 5, 7, 16, 17, 18, 19, 20, 21};
  int bad = 0;
  for (int algo : algos)
    for (int world : {2, 4})
      for (int dtype : {0, 2})                       // fp32, bf16
        for (unsigned long long n : {1ull, 1023ull, 1536ull, 40000ull}) {
          const int nnodes = ((algo == 4 || algo == 5) && world == 4) ? 2 : 1;
          // the partitioned collectives take a per-rank count that world must divide
          const unsigned long long nn = ((algo >= 16 && algo <= 18) || algo == 20) ? n * world : n;
          double err = 0.0;
          const int rc = penny_sim_run(algo, dtype, world, /*nblocks*/ 2, /*nthreads*/ 4, nn, nnodes,
                                       /*routes*/ 2, /*iters*/ 3, /*seed*/ 7u, /*stall_rank*/ -1,
                                       /*timeout_ms*/ 20000, /*in_place*/ 0, &err, nullptr);
          if (rc != 0 || !(err <= 1.0)) {
            std::fprintf(stderr, "algo %d world %d dtype %d n %llu: rc=%d err=%g\n", algo, world, dtype, nn, rc, err);
            ++bad;
          }
        }
  std::printf(bad ? "sim_tsan failed\n" : "sim_tsan ok\n");
  return bad ? 1 : 0;
}
