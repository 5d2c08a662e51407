// Host-side C++ check of the schedule math that the device kernels run
// (csrc/schedule.h, csrc/gemm_tile_order.h): compiled with g++ and executed by
// tests/test_cpu_schedule.py.  Exits non-zero at the first violated property.
//
// The reference has no tests; its only host-side artefact is
// extra/ring_visualize.py, which prints the rings for a human to inspect.
#include <cstdio>
#include <cstdlib>
#include <set>
#include <utility>
#include <vector>

#include "../../csrc/gemm_tile_order.h"
#include "../../csrc/schedule.h"

#define CHECK(cond, ...)                                  \
  do {                                                    \
    if (!(cond)) {                                        \
      std::fprintf(stderr, "FAILED %s:%d: ", __FILE__, __LINE__); \
      std::fprintf(stderr, __VA_ARGS__);                  \
      std::fprintf(stderr, "\n");                         \
      std::exit(1);                                       \
    }                                                     \
  } while (0)

using namespace penny;

// Every route of every world size is a Hamiltonian ring and pos_of inverts rank_at.
static void rings() {
  for (int world : {2, 3, 4, 6, 8})
    for (int nnodes : {1, 2, 4}) {
      if (world % nnodes != 0 || (nnodes > 1 && world / nnodes < 2)) continue;
      for (int route = 0; route < kMaxRoutes; ++route) {
        std::set<int> seen;
        for (int pos = 0; pos < world; ++pos) {
          const int r = ring_rank_at(world, nnodes, route, pos);
          CHECK(r >= 0 && r < world, "rank out of range world=%d nnodes=%d route=%d", world, nnodes, route);
          CHECK(seen.insert(r).second, "rank twice in a ring world=%d nnodes=%d route=%d", world, nnodes, route);
          CHECK(ring_pos_of(world, nnodes, route, r) == pos, "pos_of != inverse world=%d route=%d", world, route);
        }
      }
    }
}

// Ring reduce-scatter + all-gather: what position p sends at step s is what p+1
// receives; after n-1 reduce steps every chunk has visited every position once,
// and after n-1 gather steps every position holds every chunk.
static void ring_chunks() {
  for (int n = 2; n <= 8; ++n) {
    for (int s = 0; s < n - 1; ++s)
      for (int p = 0; p < n; ++p) {
        CHECK(ring_rs_send_chunk(n, p, s) == ring_rs_recv_chunk(n, (p + 1) % n, s), "rs pairing n=%d", n);
        CHECK(ring_ag_send_chunk(n, p, s) == ring_ag_recv_chunk(n, (p + 1) % n, s), "ag pairing n=%d", n);
      }
    for (int chunk = 0; chunk < n; ++chunk) {
      // contributions[p]: how many ranks' data position p's copy of `chunk` holds
      std::vector<int> contrib(n, 1);
      for (int s = 0; s < n - 1; ++s) {
        const std::vector<int> before = contrib;  // all positions send at the same time
        for (int p = 0; p < n; ++p)
          if (ring_rs_recv_chunk(n, p, s) == chunk) contrib[p] = before[(p + n - 1) % n] + 1;
      }
      int owners = 0;
      for (int p = 0; p < n; ++p) owners += contrib[p] == n;
      CHECK(owners == 1, "chunk %d fully reduced at %d positions (n=%d)", chunk, owners, n);
    }
    for (int p = 0; p < n; ++p) {
      std::set<int> have;
      have.insert(ring_ag_send_chunk(n, p, 0));  // its own reduced chunk
      for (int s = 0; s < n - 1; ++s) have.insert(ring_ag_recv_chunk(n, p, s));
      CHECK((int)have.size() == n, "position %d ends with %zu chunks (n=%d)", p, have.size(), n);
    }
  }
}

static void spans_and_trees() {
  for (size_t V : {0ul, 1ul, 7ul, 1023ul, 4096ul, 1048577ul})
    for (int parts = 1; parts <= 9; ++parts) {
      size_t covered = 0, prev_end = 0;
      for (int i = 0; i < parts; ++i) {
        Span sp = split_span(V, parts, i);
        CHECK(sp.begin == prev_end || sp.begin == V, "gap in split_span V=%zu parts=%d", V, parts);
        CHECK(sp.end >= sp.begin && sp.end <= V, "bad span");
        covered += sp.end - sp.begin;
        prev_end = sp.end;
      }
      CHECK(covered == V, "split_span covers %zu of %zu", covered, V);
    }
  for (int gpn = 1; gpn <= 8; ++gpn)
    for (int tree = 0; tree < 2; ++tree) {
      std::set<int> seen;
      for (int j = 0; j < gpn; ++j) {
        const int l = tree_local_at(gpn, tree, j);
        CHECK(l >= 0 && l < gpn && seen.insert(l).second, "tree chain gpn=%d tree=%d", gpn, tree);
        CHECK(tree_pos_of(gpn, tree, l) == j, "tree_pos_of gpn=%d", gpn);
      }
    }
}

// GEMM tiles: single-CTA order is a bijection; the CTA-pair work list (with the
// K-split last wave) computes every K step of every pair tile exactly once.
static void gemm_tiles() {
  using namespace penny::sm100;
  const int shapes[][2] = {{1, 1}, {7, 3}, {32, 14}, {33, 5}, {64, 32}, {13, 11}};
  for (auto& sh : shapes)
    for (int group : {0, 6, 16})
      for (int m_fastest : {0, 1}) {
        GemmShape s{0, 0, 0, sh[0], sh[1], 0, sh[0] * sh[1], m_fastest, group};
        std::set<std::pair<int, int>> seen;
        for (int t = 0; t < s.num_tiles; ++t) {
          int m, n;
          decode_tile(s, t, m, n);
          CHECK(m >= 0 && m < sh[0] && n >= 0 && n < sh[1], "tile out of range");
          CHECK(seen.insert({m, n}).second, "tile (%d,%d) twice", m, n);
        }
        for (int num_kb : {4, 24, 64})
          for (int max_split : {1, 4, 8}) {
            GemmShape p = s;
            const int npairs = 74;
            plan_split_tail(p, npairs, num_kb, max_split);
            std::set<std::pair<int, int>> steps;
            for (int pair = 0; pair < npairs; ++pair) {
              PairWork w;
              for (int it = 0; pair_work(p, num_kb, pair, npairs, it, w); ++it)
                for (int kb = w.kb0; kb < w.kb1; ++kb)
                  CHECK(steps.insert({w.tile, kb}).second, "K step (%d,%d) twice", w.tile, kb);
            }
            CHECK((int)steps.size() == pair_tile_count(p) * num_kb, "%zu of %d K steps covered", steps.size(),
                  pair_tile_count(p) * num_kb);
          }
      }
}

int main() {
  rings();
  ring_chunks();
  spans_and_trees();
  gemm_tiles();
  std::printf("schedule_test ok\n");
  return 0;
}
