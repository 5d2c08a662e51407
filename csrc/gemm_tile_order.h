// Which tile a persistent GEMM CTA (or CTA pair) works on at each step: plain
// index arithmetic shared by the device kernels and the host-side checks
// (the host simulator library exports it for the CPU tests).
#pragma once

#if defined(__CUDACC__)
#define PENNY_TILE_HD __host__ __device__ __forceinline__
#else
#define PENNY_TILE_HD inline
#endif

namespace penny {
namespace sm100 {

struct GemmShape {
  int M, N, K;
  int tiles_m, tiles_n;
  int m_rot;      // row-block rotation: tile row r works on block (r + m_rot) % tiles_m
  int num_tiles;
  int m_fastest;  // 1: consecutive tiles walk down M (share a B tile); 0: walk along N
  // > 0 (with m_fastest = 1): tiles are handed out in bands of `group_m` row
  // blocks, M fastest inside a band, so that the tiles in flight at one time
  // cover a square-ish patch of C and A's band stays in L2 from wave to wave
  int group_m;
  // CTA-pair kernel only.  split_s > 1: the pair tiles from split_first on (the
  // ragged last wave) are each cut into split_s ranges of K steps that different
  // pairs compute at the same time; partial sums go through split_ws (fp32) and
  // the last pair to finish a tile adds them up and runs the epilogue.
  int split_first = 0;
  int split_s = 0;
  float* split_ws = nullptr;           // [items][2 CTAs][64 column vectors][128 rows] float4
  unsigned* split_counters = nullptr;  // [tail tiles][2 CTAs], zero between launches
};

// Tile index -> (row index before rotation, column block) for `rows_m` rows
// (row blocks, or row-block pairs in the CTA-pair kernel) and band height `gm`
// in the same unit.  A bijection from [0, rows_m * tiles_n) onto the grid.
PENNY_TILE_HD void tile_order(const GemmShape& s, int tile, int rows_m, int gm, int& m_raw, int& n_blk) {
  if (!s.m_fastest) {
    m_raw = tile / s.tiles_n;
    n_blk = tile % s.tiles_n;
  } else if (gm <= 0 || gm >= rows_m) {
    m_raw = tile % rows_m;
    n_blk = tile / rows_m;
  } else {
    const int per_group = gm * s.tiles_n;
    const int g = tile / per_group, in_g = tile - g * per_group;
    const int first = g * gm;
    const int h = (rows_m - first < gm) ? rows_m - first : gm;
    m_raw = first + in_g % h;
    n_blk = in_g / h;
  }
}

// Single-CTA kernel: tile -> (row block, column block).
PENNY_TILE_HD void decode_tile(const GemmShape& s, int tile, int& m_blk, int& n_blk) {
  int m_raw;
  tile_order(s, tile, s.tiles_m, s.group_m, m_raw, n_blk);
  m_blk = (m_raw + s.m_rot) % s.tiles_m;
}

// CTA-pair kernel: a pair tile is two vertically adjacent row blocks; CTA `r`
// (0 or 1) of the pair owns row block 2 * pair_row + r, which may be == tiles_m
// (no such rows) when tiles_m is odd.  m_rot must be even.
PENNY_TILE_HD int pair_rows(const GemmShape& s) { return (s.tiles_m + 1) >> 1; }
PENNY_TILE_HD int pair_tile_count(const GemmShape& s) { return pair_rows(s) * s.tiles_n; }
PENNY_TILE_HD void decode_pair_tile(const GemmShape& s, int tile, int r, int& m_blk, int& n_blk) {
  int pm_raw;
  const int rows = pair_rows(s);
  tile_order(s, tile, rows, s.group_m >> 1, pm_raw, n_blk);
  m_blk = 2 * ((pm_raw + (s.m_rot >> 1)) % rows) + r;
}

// One unit of work of a CTA pair: K steps [kb0, kb1) of pair tile `tile`;
// seg is the index of the range within a split tile (0 when not split).
struct PairWork {
  int tile, kb0, kb1, seg;
};

// Decides the split of the last, ragged wave for a grid of `npairs` pairs (all
// of them resident).  Leaves split_s = 1 when there is nothing to gain.
PENNY_TILE_HD void plan_split_tail(GemmShape& s, int npairs, int num_kb, int max_split) {
  const int total = pair_tile_count(s);
  const int full = (total / npairs) * npairs, rest = total - full;
  s.split_first = total;
  s.split_s = 1;
  if (rest == 0) return;
  int S = npairs / rest;
  if (S > max_split) S = max_split;
  while (S > 1 && num_kb < 4 * S) --S;  // at least four K steps per range
  if (S < 2) return;
  s.split_first = full;
  s.split_s = S;
}

// The it-th unit of pair `pair` (of npairs); false when it has no more.
PENNY_TILE_HD bool pair_work(const GemmShape& s, int num_kb, int pair, int npairs, int it, PairWork& w) {
  const int total = pair_tile_count(s);
  const int first = (s.split_s > 1) ? s.split_first : total;
  const int t = pair + it * npairs;
  if (t < first) {
    w.tile = t; w.kb0 = 0; w.kb1 = num_kb; w.seg = 0;
    return true;
  }
  if (s.split_s <= 1) return false;
  const int j = t - first;
  if (j >= npairs || j >= (total - first) * s.split_s) return false;
  w.tile = first + j / s.split_s;
  w.seg = j % s.split_s;
  w.kb0 = (int)((long long)w.seg * num_kb / s.split_s);
  w.kb1 = (int)((long long)(w.seg + 1) * num_kb / s.split_s);
  return true;
}

}  // namespace sm100
}  // namespace penny
