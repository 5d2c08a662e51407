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

}  // namespace sm100
}  // namespace penny
