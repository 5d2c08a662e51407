// Work split of the weight-streaming ("skinny") GEMM used for decode batches:
// out[B, N] = x[B, K] * W[N, K]^T with B <= 128.  The weight matrix is cut into
// tiles of 128 rows and every tile into K steps of 64 columns; the (tile, K step)
// units are dealt out to the CTAs as equal contiguous ranges (stream-K), so every
// SM streams the same number of weight bytes whatever N and K are.  A tile whose
// K steps are shared by several CTAs is summed by the CTA that finishes last.
//
// Plain index arithmetic, shared by the kernel and the CPU tests.
#pragma once

#if defined(__CUDACC__)
#define PENNY_SKINNY_HD __host__ __device__ __forceinline__
#else
#define PENNY_SKINNY_HD inline
#endif

namespace penny {
namespace sm100 {

struct SkinnyPlan {
  int tiles;    // ceil(N / 128)
  int num_kb;   // ceil(K / 64)
  int ctas;     // grid size
  long long units() const { return (long long)tiles * num_kb; }
};

// First unit of CTA c; CTA c owns [begin(c), begin(c + 1)).
PENNY_SKINNY_HD long long skinny_begin(const SkinnyPlan& p, int c) {
  return (long long)c * ((long long)p.tiles * p.num_kb) / p.ctas;
}
// The CTA whose range contains unit u.
PENNY_SKINNY_HD int skinny_owner(const SkinnyPlan& p, long long u) {
  const long long U = (long long)p.tiles * p.num_kb;
  int c = (int)((u * p.ctas) / U);
  if (c >= p.ctas) c = p.ctas - 1;
  while (c + 1 < p.ctas && skinny_begin(p, c + 1) <= u) ++c;
  while (c > 0 && skinny_begin(p, c) > u) --c;
  return c;
}

struct SkinnySeg {
  int tile, kb0, kb1;  // K steps [kb0, kb1) of `tile`
  int c_lo, c_hi;      // the CTAs that share the tile (c_lo == c_hi: this CTA has all of it)
  int slot;            // which of this CTA's two partial slots it uses (0: its first tile, 1: its last)
};

// The i-th segment of CTA c (i = 0, 1, ...); false when the CTA has no more.
// `cursor` carries the position between calls: start it at skinny_begin(p, c).
PENNY_SKINNY_HD bool skinny_next(const SkinnyPlan& p, int c, long long& cursor, SkinnySeg& s) {
  const long long end = skinny_begin(p, c + 1);
  if (cursor >= end) return false;
  s.tile = (int)(cursor / p.num_kb);
  s.kb0 = (int)(cursor % p.num_kb);
  const long long left = end - cursor;
  s.kb1 = (left < (long long)(p.num_kb - s.kb0)) ? s.kb0 + (int)left : p.num_kb;
  const long long u0 = (long long)s.tile * p.num_kb;
  s.c_lo = skinny_owner(p, u0);
  s.c_hi = skinny_owner(p, u0 + p.num_kb - 1);
  s.slot = (s.tile == (int)(skinny_begin(p, c) / p.num_kb)) ? 0 : 1;
  cursor += s.kb1 - s.kb0;
  return true;
}

// Slot that CTA c used for its part of `tile` (for the CTA that adds the parts up).
PENNY_SKINNY_HD int skinny_slot_of(const SkinnyPlan& p, int c, int tile) {
  return (tile == (int)(skinny_begin(p, c) / p.num_kb)) ? 0 : 1;
}

}  // namespace sm100
}  // namespace penny
