// Argument block shared by every collective body.
#pragma once
#include "pk.h"

namespace penny {

constexpr size_t kNotInHeap = ~(size_t)0;

struct CollArgs {
  const void* in;  // this rank's input (any memory of this rank's GPU, 16-byte aligned)
  void* out;       // this rank's output (16-byte aligned)
  size_t n;        // elements: all-reduce/reduce-scatter = whole input, all-gather = one shard,
                   // all-to-all = one per-peer chunk, exchange = whole buffer
  size_t scratch_off;    // heap offset of the scratch region lent to this call
  size_t scratch_bytes;  // its size
  size_t in_heap_off;    // offset of `in` inside the heap, or kNotInHeap
  size_t out_heap_off;   // offset of `out` inside the heap, or kNotInHeap
  int nnodes;            // virtual node count (double ring, tree, node-aware ring)
  int routes;            // concurrent rings / trees are derived from it
  int peer;              // exchange partner
  uint32_t unit_vecs;    // LL protocol: 16-byte vectors owned by one block
};

// Scratch each algorithm needs for n elements of elem_size bytes on `world`
// ranks (bytes, multiple of 16).  Kept next to the bodies that index it.
PK_HD size_t vecs_for(size_t n, int elem_size) { return ceil_div(n * (size_t)elem_size, 16); }

}  // namespace penny
