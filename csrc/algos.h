// Algorithm ids (the first four keep the numbering of the reference's
// penny_cpp.all_reduce_create, csrc/torch_interface.cpp:82-97) and the dtype /
// world-size dispatch shared by the device launchers and the host simulator.
#pragma once
#include "pk.h"

namespace penny {

enum Algo : int {
  ALGO_RING_STANDARD = 0,
  ALGO_RING_SIMPLE = 1,
  ALGO_ONESHOT = 2,
  ALGO_TWOSHOT = 3,
  ALGO_DOUBLE_RING = 4,
  ALGO_TREE = 5,
  ALGO_NVLS = 6,
  ALGO_ONESHOT_LL = 7,
  ALGO_NVLS_ONESHOT = 8,
  ALGO_AUTO = -1,
  // other collectives (same dispatch machinery)
  OP_REDUCE_SCATTER = 16,
  OP_ALL_GATHER = 17,
  OP_ALL_TO_ALL = 18,
  OP_EXCHANGE = 19,
  OP_REDUCE_SCATTER_PIPELINED = 20,
  OP_ALL_TO_ALL_PIPELINED = 21,
};

inline const char* algo_name(int a) {
  switch (a) {
    case ALGO_RING_STANDARD: return "ring_standard";
    case ALGO_RING_SIMPLE: return "ring_simple";
    case ALGO_ONESHOT: return "oneshot";
    case ALGO_TWOSHOT: return "twoshot";
    case ALGO_DOUBLE_RING: return "double_ring";
    case ALGO_TREE: return "tree";
    case ALGO_NVLS: return "nvls";
    case ALGO_ONESHOT_LL: return "oneshot_ll";
    case ALGO_NVLS_ONESHOT: return "nvls_oneshot";
    case OP_REDUCE_SCATTER: return "reduce_scatter";
    case OP_ALL_GATHER: return "all_gather";
    case OP_ALL_TO_ALL: return "all_to_all";
    case OP_EXCHANGE: return "exchange";
    case OP_REDUCE_SCATTER_PIPELINED: return "reduce_scatter_pipelined";
    case OP_ALL_TO_ALL_PIPELINED: return "all_to_all_pipelined";
    default: return "auto";
  }
}

// Calls F<T>(args...) for the element type named by dt.
#define PENNY_DISPATCH_DTYPE(dt, T, ...)      \
  do {                                        \
    if ((dt) == ::penny::DT_F32) {            \
      using T = float;                        \
      __VA_ARGS__;                            \
    } else if ((dt) == ::penny::DT_F16) {     \
      using T = ::penny::f16_t;               \
      __VA_ARGS__;                            \
    } else {                                  \
      using T = ::penny::bf16_t;              \
      __VA_ARGS__;                            \
    }                                         \
  } while (0)

// Binds a compile-time world size NG in {2,4,6,8}; `bad` runs otherwise.
#define PENNY_DISPATCH_WORLD(world, NG, bad, ...) \
  do {                                            \
    switch (world) {                              \
      case 2: { constexpr int NG = 2; __VA_ARGS__; } break; \
      case 4: { constexpr int NG = 4; __VA_ARGS__; } break; \
      case 6: { constexpr int NG = 6; __VA_ARGS__; } break; \
      case 8: { constexpr int NG = 8; __VA_ARGS__; } break; \
      default: bad;                               \
    }                                             \
  } while (0)

}  // namespace penny
