"""Schedule math and the host protocol simulator, reached through ctypes.

``libpenny_sim.so`` is plain C++ built from the same headers the kernels use
(csrc/schedule.h, csrc/*.cuh with PENNY_HOST_SIM), so what is tested here is the
code that runs on the GPU, not a Python restatement of it.  The reference has a
Python replay of one schedule only (extra/ring_visualize.py).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import List, Tuple

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_LIB = None

ALGO_IDS = {
    "ring_standard": 0, "ring_simple": 1, "oneshot": 2, "twoshot": 3, "double_ring": 4, "tree": 5,
    "oneshot_ll": 7, "reduce_scatter": 16, "all_gather": 17, "all_to_all": 18, "exchange": 19,
    "reduce_scatter_pipelined": 20, "all_to_all_pipelined": 21,
}
DTYPE_IDS = {"float32": 0, "float16": 1, "bfloat16": 2}


def sim_lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    path = os.path.join(_ROOT, "libpenny_sim.so")
    src = os.path.join(_ROOT, "csrc", "sim", "host_sim.cpp")
    if not os.path.exists(path):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", "-o", path, src])
    lib = ctypes.CDLL(path)
    lib.penny_sim_run.argtypes = ([ctypes.c_int] * 5 + [ctypes.c_ulonglong] + [ctypes.c_int] * 3 + [ctypes.c_uint]
                                  + [ctypes.c_int] * 3 + [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_uint)])
    lib.penny_sim_run.restype = ctypes.c_int
    for name in ("penny_sched_ring_rank_at", "penny_sched_ring_stride", "penny_sched_ring_rs_send_chunk",
                 "penny_sched_ring_rs_recv_chunk", "penny_sched_ring_ag_send_chunk",
                 "penny_sched_ring_ag_recv_chunk", "penny_sched_tree_local_at"):
        getattr(lib, name).restype = ctypes.c_int
    _LIB = lib
    return lib


def simulate(algo: str, dtype: str = "float32", world: int = 2, nblocks: int = 4, nthreads: int = 8,
             n: int = 4096, nnodes: int = 1, routes: int = 1, iters: int = 3, seed: int = 1,
             stall_rank: int = -1, timeout_ms: int = 5000, in_place: bool = False):
    """Runs `iters` back-to-back calls on `world` simulated ranks.

    Returns (failed_ranks, worst_error_over_allowed, status_words_per_rank)."""
    lib = sim_lib()
    err = ctypes.c_double(0.0)
    words = lib.penny_status_words()
    st = (ctypes.c_uint * (words * 8))()
    rc = lib.penny_sim_run(ALGO_IDS[algo], DTYPE_IDS[dtype], world, nblocks, nthreads, n, nnodes, routes, iters,
                           seed, stall_rank, timeout_ms, int(in_place), ctypes.byref(err), st)
    status = [list(st[r * words:(r + 1) * words]) for r in range(world)]
    return rc, err.value, status


def ring_order(world: int, nnodes: int = 1, route: int = 0) -> List[int]:
    lib = sim_lib()
    return [lib.penny_sched_ring_rank_at(world, nnodes, route, p) for p in range(world)]


def ring_stride(world: int, route: int) -> int:
    return sim_lib().penny_sched_ring_stride(world, route)


def ring_step_chunks(n: int, pos: int, step: int) -> Tuple[int, int, bool]:
    """(send_chunk, recv_chunk, is_reduce_step) of ring position `pos` at step 0..2(n-1)-1."""
    lib = sim_lib()
    if step < n - 1:
        return lib.penny_sched_ring_rs_send_chunk(n, pos, step), lib.penny_sched_ring_rs_recv_chunk(n, pos, step), True
    s = step - (n - 1)
    return lib.penny_sched_ring_ag_send_chunk(n, pos, s), lib.penny_sched_ring_ag_recv_chunk(n, pos, s), False


def tree_chain(gpn: int, tree: int) -> List[int]:
    """Local ranks of chain-tree `tree` from the far leaf to the root."""
    lib = sim_lib()
    return [lib.penny_sched_tree_local_at(gpn, tree, j) for j in range(gpn)]


def split_span(total: int, parts: int, i: int) -> Tuple[int, int]:
    lib = sim_lib()
    b = ctypes.c_ulonglong(0)
    e = ctypes.c_ulonglong(0)
    lib.penny_sched_split_span(ctypes.c_ulonglong(total), parts, i, ctypes.byref(b), ctypes.byref(e))
    return b.value, e.value


def gemm_tile_at(tiles_m: int, tiles_n: int, tile: int, m_rot: int = 0, m_fastest: int = 1, group_m: int = 0,
                 pair_rank: int = -1) -> Tuple[int, int, int]:
    """(row block, column block, tiles in the grid) that the persistent tcgen05 GEMM
    gives to step `tile`: the single-CTA kernel for pair_rank < 0, CTA 0 / 1 of a
    CTA pair otherwise.  Same code as the device kernels (csrc/gemm_tile_order.h)."""
    lib = sim_lib()
    m, n = ctypes.c_int(0), ctypes.c_int(0)
    total = lib.penny_gemm_tile_at(tiles_m, tiles_n, m_rot, m_fastest, group_m, pair_rank, tile,
                                   ctypes.byref(m), ctypes.byref(n))
    return m.value, n.value, total


def gemm_pair_work(tiles_m: int, tiles_n: int, npairs: int, num_kb: int, pair: int, it: int, max_split: int = 8):
    """The it-th work unit of CTA pair `pair`: dict(tile, kb0, kb1, seg, split_s, split_first) or None.
    The ragged last wave of pair tiles is split along K over the idle pairs (csrc/gemm_tile_order.h)."""
    lib = sim_lib()
    out = (ctypes.c_int * 6)()
    ok = lib.penny_gemm_pair_work(tiles_m, tiles_n, npairs, num_kb, max_split, pair, it, out)
    if not ok:
        return None
    return dict(zip(("tile", "kb0", "kb1", "seg", "split_s", "split_first"), list(out)))


def decode_plan(num_kb: int, splits: int, r: int, bt: int = 64):
    """K range and reduction layout of CTA `r` in a cluster of `splits` of the decode GEMM
    (csrc/decode_gemm_plan.h): dict(kb0, kb1, slice, recv_floats)."""
    lib = sim_lib()
    out = (ctypes.c_longlong * 4)()
    lib.penny_decode_plan(num_kb, splits, r, bt, out)
    return dict(zip(("kb0", "kb1", "slice", "recv_floats"), [int(v) for v in out]))


def decode_recv_slot(src: int, dst: int) -> int:
    return sim_lib().penny_decode_recv_slot(src, dst)


def decode_choose_splits(tiles: int, num_kb: int, sms: int = 148, gpc_sms: int = 18) -> int:
    """Cluster size the decode GEMM picks for `tiles` weight tiles of 128 rows and `num_kb` K steps of
    64 on a GPU of `sms` SMs in GPCs of `gpc_sms` (the launcher uses the occupancy API's figure)."""
    return sim_lib().penny_decode_choose_splits(tiles, num_kb, sms, gpc_sms)
