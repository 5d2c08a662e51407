"""Communicator: the Python face of the symmetric heap and its collectives.

Two kinds, one API:

* ``Communicator.create(group)`` – one process per GPU.  Rank 0 of ``group``
  (any torch.distributed group; gloo is enough) draws a unique id, the id is
  broadcast as an object, and every rank joins the native bootstrap (Unix
  sockets + fd passing) that builds the peer-mapped heap and, when the driver
  allows it, the NVLS multicast mapping.  torch.distributed is not used again.
* ``Communicator.emulated(world)`` – all ranks on ONE GPU, every collective one
  cooperative launch.  Arguments are then lists with one tensor per virtual
  rank.  This is how the multi-rank kernels are tested on a single GPU.

The reference reaches the same point with ``initialize_distributed`` + NVSHMEM
(penny/utils.py:39-52) and per-algorithm objects (csrc/common.h:89-118).
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Union

import torch

from .._ext import ops
from ..config import PennyConfig
from .tuner import Tuner

TensorOrList = Union[torch.Tensor, Sequence[torch.Tensor]]

ALGOS = {
    "auto": ops.ALGO_AUTO,
    "ring_standard": ops.ALGO_RING_STANDARD,
    "ring": ops.ALGO_RING_STANDARD,
    "ring_simple": ops.ALGO_RING_SIMPLE,
    "oneshot": ops.ALGO_ONESHOT,
    "twoshot": ops.ALGO_TWOSHOT,
    "double_ring": ops.ALGO_DOUBLE_RING,
    "tree": ops.ALGO_TREE,
    "nvls": ops.ALGO_NVLS,
    "oneshot_ll": ops.ALGO_ONESHOT_LL,
    "nvls_oneshot": ops.ALGO_NVLS_ONESHOT,
}
ALGO_NAMES = {v: k for k, v in ALGOS.items() if k not in ("ring",)}
PROTOS = {"ll": ops.PROTO_LL, "flag": ops.PROTO_FLAG, "nvls": ops.PROTO_NVLS, "nvls_oneshot": ops.PROTO_NVLS_ONESHOT,
          "ll_twoshot": ops.PROTO_LL_TWOSHOT}

STATUS_NAMES = {
    0: "ok", 1: "timeout in a barrier", 2: "timeout waiting for data", 3: "timeout waiting for a credit",
    4: "timeout waiting for a low-latency line", 5: "timeout waiting for a tile", 6: "self test",
    7: "bad arguments",
}


class PennyTimeoutError(RuntimeError):
    """A device-side wait ran out; ``record`` says who waited for whom."""

    def __init__(self, record: dict):
        self.record = record
        super().__init__(
            f"penny: {STATUS_NAMES.get(record['code'], record['code'])}: rank {record['rank']} "
            f"block {record['block']} waited for rank {record['peer']} "
            f"(want {record['want']}, saw {record['seen']})")


def _algo_id(algo) -> int:
    if isinstance(algo, str):
        if algo not in ALGOS:
            raise ValueError(f"unknown algorithm {algo!r}; one of {sorted(ALGOS)}")
        return ALGOS[algo]
    return int(algo)


class Communicator:
    def __init__(self, handle: int, emulated: bool, owned: bool = True):
        self._h = handle
        self._owned = owned  # False: the extension's global communicator (penny_cpp.finalize frees it)
        self.emulated = emulated
        self.rank = ops.comm_rank(handle)
        self.world_size = ops.comm_world(handle)
        self.views = ops.comm_views(handle)
        # data_ptr of tensors handed out by empty(): symmetric by construction
        self._symmetric = {}
        # PennyConfig.debug_poison: check() also overwrites all scratch with NaN patterns
        self.debug_poison = False
        # measured (op, world, dtype, memory class, size) -> algorithm table; its all-reduce rows
        # also go to the native communicator, so "auto" means the same through every entry point
        self.tuner = Tuner.load()
        self._pick_cache = {}
        self._install_tuning()

    def _install_tuning(self):
        for es, dt in ((2, "bf16"), (4, "fp32")):
            for sym in (False, True):
                rows = self.tuner.rows("all_reduce", self.world_size, dt, sym)
                if not rows:
                    continue
                try:
                    ops.comm_set_tuning(self._h, es, sym, [(-1 if b is None else int(b), ALGOS[a]) for b, a in rows])
                except KeyError:
                    continue  # a table naming an algorithm this build does not have: keep the native rule

    def set_tuner(self, tuner: Tuner):
        """Replaces the algorithm table (e.g. one just built by Tuner.from_sweep)."""
        self.tuner = tuner
        self._pick_cache = {}
        self._install_tuning()

    # ------------------------------------------------------------------ creation
    @classmethod
    def create(cls, group=None, heap_bytes: Optional[int] = None, multicast: Optional[bool] = None,
               heap_mode: Optional[str] = None, timeout_ms: Optional[int] = None,
               config: Optional[PennyConfig] = None) -> "Communicator":
        """One communicator over the ranks of `group` (default: the world group).

        Settings come from `config` (default `PennyConfig.from_env()`); the
        keyword arguments override single fields of it."""
        import torch.distributed as dist

        cfg = config if config is not None else PennyConfig.from_env()
        if heap_bytes is None:
            heap_bytes = cfg.heap_bytes
        if multicast is None:
            multicast = not cfg.disable_nvls
        if heap_mode is None:
            heap_mode = cfg.heap_mode
        if timeout_ms is None:
            timeout_ms = cfg.timeout_ms
        rank = dist.get_rank(group)
        world = dist.get_world_size(group)
        box = [bytes(ops.get_unique_id()) if rank == 0 else None]
        src = dist.get_global_rank(group, 0) if group is not None else 0
        dist.broadcast_object_list(box, src=src, group=group, device="cpu")
        mode = {"auto": 0, "vmm": 1, "ipc": 2}[heap_mode]
        h = ops.comm_create(box[0], rank, world, int(heap_bytes), mode, bool(multicast), int(timeout_ms))
        comm = cls(h, emulated=False)
        comm.debug_poison = cfg.debug_poison
        return comm

    @classmethod
    def emulated(cls, world: int, heap_bytes: int = 256 << 20, timeout_ms: int = 2000,
                 debug_poison: Optional[bool] = None) -> "Communicator":
        """All `world` ranks on ONE GPU (one cooperative launch per collective): for tests and profiling."""
        comm = cls(ops.comm_create_emulated(world, int(heap_bytes), int(timeout_ms)), emulated=True)
        comm.debug_poison = PennyConfig.from_env().debug_poison if debug_poison is None else bool(debug_poison)
        return comm

    def close(self):
        if self._h:
            if self._owned:
                ops.comm_destroy(self._h)
            self._h = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------- queries
    @property
    def has_multicast(self) -> bool:
        return ops.comm_has_multicast(self._h)

    def describe(self) -> str:
        return ops.comm_describe(self._h)

    def heap_free(self) -> int:
        return ops.comm_heap_free(self._h)

    def barrier(self):
        """Host-side barrier over the native bootstrap (no-op when emulated)."""
        ops.comm_barrier(self._h)

    def set_timeout_ms(self, ms: int):
        ops.comm_set_timeout_ms(self._h, int(ms))

    def pick_algo(self, dtype: torch.dtype, numel: int, symmetric: bool = False) -> str:
        """The all-reduce algorithm `algo="auto"` resolves to for this message."""
        forced = os.environ.get("PENNY_ALGO")
        if forced:
            return forced
        dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
        return ALGO_NAMES[ops.comm_pick_algo(self._h, dt, int(numel), bool(symmetric))]

    def _pick(self, op: str, nbytes: int, dtype, symmetric: bool) -> Optional[str]:
        """Table lookup, remembered per (op, size, dtype, memory class): an eager call pays a dict hit."""
        key = (op, nbytes, dtype, symmetric)
        hit = self._pick_cache.get(key, self)
        if hit is self:
            hit = self._pick_cache[key] = self.tuner.pick(op, nbytes, self.world_size, dtype, symmetric,
                                                          self.has_multicast)
        return hit

    def pick_fused_proto(self, rows: int, hidden: int, dtype=torch.bfloat16, symmetric_in: bool = True,
                         symmetric_out: bool = True, alternating_inputs: bool = False) -> str:
        """Transport of fused_all_reduce_rmsnorm(proto="auto"): the measured table when it has an
        entry that these tensors allow, else a handful of rows -> flag-in-data lines, heap tensors ->
        the switch, anything else -> pushes + a flag barrier.
        alternating_inputs: the caller promises that consecutive calls read different input buffers,
        which the one-shot switch transport needs (it has no barrier after the reduction); without
        the promise the table's "nvls_oneshot" rows are served by "nvls"."""
        nbytes = rows * hidden * torch.empty((), dtype=dtype).element_size()
        mc = self.has_multicast and not self.emulated

        def allowed(p):
            return p in ("ll", "flag", "ll_twoshot") or (mc and symmetric_in and (symmetric_out or p == "nvls_oneshot"))
        p = self._pick("fused_norm", nbytes, dtype, symmetric_in)
        if p == "nvls_oneshot" and not alternating_inputs:
            p = "nvls" if rows > 16 else "ll"
        if p in PROTOS and allowed(p):
            return p
        if rows <= 16:
            return "ll"
        return "nvls" if allowed("nvls") else "flag"

    # ------------------------------------------------------------------ tensors
    def empty(self, *shape, dtype=torch.bfloat16):
        """A tensor in the symmetric heap: same offset on every rank, so peers
        (and the NVSwitch) can address it directly.  Every rank must call this in
        the same order.  Emulated: a list with one tensor per virtual rank."""
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = tuple(shape[0])
        ts = ops.comm_empty(self._h, list(shape), dtype)
        for t in ts:
            self._symmetric[t.data_ptr()] = t.numel() * t.element_size()
        return list(ts) if self.emulated else ts[0]

    def is_symmetric(self, t: TensorOrList) -> bool:
        ts = self._as_list(t)
        return all(x.data_ptr() in self._symmetric for x in ts)

    def _as_list(self, t: TensorOrList) -> List[torch.Tensor]:
        if isinstance(t, torch.Tensor):
            ts = [t]
        else:
            ts = list(t)
        if len(ts) != self.views:
            raise ValueError(f"expected {self.views} tensor(s), got {len(ts)}")
        return ts

    def _ret(self, ts: List[torch.Tensor]):
        return ts if self.emulated else ts[0]

    # -------------------------------------------------------------- collectives
    def all_reduce(self, inp: TensorOrList, out: Optional[TensorOrList] = None, algo="auto",
                   blocks: int = 0, threads: int = 0, nnodes: int = 1, routes: int = 0):
        """algo: a name from ALGOS, the reference's ids 0-3, or "auto" (the measured table).

        The switch algorithms take tensors anywhere in device memory: "nvls_oneshot" stages its input
        inside the kernel (one flag exchange, every rank pulls the whole sum; in place is fine);
        "nvls" reduces and multicasts in place for tensors from `empty()`, goes through two staging
        copies for other tensors and, from 256 MiB, runs the copies of piece i + 1 and piece i - 1 on
        side streams under the reduction of piece i."""
        ins = self._as_list(inp)
        outs = self._as_list(out) if out is not None else [torch.empty_like(x) for x in ins]
        if algo == "auto" and os.environ.get("PENNY_ALGO"):
            algo = os.environ["PENNY_ALGO"]
        ops.comm_all_reduce(self._h, ins, outs, _algo_id(algo), blocks, threads, nnodes, routes,
                            self.is_symmetric(ins), self.is_symmetric(outs))
        return self._ret(outs)

    def reduce_scatter(self, inp: TensorOrList, out: Optional[TensorOrList] = None, nvls: Optional[bool] = None,
                       blocks: int = 0, threads: int = 0, pipelined: Optional[bool] = None, algo: str = "auto"):
        """out[numel / world] = this rank's shard of the sum.

        algo: "push" (peers write their slices into the owner's scratch, the owner adds them up),
        "pipelined" (the same, one chunk reduced while the next is on the wire: large shards),
        "nvls" (the switch adds; inputs outside the heap are staged) or "auto" (the measured
        table).  The `nvls=` / `pipelined=` flags of earlier versions still select directly."""
        ins = self._as_list(inp)
        if out is None:
            outs = [torch.empty(x.numel() // self.world_size, dtype=x.dtype, device=x.device) for x in ins]
        else:
            outs = self._as_list(out)
        sym = self.is_symmetric(ins)
        if nvls is not None or pipelined is not None:
            algo = "nvls" if nvls else ("pipelined" if pipelined else "push")
        elif algo == "auto":
            nbytes = ins[0].numel() * ins[0].element_size()
            algo = self._pick("reduce_scatter", nbytes // self.world_size, ins[0].dtype, sym) or "push"
        shard_bytes = ins[0].numel() // self.world_size * ins[0].element_size()
        if algo == "nvls" and (self.emulated or not self.has_multicast or shard_bytes % 16 != 0):
            algo = "push"
        if algo not in ("push", "pipelined", "nvls"):
            raise ValueError(f"unknown reduce-scatter algorithm {algo!r}")
        ops.comm_reduce_scatter(self._h, ins, outs, algo == "nvls", blocks, threads, sym, algo == "pipelined")
        return self._ret(outs)

    def all_gather(self, inp: TensorOrList, out: Optional[TensorOrList] = None, nvls: Optional[bool] = None,
                   blocks: int = 0, threads: int = 0, algo: str = "auto"):
        """out = concatenation of every rank's `inp`.  algo: "push" (every rank writes its shard into
        every peer), "nvls" (one multicast store per vector; needs an output from `empty()` and a
        16-byte-multiple shard) or "auto" (the measured table)."""
        ins = self._as_list(inp)
        if out is None:
            outs = [torch.empty(x.numel() * self.world_size, dtype=x.dtype, device=x.device) for x in ins]
        else:
            outs = self._as_list(out)
        sym = self.is_symmetric(outs)
        nbytes = ins[0].numel() * ins[0].element_size()
        if nvls is not None:
            algo = "nvls" if nvls else "push"
        elif algo == "auto":
            algo = self._pick("all_gather", nbytes, ins[0].dtype, sym) or "push"
            if algo == "nvls" and (self.emulated or not self.has_multicast or not sym or nbytes % 16 != 0):
                algo = "push"
        if algo not in ("push", "nvls"):
            raise ValueError(f"unknown all-gather algorithm {algo!r}")
        ops.comm_all_gather(self._h, ins, outs, algo == "nvls", blocks, threads, sym)
        return self._ret(outs)

    def all_to_all(self, inp: TensorOrList, out: Optional[TensorOrList] = None, blocks: int = 0,
                   threads: int = 0, pipelined: Optional[bool] = None, algo: str = "auto"):
        """out[s * n : (s + 1) * n] = rank s's in[rank * n : (rank + 1) * n].  algo: "push", "pipelined"
        (ordinary output tensors only: one piece is copied out of scratch while the next is on the
        wire) or "auto" (the measured table)."""
        ins = self._as_list(inp)
        outs = self._as_list(out) if out is not None else [torch.empty_like(x) for x in ins]
        sym = self.is_symmetric(outs)
        if pipelined is not None:
            algo = "pipelined" if pipelined else "push"
        elif algo == "auto":
            nbytes = ins[0].numel() // self.world_size * ins[0].element_size()
            algo = self._pick("all_to_all", nbytes, ins[0].dtype, sym) or "push"
        if algo not in ("push", "pipelined"):
            raise ValueError(f"unknown all-to-all algorithm {algo!r}")
        ops.comm_all_to_all(self._h, ins, outs, blocks, threads, sym, algo == "pipelined")
        return self._ret(outs)

    def exchange(self, buf: TensorOrList, peer: Union[int, Sequence[int]], blocks: int = 0, threads: int = 0):
        """In-place pairwise swap.  Every rank must call it; a rank that sits a
        round out passes its own rank as ``peer``."""
        bufs = self._as_list(buf)
        peers = [int(peer)] if isinstance(peer, int) else [int(p) for p in peer]
        ops.comm_exchange(self._h, bufs, peers, blocks, threads)
        return self._ret(bufs)

    def fused_all_reduce_rmsnorm(self, inp: TensorOrList, weight: torch.Tensor, residual: Optional[TensorOrList] = None,
                                 out: Optional[TensorOrList] = None, residual_out: Optional[TensorOrList] = None,
                                 eps: float = 1e-5, proto: str = "ll", blocks: int = 0, threads: int = 0,
                                 pushed: bool = False):
        """out = rmsnorm(all_reduce(inp) + residual) * weight; residual_out = all_reduce(inp) + residual.

        proto: "auto" (the measured table, restricted to what these tensors allow),
        "ll" (flag-in-data pushes, a handful of rows), "ll_twoshot" (rows sharded over the ranks,
        flag-in-data lines to the owner and back; the residual stays sharded), "flag" (pushes + one flag barrier),
        "nvls" (switch reduction, rows sharded over the ranks, result multicast: `inp` and `out`
        must come from `empty()`; each rank keeps the residual of its own rows only) or
        "nvls_oneshot" (every rank pulls all rows switch-reduced: `inp` from `empty()`, and
        consecutive calls must alternate between two input buffers, see csrc/fused_ar_rmsnorm.cu).
        pushed=True ("ll_twoshot" only): the GEMM that produced `inp` was given `fused_norm_push_target`
        and has already written the rows other ranks own into their receive lines."""
        ins = self._as_list(inp)
        outs = self._as_list(out) if out is not None else [torch.empty_like(x) for x in ins]
        res = self._as_list(residual) if residual is not None else []
        if proto == "auto":
            proto = self.pick_fused_proto(ins[0].shape[0], ins[0].shape[1], ins[0].dtype, self.is_symmetric(ins),
                                          self.is_symmetric(outs))
        if residual_out is not None:
            rout = self._as_list(residual_out)
        else:
            rout = res  # in place on the residual stream
        ops.comm_fused_ar_rmsnorm(self._h, ins, res, weight, outs, rout, float(eps), PROTOS[proto],
                                  blocks, threads, self.is_symmetric(ins), int(self.is_symmetric(outs)), bool(pushed))
        return self._ret(outs), (self._ret(rout) if rout else None)

    def fused_norm_push_target(self, rows: int, hidden: int, view: int = 0) -> torch.Tensor:
        """Epilogue target for `ops.gemm_decode(..., push=target)`: the row-parallel linear in front of a
        `fused_all_reduce_rmsnorm(proto="ll_twoshot", pushed=True)` on a [rows, hidden] bf16 tensor then
        writes the rows another rank owns straight into that rank's receive lines (flag-in-data), and the
        all-reduce kernel starts by polling instead of pushing.  Reserves the all-reduce's scratch; ask
        again if another flag-in-data collective with a larger footprint has run in between."""
        return ops.comm_fused_norm_push_target(self._h, int(rows), int(hidden), int(view))

    # ---------------------------------------------------------------------- MoE
    def moe_dispatch(self, x, order, expert_of_sorted, send_off, dst_base, dst_row_of_pair, recv, meta,
                     topk: int, experts: int, blocks: int = 0):
        """Pushes every (token, k) row of `x` to the rank that owns its expert, into
        the symmetric tensors `recv` (rows) and `meta` (return addresses).  The
        routing tables come from penny_b200.models.moe_ep.build_routing."""
        L = self._as_list
        ops.comm_moe_dispatch(self._h, L(x), L(order), L(expert_of_sorted), L(send_off), L(dst_base),
                              L(dst_row_of_pair), L(recv), L(meta), int(topk), int(experts), blocks)

    def moe_combine(self, y, out, topk_ids, gates, meta, dst_row_of_pair, comb, recv_rows, experts: int,
                    blocks: int = 0):
        """Returns the expert outputs `y` to their sources and forms
        out[t] = sum_k gates[t, k] * y[t, k] in the same kernel."""
        L = self._as_list
        rr = [int(recv_rows)] if isinstance(recv_rows, int) else [int(r) for r in recv_rows]
        ops.comm_moe_combine(self._h, L(y), L(out), L(topk_ids), L(gates), L(meta), L(dst_row_of_pair),
                             L(comb), rr, int(experts), blocks)

    def gemm_reduce_scatter(self, a: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None):
        """Row-parallel linear fused with its reduce-scatter (one tcgen05 kernel):
        out[M / world, N] = this rank's row shard of sum_r a_r[M, K_r] @ weight_r[N, K_r]^T."""
        if out is None:
            out = torch.empty(a.shape[0] // self.world_size, weight.shape[0], dtype=a.dtype, device=a.device)
        ops.comm_gemm_rs(self._h, a, weight, out)
        return out

    def all_gather_gemm(self, a_shard: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
                        side_ctas: int = 0):
        """Column-parallel linear fused with the all-gather of its input (one
        tcgen05 kernel): out[M, N] = all_gather(a_shard)[M, K] @ weight[N, K]^T."""
        if out is None:
            out = torch.empty(a_shard.shape[0] * self.world_size, weight.shape[0], dtype=a_shard.dtype,
                              device=a_shard.device)
        ops.comm_ag_gemm(self._h, a_shard, weight, out, side_ctas)
        return out

    def gemm_error(self) -> int:
        """Synchronises; non-zero if a pipeline wait inside a GEMM kernel ran out."""
        return ops.gemm_error()

    # ------------------------------------------------------------------- status
    def status(self, view: int = 0, clear: bool = True) -> dict:
        return dict(ops.comm_status(self._h, view, clear))

    def check(self):
        """Synchronise and raise PennyTimeoutError if any device-side wait ran out.
        With `debug_poison` set it then poisons the scratch (see poison_scratch)."""
        recs = [self.status(v, clear=True) for v in range(self.views)]
        for rec in recs:
            if rec["code"] != 0:
                raise PennyTimeoutError(rec)
        if self.debug_poison:
            self.poison_scratch()

    def poison_scratch(self):
        """Debug aid, collective (every rank calls it): with all ranks idle, fill
        every scratch region with 0xFF bytes, so that a kernel reading scratch that
        nobody wrote in the current call produces NaNs rather than the previous
        call's plausible values."""
        ops.comm_poison_scratch(self._h)

    def wait_selftest(self):
        ops.comm_wait_selftest(self._h)
