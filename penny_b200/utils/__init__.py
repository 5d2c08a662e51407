"""Process setup and measurement helpers.

`initialize_distributed` and `bench_kineto` keep the names of the reference
(penny/utils.py:8-52); `bench_device` is the timing method used for every
number this project reports: CUDA events on the launching stream, warm-up,
an L2 flush before every timed call, and the maximum over ranks.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional

import torch

_GLOBAL_COMM = None
_L2_FLUSH = None


def initialize_distributed(backend: str = "cpu:gloo,cuda:nccl", heap_bytes: Optional[int] = None,
                           init_native: bool = True, config=None):
    """One process per GPU: torch.distributed (gloo for objects, NCCL as the
    baseline) + the native communicator.  Reads torchrun's environment; `config`
    (a PennyConfig, default PennyConfig.from_env()) carries the library's knobs."""
    import torch.distributed as dist

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    nnodes = int(os.environ.get("NNODES", "1"))
    local_size = max(1, world // nnodes)
    local_rank = int(os.environ.get("LOCAL_RANK", rank % local_size))
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
    else:
        backend = "gloo"
    if not dist.is_initialized():
        kw = {}
        if torch.cuda.is_available():
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kw)
    comm = None
    if init_native and torch.cuda.is_available() and world > 1:
        comm = global_communicator(heap_bytes=heap_bytes, config=config)
    return rank, world, comm


def global_communicator(heap_bytes: Optional[int] = None, config=None):
    """The process-wide communicator over the default group (created on first use).
    The native side reads its settings from the environment, so the PennyConfig
    (env + `heap_bytes` override) is exported there before init_with_uid."""
    global _GLOBAL_COMM
    if _GLOBAL_COMM is None:
        import torch.distributed as dist
        from .._ext import ops
        from ..config import PennyConfig
        from ..parallel.comm import Communicator
        cfg = config if config is not None else PennyConfig.from_env(heap_bytes=heap_bytes)
        if config is not None and heap_bytes is not None:
            cfg.heap_bytes = int(heap_bytes)
        if not ops.is_initialized():
            # the same two steps as the reference: unique id from rank 0, init on all
            box = [bytes(ops.get_unique_id()) if dist.get_rank() == 0 else None]
            dist.broadcast_object_list(box, src=0, device="cpu")
            cfg.apply_env()
            ops.init_with_uid(box[0], dist.get_rank(), dist.get_world_size())
        _GLOBAL_COMM = Communicator(ops.global_comm(), emulated=False, owned=False)
        _GLOBAL_COMM.debug_poison = cfg.debug_poison
    return _GLOBAL_COMM


def shutdown():
    global _GLOBAL_COMM
    import torch.distributed as dist
    if _GLOBAL_COMM is not None:
        _GLOBAL_COMM.close()
        _GLOBAL_COMM = None
    from .._ext import ops
    if ops.is_initialized():
        ops.finalize()
    if dist.is_initialized():
        dist.destroy_process_group()


def flush_l2():
    """Overwrites a buffer larger than the 126 MB L2."""
    global _L2_FLUSH
    if _L2_FLUSH is None:
        _L2_FLUSH = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    _L2_FLUSH.zero_()


def bench_device(fn: Callable[[], None], warmup: int = 20, iters: int = 100, flush: bool = True,
                 group=None, sync_ranks: bool = True) -> dict:
    """Device time of `fn` in microseconds: per-call CUDA events, max over ranks.

    Every timed call is preceded (outside the timed interval) by an L2 flush and,
    on several ranks, by a barrier so that all ranks enter the call together –
    otherwise a collective's time would include the skew of the slowest rank."""
    import torch.distributed as dist
    multi = sync_ranks and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        if flush:
            flush_l2()
        if multi:
            torch.cuda.synchronize()
            dist.barrier(group=group)
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    times = torch.tensor([s.elapsed_time(e) * 1e3 for s, e in zip(starts, ends)], dtype=torch.float64)
    if multi:
        t = times.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        times = t.cpu()
    return {"mean_us": times.mean().item(), "median_us": times.median().item(), "min_us": times.min().item(),
            "max_us": times.max().item(), "iters": iters}


def bench_graph(fn: Callable[[], None], inner: int = 10, warmup: int = 5, iters: int = 30, group=None) -> dict:
    """Device time per call (us) with the CPU out of the picture: `inner`
    back-to-back calls are captured in one CUDA graph and the replay is timed
    (max over ranks).  This is what a serving engine pays per call inside its
    decode graph; `bench_device` measures an eager call including its launch."""
    import torch.distributed as dist
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(inner):
            fn()
    for _ in range(warmup):
        g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush_l2()
        if multi:
            torch.cuda.synchronize()
            dist.barrier(group=group)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / inner)
    t = torch.tensor(times, dtype=torch.float64)
    if multi:
        tc = t.cuda()
        dist.all_reduce(tc, op=dist.ReduceOp.MAX, group=group)
        t = tc.cpu()
    return {"mean_us": t.mean().item(), "median_us": t.median().item(), "min_us": t.min().item(), "inner": inner}


def bench_kineto(fn, kernel_name: str, num_tests: int = 30, suppress_kineto_output: bool = False,
                 barrier_comm_profiling: bool = True):
    """Mean device time (us) of the kernels whose name contains `kernel_name`, taken
    from a torch-profiler trace; same contract as the reference's bench_kineto
    (L2 flushed before each call, samples outside 0.5-1.5x the median dropped)."""
    import torch.distributed as dist
    schedule = torch.profiler.schedule(wait=0, warmup=1, active=1, repeat=1)
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA], schedule=schedule) as prof:
        for _ in range(2):
            if barrier_comm_profiling and dist.is_initialized():
                torch.cuda.synchronize()
                dist.barrier()
            for _ in range(num_tests):
                flush_l2()
                fn()
            prof.step()
    times: List[float] = [e.device_time_total for e in prof.profiler.function_events if kernel_name in e.name]
    if not times:
        raise RuntimeError(f"no kernel matching {kernel_name!r} in the trace")
    median = sorted(times)[len(times) // 2]
    kept = [t for t in times if 0.5 < t / median < 1.5]
    return sum(kept) / len(kept)


def bus_bandwidth_gbs(op: str, bytes_per_rank: int, world: int, time_us: float) -> float:
    """NCCL-style bus bandwidth.  all_reduce: bytes = message size; all_gather /
    reduce_scatter: bytes = size of the whole (gathered / scattered) buffer."""
    if time_us <= 0:
        return 0.0
    factor = {"all_reduce": 2.0 * (world - 1) / world, "all_gather": (world - 1) / world,
              "reduce_scatter": (world - 1) / world, "all_to_all": (world - 1) / world, "exchange": 1.0}[op]
    return factor * bytes_per_rank / (time_us * 1e-6) / 1e9
