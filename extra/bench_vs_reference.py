"""Times the UNMODIFIED reference (the NVSHMEM build installed under baseline/_ref) on this box, with
the event timing of this repository's sweeps, so that the two can be put side by side.

    torchrun --nproc-per-node 8 extra/bench_vs_reference.py [--out ref.jsonl] [--skip-algos]

Nothing of this repository's package is imported: the process sees baseline/_ref only.
  part 1  the reference's drop-in class - `CustomAllreduce.custom_all_reduce /
          custom_reduce_scatter / custom_all_gather` (penny/custom_all_reduce.py:250-349) - eager
          and replayed from a CUDA graph captured under its `capture()`, 1 KiB - 4 MiB;
  part 2  `penny_cpp.all_reduce_create / all_reduce_run` for the reference's algorithms 0-3
          (ring_standard, ring_simple, oneshot, twoshot; csrc/torch_interface.cpp:82-112) on fp16,
          over a reduced grid of its packet x block x routes search with the divisibility filters
          of its own harness (extra/benchmark_allreduce.py:62-89), best configuration per size.
Timing of every point: warm-up, then per-call CUDA events, L2 flushed (256 MiB write) and ranks
aligned before every timed call, median over calls, max over ranks.  The reference's device waits
have no bound: a watchdog ends the process (exit code 3, record "unavailable") if one configuration
does not finish in time, and later parts are then not run.
"""
import argparse
import json
import os
import sys
import threading

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
sys.path = [REF] + [p for p in sys.path if os.path.abspath(p or ".") not in (ROOT, os.path.join(ROOT, "extra"))]
os.environ.setdefault("NNODES", "1")
os.environ.setdefault("NVSHMEM_REMOTE_TRANSPORT", "none")
os.environ.setdefault("NVSHMEM_DISABLE_NVLS", "1")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

ALGO_NAMES = {0: "ring_standard", 1: "ring_simple", 2: "oneshot", 3: "twoshot"}
_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def timed(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    t = torch.tensor(sorted(ts)[len(ts) // 2], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def timed_graph(fn, inner, car, warmup=5, iters=30):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with car.capture():
        with torch.cuda.graph(g):
            for _ in range(inner):
                fn()
    return timed(g.replay, warmup, iters) / inner


class Watchdog:
    def __init__(self, seconds, rank, what):
        self.t = threading.Timer(seconds, self._fire)
        self.rank, self.what = rank, what

    def _fire(self):
        print(json.dumps({"impl": "reference", "event": "unavailable", "rank": self.rank,
                          "why": f"{self.what} did not finish (the reference's waits are unbounded)"}), flush=True)
        os._exit(3)

    def __enter__(self):
        self.t.start()

    def __exit__(self, *a):
        self.t.cancel()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--num-tests", type=int, default=100)
    ap.add_argument("--skip-algos", action="store_true", help="part 1 only")
    ap.add_argument("--skip-custom", action="store_true", help="part 2 only")
    ap.add_argument("--watchdog-s", type=float, default=45.0)
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(REF, "penny")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}))
        return
    import penny_cpp  # the reference's extension
    from penny.custom_all_reduce import CustomAllreduce
    from penny.utils import initialize_distributed
    assert os.path.abspath(penny_cpp.__file__).startswith(REF), penny_cpp.__file__
    initialize_distributed()
    rank, world = dist.get_rank(), dist.get_world_size()
    rows = []

    def emit(**rec):
        rec = dict(impl="reference", world=world, **rec)
        rows.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    # ------------------------------------------------------------------ part 1
    if not args.skip_custom:
        gloo = dist.new_group(backend="gloo")
        car = CustomAllreduce(gloo, torch.cuda.current_device(), nvshmem_registered=True)
        for p in range(10, 23):
            nbytes = 1 << p
            n = nbytes // 2
            g = torch.Generator(device="cuda").manual_seed(rank)
            x = (torch.rand(n, device="cuda", generator=g) * 2 - 1).bfloat16()
            ref = x.clone()
            dist.all_reduce(ref)
            rs_out = torch.empty(max(1, n // world), device="cuda", dtype=x.dtype)
            for op, call, check in (
                    ("all_reduce", lambda: car.custom_all_reduce(x),
                     lambda o: torch.allclose(o.float(), ref.float(), atol=1e-1, rtol=1e-2)),
                    # the reference's kernel wants an output of exactly one shard (csrc/custom_all_reduce.cu:121;
                    # its Python default, empty_like(input), fails that check)
                    ("reduce_scatter", lambda: car.custom_reduce_scatter(x, out=rs_out),
                     lambda o: torch.allclose(o.float(), ref[rank * (n // world):(rank + 1) * (n // world)].float(),
                                              atol=1e-1, rtol=1e-2)),
                    ("all_gather", lambda: car.custom_all_gather(x), lambda o: True)):
                if op == "all_gather" and nbytes * world >= car.max_size:
                    continue
                if op == "reduce_scatter" and (n % world or (n // world * 2) % 16):
                    continue
                with Watchdog(args.watchdog_s, rank, f"CustomAllreduce.{op} @ {nbytes} B"):
                    try:
                        o = call()
                    except RuntimeError as e:  # e.g. "requires a minimum size of 2048" (csrc/custom_all_reduce.cuh:891-893)
                        emit(op=op, algo="custom_all_reduce", dtype="bf16", bytes=nbytes,
                             unsupported=str(e).strip().splitlines()[-1][:120])
                        continue
                    torch.cuda.synchronize()
                    if o is None:
                        emit(op=op, algo="custom_all_reduce", dtype="bf16", bytes=nbytes, declined=True)
                        continue
                    ok = bool(check(o))
                    t = timed(call, args.warmup, args.num_tests)
                    tg = None
                    try:
                        tg = timed_graph(call, 10, car)
                    except Exception as e:  # noqa: BLE001
                        if rank == 0:
                            print(json.dumps({"event": "graph_failed", "op": op, "bytes": nbytes, "why": str(e)[:120]}), flush=True)
                emit(op=op, algo="custom_all_reduce", dtype="bf16", bytes=nbytes, correct=ok, t_us=round(t, 2),
                     t_graph_us=round(tg, 2) if tg else None)
    # ------------------------------------------------------------------ part 2
    if not args.skip_algos:
        nnodes = int(os.environ.get("NNODES", "1"))
        packet_sizes, block_sizes = [16, 64, 256, 2048], [128, 512, 1024]
        for algo in (0, 3, 2, 1):
            if algo in (2, 3) and world != 8:
                emit(op="all_reduce", algo=ALGO_NAMES[algo], unavailable="the reference's kernel is instantiated for 8 PEs")
                continue
            for p in (13, 17, 21, 25, 28):
                nbytes = 1 << p
                num = nbytes // 2
                if algo == 2 and nbytes > (2 << 20):
                    continue  # its scratch is numel x PEs
                best = None
                for packet in packet_sizes:
                    for block in block_sizes:
                        for routes in ([1, 4] if algo == 3 else [1]):
                            # the divisibility filters of the reference's own harness
                            if p > 23 and packet < 32:
                                continue
                            if algo == 0 and nbytes % (packet * block * world * routes) != 0:
                                continue
                            if algo == 1 and nbytes % (packet * block * routes) != 0:
                                continue
                            if algo == 2 and (nbytes % (packet * block) != 0 or nbytes // (packet * block) == 0):
                                continue
                            if algo == 3 and (nbytes % (packet * block * world) != 0 or nbytes // (packet * block * world) == 0):
                                continue
                            if algo in (2, 3):
                                reduce_size = (packet * block) // (world * routes)
                                if reduce_size == 0 or reduce_size % 16 != 0:
                                    continue
                            data = torch.empty(num, device="cuda", dtype=torch.float16).normal_(mean=0, std=1) + 1
                            want = data.clone()
                            dist.all_reduce(want)
                            out = torch.empty_like(data)
                            with Watchdog(args.watchdog_s, rank, f"{ALGO_NAMES[algo]} packet {packet} block {block} "
                                                                 f"routes {routes} @ {nbytes} B"):
                                penny_cpp.nvshmem_register(out)
                                h = penny_cpp.all_reduce_create(data, packet, block, nnodes, routes, algo)
                                penny_cpp.all_reduce_run(h, out)
                                torch.cuda.synchronize()
                                ok = torch.allclose(want, out, atol=1e-1, rtol=1e-2)
                                t = timed(lambda: penny_cpp.all_reduce_run(h, out), 5, 20) if ok else None
                                penny_cpp.all_reduce_destroy(h)
                                penny_cpp.nvshmem_unregister(out)
                            if ok and (best is None or t < best[0]):
                                best = (t, packet, block, routes)
                if best is None:
                    emit(op="all_reduce", algo=ALGO_NAMES[algo], dtype="fp16", bytes=nbytes,
                         unavailable="no configuration of the grid gave the right sum")
                else:
                    emit(op="all_reduce", algo=ALGO_NAMES[algo], dtype="fp16", bytes=nbytes, t_us=round(best[0], 2),
                         packet_size=best[1], block_size=best[2], routes=best[3],
                         busbw_gbs=round(2 * (world - 1) / world * nbytes / best[0] / 1e3, 2))
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)  # the reference's tear-down paths were seen to block after graph capture


if __name__ == "__main__":
    main()
