"""All-reduce sweep: every algorithm and the auto-selected one against NCCL.

    torchrun --nproc-per-node 8 extra/benchmark_allreduce.py --start-pow 10 --range 21 --dtype bf16

For each message size it times every requested algorithm (CUDA events on the
device, L2 flushed and ranks aligned before each timed call, max over ranks),
checks the result against NCCL's (`--atol/--rtol`, failing loudly), and prints
one JSON line per (size, algorithm) with the NCCL-style bus bandwidth
2(n-1)/n * bytes / t and its fraction of the 900 GB/s NVLink 5 line rate.

Same role and flags as the reference's extra/benchmark_allreduce.py (which
sweeps packet/block/routes per size with a profiler-based timer and prints
2*bytes/t, :62-179); `--algo` accepts the reference's numbers 0-3 as well as
names.  `--tune` sweeps the launch grid per algorithm like the reference does.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from penny_b200.parallel.comm import ALGOS, ALGO_NAMES  # noqa: E402
from penny_b200.utils import bench_device, bench_graph, bus_bandwidth_gbs, initialize_distributed, shutdown  # noqa: E402

NVLINK_GBS = 900.0


def parse(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--algo", nargs="*", default=["all"], help="names or the reference's ids 0-3; 'all'; 'auto'")
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    p.add_argument("--start-pow", type=int, default=10, help="first size = 2^start_pow bytes")
    p.add_argument("--range", type=int, default=21, help="number of power-of-two sizes")
    p.add_argument("--num-tests", type=int, default=100)
    p.add_argument("--warmup", type=int, default=20)
    p.add_argument("--atol", type=float, default=1e-1)
    p.add_argument("--rtol", type=float, default=1e-2)
    p.add_argument("--nnodes", type=int, default=int(os.environ.get("NNODES", "1")), help="virtual nodes")
    p.add_argument("--symmetric", action="store_true", help="tensors in the symmetric heap (no staging)")
    p.add_argument("--tune", action="store_true", help="sweep blocks x threads per algorithm and size")
    p.add_argument("--no-nccl", action="store_true")
    p.add_argument("--bench-custom", action="store_true", help="also time penny.CustomAllreduce (<= 8 MiB)")
    p.add_argument("--profile-mode", default="none", choices=["none", "file"])
    p.add_argument("--heap-gib", type=float, default=6.0)
    p.add_argument("--graph-inner", type=int, default=10,
                   help="also time N back-to-back calls inside one CUDA graph (sizes <= 8 MiB); 0 = off")
    p.add_argument("--out", default="")
    p.add_argument("--max-slow-mib", type=int, default=256,
                   help="largest message (MiB) for the parity algorithms (simple ring, tree, double ring)")
    return p.parse_args(argv)


def main(argv=None, ctx=None):
    """ctx: (rank, world, comm) of an already initialised process (extra/sweep_all.py); else set up here."""
    args = parse(argv)
    rank, world, comm = ctx if ctx is not None else initialize_distributed(heap_bytes=int(args.heap_gib * (1 << 30)))
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    es = torch.empty((), dtype=dtype).element_size()
    names = []
    for a in args.algo:
        if a == "all":
            names += ["oneshot_ll", "oneshot", "twoshot", "ring_simple", "ring_standard", "double_ring", "tree"]
            if comm.has_multicast:
                names += ["nvls_oneshot", "nvls"]
            names += ["auto"]
        elif a.isdigit():
            names.append(ALGO_NAMES[int(a)])
        else:
            assert a in ALGOS, a
            names.append(a)
    if rank == 0:
        print(json.dumps({"event": "setup", "world": world, "describe": comm.describe(), "dtype": args.dtype}),
              flush=True)
    custom = None
    if args.bench_custom:
        from penny_b200.parallel.custom_all_reduce import CustomAllreduce
        gloo = dist.new_group(backend="gloo")
        custom = CustomAllreduce(gloo, torch.cuda.current_device())
    results = []
    prof = None
    if args.profile_mode == "file":
        prof = torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU,
                                                  torch.profiler.ProfilerActivity.CUDA], record_shapes=True)
        prof.__enter__()
    for p in range(args.start_pow, args.start_pow + args.range):
        nbytes = 1 << p
        n = nbytes // es
        if n < 1:
            continue
        g = torch.Generator(device="cuda").manual_seed(rank)
        src = (torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dtype)
        if args.symmetric:
            try:
                x = comm.empty(n, dtype=dtype)
                y = comm.empty(n, dtype=dtype)
            except RuntimeError as e:
                if rank == 0:
                    print(json.dumps({"event": "skip", "bytes": nbytes, "why": str(e)[:120]}), flush=True)
                break
            x.copy_(src)
        else:
            x, y = src, torch.empty_like(src)
        ref = x.clone()
        dist.all_reduce(ref)
        nccl_us, nccl_graph_us = None, None
        if not args.no_nccl:
            buf = x.clone()
            nccl_us = bench_device(lambda: dist.all_reduce(buf), args.warmup, args.num_tests)["median_us"]
            rec = {"op": "all_reduce", "impl": "nccl", "world": world, "dtype": args.dtype, "bytes": nbytes,
                   "t_us": round(nccl_us, 2),
                   "busbw_gbs": round(bus_bandwidth_gbs("all_reduce", nbytes, world, nccl_us), 2)}
            if args.graph_inner > 0 and nbytes <= (8 << 20):
                try:
                    nccl_graph_us = bench_graph(lambda: dist.all_reduce(buf), args.graph_inner)["median_us"]
                    rec["t_graph_us"] = round(nccl_graph_us, 2)
                except RuntimeError:
                    nccl_graph_us = None
            results.append(rec)
            if rank == 0:
                print(json.dumps(rec), flush=True)
        for name in names:
            # size limits of the latency-oriented algorithms
            if name in ("oneshot_ll",) and nbytes > (4 << 20):
                continue
            if name in ("oneshot", "nvls_oneshot") and nbytes > (32 << 20):
                continue
            if name in ("ring_simple", "tree", "double_ring") and nbytes > (args.max_slow_mib << 20):
                continue
            nnodes = args.nnodes if name in ("double_ring", "tree", "ring_standard") else 1
            if name in ("double_ring", "tree") and nnodes == 1 and world >= 4:
                nnodes = 2
            grids = [(0, 0)]
            if args.tune:
                grids = [(b, t) for b in (8, 16, 32, 64, 128) for t in (256, 512)]
            best = None
            for blocks, threads in grids:
                def call():
                    comm.all_reduce(x, out=y, algo=name, nnodes=nnodes, blocks=blocks, threads=threads)
                try:
                    call()
                    comm.check()
                except RuntimeError as e:
                    if rank == 0:
                        print(json.dumps({"event": "error", "algo": name, "bytes": nbytes, "why": str(e)[:200]}),
                              flush=True)
                    break
                ok = torch.allclose(y.float(), ref.float(), atol=args.atol, rtol=args.rtol)
                if not ok:
                    bad = (y.float() - ref.float()).abs().max().item()
                    raise SystemExit(f"rank {rank}: {name} @ {nbytes} B differs from NCCL (max abs diff {bad})")
                t = bench_device(call, args.warmup, args.num_tests)["median_us"]
                if best is None or t < best[0]:
                    best = (t, blocks, threads)
            if best is None:
                continue
            comm.check()
            t, blocks, threads = best
            bw = bus_bandwidth_gbs("all_reduce", nbytes, world, t)
            rec = {"op": "all_reduce", "impl": "penny", "algo": name, "world": world, "dtype": args.dtype,
                   "bytes": nbytes, "t_us": round(t, 2), "busbw_gbs": round(bw, 2),
                   "frac_nvlink": round(bw / NVLINK_GBS, 4), "symmetric": args.symmetric,
                   "picked": comm.pick_algo(dtype, n, args.symmetric) if name == "auto" else name}
            if args.tune:
                rec["blocks"], rec["threads"] = blocks, threads
            if nccl_us:
                rec["vs_nccl"] = round(nccl_us / t, 3)
            if args.graph_inner > 0 and nbytes <= (8 << 20):
                def gcall():
                    comm.all_reduce(x, out=y, algo=name, nnodes=nnodes, blocks=blocks, threads=threads)
                tg = bench_graph(gcall, args.graph_inner)["median_us"]
                comm.check()
                rec["t_graph_us"] = round(tg, 2)
                if nccl_graph_us:
                    rec["vs_nccl_graph"] = round(nccl_graph_us / tg, 3)
            results.append(rec)
            if rank == 0:
                print(json.dumps(rec), flush=True)
        if custom is not None and not custom.disabled and nbytes < custom.max_size and nbytes % 16 == 0:
            out = custom.custom_all_reduce(x)
            assert out is not None and torch.allclose(out.float(), ref.float(), atol=args.atol, rtol=args.rtol)
            t = bench_device(lambda: custom.custom_all_reduce(x), args.warmup, args.num_tests)["median_us"]
            rec = {"op": "all_reduce", "impl": "penny", "algo": "custom_all_reduce", "world": world,
                   "dtype": args.dtype, "bytes": nbytes, "t_us": round(t, 2),
                   "busbw_gbs": round(bus_bandwidth_gbs("all_reduce", nbytes, world, t), 2)}
            results.append(rec)
            if rank == 0:
                print(json.dumps(rec), flush=True)
    if prof is not None:
        prof.__exit__(None, None, None)
        if rank == 0:
            prof.export_chrome_trace("trace_penny.json")
    if rank == 0 and args.out:
        with open(args.out, "a") as f:
            for r in results:
                f.write(json.dumps(r) + "\n")
    if custom is not None:
        custom.close()
    if ctx is None:
        shutdown()


if __name__ == "__main__":
    main()
