"""Every fused compute + collective benchmark in ONE set of processes.

    torchrun --nproc-per-node 8 extra/bench_fused_all.py --tokens 4096 --moe-tokens 2048

Runs, on one communicator (start-up of an 8-rank job costs more than the
measurements themselves):
  1. the four sequence-parallel linears of extra/bench_fused_gemm.py
     (tcgen05 GEMM -> reduce-scatter, all-gather -> tcgen05 GEMM) against
     cuBLAS + NCCL,
  2. the Mixtral-shaped expert-parallel layer of extra/bench_moe_ep.py against
     NCCL all_to_all_single,
  3. all-to-all and pairwise exchange at three sizes against NCCL
     (all_to_all_single, batch_isend_irecv),
  4. the sequence-parallel prefill stack of extra/bench_sp_prefill.py (fused
     linears against cuBLAS + NCCL).
Rank 0 prints one JSON line per measurement.  Device time everywhere: CUDA
events, L2 flushed between calls, ranks aligned, median, max over ranks.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import bench_fused_gemm  # noqa: E402
import bench_moe_ep  # noqa: E402
import bench_sp_prefill  # noqa: E402
from penny_b200.utils import bench_device, initialize_distributed, shutdown  # noqa: E402


def run_exchange(rank, world, comm, sizes, warmup, iters):
    """all_to_all (bytes per peer) and exchange with rank ^ 1 against their NCCL counterparts."""
    peer = rank ^ 1
    for nbytes in sizes:
        n = nbytes // 2
        x = torch.full((world * n,), float(rank + 1), device="cuda", dtype=torch.bfloat16)
        want = torch.empty_like(x)
        dist.all_to_all_single(want, x)
        got = comm.all_to_all(x)
        comm.check()
        if not torch.equal(got, want):
            raise SystemExit(f"rank {rank}: all_to_all differs from all_to_all_single at {nbytes} bytes per peer")
        out = torch.empty_like(x)
        t_p = bench_device(lambda: comm.all_to_all(x, out=out), warmup, iters)["median_us"]
        t_n = bench_device(lambda: dist.all_to_all_single(want, x), warmup, iters)["median_us"]
        line = {"op": "all_to_all", "world": world, "bytes_per_peer": nbytes, "penny_us": round(t_p, 1),
                "nccl_us": round(t_n, 1), "speedup": round(t_n / t_p, 3),
                "penny_gbs_out": round(nbytes * (world - 1) / t_p / 1e3, 1)}
        if rank == 0:
            print(json.dumps(line), flush=True)
        if world % 2 == 0:
            y = torch.full((n,), float(rank + 1), device="cuda", dtype=torch.bfloat16)
            r_n = torch.empty_like(y)

            def nccl_pair():
                ops_ = [dist.P2POp(dist.isend, y, peer), dist.P2POp(dist.irecv, r_n, peer)]
                for w in dist.batch_isend_irecv(ops_):
                    w.wait()
            nccl_pair()
            comm.exchange(y, peer)  # in place: y now holds the peer's values
            comm.check()
            if not torch.equal(y, r_n):
                raise SystemExit(f"rank {rank}: exchange differs from batch_isend_irecv at {nbytes} bytes")
            t_p = bench_device(lambda: comm.exchange(y, peer), warmup, iters)["median_us"]
            t_n = bench_device(nccl_pair, warmup, iters)["median_us"]
            if rank == 0:
                print(json.dumps({"op": "exchange", "world": world, "bytes": nbytes, "penny_us": round(t_p, 1),
                                  "nccl_us": round(t_n, 1), "speedup": round(t_n / t_p, 3),
                                  "penny_gbs": round(nbytes / t_p / 1e3, 1)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096, help="prefill tokens of the fused linears")
    ap.add_argument("--moe-tokens", type=int, default=2048, help="tokens per rank of the MoE layer")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--heap-gib", type=float, default=4.0)
    ap.add_argument("--skip", nargs="*", default=[], choices=["gemm", "moe", "exchange", "sp"])
    ap.add_argument("--sp-layers", type=int, default=8, help="layers of the sequence-parallel prefill stack")
    args = ap.parse_args()
    rank, world, comm = initialize_distributed(heap_bytes=int(args.heap_gib * (1 << 30)))
    if "gemm" not in args.skip:
        bench_fused_gemm.run(rank, world, comm, argparse.Namespace(tokens=args.tokens, iters=args.iters,
                                                                   warmup=args.warmup, side_ctas=0))
    if "moe" not in args.skip:
        bench_moe_ep.run(rank, world, comm, argparse.Namespace(tokens=args.moe_tokens, iters=max(5, args.iters // 2),
                                                               warmup=args.warmup, ffn=14336))
    if "exchange" not in args.skip:
        run_exchange(rank, world, comm, [64 << 10, 1 << 20, 16 << 20], args.warmup, args.iters)
    if "sp" not in args.skip:
        bench_sp_prefill.run(rank, world, comm, argparse.Namespace(tokens=args.tokens, layers=args.sp_layers,
                                                                   iters=5, warmup=2))
    comm.check()
    shutdown()


if __name__ == "__main__":
    main()
