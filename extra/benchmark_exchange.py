"""Pairwise exchange and all-to-all sweep against NCCL.

    torchrun --nproc-per-node 8 extra/benchmark_exchange.py --mode intranode --start-pow 12 --range 15

`--mode intranode` pairs neighbours (0<->1, 2<->3, ...), `--mode internode`
pairs rank r with r + world/2 (the two virtual nodes of the box), like the
reference's extra/benchmark_exchange.py:54-60.  The swap is checked bit-exactly
against batch_isend_irecv.  `--all-to-all` adds the N-way exchange with equal
per-peer chunks of the same size against all_to_all_single.
"""
import os

import torch
import torch.distributed as dist

from _bench_common import DTYPES, NVLINK_GBS, Recorder, base_parser, uniform
from penny_b200.utils import bench_device, initialize_distributed, shutdown


def main(argv=None, ctx=None):
    """ctx: (rank, world, comm) of an already initialised process (extra/sweep_all.py); else set up here."""
    p = base_parser(default_start=12, default_range=15)
    p.add_argument("--mode", default="intranode", choices=["intranode", "internode"])
    p.add_argument("--all-to-all", action="store_true")
    args = p.parse_args(argv)
    rank, world, comm = ctx if ctx is not None else initialize_distributed(heap_bytes=int(args.heap_gib * (1 << 30)))
    dtype = DTYPES[args.dtype]
    es = torch.empty((), dtype=dtype).element_size()
    rec = Recorder(rank, args.out)
    peer = rank ^ 1 if args.mode == "intranode" else (rank + world // 2) % world
    if world == 2:
        peer = rank ^ 1
    for pw in range(args.start_pow, args.start_pow + args.range):
        nbytes = 1 << pw
        n = nbytes // es
        x = uniform(n, dtype, rank)
        want = torch.empty_like(x)
        ops = [dist.P2POp(dist.isend, x, peer), dist.P2POp(dist.irecv, want, peer)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        torch.cuda.synchronize()
        nccl_us = None
        if not args.no_nccl:
            def nccl_swap():
                for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, x, peer), dist.P2POp(dist.irecv, want, peer)]):
                    w.wait()
            nccl_us = bench_device(nccl_swap, args.warmup, args.num_tests)["median_us"]
            rec.add(op="exchange", impl="nccl", world=world, dtype=args.dtype, bytes=nbytes, mode=args.mode,
                    t_us=round(nccl_us, 2), gbs=round(nbytes / nccl_us / 1e3, 2))
        buf = x.clone()
        comm.exchange(buf, peer)
        comm.check()
        if not torch.equal(buf, want):
            raise SystemExit(f"rank {rank}: exchange @ {nbytes} B is not bit-exact")
        # an even number of swaps restores the buffer, so timing does not disturb it
        t = bench_device(lambda: comm.exchange(buf, peer), args.warmup, args.num_tests)["median_us"]
        gbs = nbytes / t / 1e3
        rec.add(op="exchange", impl="penny", world=world, dtype=args.dtype, bytes=nbytes, mode=args.mode,
                t_us=round(t, 2), gbs=round(gbs, 2), frac_nvlink=round(gbs / NVLINK_GBS, 4),
                vs_nccl=round(nccl_us / t, 3) if nccl_us else None)
        if args.all_to_all:
            xs = uniform(n * world, dtype, rank)
            ref = torch.empty_like(xs)
            dist.all_to_all_single(ref, xs)
            t_nccl = None if args.no_nccl else bench_device(lambda: dist.all_to_all_single(ref, xs), args.warmup,
                                                            args.num_tests)["median_us"]
            sent = nbytes * (world - 1)
            for name in ("push", "pipelined", "auto"):
                if name == "pipelined" and nbytes < (64 << 10):
                    continue
                out = comm.all_to_all(xs, algo=name)
                comm.check()
                if not torch.equal(out, ref):
                    raise SystemExit(f"rank {rank}: all_to_all/{name} @ {nbytes} B per peer differs from NCCL")
                t = bench_device(lambda: comm.all_to_all(xs, out=out, algo=name), args.warmup, args.num_tests)["median_us"]
                rec.add(op="all_to_all", impl="penny", algo=name, world=world, dtype=args.dtype, bytes=nbytes,
                        bytes_per_peer=nbytes, symmetric=False, t_us=round(t, 2), egress_gbs=round(sent / t / 1e3, 2),
                        frac_nvlink=round(sent / t / 1e3 / NVLINK_GBS, 4),
                        nccl_us=round(t_nccl, 2) if t_nccl else None, vs_nccl=round(t_nccl / t, 3) if t_nccl else None)
    comm.check()
    rec.close()
    if ctx is None:
        shutdown()


if __name__ == "__main__":
    main()
