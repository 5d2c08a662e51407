"""All-gather sweep against NCCL's all_gather_into_tensor.

    torchrun --nproc-per-node 8 extra/benchmark_all_gather.py --start-pow 10 --range 19

Sizes are per-rank shard bytes.  Variants: peer pushes through scratch
("push"), pushes straight into a symmetric output ("push_direct"), NVLS
multimem.st ("nvls") and the drop-in CustomAllreduce.all_gather (<= 8 MiB).
Bus bandwidth = (n-1)/n * gathered_bytes / t.  Counterpart of the reference's
extra/benchmark_all_gather.py (data = rank so that misplaced shards show).
"""
import torch
import torch.distributed as dist

from _bench_common import DTYPES, NVLINK_GBS, Recorder, base_parser, uniform
from penny_b200.utils import bench_device, bus_bandwidth_gbs, initialize_distributed, shutdown


def main(argv=None, ctx=None):
    """ctx: (rank, world, comm) of an already initialised process (extra/sweep_all.py); else set up here."""
    args = base_parser().parse_args(argv)
    rank, world, comm = ctx if ctx is not None else initialize_distributed(heap_bytes=int(args.heap_gib * (1 << 30)))
    dtype = DTYPES[args.dtype]
    es = torch.empty((), dtype=dtype).element_size()
    rec = Recorder(rank, args.out)
    from penny_b200.parallel.custom_all_reduce import CustomAllreduce
    car = CustomAllreduce(dist.new_group(backend="gloo"), torch.cuda.current_device())
    for p in range(args.start_pow, args.start_pow + args.range):
        shard_bytes = 1 << p
        n = shard_bytes // es
        x = torch.full((n,), float(rank), device="cuda", dtype=dtype) + uniform(n, dtype, rank) * 0.25
        ref = torch.empty(n * world, device="cuda", dtype=dtype)
        dist.all_gather_into_tensor(ref, x)
        total = shard_bytes * world
        nccl_us = None
        if not args.no_nccl:
            nccl_us = bench_device(lambda: dist.all_gather_into_tensor(ref, x), args.warmup, args.num_tests)["median_us"]
            rec.add(op="all_gather", impl="nccl", world=world, dtype=args.dtype, shard_bytes=shard_bytes,
                    t_us=round(nccl_us, 2), busbw_gbs=round(bus_bandwidth_gbs("all_gather", total, world, nccl_us), 2))
        variants = [("push", False, False)]
        try:
            sym_out = comm.empty(n * world, dtype=dtype)
            variants.append(("push_direct", True, False))
            if comm.has_multicast and shard_bytes % 16 == 0:
                variants.append(("nvls", True, True))
        except RuntimeError:
            sym_out = None
        for name, direct, nvls in variants:
            out = sym_out if direct else torch.empty(n * world, device="cuda", dtype=dtype)
            comm.all_gather(x, out=out, nvls=nvls)
            comm.check()
            algo = "nvls" if nvls else "push"   # the name the tuner table uses; `direct` is the memory class
            if not torch.equal(out, ref):
                raise SystemExit(f"rank {rank}: all_gather/{name} @ {shard_bytes} B differs from NCCL")
            t = bench_device(lambda: comm.all_gather(x, out=out, nvls=nvls), args.warmup, args.num_tests)["median_us"]
            bw = bus_bandwidth_gbs("all_gather", total, world, t)
            rec.add(op="all_gather", impl="penny", algo=algo, variant=name, world=world, dtype=args.dtype,
                    bytes=shard_bytes, shard_bytes=shard_bytes, symmetric=direct,
                    t_us=round(t, 2), busbw_gbs=round(bw, 2), frac_nvlink=round(bw / NVLINK_GBS, 4),
                    vs_nccl=round(nccl_us / t, 3) if nccl_us else None)
        # what `algo="auto"` (the measured table) makes of it, for both kinds of output tensor
        for direct in ([False, True] if sym_out is not None else [False]):
            out = sym_out if direct else torch.empty(n * world, device="cuda", dtype=dtype)
            comm.all_gather(x, out=out)
            comm.check()
            if not torch.equal(out, ref):
                raise SystemExit(f"rank {rank}: all_gather/auto @ {shard_bytes} B differs from NCCL")
            t = bench_device(lambda: comm.all_gather(x, out=out), args.warmup, args.num_tests)["median_us"]
            bw = bus_bandwidth_gbs("all_gather", total, world, t)
            rec.add(op="all_gather", impl="penny", algo="auto", world=world, dtype=args.dtype, bytes=shard_bytes,
                    shard_bytes=shard_bytes, symmetric=direct, t_us=round(t, 2), busbw_gbs=round(bw, 2),
                    vs_nccl=round(nccl_us / t, 3) if nccl_us else None)
        if not car.disabled and total < car.max_size and shard_bytes % 16 == 0:
            out = car.custom_all_gather(x)
            assert out is not None and torch.equal(out, ref)
            t = bench_device(lambda: car.custom_all_gather(x), args.warmup, args.num_tests)["median_us"]
            rec.add(op="all_gather", impl="penny", algo="custom_all_reduce", world=world, dtype=args.dtype,
                    shard_bytes=shard_bytes, t_us=round(t, 2),
                    busbw_gbs=round(bus_bandwidth_gbs("all_gather", total, world, t), 2))
    comm.check()
    rec.close()
    car.close()
    if ctx is None:
        shutdown()


if __name__ == "__main__":
    main()
