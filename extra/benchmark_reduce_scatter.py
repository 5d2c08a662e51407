"""Reduce-scatter sweep against NCCL's reduce_scatter_tensor.

    torchrun --nproc-per-node 8 extra/benchmark_reduce_scatter.py --start-pow 10 --range 19

Sizes are per-rank OUTPUT shard bytes (the input is world times larger).
Variants: peer pushes + local reduce ("push"), NVLS multimem.ld_reduce ("nvls")
and the drop-in CustomAllreduce.reduce_scatter (<= 8 MiB inputs).  Bus bandwidth
= (n-1)/n * input_bytes / t.  Counterpart of the reference's
extra/benchmark_reduce_scatter.py.
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
        shard = shard_bytes // es
        n = shard * world
        src = uniform(n, dtype, rank)
        x = src
        if args.symmetric:
            try:
                x = comm.empty(n, dtype=dtype)
                x.copy_(src)
            except RuntimeError:
                break
        ref = torch.empty(shard, device="cuda", dtype=dtype)
        dist.reduce_scatter_tensor(ref, x.clone())
        total = n * es
        nccl_us = None
        if not args.no_nccl:
            buf = x.clone()
            nccl_us = bench_device(lambda: dist.reduce_scatter_tensor(ref, buf), args.warmup, args.num_tests)["median_us"]
            rec.add(op="reduce_scatter", impl="nccl", world=world, dtype=args.dtype, shard_bytes=shard_bytes,
                    t_us=round(nccl_us, 2), busbw_gbs=round(bus_bandwidth_gbs("reduce_scatter", total, world, nccl_us), 2))
        variants = [("push", False, False)]
        if shard_bytes >= (256 << 10):
            variants.append(("pipelined", False, True))
        if comm.has_multicast and shard_bytes % 16 == 0:
            variants.append(("nvls", True, False))
        variants.append(("auto", None, None))
        out = torch.empty(shard, device="cuda", dtype=dtype)
        for name, nvls, pipe in variants:
            comm.reduce_scatter(x, out=out, nvls=nvls, pipelined=pipe)
            comm.check()
            if not torch.allclose(out.float(), ref.float(), atol=args.atol, rtol=args.rtol):
                raise SystemExit(f"rank {rank}: reduce_scatter/{name} @ {shard_bytes} B differs from NCCL")
            t = bench_device(lambda: comm.reduce_scatter(x, out=out, nvls=nvls, pipelined=pipe), args.warmup,
                             args.num_tests)["median_us"]
            bw = bus_bandwidth_gbs("reduce_scatter", total, world, t)
            rec.add(op="reduce_scatter", impl="penny", algo=name, world=world, dtype=args.dtype,
                    bytes=shard_bytes, shard_bytes=shard_bytes, t_us=round(t, 2), busbw_gbs=round(bw, 2),
                    frac_nvlink=round(bw / NVLINK_GBS, 4), symmetric=args.symmetric,
                    vs_nccl=round(nccl_us / t, 3) if nccl_us else None)
        if not car.disabled and total < car.max_size and shard_bytes % 16 == 0:
            o = car.custom_reduce_scatter(x)
            assert o is not None and torch.allclose(o[:shard].float(), ref.float(), atol=args.atol, rtol=args.rtol)
            t = bench_device(lambda: car.custom_reduce_scatter(x), args.warmup, args.num_tests)["median_us"]
            rec.add(op="reduce_scatter", impl="penny", algo="custom_all_reduce", world=world, dtype=args.dtype,
                    shard_bytes=shard_bytes, t_us=round(t, 2),
                    busbw_gbs=round(bus_bandwidth_gbs("reduce_scatter", total, world, t), 2))
    comm.check()
    rec.close()
    car.close()
    if ctx is None:
        shutdown()


if __name__ == "__main__":
    main()
