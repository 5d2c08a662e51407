"""Every sweep the tuner table and the results tables are built from, in ONE process group:

    torchrun --nproc-per-node N extra/sweep_all.py --out sweep_wN.jsonl [--quick]

  all-reduce      bf16 and fp32, 1 KiB - 1 GiB, ordinary tensors: every algorithm, `auto`, NCCL
                  the same in the symmetric heap for the algorithms whose path differs there
  reduce-scatter  bf16 and fp32 shards of 1 KiB - 256 MiB (ordinary and symmetric input)
  all-gather      bf16 shards of 1 KiB - 256 MiB (ordinary and symmetric output)
  exchange / all-to-all   4 KiB - 64 MiB per peer
  fused all-reduce + residual + RMSNorm   1 - 256 rows of 4096
Protocol of every point: 20 warm-up + 100 timed calls, CUDA events on the launching stream, L2
flushed and ranks aligned before every timed call, median, max over ranks; sizes up to 8 MiB are
also timed as 10 back-to-back calls inside a CUDA graph.  `--quick` (5 + 20 calls, fewer sizes) is
for checking the script.  Output: JSON lines (appended to --out), the input of
`python -m penny_b200.parallel.tuner`.
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import benchmark_all_gather  # noqa: E402
import benchmark_allreduce  # noqa: E402
import benchmark_exchange  # noqa: E402
import benchmark_reduce_scatter  # noqa: E402
import bench_fused_norm  # noqa: E402
from penny_b200.utils import initialize_distributed, shutdown  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--heap-gib", type=float, default=40.0)
    ap.add_argument("--skip", nargs="*", default=[], help="parts to leave out: ar ar_sym rs ag a2a fused")
    args = ap.parse_args()
    rank, world, comm = initialize_distributed(heap_bytes=int(args.heap_gib * (1 << 30)))
    ctx = (rank, world, comm)
    if rank == 0 and os.path.exists(args.out):
        os.remove(args.out)
    it = ["--warmup", "5", "--num-tests", "20"] if args.quick else ["--warmup", "20", "--num-tests", "100"]
    out = ["--out", args.out]
    t0 = time.time()

    def note(what):
        if rank == 0:
            print(f'{{"event": "part", "what": "{what}", "elapsed_s": {time.time() - t0:.1f}}}', flush=True)

    big = "12" if args.quick else "21"      # all-reduce sizes from 1 KiB
    shard = "10" if args.quick else "19"    # shard sizes from 1 KiB
    for dtype in ("bf16", "fp32"):
        if "ar" not in args.skip:
            note(f"all_reduce {dtype}")
            benchmark_allreduce.main(["--dtype", dtype, "--start-pow", "10", "--range", big, "--max-slow-mib", "64"]
                                     + it + out, ctx)
        if "ar_sym" not in args.skip:
            note(f"all_reduce {dtype} symmetric")
            algos = ["oneshot_ll", "oneshot", "twoshot"] + (["nvls_oneshot", "nvls"] if comm.has_multicast else []) + ["auto"]
            benchmark_allreduce.main(["--dtype", dtype, "--start-pow", "10", "--range", big if dtype == "bf16" else "19",
                                      "--symmetric", "--no-nccl", "--algo"] + algos + it + out, ctx)
        if "rs" not in args.skip:
            note(f"reduce_scatter {dtype}")
            benchmark_reduce_scatter.main(["--dtype", dtype, "--start-pow", "10", "--range", shard] + it + out, ctx)
            if dtype == "bf16":
                benchmark_reduce_scatter.main(["--dtype", dtype, "--start-pow", "10", "--range", shard, "--symmetric",
                                               "--no-nccl"] + it + out, ctx)
    if "ag" not in args.skip:
        note("all_gather bf16")
        benchmark_all_gather.main(["--dtype", "bf16", "--start-pow", "10", "--range", shard] + it + out, ctx)
    if "a2a" not in args.skip:
        note("exchange + all_to_all bf16")
        benchmark_exchange.main(["--dtype", "bf16", "--start-pow", "12", "--range", "8" if args.quick else "15",
                                 "--all-to-all"] + it + out, ctx)
    if "fused" not in args.skip:
        note("fused all-reduce + RMSNorm")
        bench_fused_norm.main(out, ctx)
    note("done")
    shutdown()


if __name__ == "__main__":
    main()
