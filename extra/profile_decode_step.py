"""Per-kernel timeline of the TP decode step as it runs inside its CUDA graph.

    python extra/profile_decode_step.py [--batch 64] [--kv-len 2048] [--layers 32] [--linears penny]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 extra/profile_decode_step.py

The step is captured exactly as bench.py runs it and replayed under the torch
profiler (CUPTI activity records: the kernels are not serialised, so overlap from
programmatic dependent launch is visible).  Rank 0 prints
  * per kernel name: launches per step, summed and mean device time, share of the step;
  * the timeline of one middle layer: start offset, duration, and the gap (negative =
    overlap) to the end of the previous kernel.
Device time of a kernel that waits for its predecessor (griddepcontrol.wait) or for
its peers includes that wait.
"""
import argparse
import os
import sys
from collections import defaultdict

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def short(name: str) -> str:
    for key in ("gemm_decode_kernel", "k_decode_attn_fused", "k_fused_nvls_norm", "k_add_rmsnorm", "k_argmax",
                "k_silu_mul", "k_decode_attn", "k_attn_merge", "k_rope_append"):
        if key in name:
            return key
    if "k_real" in name:
        for key in ("FusedOneShotNorm", "AllGather", "OneShot", "TwoShot", "Nvls"):
            if key in name:
                return "collective:" + key
        return "collective"
    return name.split("(")[0][-48:]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--kv-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--linears", default="auto", choices=["auto", "penny", "cublas"])
    ap.add_argument("--backend", default="penny", choices=["penny", "penny_unfused", "nccl"])
    ap.add_argument("--proto", default="auto")
    args = ap.parse_args()
    from penny_b200.models.llama_tp import LlamaConfig, LlamaTPDecoder
    from penny_b200.utils import initialize_distributed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, comm = 0, None
    if world > 1:
        rank, world, comm = initialize_distributed(heap_bytes=1 << 30)
    else:
        torch.cuda.set_device(0)
    cfg = LlamaConfig.llama3_8b()
    cfg.layers = args.layers
    model = LlamaTPDecoder(cfg, comm=comm, rank=rank, world=world, max_batch=args.batch, max_len=args.kv_len + 64,
                           backend=args.backend, proto=args.proto, linears=args.linears)
    model.fill_synthetic_kv(args.kv_len)
    model.capture()
    for _ in range(3):
        model.step_device()
    torch.cuda.synchronize()
    steps = 3
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            model.step_device()
        torch.cuda.synchronize()
    if comm is not None:
        comm.check()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and e.device_time > 0
                 and "Memcpy" not in e.name and "Memset" not in e.name),
                key=lambda e: e.time_range.start)
    if rank == 0 and ev:
        per_step = len(ev) // steps
        last = ev[-per_step:]
        t0, t1 = last[0].time_range.start, max(e.time_range.end for e in last)
        print(f"world {world}, batch {args.batch}, kv {args.kv_len}, linears {model.linears}, proto {model.proto}: "
              f"{per_step} kernels per step, step {t1 - t0:.1f} us (first kernel start to last kernel end)")
        agg = defaultdict(lambda: [0, 0.0])
        for e in last:
            a = agg[short(e.name)]
            a[0] += 1
            a[1] += e.device_time
        print(f"{'kernel':34s} {'count':>6s} {'sum us':>9s} {'mean us':>8s} {'share':>6s}")
        for k, (n, t) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
            print(f"{k:34s} {n:6d} {t:9.1f} {t / n:8.2f} {100 * t / (t1 - t0):5.1f}%")
        # one middle layer: from a qkv GEMM (the kernel after a norm) to the next one
        names = [short(e.name) for e in last]
        per_layer = None
        starts = [i for i, n in enumerate(names) if n in ("k_decode_attn_fused", "k_decode_attn")]
        if len(starts) > 3:
            per_layer = starts[2] - starts[1]
            lo = starts[len(starts) // 2] - 1
            print(f"\ntimeline of one layer ({per_layer} kernels), us from the start of its first kernel:")
            base = last[lo].time_range.start
            prev_end = None
            for e in last[lo:lo + per_layer + 1]:
                gap = "" if prev_end is None else f"{e.time_range.start - prev_end:+7.2f}"
                print(f"  {e.time_range.start - base:8.2f}  +{e.device_time:7.2f}  gap {gap:>8s}  {short(e.name)}")
                prev_end = e.time_range.end
    if comm is not None:
        torch.cuda.synchronize()
        comm.barrier()
        comm.close()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
