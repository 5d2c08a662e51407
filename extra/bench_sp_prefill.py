"""Sequence-parallel prefill of a Llama-3-8B-shaped stack: fused tcgen05 GEMM + collective
kernels in every linear against cuBLAS GEMMs with NCCL all-gather / reduce-scatter around them.

    torchrun --nproc-per-node 8 extra/bench_sp_prefill.py --tokens 4096 --layers 32

One forward = `layers` transformer layers over one `tokens`-token sequence whose
residual stream is sharded along the sequence (penny_b200/models/llama_sp.py).
Both backends run the same attention (library SDPA), norm, RoPE and silu*mul
kernels, so the difference is the four linears per layer.  Device time: CUDA
events, L2 flushed between forwards, ranks aligned, median, max over ranks;
the two backends are checked against each other first.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from penny_b200.models.llama_sp import LlamaSPPrefill  # noqa: E402
from penny_b200.models.llama_tp import LlamaConfig  # noqa: E402
from penny_b200.utils import bench_device, initialize_distributed, shutdown  # noqa: E402


def add_args(ap):
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)


def run(rank, world, comm, args):
    """Both backends on an initialised communicator (heap >= 1 GiB); rank 0 prints one JSON line."""
    cfg = LlamaConfig.llama3_8b()
    rows = args.tokens // world
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(args.tokens, cfg.hidden, device="cuda", generator=g).bfloat16()[rank * rows:(rank + 1) * rows]
    x = x.contiguous()
    penny = LlamaSPPrefill(cfg, comm=comm, rank=rank, world=world, tokens=args.tokens, layers=args.layers,
                           backend="penny", seed=2)
    nccl = LlamaSPPrefill(cfg, comm=comm, rank=rank, world=world, tokens=args.tokens, layers=args.layers,
                          backend="nccl", seed=2)
    nccl.layers = penny.layers  # same tensors: one copy of the weights
    # agreement is checked on the first two layers: the fused linears sum the ranks' partials in fp32 and
    # round once, the two-step path rounds every partial to bf16 first, and over 2 x layers reductions
    # that rounding noise adds up (about 5 % of the norm after 32 layers)
    full = penny.layers
    penny.layers = nccl.layers = full[:2]
    a = penny.forward(x).float()
    comm.check()
    b = nccl.forward(x).float()
    rel = ((a - b).norm() / b.norm()).item()
    if not rel < 2e-2:
        raise SystemExit(f"rank {rank}: fused and two-step prefill disagree after 2 layers (relative error {rel})")
    penny.layers = nccl.layers = full
    a, b = penny.forward(x).float(), nccl.forward(x).float()
    rel_full = ((a - b).norm() / b.norm()).item()
    t_p = bench_device(lambda: penny.forward(x), args.warmup, args.iters)["median_us"]
    comm.check()
    t_n = bench_device(lambda: nccl.forward(x), args.warmup, args.iters)["median_us"]
    if rank == 0:
        print(json.dumps({"op": "sp_prefill", "world": world, "tokens": args.tokens, "layers": args.layers,
                          "penny_us": round(t_p, 1), "cublas_nccl_us": round(t_n, 1), "speedup": round(t_n / t_p, 3),
                          "penny_tokens_per_s": round(args.tokens / t_p * 1e6, 1),
                          "baseline_tokens_per_s": round(args.tokens / t_n * 1e6, 1),
                          "relative_difference_2_layers": round(rel, 5),
                          "relative_difference_all_layers": round(rel_full, 5)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    add_args(ap)
    args = ap.parse_args()
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        rank, world, comm = initialize_distributed(heap_bytes=2 << 30)
        run(rank, world, comm, args)
        shutdown()
    else:
        from penny_b200.parallel.comm import Communicator
        torch.cuda.set_device(0)
        comm = Communicator.emulated(1, heap_bytes=2 << 30, timeout_ms=5000)
        try:
            run(0, 1, comm, args)
        finally:
            comm.close()


if __name__ == "__main__":
    main()
