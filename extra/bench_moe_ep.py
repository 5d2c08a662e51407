"""Mixtral-8x7B-shaped MoE layer with expert parallelism = world size.

    torchrun --nproc-per-node 8 extra/bench_moe_ep.py --tokens 4096

Times one layer forward (router, dispatch, expert FFN, combine) with this
library's dispatch / combine kernels against the same layer over NCCL
all_to_all_single, checks the two against each other, and prints the
dispatch + combine wire bytes per rank.  Device time: CUDA events, L2 flushed,
ranks aligned, max over ranks.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from penny_b200.models.moe_ep import MoeConfig, MoeEPLayer  # noqa: E402
from penny_b200.utils import bench_device, initialize_distributed, shutdown  # noqa: E402


def add_args(ap):
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ffn", type=int, default=14336)


def run(rank, world, comm, args):
    """One layer, both backends, on an initialised communicator (heap >= 3 GiB); rank 0 prints one JSON line."""
    cfg = MoeConfig.mixtral_8x7b()
    cfg.ffn = args.ffn
    if cfg.experts % world:
        cfg.experts = world
    penny = MoeEPLayer(cfg, comm, tokens=args.tokens, cap_factor=2.0, backend="penny", seed=1)
    nccl = MoeEPLayer(cfg, comm, tokens=args.tokens, cap_factor=2.0, backend="nccl", seed=1)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x = torch.randn(args.tokens, cfg.hidden, device="cuda", generator=g).bfloat16()
    a = penny.forward(x)
    comm.check()
    b = nccl.forward(x)
    err = (a.float() - b.float()).abs().max().item()
    if err > 0.02 * (b.float().abs().max().item() + 1e-6) + 1e-3:
        raise SystemExit(f"rank {rank}: penny and NCCL MoE layers disagree (max abs {err})")
    t_p = bench_device(lambda: penny.forward(x), args.warmup, args.iters)["median_us"]
    comm.check()
    t_n = bench_device(lambda: nccl.forward(x), args.warmup, args.iters)["median_us"]
    if rank == 0:
        rows = args.tokens * cfg.topk
        print(json.dumps({"op": "moe_ep_layer", "world": world, "tokens_per_rank": args.tokens, "experts": cfg.experts,
                          "topk": cfg.topk, "hidden": cfg.hidden, "ffn": cfg.ffn, "penny_us": round(t_p, 1),
                          "nccl_all_to_all_us": round(t_n, 1), "speedup": round(t_n / t_p, 3),
                          "wire_mb_per_rank_each_way": round(rows * cfg.hidden * 2 * (world - 1) / world / 1e6, 1)}),
              flush=True)


def main():
    ap = argparse.ArgumentParser()
    add_args(ap)
    args = ap.parse_args()
    rank, world, comm = initialize_distributed(heap_bytes=3 << 30)
    if comm is None or world < 2:
        raise SystemExit("expert parallelism needs >= 2 ranks: launch with torchrun --nproc-per-node N")
    run(rank, world, comm, args)
    shutdown()


if __name__ == "__main__":
    main()
