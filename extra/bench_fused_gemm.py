"""Sequence-parallel linears at prefill size: fused tcgen05 GEMM + collective in one
kernel against the two-step baseline (cuBLAS GEMM, then NCCL).

    torchrun --nproc-per-node 8 extra/bench_fused_gemm.py --tokens 4096

Shapes are the Llama-3-8B layer at TP = world: o_proj and down_proj as
GEMM -> reduce-scatter, qkv and gate/up as all-gather -> GEMM.  For every op it
prints device time (CUDA events, L2 flushed, ranks aligned, max over ranks) and
the fraction of the roofline max(FLOPs / measured GEMM peak, NVLink bytes /
measured link bandwidth).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from penny_b200._ext import ops  # noqa: E402
from penny_b200.utils import bench_device, initialize_distributed, shutdown  # noqa: E402


def peaks():
    tf, link = 1590.0, 770.0  # fallback GEMM peak (TFLOP/s) and measured peer-copy bandwidth (GB/s)
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        tf = float(json.load(open(p))["bf16_tflops"])
        src = "measured"
    except (OSError, KeyError, ValueError):
        src = "fallback"
    return tf, link, src


def add_args(ap):
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--side-ctas", type=int, default=0)


def run(rank, world, comm, args):
    """All four linears on an initialised communicator (heap >= 2 GiB); rank 0 prints one JSON line per op."""
    tf, link, src = peaks()
    M, H, F, D = args.tokens, 4096, 14336, 128
    qkv_n = (32 + 2 * 8) * D // world
    g = torch.Generator(device="cuda").manual_seed(rank)

    def rnd(*s):
        return (torch.randn(*s, device="cuda", generator=g) * 0.05).bfloat16()
    cases = [("o_proj gemm->rs", "rs", H, 32 * D // world), ("down gemm->rs", "rs", H, F // world),
             ("qkv ag->gemm", "ag", qkv_n, H), ("gate_up ag->gemm", "ag", 2 * F // world, H)]
    for name, kind, N, K in cases:
        w = rnd(N, K)
        if kind == "rs":
            a = rnd(M, K)
            out = torch.empty(M // world, N, device="cuda", dtype=torch.bfloat16)
            full = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

            def fused():
                comm.gemm_reduce_scatter(a, w, out=out)

            def base():
                torch.matmul(a, w.t(), out=full)
                dist.reduce_scatter_tensor(out, full)
            fused()
            ref = torch.empty_like(out)
            torch.matmul(a, w.t(), out=full)
            dist.reduce_scatter_tensor(ref, full)
            wire = M * N * 2 * (world - 1) / world  # bytes leaving each GPU
        else:
            a = rnd(M // world, K)
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            gathered = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)

            def fused():
                comm.all_gather_gemm(a, w, out=out, side_ctas=args.side_ctas)

            def base():
                dist.all_gather_into_tensor(gathered, a)
                torch.matmul(gathered, w.t(), out=out)
            fused()
            got = out.clone()
            base()
            ref, out_chk = out.clone(), got
            wire = M * K * 2 * (world - 1) / world
        assert ops.gemm_error() == 0
        comm.check()
        chk = out if kind == "rs" else out_chk
        err = (chk.float() - ref.float()).abs().max().item()
        scale = ref.float().abs().max().item() + 1e-6
        if err > 0.05 * scale:
            raise SystemExit(f"rank {rank}: {name} differs from the two-step baseline (max abs {err}, scale {scale})")
        t_f = bench_device(fused, args.warmup, args.iters)["median_us"]
        t_b = bench_device(base, args.warmup, args.iters)["median_us"]
        flops = 2.0 * M * N * K
        roof_us = max(flops / (tf * 1e6), wire / (link * 1e3))
        if rank == 0:
            print(json.dumps({"op": name, "world": world, "M": M, "N": N, "K": K, "fused_us": round(t_f, 1),
                              "cublas_plus_nccl_us": round(t_b, 1), "speedup": round(t_b / t_f, 3),
                              "tflops": round(flops / t_f / 1e6, 1), "roofline_us": round(roof_us, 1),
                              "frac_of_roofline": round(roof_us / t_f, 3), "peaks": src,
                              "bound": "compute" if flops / (tf * 1e6) > wire / (link * 1e3) else "nvlink"}), flush=True)
    assert ops.gemm_error() == 0
    comm.check()


def main():
    ap = argparse.ArgumentParser()
    add_args(ap)
    args = ap.parse_args()
    rank, world, comm = initialize_distributed(heap_bytes=2 << 30)
    run(rank, world, comm, args)
    shutdown()


if __name__ == "__main__":
    main()
