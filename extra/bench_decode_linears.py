"""The four linears of a Llama-3-8B layer at a decode batch, one GPU: this library's
decode GEMM (`gemm_decode`: tcgen05, cluster split-K, programmatic dependent launch)
against cuBLAS.

    python extra/bench_decode_linears.py [--batch 64] [--tp 1] [--layers 8] [--sweep]

`--tp N` uses the shard shapes a rank of an N-way tensor-parallel group sees.
Three views:
  * each GEMM alone, eager calls, CUDA events, L2 flushed between calls (includes
    the launch path of each implementation); `--sweep` adds every cluster size;
  * the same GEMM replayed back to back from a CUDA graph over 8 distinct weight
    copies (so the weights come from HBM): device time per call without the host;
  * the four linears (+ silu*mul) of `--layers` layers with distinct weights
    replayed from ONE CUDA graph, with and without programmatic dependent launch:
    microseconds per layer and streamed GB/s.
Results are compared between the two implementations before timing.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from penny_b200._ext import ops  # noqa: E402
from penny_b200.utils import bench_device, bench_graph  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--sweep", action="store_true", help="time every cluster size of the decode GEMM")
    args = ap.parse_args()
    B, H, L, tp = args.batch, 4096, args.layers, args.tp
    F = 14336 // tp
    QKV = 6144 // tp
    HA = 4096 // tp      # o_proj input width on one rank
    V = 128256 // tp

    def rnd(*s):
        return (torch.randn(*s, device="cuda") * 0.02).bfloat16()

    shapes = [("qkv", QKV, H), ("o_proj", H, HA), ("gate_up", 2 * F, H), ("down", H, F), ("lm_head", V, H)]
    # ---- single GEMMs: eager (with launch path) and in-graph over distinct weights
    for name, N, K in shapes:
        copies = max(1, min(8, (1 << 30) // (N * K * 2)))
        x = rnd(B, K).mul_(50)
        ws = [rnd(N, K) for _ in range(copies)]
        o1 = torch.empty(B, N, device="cuda", dtype=torch.bfloat16)
        o2 = torch.empty_like(o1)
        t_c = bench_device(lambda: torch.matmul(x, ws[0].t(), out=o1), 3, 20)["median_us"]
        t_s = bench_device(lambda: ops.gemm_decode(x, ws[0], o2), 3, 20)["median_us"]
        assert ops.gemm_error() == 0
        err = (o1.float() - o2.float()).abs().max().item()
        gb = N * K * 2 / 1e9

        def many(f):
            def run():
                for w in ws:
                    f(w)
            return run
        g_c = bench_graph(many(lambda w: torch.matmul(x, w.t(), out=o1)), inner=1, warmup=3, iters=20)["median_us"] / copies
        g_s = bench_graph(many(lambda w: ops.gemm_decode(x, w, o2)), inner=1, warmup=3, iters=20)["median_us"] / copies
        print(f"{name:8s} N={N:6d} K={K:5d} S={ops.gemm_decode_splits(B, N, K)}: eager cuBLAS {t_c:7.1f} us | gemm_decode "
              f"{t_s:7.1f} us || in graph cuBLAS {g_c:7.2f} us ({gb / g_c * 1e6:5.0f} GB/s) | gemm_decode {g_s:7.2f} us "
              f"({gb / g_s * 1e6:5.0f} GB/s) | max abs diff {err:.3g}", flush=True)
        if args.sweep:
            row = []
            for s in range(1, min(8, K // 64) + 1):
                t = bench_graph(many(lambda w: ops.gemm_decode(x, w, o2, False, s)), inner=1, warmup=3,
                                iters=10)["median_us"] / copies
                row.append(f"S={s}: {t:.2f}")
            print("         in graph by cluster size, us: " + "  ".join(row), flush=True)
            row = []
            for s in range(1, min(8, K // 64) + 1):
                t = bench_graph(many(lambda w: ops.gemm_decode(x, w, o2, False, s, True, -1, 200)), inner=1, warmup=3,
                                iters=10)["median_us"] / copies
                row.append(f"S={s}: {t:.2f}")
            print("         ... with a 200 KB ring:           " + "  ".join(row), flush=True)
        assert ops.gemm_error() == 0
        del x, ws, o1, o2

    # ---- a layer's linears from one CUDA graph
    layers = []
    for _ in range(L):
        wg, wu = rnd(F, H), rnd(F, H)
        layers.append(dict(qkv=rnd(QKV, H), o=rnd(H, HA), gu=torch.cat([wg, wu], 0).contiguous(),
                           gu_il=torch.stack([wg.view(F // 64, 64, H), wu.view(F // 64, 64, H)], 1)
                           .reshape(2 * F, H).contiguous(), down=rnd(H, F)))
    x, a_in, act_in = rnd(B, H).mul_(50), rnd(B, HA).mul_(50), rnd(B, F).mul_(50)
    e = lambda n: torch.empty(B, n, device="cuda", dtype=torch.bfloat16)  # noqa: E731
    qkv, o, gu, act, d = e(QKV), e(H), e(2 * F), e(F), e(H)

    def cublas():
        for l in layers:
            torch.matmul(x, l["qkv"].t(), out=qkv)
            torch.matmul(a_in, l["o"].t(), out=o)
            torch.matmul(x, l["gu"].t(), out=gu)
            ops.silu_mul(gu, act)
            torch.matmul(act_in, l["down"].t(), out=d)

    def decode(pdl):
        def run():
            for l in layers:
                ops.gemm_decode(x, l["qkv"], qkv, False, 0, pdl)
                ops.gemm_decode(a_in, l["o"], o, False, 0, pdl)
                ops.gemm_decode(x, l["gu_il"], act, True, 0, pdl)
                ops.gemm_decode(act_in, l["down"], d, False, 0, pdl)
        return run

    cublas()
    ref_act = act.clone()
    decode(True)()
    torch.cuda.synchronize()
    assert ops.gemm_error() == 0
    diff = (ref_act.float() - act.float()).abs().max().item()
    assert diff < 0.05 * ref_act.float().abs().max().item() + 1e-2, diff
    gb = L * (QKV * H + H * HA + 2 * F * H + H * F) * 2 / 1e9
    for name, f in (("cuBLAS + silu_mul", cublas), ("gemm_decode, serialised", decode(False)),
                    ("gemm_decode, dependent launch", decode(True))):
        us = bench_graph(f, inner=1, warmup=3, iters=20)["median_us"]
        print(f"{name:30s}: {us / L:7.2f} us per layer ({gb / us * 1e6:5.0f} GB/s of weights)", flush=True)
    assert ops.gemm_error() == 0


if __name__ == "__main__":
    main()
