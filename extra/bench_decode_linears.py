"""The four linears of a Llama-3-8B layer at a decode batch, one GPU: cuBLAS against
this library's weight-streaming `gemm_skinny`.

    python extra/bench_decode_linears.py [--batch 64] [--layers 8]

Two views:
  * each GEMM alone, eager calls, CUDA events, L2 flushed between calls (includes
    the launch path of each implementation);
  * the four linears (+ silu*mul) of `--layers` layers with distinct weights
    replayed from ONE CUDA graph, so no weight is in L2 when it is read and the
    host is out of the picture: microseconds per layer and streamed GB/s.
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
    ap.add_argument("--layers", type=int, default=8)
    args = ap.parse_args()
    B, H, F, L = args.batch, 4096, 14336, args.layers

    def rnd(*s):
        return (torch.randn(*s, device="cuda") * 0.02).bfloat16()

    # ---- single GEMMs, eager
    for name, N, K in [("qkv", 6144, H), ("o_proj", H, H), ("gate_up", 2 * F, H), ("down", H, F), ("lm_head", 128256, H)]:
        x, w = rnd(B, K).mul_(50), rnd(N, K)
        o1 = torch.empty(B, N, device="cuda", dtype=torch.bfloat16)
        o2 = torch.empty_like(o1)
        t_c = bench_device(lambda: torch.matmul(x, w.t(), out=o1), 3, 20)["median_us"]
        t_s = bench_device(lambda: ops.gemm_skinny(x, w, o2), 3, 20)["median_us"]
        assert ops.gemm_error() == 0
        err = (o1.float() - o2.float()).abs().max().item()
        gb = N * K * 2 / 1e9
        print(f"{name:8s} N={N:6d} K={K:5d}: cuBLAS {t_c:7.1f} us ({gb / t_c * 1e6:5.0f} GB/s) | gemm_skinny {t_s:7.1f} us "
              f"({gb / t_s * 1e6:5.0f} GB/s) | max abs diff {err:.3g}", flush=True)
        del x, w, o1, o2

    # ---- a layer's linears from one CUDA graph
    layers = []
    for _ in range(L):
        wg, wu = rnd(F, H), rnd(F, H)
        layers.append(dict(qkv=rnd(6144, H), o=rnd(H, H), gu=torch.cat([wg, wu], 0).contiguous(),
                           gu_il=torch.stack([wg.view(F // 64, 64, H), wu.view(F // 64, 64, H)], 1)
                           .reshape(2 * F, H).contiguous(), down=rnd(H, F)))
    x, a_in, act_in = rnd(B, H).mul_(50), rnd(B, H).mul_(50), rnd(B, F).mul_(50)
    e = lambda n: torch.empty(B, n, device="cuda", dtype=torch.bfloat16)  # noqa: E731
    qkv, o, gu, act, d = e(6144), e(H), e(2 * F), e(F), e(H)

    def cublas():
        for l in layers:
            torch.matmul(x, l["qkv"].t(), out=qkv)
            torch.matmul(a_in, l["o"].t(), out=o)
            torch.matmul(x, l["gu"].t(), out=gu)
            ops.silu_mul(gu, act)
            torch.matmul(act_in, l["down"].t(), out=d)

    def skinny():
        for l in layers:
            ops.gemm_skinny(x, l["qkv"], qkv)
            ops.gemm_skinny(a_in, l["o"], o)
            ops.gemm_skinny(x, l["gu"], gu)
            ops.silu_mul(gu, act)
            ops.gemm_skinny(act_in, l["down"], d)

    def skinny_fused():
        for l in layers:
            ops.gemm_skinny(x, l["qkv"], qkv)
            ops.gemm_skinny(a_in, l["o"], o)
            ops.gemm_skinny(x, l["gu_il"], act, True)
            ops.gemm_skinny(act_in, l["down"], d)

    def mixed():  # cuBLAS for the narrow ones, fused gemm_skinny for gate/up
        for l in layers:
            torch.matmul(x, l["qkv"].t(), out=qkv)
            torch.matmul(a_in, l["o"].t(), out=o)
            ops.gemm_skinny(x, l["gu_il"], act, True)
            torch.matmul(act_in, l["down"].t(), out=d)

    cublas()
    ref_act = act.clone()
    skinny_fused()
    torch.cuda.synchronize()
    assert ops.gemm_error() == 0
    diff = (ref_act.float() - act.float()).abs().max().item()
    assert diff < 0.05 * ref_act.float().abs().max().item() + 1e-2, diff
    gb = L * (6144 * H + H * H + 2 * F * H + H * F) * 2 / 1e9
    for name, f in (("cuBLAS + silu_mul", cublas), ("gemm_skinny + silu_mul", skinny),
                    ("gemm_skinny, fused silu", skinny_fused), ("cuBLAS + fused gate/up", mixed)):
        us = bench_graph(f, inner=1, warmup=3, iters=20)["median_us"]
        print(f"{name:24s}: {us / L:7.1f} us per layer ({gb / us * 1e6:5.0f} GB/s of weights)", flush=True)
    assert ops.gemm_error() == 0


if __name__ == "__main__":
    main()
