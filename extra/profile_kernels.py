"""Small, self-contained launches of this library's hot kernels, sized for a
profiler capture on ONE GPU (a few launches, well under a GB on the device
except where DRAM figures need inputs larger than L2).

    python extra/profile_kernels.py gemm        # tcgen05 GEMM 4096^3, 3 launches
    python extra/profile_kernels.py gemm_pair   # the same on CTA pairs (cta_group::2), 8192^3, 3 launches
    python extra/profile_kernels.py attention   # decode attention, batch 64 x 8 KV heads x 2048
    python extra/profile_kernels.py fused       # all-reduce+residual+RMSNorm, 8 emulated ranks
    python extra/profile_kernels.py allreduce   # two-shot / LL all-reduce, 8 emulated ranks
    python extra/profile_kernels.py attention_fused   # one-launch decode attention (RoPE + KV append + split merge)
    python extra/profile_kernels.py gemm_decode       # decode-batch GEMM: a wide matrix (no cluster) and a narrow one (cluster split-K)
    python extra/profile_kernels.py fused_twoshot     # flag-in-data two-shot all-reduce+RMSNorm, 8 emulated ranks
    python extra/profile_kernels.py collectives       # reduce-scatter / all-gather / all-to-all (push and pipelined), 8 emulated ranks
    python extra/profile_kernels.py moe               # MoE dispatch + combine (and the routing kernels), 8 emulated ranks

Each prints the CUDA-event time per launch so that the same command line can be
run plainly first and under `ncu --clock-control none -k regex:<kernel> -c <n>`
afterwards.
"""
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from penny_b200._ext import ops  # noqa: E402


def timed(fn, n=3):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e3


def main():
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    torch.manual_seed(0)
    if what == "gemm":
        M = N = K = 4096
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t = timed(lambda: ops.gemm_bf16(a, b, c, 256))
        assert ops.gemm_error() == 0
        print(f"gemm_bf16 {M}x{N}x{K}: {t:.1f} us, {2 * M * N * K / t / 1e6:.1f} TFLOP/s")
    elif what == "gemm_pair":
        M = N = K = 8192
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t = timed(lambda: ops.gemm_bf16(a, b, c, 512), n=2)
        assert ops.gemm_error() == 0
        print(f"gemm_bf16 (CTA pairs) {M}x{N}x{K}: {t:.1f} us, {2 * M * N * K / t / 1e6:.1f} TFLOP/s")
    elif what == "attention":
        B, Hq, Hkv, D, L = 64, 32, 8, 128, 2048
        qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
        kc = torch.randn(B, Hkv, L + 16, D, device="cuda").bfloat16()
        vc = torch.randn(B, Hkv, L + 16, D, device="cuda").bfloat16()
        pos = torch.full((B,), L, dtype=torch.int32, device="cuda")
        out = torch.empty(B, Hq * D, device="cuda", dtype=torch.bfloat16)
        splits = 1
        ws = torch.empty(ops.decode_attn_workspace_bytes(B, Hq, splits), dtype=torch.uint8, device="cuda")
        t = timed(lambda: ops.decode_attention(qkv, kc, vc, pos, out, ws, Hq, Hkv, splits, 1 / math.sqrt(D)))
        gb = B * Hkv * (L + 1) * D * 2 * 2 / 1e9
        print(f"decode_attention B={B} Hkv={Hkv} L={L}: {t:.1f} us, {gb / t * 1e6:.0f} GB/s of K+V")
    elif what == "attention_fused":
        # the shard one rank of a TP-8 group sees (4 splits: 256 CTAs) and the TP-1 shape (no split)
        for Hq, Hkv, splits in ((4, 1, 4), (32, 8, 1)):
            B, D, L = 64, 128, 2048
            qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
            kc = torch.randn(B, Hkv, L + 16, D, device="cuda").bfloat16()
            vc = torch.randn(B, Hkv, L + 16, D, device="cuda").bfloat16()
            pos = torch.full((B,), L, dtype=torch.int32, device="cuda")
            out = torch.empty(B, Hq * D, device="cuda", dtype=torch.bfloat16)
            ws = torch.zeros(ops.decode_attn_fused_workspace_bytes(B, Hq, Hkv, splits), dtype=torch.uint8, device="cuda")
            t = timed(lambda: ops.decode_attention_fused(qkv, kc, vc, pos, out, ws, Hq, Hkv, splits, 1 / math.sqrt(D),
                                                         500000.0, False))
            gb = B * Hkv * (L + 1) * D * 2 * 2 / 1e9
            print(f"decode_attention_fused B={B} Hq={Hq} Hkv={Hkv} L={L} splits={splits}: {t:.1f} us, "
                  f"{gb / t * 1e6:.0f} GB/s of K+V (L2-warm when the cache fits)")
    elif what == "gemm_decode":
        B = 64
        x4096 = torch.randn(B, 4096, device="cuda").bfloat16() * 0.1
        for name, N, K in (("gate_up TP1", 28672, 4096), ("qkv TP8", 768, 4096), ("down TP8", 4096, 1792)):
            x = x4096 if K == 4096 else torch.randn(B, K, device="cuda").bfloat16() * 0.1
            w = torch.randn(N, K, device="cuda").bfloat16() * 0.05
            out = torch.empty(B, N, device="cuda", dtype=torch.bfloat16)
            t = timed(lambda: ops.gemm_decode(x, w, out, False, 0, False))
            assert ops.gemm_error() == 0
            print(f"gemm_decode {name} {N}x{K} batch {B}, cluster {ops.gemm_decode_splits(B, N, K)}: {t:.1f} us, "
                  f"{N * K * 2 / t / 1e3:.0f} GB/s of W (back-to-back launches: W of {N * K * 2 >> 20} MiB "
                  f"{'stays in' if N * K * 2 < (100 << 20) else 'exceeds'} L2)")
    elif what in ("fused_twoshot", "collectives"):
        from penny_b200.parallel.comm import Communicator
        comm = Communicator.emulated(8, heap_bytes=256 << 20)
        if what == "fused_twoshot":
            rows, hidden = 64, 4096
            x = [torch.randn(rows, hidden, device="cuda").bfloat16() for _ in range(8)]
            r = [torch.randn(rows, hidden, device="cuda").bfloat16() for _ in range(8)]
            w = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
            o = [torch.empty_like(t) for t in x]
            t = timed(lambda: comm.fused_all_reduce_rmsnorm(x, w, residual=r, out=o, proto="ll_twoshot"))
            print(f"fused all-reduce+rmsnorm (ll_twoshot) rows={rows}, 8 emulated ranks on one GPU: {t:.1f} us")
        else:
            n = 1 << 22  # 8 MiB per rank
            x = [torch.randn(n, device="cuda").bfloat16() for _ in range(8)]
            for name, fn in (("reduce_scatter push", lambda: comm.reduce_scatter(x, algo="push")),
                             ("reduce_scatter pipelined", lambda: comm.reduce_scatter(x, algo="pipelined")),
                             ("all_gather push", lambda: comm.all_gather(x, algo="push")),
                             ("all_to_all push", lambda: comm.all_to_all(x, algo="push")),
                             ("all_to_all pipelined", lambda: comm.all_to_all(x, algo="pipelined"))):
                t = timed(fn)
                print(f"{name} {n * 2 >> 20} MiB per rank bf16, 8 emulated ranks on one GPU: {t:.1f} us")
        comm.check()
        comm.close()
    elif what == "moe":
        from penny_b200.models.moe_ep import MoeConfig, MoeEPLayer
        from penny_b200.parallel.comm import Communicator
        comm = Communicator.emulated(8, heap_bytes=256 << 20)
        cfg = MoeConfig(hidden=1024, ffn=2048, experts=8, topk=2)
        tokens = 1024
        layer = MoeEPLayer(cfg, comm, tokens)
        xs = [torch.randn(tokens, cfg.hidden, device="cuda").bfloat16() for _ in range(8)]
        t = timed(lambda: layer.forward(xs))
        print(f"MoE EP layer, 8 emulated ranks on one GPU, {tokens} tokens per rank, hidden {cfg.hidden}, "
              f"ffn {cfg.ffn}: {t:.1f} us per forward (routing + dispatch + expert GEMMs + combine)")
        comm.check()
        comm.close()
    elif what in ("fused", "allreduce"):
        from penny_b200.parallel.comm import Communicator
        comm = Communicator.emulated(8, heap_bytes=256 << 20)
        if what == "fused":
            rows, hidden = 64, 4096
            x = [torch.randn(rows, hidden, device="cuda").bfloat16() for _ in range(8)]
            r = [torch.randn(rows, hidden, device="cuda").bfloat16() for _ in range(8)]
            w = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
            o = [torch.empty_like(t) for t in x]
            for proto in ("ll", "flag"):
                t = timed(lambda: comm.fused_all_reduce_rmsnorm(x, w, residual=r, out=o, proto=proto))
                print(f"fused all-reduce+rmsnorm ({proto}) rows={rows}, 8 emulated ranks on one GPU: {t:.1f} us")
        else:
            for n, algo in ((4096, "oneshot_ll"), (1 << 24, "twoshot")):
                x = [torch.randn(n, device="cuda").bfloat16() for _ in range(8)]
                o = [torch.empty_like(t) for t in x]
                t = timed(lambda: comm.all_reduce(x, out=o, algo=algo))
                print(f"all_reduce {algo} n={n} bf16, 8 emulated ranks on one GPU: {t:.1f} us")
        comm.check()
        comm.close()
    else:
        raise SystemExit(f"unknown target {what}")


if __name__ == "__main__":
    main()
