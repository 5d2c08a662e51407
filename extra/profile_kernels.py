"""Small, self-contained launches of this library's hot kernels, sized for a
profiler capture on ONE GPU (a few launches, well under a GB on the device
except where DRAM figures need inputs larger than L2).

    python extra/profile_kernels.py gemm        # tcgen05 GEMM 4096^3, 3 launches
    python extra/profile_kernels.py gemm_pair   # the same on CTA pairs (cta_group::2), 8192^3, 3 launches
    python extra/profile_kernels.py attention   # decode attention, batch 64 x 8 KV heads x 2048
    python extra/profile_kernels.py fused       # all-reduce+residual+RMSNorm, 8 emulated ranks
    python extra/profile_kernels.py allreduce   # two-shot / LL all-reduce, 8 emulated ranks

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
