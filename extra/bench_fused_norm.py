"""All-reduce + residual add + RMSNorm in one kernel: every transport against NCCL all-reduce +
this library's add_rmsnorm kernel, at the row counts of a decode batch.

    torchrun --nproc-per-node 8 extra/bench_fused_norm.py [--hidden 4096] [--rows 1 8 64 256] [--out f.jsonl]

Each transport runs where serving runs it: 10 back-to-back calls inside one CUDA graph, alternating
between two input buffers (the way a transformer layer alternates between its two row-parallel
GEMM outputs), L2 flushed and ranks aligned before each replay, device time per call, max over
ranks.  Records carry op="fused_norm" and the message size in bytes, the form the tuner reads.
"""
import torch
import torch.distributed as dist

from _bench_common import Recorder, base_parser
from penny_b200._ext import ops
from penny_b200.utils import bench_graph, initialize_distributed, shutdown


def main(argv=None, ctx=None):
    """ctx: (rank, world, comm) of an already initialised process (extra/sweep_all.py); else set up here."""
    p = base_parser()
    p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--rows", type=int, nargs="*", default=[1, 8, 16, 32, 64, 128, 256])
    args = p.parse_args(argv)
    rank, world, comm = ctx if ctx is not None else initialize_distributed(heap_bytes=int(args.heap_gib * (1 << 30)))
    rec = Recorder(rank, args.out)
    H = args.hidden
    dt = torch.bfloat16
    for rows in args.rows:
        g = torch.Generator(device="cuda").manual_seed(100 + rank + rows)
        src = [(torch.randn(rows, H, device="cuda", generator=g) * 0.5).to(dt) for _ in range(2)]
        g2 = torch.Generator(device="cuda").manual_seed(7)
        res0 = torch.randn(rows, H, device="cuda", generator=g2).to(dt)
        w = (torch.rand(H, device="cuda", generator=g2) + 0.5).to(dt)
        xin = [comm.empty(rows, H, dtype=dt) for _ in range(2)]   # symmetric: every transport may use them
        for a, b in zip(xin, src):
            a.copy_(b)
        out_sym = comm.empty(rows, H, dtype=dt)
        out_loc = torch.empty(rows, H, device="cuda", dtype=dt)
        res = res0.clone()
        nbytes = rows * H * 2
        # oracle: NCCL sum + fp32 norm
        ref = src[0].clone()
        dist.all_reduce(ref)
        z = ref.float() + res0.float()
        want = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()

        buf = [s.clone() for s in src]

        def nccl_pair():
            for i in range(2):
                dist.all_reduce(buf[i])
                ops.add_rmsnorm(buf[i], res, w, out_loc, res, 1e-5)
        t_nccl = None
        if not args.no_nccl:
            t_nccl = bench_graph(nccl_pair, inner=5, warmup=5, iters=30)["median_us"] / 2
            rec.add(op="fused_norm", impl="nccl", algo="all_reduce + add_rmsnorm", world=world, dtype="bf16",
                    rows=rows, hidden=H, bytes=nbytes, t_graph_us=round(t_nccl, 2))
        protos = ["ll", "ll_twoshot", "flag"] + (["nvls", "nvls_oneshot"] if comm.has_multicast else []) + ["auto"]
        for proto in protos:
            if proto == "ll" and rows > 128:
                continue
            out = out_sym if proto in ("nvls", "auto") else out_loc
            res.copy_(res0)
            comm.fused_all_reduce_rmsnorm(xin[0], w, residual=res, out=out, proto=proto)
            comm.check()
            err = (out.float() - want).abs().max().item()
            if not torch.allclose(out.float(), want, atol=args.atol, rtol=2e-2):
                raise SystemExit(f"rank {rank}: fused_norm/{proto} @ {rows} rows differs from NCCL + norm (max abs diff {err})")

            def pair(proto=proto, out=out):
                for i in range(2):
                    comm.fused_all_reduce_rmsnorm(xin[i], w, residual=res, out=out, proto=proto)
            t = bench_graph(pair, inner=5, warmup=5, iters=30)["median_us"] / 2
            comm.check()
            rec.add(op="fused_norm", impl="penny", algo=proto, world=world, dtype="bf16", rows=rows, hidden=H,
                    bytes=nbytes, symmetric=True, t_graph_us=round(t, 2),
                    picked=comm.pick_fused_proto(rows, H, dt) if proto == "auto" else proto,
                    vs_nccl=round(t_nccl / t, 3) if t_nccl else None)
    comm.check()
    rec.close()
    if ctx is None:
        shutdown()


if __name__ == "__main__":
    main()
