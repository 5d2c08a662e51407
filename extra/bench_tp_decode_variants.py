"""TP decode step time for several configurations in one process group (the headline numbers come
from bench.py; this is the ablation around them).

    torchrun --nproc-per-node 8 extra/bench_tp_decode_variants.py [--batches 1 8 64 256]
        [--protos auto ll flag nvls nvls_oneshot] [--linears penny cublas] [--steps 20]

For every (batch, transport of the fused all-reduce + RMSNorm, linear implementation) it builds the
Llama-3-8B-shaped decoder with a 2048-token synthetic KV cache, captures the step in a CUDA graph and
times `--steps` replays with CUDA events (5 warm-up replays, barrier + synchronize on both sides, max
over ranks).  One JSON line per configuration.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batches", type=int, nargs="*", default=[64])
    ap.add_argument("--protos", nargs="*", default=["auto"])
    ap.add_argument("--linears", nargs="*", default=["auto"])
    ap.add_argument("--backends", nargs="*", default=["penny"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--kv-len", type=int, default=2048)
    ap.add_argument("--no-pdl", action="store_true", help="also time every configuration without dependent launch")
    args = ap.parse_args()
    from penny_b200._ext import ops
    from penny_b200.models.llama_tp import LlamaConfig, LlamaTPDecoder
    from penny_b200.utils import initialize_distributed
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, comm = 0, None
    if world > 1:
        rank, world, comm = initialize_distributed(heap_bytes=2 << 30)
    else:
        torch.cuda.set_device(0)
    cfg = LlamaConfig.llama3_8b()
    for batch in args.batches:
        for backend in args.backends:
            for linears in args.linears:
                for proto in (args.protos if backend == "penny" and world > 1 else ["auto"]):
                    if proto == "ll" and batch > 128:
                        continue
                    for pdl in ([True, False] if args.no_pdl else [True]):
                        ops.set_pdl(1 if pdl else 0)
                        model = LlamaTPDecoder(cfg, comm=comm, rank=rank, world=world, max_batch=batch,
                                               max_len=args.kv_len + args.steps + 16, backend=backend, proto=proto,
                                               linears=linears, pdl=pdl, process_group=None)
                        model.fill_synthetic_kv(args.kv_len)
                        model.capture()
                        for _ in range(5):
                            model.step_device()
                        torch.cuda.synchronize()
                        if world > 1:
                            dist.barrier()
                            torch.cuda.synchronize()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                        for _ in range(args.steps):
                            model.step_device()
                        e1.record()
                        torch.cuda.synchronize()
                        ms = e0.elapsed_time(e1) / args.steps
                        if world > 1:
                            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
                            dist.all_reduce(t, op=dist.ReduceOp.MAX)
                            ms = t.item()
                            comm.check()
                        if rank == 0:
                            print(json.dumps({"world": world, "batch": batch, "backend": backend, "proto": model.proto,
                                              "asked_proto": proto, "linears": model.linears, "pdl": pdl,
                                              "ms_per_step": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3, 1)}),
                                  flush=True)
                        del model
                        torch.cuda.empty_cache()
    ops.set_pdl(-1)
    if comm is not None:
        torch.cuda.synchronize()
        comm.barrier()
        comm.close()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
