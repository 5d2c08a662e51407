"""Shared plumbing of the extra/benchmark_*.py scripts: arguments, data, JSON lines."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS = 900.0
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def base_parser(default_start=10, default_range=19):
    p = argparse.ArgumentParser()
    p.add_argument("--dtype", default="bf16", choices=list(DTYPES))
    p.add_argument("--start-pow", type=int, default=default_start, help="first size = 2^start_pow bytes")
    p.add_argument("--range", type=int, default=default_range, help="number of power-of-two sizes")
    p.add_argument("--num-tests", type=int, default=100)
    p.add_argument("--warmup", type=int, default=20)
    p.add_argument("--atol", type=float, default=1e-1)
    p.add_argument("--rtol", type=float, default=1e-2)
    p.add_argument("--symmetric", action="store_true", help="tensors in the symmetric heap")
    p.add_argument("--no-nccl", action="store_true")
    p.add_argument("--profile-mode", default="none", choices=["none", "file"])
    p.add_argument("--heap-gib", type=float, default=6.0)
    p.add_argument("--out", default="")
    return p


class Recorder:
    def __init__(self, rank, out):
        self.rank, self.out, self.rows = rank, out, []

    def add(self, **rec):
        self.rows.append(rec)
        if self.rank == 0:
            print(json.dumps(rec), flush=True)

    def close(self):
        if self.rank == 0 and self.out:
            with open(self.out, "a") as f:
                for r in self.rows:
                    f.write(json.dumps(r) + "\n")


def uniform(n, dtype, rank):
    g = torch.Generator(device="cuda").manual_seed(rank)
    return (torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dtype)
