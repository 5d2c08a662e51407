"""Algorithm choice per (operation, dtype, world size, message size) from MEASURED times.

`extra/benchmark_allreduce.py --out sweep.jsonl` writes one JSON line per (size,
algorithm); `Tuner.from_sweep` keeps, for every size, the fastest algorithm, and
`Tuner.pick` looks a size up (nearest measured size at or above it).  The table
is cached as JSON (`PENNY_TUNER_CACHE`, default ~/.cache/penny_b200/tuner.json)
and a built-in default – taken from sweeps of this script on an 8 x B200
NVSwitch box – is used when no cache exists.  Overrides: `PENNY_ALGO=<name>`
forces one algorithm; `VLLM_CUSTOM_ALLREDUCE_ALGO` keeps its meaning for the
drop-in CustomAllreduce (1stage|oneshot|2stage|twoshot), as in the reference
(csrc/custom_all_reduce.cuh:803-818), whose own choice is a fixed size threshold
(:831-841).
"""
from __future__ import annotations

import json
import os
from bisect import bisect_left
from typing import Dict, List, Optional, Tuple

DEFAULT_CACHE = os.path.join(os.path.expanduser("~"), ".cache", "penny_b200", "tuner.json")

# (upper size bound in bytes, algorithm) per world size; the last entry has no bound.
# Symmetric (heap) tensors may use "nvls" without staging; others fall back to "twoshot".
BUILTIN: Dict[str, List[Tuple[Optional[int], str]]] = {
    "2": [(64 << 10, "oneshot_ll"), (2 << 20, "oneshot"), (None, "twoshot")],
    "4": [(32 << 10, "oneshot_ll"), (None, "nvls")],
    "8": [(32 << 10, "oneshot_ll"), (None, "nvls")],
}


class Tuner:
    def __init__(self, table: Optional[Dict[str, List[Tuple[Optional[int], str]]]] = None, source: str = "builtin"):
        self.table = table or {k: list(v) for k, v in BUILTIN.items()}
        self.source = source
        self.records = 0

    # ---------------------------------------------------------------- building
    @classmethod
    def from_sweep(cls, path: str, op: str = "all_reduce", dtype: Optional[str] = None) -> "Tuner":
        best: Dict[Tuple[int, int], Tuple[float, str]] = {}
        with open(path) as f:
            for line in f:
                try:
                    r = json.loads(line)
                except ValueError:
                    continue
                if r.get("op") != op or r.get("impl") != "penny" or r.get("algo") in (None, "auto", "custom_all_reduce"):
                    continue
                if dtype and r.get("dtype") != dtype:
                    continue
                t = r.get("t_graph_us") or r["t_us"]
                key = (int(r["world"]), int(r["bytes"]))
                if key not in best or t < best[key][0]:
                    best[key] = (t, r["algo"])
        table: Dict[str, List[Tuple[Optional[int], str]]] = {}
        for (world, size), (_, algo) in sorted(best.items()):
            rows = table.setdefault(str(world), [])
            if rows and rows[-1][1] == algo:
                rows[-1] = (size, algo)
            else:
                rows.append((size, algo))
        for rows in table.values():
            rows[-1] = (None, rows[-1][1])
        t = cls(table, source=path)
        t.records = len(best)  # (world, size) points the table was built from; 0: the built-in table is in use
        return t

    @classmethod
    def load(cls, path: Optional[str] = None) -> "Tuner":
        path = path or os.environ.get("PENNY_TUNER_CACHE", DEFAULT_CACHE)
        try:
            with open(path) as f:
                raw = json.load(f)
            return cls({k: [(b, a) for b, a in v] for k, v in raw.items()}, source=path)
        except (OSError, ValueError):
            return cls()

    def save(self, path: Optional[str] = None) -> str:
        path = path or os.environ.get("PENNY_TUNER_CACHE", DEFAULT_CACHE)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as f:
            json.dump(self.table, f, indent=1)
        return path

    # ----------------------------------------------------------------- lookup
    def pick(self, nbytes: int, world: int, has_multicast: bool = True, symmetric: bool = True) -> str:
        forced = os.environ.get("PENNY_ALGO")
        if forced:
            return forced
        rows = self.table.get(str(world))
        if not rows:
            return "ring_standard" if world not in (2, 4, 6, 8) else "twoshot"
        bounds = [b if b is not None else float("inf") for b, _ in rows]
        algo = rows[min(bisect_left(bounds, nbytes), len(rows) - 1)][1]
        if algo.startswith("nvls") and not has_multicast:
            algo = "oneshot" if nbytes <= (256 << 10) else "twoshot"
        return algo


def _main(argv=None) -> int:
    """python -m penny_b200.parallel.tuner sweep.jsonl [--out cache.json] [--dtype bf16]

    Turns the JSON lines of `extra/benchmark_allreduce.py --out sweep.jsonl` into the cached table."""
    import argparse
    ap = argparse.ArgumentParser(prog="python -m penny_b200.parallel.tuner", description=_main.__doc__)
    ap.add_argument("sweep", help="JSON-lines file written by extra/benchmark_allreduce.py --out")
    ap.add_argument("--out", default=None, help=f"cache file (default: PENNY_TUNER_CACHE or {DEFAULT_CACHE})")
    ap.add_argument("--dtype", default=None, help="only use records of this dtype (e.g. bf16)")
    args = ap.parse_args(argv)
    t = Tuner.from_sweep(args.sweep, dtype=args.dtype)
    if not t.records:
        print("no usable records (op=all_reduce, impl=penny, a named algorithm) in", args.sweep)
        return 1
    path = t.save(args.out)
    for world, rows in sorted(t.table.items(), key=lambda kv: int(kv[0])):
        print(f"world {world}: " + ", ".join(f"<= {b} B: {a}" if b is not None else f"above: {a}" for b, a in rows))
    print("written to", path)
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
