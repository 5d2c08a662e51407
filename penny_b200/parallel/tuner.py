"""Algorithm choice per (operation, world size, dtype, memory class, message size) from MEASURED times.

The sweep scripts (`extra/benchmark_allreduce.py`, `benchmark_all_gather.py`,
`benchmark_reduce_scatter.py`, `benchmark_exchange.py --all-to-all`,
`bench_fused_norm.py`) write one JSON line per (size, algorithm).
`Tuner.from_sweep` keeps the fastest algorithm of every size and merges runs of
equal winners into (upper byte bound, algorithm) rows; `Tuner.pick` looks a size
up.  Every `Communicator` is given a tuner when it is created:

  * `PENNY_TUNER_CACHE` (a JSON file written by `python -m penny_b200.parallel.tuner`),
    when it exists;
  * else the built-in table `tuner_table.json` next to this file, produced by the
    same command from sweeps on an 8 x B200 NVSwitch box at 2, 4 and 8 GPUs in
    bf16 and fp32 (20 warm-up + 100 timed calls per point);
  * world sizes or operations a table does not cover fall back to the rule
    compiled into the native communicator.

The all-reduce rows are also installed in the native communicator
(`comm_set_tuning`), so `algo="auto"` means the same thing through every entry
point (Python, the handle API, the drop-in CustomAllreduce).  Overrides:
`PENNY_ALGO=<name>` forces one all-reduce algorithm; `VLLM_CUSTOM_ALLREDUCE_ALGO`
keeps its meaning for the drop-in CustomAllreduce (1stage|oneshot|2stage|twoshot),
as in the reference (csrc/custom_all_reduce.cuh:803-818), whose own choice is a
fixed size threshold (:831-841).

Table layout: table[op][world][dtype][memory class] = [[max_bytes or null, algo], ...]
with memory class "sym" (tensors from `Communicator.empty`) or "any".
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Tuple

DEFAULT_CACHE = os.path.join(os.path.expanduser("~"), ".cache", "penny_b200", "tuner.json")
BUILTIN_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tuner_table.json")

OPS = ("all_reduce", "reduce_scatter", "all_gather", "all_to_all", "fused_norm")
Rows = List[Tuple[Optional[int], str]]

# Used only when neither a cache nor the built-in file can be read.
FALLBACK: Dict[str, dict] = {
    "all_reduce": {
        "2": {"bf16": {"any": [(64 << 10, "oneshot_ll"), (2 << 20, "oneshot"), (None, "twoshot")]}},
        "4": {"bf16": {"any": [(64 << 10, "oneshot_ll"), (None, "nvls")]}},
        "8": {"bf16": {"any": [(64 << 10, "oneshot_ll"), (None, "nvls")]}},
    },
}


def _dtype_key(dtype) -> str:
    s = str(dtype).replace("torch.", "")
    return {"bfloat16": "bf16", "float16": "fp16", "float32": "fp32"}.get(s, s)


class Tuner:
    def __init__(self, table: Optional[dict] = None, source: str = "fallback"):
        self.table = table if table is not None else json.loads(json.dumps(FALLBACK))
        self.source = source
        self.records = 0

    # ---------------------------------------------------------------- building
    @classmethod
    def from_sweep(cls, paths, dtype: Optional[str] = None, tolerance: float = 0.0, both_dtypes=()) -> "Tuner":
        """Builds the table from one or several JSON-lines files.  Records need
        op, impl == "penny", algo, world, dtype, bytes and t_us (t_graph_us is preferred
        when present: it is what a call costs inside a serving engine's CUDA graph).
        Several records of one point (re-measurements in later files): the fastest counts.
        tolerance: an algorithm within this fraction of the best keeps the previous
        size's winner (fewer, longer rows).
        both_dtypes: files whose bf16 records also count for fp32 (a partial re-measurement in
        one element size: every kernel moves 16-byte vectors, and in the full sweeps the two
        differ by 1 % in the median at equal bytes)."""
        if isinstance(paths, str):
            paths = [paths]
        paths = list(paths) + [p for p in both_dtypes if p not in paths]
        times: Dict[tuple, Dict[str, float]] = {}
        n_rec = 0
        for path in paths:
            with open(path) as f:
                for line in f:
                    try:
                        r = json.loads(line)
                    except ValueError:
                        continue
                    if r.get("op") not in OPS or r.get("impl") != "penny":
                        continue
                    algo = r.get("algo")
                    if algo in (None, "auto", "custom_all_reduce"):
                        continue
                    if dtype and r.get("dtype") != dtype:
                        continue
                    t = r.get("t_graph_us") or r.get("t_us")
                    if not t:
                        continue
                    mem = "sym" if r.get("symmetric") else "any"
                    dts = [r.get("dtype", "bf16")]
                    if path in both_dtypes and dts[0] == "bf16" and r["op"] != "fused_norm":
                        dts.append("fp32")
                    for dt in dts:
                        key = (r["op"], str(int(r["world"])), dt, mem, int(r["bytes"]))
                        slot = times.setdefault(key, {})
                        slot[algo] = min(float(t), slot.get(algo, float("inf")))
                    n_rec += 1
        table: dict = {}
        prev_key, prev_algo = None, None
        for key in sorted(times):
            op, world, dt, mem, size = key
            cand = times[key]
            best_algo = min(cand, key=cand.get)
            if prev_key == key[:4] and prev_algo in cand and cand[prev_algo] <= cand[best_algo] * (1.0 + tolerance):
                best_algo = prev_algo
            rows = table.setdefault(op, {}).setdefault(world, {}).setdefault(dt, {}).setdefault(mem, [])
            if rows and rows[-1][1] == best_algo:
                rows[-1] = [size, best_algo]
            else:
                rows.append([size, best_algo])
            prev_key, prev_algo = key[:4], best_algo
        for op in table.values():
            for world in op.values():
                for dt in world.values():
                    for rows in dt.values():
                        rows[-1] = [None, rows[-1][1]]
        t = cls(table, source=",".join(paths))
        t.records = n_rec
        return t

    @classmethod
    def load(cls, path: Optional[str] = None) -> "Tuner":
        """PENNY_TUNER_CACHE (or `path`) when readable, else the built-in table, else the fallback rows."""
        for cand in (path or os.environ.get("PENNY_TUNER_CACHE", DEFAULT_CACHE), BUILTIN_PATH):
            try:
                with open(cand) as f:
                    raw = json.load(f)
                if isinstance(raw, dict) and any(op in raw for op in OPS):
                    # (op, world) pairs the file has no sweep for keep the fallback rows
                    for op, per_world in json.loads(json.dumps(FALLBACK)).items():
                        for world, per_dt in per_world.items():
                            raw.setdefault(op, {}).setdefault(world, per_dt)
                    return cls(raw, source=cand)
            except (OSError, ValueError):
                continue
        return cls()

    def save(self, path: Optional[str] = None) -> str:
        path = path or os.environ.get("PENNY_TUNER_CACHE", DEFAULT_CACHE)
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump(self.table, f, indent=1, sort_keys=True)
        return path

    # ----------------------------------------------------------------- lookup
    def rows(self, op: str, world: int, dtype="bf16", symmetric: bool = False) -> Optional[Rows]:
        """The rows of one (op, world, dtype, memory class); a missing dtype falls back to
        the other element size's rows, a missing "sym" class to "any"."""
        per_world = self.table.get(op, {}).get(str(world))
        if not per_world:
            return None
        dt = _dtype_key(dtype)
        per_dt = per_world.get(dt) or per_world.get("bf16" if dt == "fp16" else dt) or next(iter(per_world.values()))
        rows = per_dt.get("sym" if symmetric else "any") or per_dt.get("any") or per_dt.get("sym")
        return [(b, a) for b, a in rows] if rows else None

    def pick(self, op: str, nbytes: int, world: int, dtype="bf16", symmetric: bool = False,
             has_multicast: bool = True) -> Optional[str]:
        """The algorithm name for this call, or None when the table has nothing for it."""
        if op == "all_reduce":
            forced = os.environ.get("PENNY_ALGO")
            if forced:
                return forced
        rows = self.rows(op, world, dtype, symmetric)
        if not rows:
            return None
        algo = rows[-1][1]
        for bound, name in rows:
            if bound is None or nbytes <= bound:
                algo = name
                break
        if algo.startswith("nvls") and not has_multicast:
            return None
        return algo

    def describe(self) -> str:
        out = [f"tuner table from {self.source}"]
        for op in OPS:
            for world, per_world in sorted(self.table.get(op, {}).items(), key=lambda kv: int(kv[0])):
                for dt, per_dt in sorted(per_world.items()):
                    for mem, rows in sorted(per_dt.items()):
                        txt = ", ".join(f"<= {b} B: {a}" if b is not None else f"above: {a}" for b, a in rows)
                        out.append(f"  {op} world {world} {dt} {mem}: {txt}")
        return "\n".join(out)


def _main(argv=None) -> int:
    """python -m penny_b200.parallel.tuner sweep1.jsonl [sweep2.jsonl ...] [--out table.json] [--builtin]

    Turns the JSON lines of the sweep scripts into the table `Communicator` loads."""
    import argparse
    ap = argparse.ArgumentParser(prog="python -m penny_b200.parallel.tuner", description=_main.__doc__)
    ap.add_argument("sweep", nargs="+", help="JSON-lines files written by the sweep scripts (--out)")
    ap.add_argument("--out", default=None, help=f"table file (default: PENNY_TUNER_CACHE or {DEFAULT_CACHE})")
    ap.add_argument("--builtin", action="store_true", help="write the package's built-in table instead")
    ap.add_argument("--dtype", default=None, help="only use records of this dtype (e.g. bf16)")
    ap.add_argument("--both-dtypes", nargs="*", default=[],
                    help="further sweep files whose bf16 records also count for fp32 (partial re-measurements)")
    ap.add_argument("--tolerance", type=float, default=0.03,
                    help="keep the previous size's winner while it is within this fraction of the best")
    args = ap.parse_args(argv)
    t = Tuner.from_sweep(args.sweep, dtype=args.dtype, tolerance=args.tolerance, both_dtypes=args.both_dtypes)
    if not t.records:
        print("no usable records (impl=penny, a named algorithm) in", ", ".join(args.sweep))
        return 1
    path = t.save(BUILTIN_PATH if args.builtin else args.out)
    print(t.describe())
    print("written to", path)
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
