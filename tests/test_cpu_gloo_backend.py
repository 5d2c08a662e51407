"""The collectives on CPU tensors over gloo, world_size = 2 (no GPU): fp32 and
bf16 vectors of 1, 1023, 4096, 65536 and 1,048,576 elements, values N(0, 1) from
seed 1234 + rank, against the torch sum of all ranks' tensors; the same tensors
exercise all-gather (concatenation) and reduce-scatter (equal shards)."""
import os
import socket
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SIZES = [1, 1023, 4096, 65536, 1 << 20]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import penny_b200.ops as P
    comm = P.init(force_cpu=True)
    fails = []
    try:
        for dtype, tol in ((torch.float32, dict(atol=1e-5, rtol=1e-5)), (torch.bfloat16, dict(atol=1e-2, rtol=1e-2))):
            for n in SIZES:
                mine = torch.randn(n, generator=torch.Generator().manual_seed(1234 + rank)).to(dtype)
                every = [torch.randn(n, generator=torch.Generator().manual_seed(1234 + r)).to(dtype) for r in range(world)]
                want = torch.stack([e.float() for e in every]).sum(0)
                for algo in ("auto", "oneshot", "twoshot", "ring_standard", "ring_simple", "tree", "double_ring"):
                    got = P.all_reduce(mine, algo=algo)
                    if got.dtype != dtype or not torch.allclose(got.float(), want, **tol):
                        fails.append(f"all_reduce {algo} {dtype} {n}")
                if not torch.equal(P.all_gather(mine), torch.cat(every)):
                    fails.append(f"all_gather {dtype} {n}")
                if n % world == 0:
                    sh = n // world
                    got = P.reduce_scatter(mine)
                    if not torch.allclose(got.float(), want[rank * sh:(rank + 1) * sh], **tol):
                        fails.append(f"reduce_scatter {dtype} {n}")
                    got = P.all_to_all(mine)
                    exp = torch.cat([e[rank * sh:(rank + 1) * sh] for e in every])
                    if not torch.equal(got, exp):
                        fails.append(f"all_to_all {dtype} {n}")
                buf = mine.clone()
                P.exchange(buf, rank ^ 1)
                if not torch.equal(buf, every[rank ^ 1]):
                    fails.append(f"exchange {dtype} {n}")
        # fused op semantics
        x = torch.randn(4, 64, generator=torch.Generator().manual_seed(rank))
        res = torch.randn(4, 64, generator=torch.Generator().manual_seed(99))
        w = torch.rand(64, generator=torch.Generator().manual_seed(98)) + 0.5
        xs = [torch.randn(4, 64, generator=torch.Generator().manual_seed(r)) for r in range(world)]
        z = torch.stack(xs).sum(0) + res
        out, newres = P.all_reduce_rmsnorm(x, w, residual=res.clone())
        if not torch.allclose(out, z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1e-5) * w, atol=1e-5):
            fails.append("fused norm")
        if not torch.allclose(newres, z, atol=1e-6):
            fails.append("fused residual")
        # sequence-parallel linears: row-parallel GEMM -> reduce-scatter, all-gather -> column-parallel GEMM
        M, N, K = 8 * world, 24, 16 * world
        gen = torch.Generator().manual_seed(5)
        a_full, w_full = torch.randn(M, K, generator=gen), torch.randn(N, K, generator=gen)
        ks, rows = K // world, M // world
        want = a_full @ w_full.t()
        got = comm.gemm_reduce_scatter(a_full[:, rank * ks:(rank + 1) * ks].contiguous(),
                                       w_full[:, rank * ks:(rank + 1) * ks].contiguous())
        if got.shape != (rows, N) or not torch.allclose(got, want[rank * rows:(rank + 1) * rows], atol=1e-4):
            fails.append("gemm_reduce_scatter")
        got = comm.all_gather_gemm(a_full[rank * rows:(rank + 1) * rows].contiguous(), w_full)
        if got.shape != (M, N) or not torch.allclose(got, want, atol=1e-4):
            fails.append("all_gather_gemm")
    finally:
        with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
            f.write("\n".join(fails))
        dist.destroy_process_group()


def test_gloo_world2_all_collectives():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(2, _free_port(), d), nprocs=2, join=True)
        for r in range(2):
            text = open(os.path.join(d, f"r{r}.txt")).read().strip()
            assert text == "", f"rank {r}: {text}"


def _sp_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from penny_b200.models.llama_sp import LlamaSPPrefill
    from penny_b200.models.llama_tp import LlamaConfig
    from penny_b200.parallel.cpu_backend import CpuCommunicator
    verdict = ""
    try:
        cfg = LlamaConfig(hidden=256, layers=2, heads=4, kv_heads=2, head_dim=128, ffn=512, vocab=512)
        T, L = 32, 2
        x = torch.randn(T, cfg.hidden, generator=torch.Generator().manual_seed(3)).bfloat16()
        want = LlamaSPPrefill.reference_forward(cfg, x, L, seed=4)
        comm = CpuCommunicator()
        m = LlamaSPPrefill(cfg, comm=comm, rank=rank, world=world, tokens=T, layers=L, seed=4, device="cpu")
        rows = T // world
        got = m.forward(x[rank * rows:(rank + 1) * rows].contiguous()).float()
        ref = want[rank * rows:(rank + 1) * rows]
        rel = ((got - ref).norm() / ref.norm()).item()
        if not rel < 3e-2:
            verdict = f"relative error {rel}"
    except Exception as e:  # noqa: BLE001
        import traceback
        verdict = "exception: " + traceback.format_exc()[-800:]
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(verdict)
    dist.destroy_process_group()


def test_sp_prefill_partitioning_on_gloo():
    """The sequence-parallel prefill model on two CPU ranks (torch ops, gloo collectives): the
    weight slicing, the sequence sharding and the layer wiring against the fp32 one-device oracle."""
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_sp_worker, args=(2, _free_port(), d), nprocs=2, join=True)
        for r in range(2):
            text = open(os.path.join(d, f"r{r}.txt")).read().strip()
            assert text == "", f"rank {r}: {text}"


def _dead_rank_worker(rank, world, port, out_dir):
    """Failure detection on the host: rank 1 raises before joining the collective;
    rank 0's collective must end with an error within the group timeout."""
    import datetime
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    import penny_b200.ops as P
    P.init(force_cpu=True)
    if rank == 1:
        os._exit(0)  # leaves without a word, between steps
    try:
        P.all_reduce(torch.ones(1024), algo="ring_standard")
        verdict = "no error"
    except Exception as e:  # noqa: BLE001
        verdict = "error: " + type(e).__name__
    with open(os.path.join(out_dir, "r0.txt"), "w") as f:
        f.write(verdict)
    os._exit(0)


def test_gloo_peer_exit_is_detected():
    with tempfile.TemporaryDirectory() as d:
        ctx = mp.spawn(_dead_rank_worker, args=(2, _free_port(), d), nprocs=2, join=False)
        import time
        deadline = time.time() + 90
        while not ctx.join(timeout=5) and time.time() < deadline:
            pass
        assert open(os.path.join(d, "r0.txt")).read().startswith("error")


def test_tuner_roundtrip(tmp_path):
    """Sweep records -> table keyed by (op, world, dtype, memory class) -> lookups -> JSON and back,
    through the class and through the command line."""
    import json
    sys.path.insert(0, ROOT)
    from penny_b200.parallel.tuner import Tuner, _main
    rows = []
    for size, times in ((1024, {"oneshot_ll": 5, "oneshot": 7, "nvls": 12}), (1 << 20, {"oneshot_ll": 80, "oneshot": 30, "nvls": 25}),
                        (1 << 26, {"twoshot": 400, "nvls": 250})):
        for algo, t in times.items():
            rows.append(dict(op="all_reduce", impl="penny", algo=algo, world=8, dtype="bf16", bytes=size, t_us=t, symmetric=True))
    # ordinary memory: the switch pays staging copies and loses at the top end
    for size, times in ((1024, {"oneshot_ll": 5, "nvls": 14}), (1 << 26, {"twoshot": 300, "nvls": 330})):
        for algo, t in times.items():
            rows.append(dict(op="all_reduce", impl="penny", algo=algo, world=8, dtype="bf16", bytes=size, t_us=t))
    # a graph time wins over the eager time of the same point; "auto" and NCCL rows are ignored
    rows.append(dict(op="all_reduce", impl="penny", algo="oneshot", world=4, dtype="fp32", bytes=4096, t_us=9, t_graph_us=3))
    rows.append(dict(op="all_reduce", impl="penny", algo="oneshot_ll", world=4, dtype="fp32", bytes=4096, t_us=5, t_graph_us=4))
    rows.append(dict(op="all_reduce", impl="penny", algo="auto", world=4, dtype="fp32", bytes=4096, t_us=1))
    rows.append(dict(op="all_reduce", impl="nccl", world=4, dtype="fp32", bytes=4096, t_us=1))
    for size, times in ((1 << 12, {"push": 20, "nvls": 25}), (1 << 24, {"push": 300, "pipelined": 250, "nvls": 260})):
        for algo, t in times.items():
            rows.append(dict(op="reduce_scatter", impl="penny", algo=algo, world=8, dtype="bf16", bytes=size, t_us=t))
    for nbytes, times in ((8 * 8192, {"ll": 6, "nvls": 14, "nvls_oneshot": 9}), (64 * 8192, {"ll": 30, "nvls": 16, "nvls_oneshot": 11})):
        for algo, t in times.items():
            rows.append(dict(op="fused_norm", impl="penny", algo=algo, world=8, dtype="bf16", bytes=nbytes, t_graph_us=t, symmetric=True))
    p = tmp_path / "sweep.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in rows))
    t = Tuner.from_sweep(str(p))
    ar = lambda n, **kw: t.pick("all_reduce", n, 8, "bf16", **kw)  # noqa: E731
    assert ar(512, symmetric=True) == "oneshot_ll" and ar(1 << 19, symmetric=True) == "nvls" and ar(1 << 30, symmetric=True) == "nvls"
    assert ar(1 << 30) == "twoshot" and ar(512) == "oneshot_ll"            # ordinary memory has its own rows
    assert ar(1 << 30, symmetric=True, has_multicast=False) is None         # the caller falls back to its rule
    assert t.pick("all_reduce", 4096, 4, "fp32") == "oneshot"               # graph time decides
    assert t.pick("all_reduce", 4096, 4, torch.float32) == "oneshot"        # torch dtypes are accepted
    assert t.pick("all_reduce", 4096, 2, "bf16") is None                    # nothing measured at 2 ranks
    assert t.pick("reduce_scatter", 1 << 10, 8) == "push" and t.pick("reduce_scatter", 1 << 26, 8) == "pipelined"
    assert t.pick("fused_norm", 8 * 8192, 8, symmetric=True) == "ll" and t.pick("fused_norm", 64 * 8192, 8, symmetric=True) == "nvls_oneshot"
    saved = t.save(str(tmp_path / "cache.json"))
    again = Tuner.load(saved)
    assert again.source == saved and again.pick("all_reduce", 1 << 19, 8, "bf16", symmetric=True) == "nvls"
    assert "all_reduce world 8 bf16 sym" in again.describe()
    # the package ships a built-in table (or, failing that, fallback rows) for 2, 4 and 8 ranks
    builtin = Tuner.load(str(tmp_path / "does_not_exist.json"))
    for world in (2, 4, 8):
        assert builtin.pick("all_reduce", 4096, world, "bf16") is not None
    # the command-line form writes the same table
    cli_out = tmp_path / "cli_cache.json"
    assert _main([str(p), "--out", str(cli_out), "--tolerance", "0"]) == 0
    cli = Tuner.load(str(cli_out)).table                                    # + fallback rows for 2 ranks
    want = json.loads(json.dumps(t.table))
    assert all(cli[op][w] == want[op][w] for op in want for w in want[op]) and "2" in cli["all_reduce"]
    # a later, partial re-measurement in bf16: the fastest record of a point counts, for fp32 too when asked
    again2 = tmp_path / "again.jsonl"
    again2.write_text(json.dumps(dict(op="all_reduce", impl="penny", algo="oneshot_ll", world=4, dtype="bf16", bytes=4096,
                                      t_us=9, t_graph_us=2)))
    t2 = Tuner.from_sweep([str(p)], both_dtypes=[str(again2)])
    assert t2.pick("all_reduce", 4096, 4, "fp32") == "oneshot_ll" and t2.pick("all_reduce", 4096, 4, "bf16") == "oneshot_ll"
    assert Tuner.from_sweep([str(p), str(again2)]).pick("all_reduce", 4096, 4, "fp32") == "oneshot"
    empty = tmp_path / "empty.jsonl"
    empty.write_text("")
    assert _main([str(empty), "--out", str(tmp_path / "none.json")]) == 1


def test_builtin_tuner_table_names_are_known():
    """Every algorithm the shipped table can hand out is a name the API it is handed to accepts."""
    from penny_b200.parallel.tuner import BUILTIN_PATH, Tuner
    t = Tuner.load(BUILTIN_PATH)
    assert t.source == BUILTIN_PATH
    known = {
        "all_reduce": {"oneshot", "oneshot_ll", "twoshot", "nvls", "nvls_oneshot", "ring_simple", "ring_standard",
                       "double_ring", "tree"},
        "reduce_scatter": {"push", "pipelined", "nvls"},
        "all_gather": {"push", "nvls"},
        "all_to_all": {"push", "pipelined"},
        "fused_norm": {"ll", "ll_twoshot", "flag", "nvls", "nvls_oneshot"},
    }
    seen_worlds = set()
    for op, per_world in t.table.items():
        assert op in known, op
        for world, per_dt in per_world.items():
            seen_worlds.add(int(world))
            for dt, per_mem in per_dt.items():
                assert dt in ("bf16", "fp32", "fp16"), dt
                for mem, rows in per_mem.items():
                    assert mem in ("sym", "any") and rows and rows[-1][0] is None
                    bounds = [b for b, _ in rows[:-1]]
                    assert bounds == sorted(bounds)
                    for _, algo in rows:
                        assert algo in known[op], (op, world, dt, mem, algo)
    assert {2, 8} <= seen_worlds
    # sizes between, below and above the measured points all resolve
    for world in (2, 4, 8):
        for nbytes in (1, 4096, 3 << 20, 5 << 30):
            for sym in (False, True):
                assert t.pick("all_reduce", nbytes, world, "bf16", symmetric=sym) in known["all_reduce"]
                assert t.pick("all_reduce", nbytes, world, torch.float32, symmetric=sym) in known["all_reduce"]


def test_tuner_picks_the_fastest_measured_algorithm(tmp_path):
    """Property: with tolerance 0, at every measured size `pick` returns an algorithm whose time
    equals the minimum over the algorithms measured at that size (ties may go either way), and
    between two measured sizes it returns the choice of the next larger one."""
    import json
    import random
    from penny_b200.parallel.tuner import Tuner
    rng = random.Random(7)
    algos = ["oneshot_ll", "oneshot", "twoshot", "nvls"]
    for trial in range(20):
        sizes = sorted(rng.sample([1 << p for p in range(10, 31)], rng.randint(2, 8)))
        recs, best = [], {}
        for sz in sizes:
            times = {a: rng.uniform(5, 500) for a in rng.sample(algos, rng.randint(1, 4))}
            best[sz] = times
            for a, t in times.items():
                recs.append(dict(op="all_reduce", impl="penny", algo=a, world=8, dtype="bf16", bytes=sz, t_us=t))
        rng.shuffle(recs)
        path = tmp_path / f"s{trial}.jsonl"
        path.write_text("\n".join(json.dumps(r) for r in recs))
        t = Tuner.from_sweep(str(path), tolerance=0.0)
        for i, sz in enumerate(sizes):
            got = t.pick("all_reduce", sz, 8, "bf16")
            assert best[sz][got] == min(best[sz].values())
            if i + 1 < len(sizes) and sizes[i + 1] > sz + 1:
                assert t.pick("all_reduce", sz + 1, 8, "bf16") == t.pick("all_reduce", sizes[i + 1], 8, "bf16")
        assert t.pick("all_reduce", sizes[-1] * 4, 8, "bf16") == t.pick("all_reduce", sizes[-1], 8, "bf16")
