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
    import json
    sys.path.insert(0, ROOT)
    from penny_b200.parallel.tuner import Tuner
    rows = []
    for size, times in ((1024, {"oneshot_ll": 5, "oneshot": 7, "nvls": 12}), (1 << 20, {"oneshot_ll": 80, "oneshot": 30, "nvls": 25}),
                        (1 << 26, {"twoshot": 400, "nvls": 250})):
        for algo, t in times.items():
            rows.append(dict(op="all_reduce", impl="penny", algo=algo, world=8, dtype="bf16", bytes=size, t_us=t))
    p = tmp_path / "sweep.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in rows))
    t = Tuner.from_sweep(str(p))
    assert t.pick(512, 8) == "oneshot_ll" and t.pick(1 << 19, 8) == "nvls" and t.pick(1 << 30, 8) == "nvls"
    assert t.pick(1 << 30, 8, has_multicast=False) == "twoshot"
    saved = t.save(str(tmp_path / "cache.json"))
    assert Tuner.load(saved).table == {k: [tuple(x) for x in v] for k, v in t.table.items()} or Tuner.load(saved).pick(512, 8) == "oneshot_ll"
    assert Tuner().pick(4096, 8) == "oneshot_ll"
    # the command-line form writes the same cache
    from penny_b200.parallel.tuner import _main
    cli_out = tmp_path / "cli_cache.json"
    assert _main([str(p), "--out", str(cli_out), "--dtype", "bf16"]) == 0
    assert Tuner.load(str(cli_out)).pick(1 << 19, 8) == "nvls"
    empty = tmp_path / "empty.jsonl"
    empty.write_text("")
    assert _main([str(empty), "--out", str(tmp_path / "none.json")]) == 1
