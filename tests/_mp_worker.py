"""Worker of the multi-process GPU tests: one process per GPU, launched by
torch.distributed.run.  Writes a JSON report that the test reads."""
import json
import os
import sys
import traceback

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

TOL = {torch.float32: dict(atol=1e-5, rtol=1e-5), torch.bfloat16: dict(atol=6e-2, rtol=2e-2),
       torch.float16: dict(atol=1e-2, rtol=1e-2)}


def gather_cpu(t):
    """All ranks' tensors on the CPU (through gloo), as the oracle's input."""
    parts = [torch.empty(t.shape, dtype=t.dtype) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, t.cpu())
    return parts


def main():
    out_path = sys.argv[1]
    use_nvls = os.environ.get("PENNY_TEST_NVLS", "1") == "1"
    from penny_b200.utils import initialize_distributed, shutdown
    rank, world, _ = initialize_distributed(init_native=False)
    from penny_b200.parallel.comm import Communicator
    report = {"world": world, "failures": [], "checked": 0}
    comm = Communicator.create(None, heap_bytes=2 << 30, multicast=use_nvls, timeout_ms=5000)
    report["describe"] = comm.describe()
    report["multicast"] = comm.has_multicast

    def check(name, fn):
        try:
            fn()
            report["checked"] += 1
        except Exception as e:  # noqa: BLE001
            report["failures"].append(f"{name}: {type(e).__name__}: {str(e)[:300]}")
            traceback.print_exc()

    algos = ["oneshot", "oneshot_ll", "twoshot", "ring_simple", "ring_standard", "double_ring", "tree"]
    if comm.has_multicast:
        algos += ["nvls", "nvls_oneshot"]

    if comm.has_multicast:
        # a very large tensor in ordinary memory: the staging copies of the switch all-reduce run piece by
        # piece on side streams under the reductions; eager, in place, and replayed from a CUDA graph
        def run_pipelined_nvls():
            n = (64 << 20) + 1000  # fp32: just above the size where the pipeline starts, ragged pieces
            base = (torch.arange(n, device="cuda") % 251).float()
            x = base + rank
            want = base * world + sum(range(world))
            out = comm.all_reduce(x, algo="nvls")
            comm.check()
            assert torch.equal(out, want), "eager"
            y = x.clone()
            comm.all_reduce(y, out=y, algo="nvls")
            assert torch.equal(y, want), "in place"
            o2 = torch.empty_like(x)
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                comm.all_reduce(x, out=o2, algo="nvls")
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                comm.all_reduce(x, out=o2, algo="nvls")
            for _ in range(2):
                o2.zero_()
                gr.replay()
                torch.cuda.synchronize()
                assert torch.equal(o2, want), "graph replay"
            comm.check()
        check("all_reduce/nvls-pipelined-staging", run_pipelined_nvls)

    for dtype in (torch.float32, torch.bfloat16):
        for n in (1, 1023, 4096, 65536, 1 << 20):
            g = torch.Generator(device="cuda").manual_seed(1234 + rank + n)
            x = (torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dtype)
            parts = gather_cpu(x)
            want = torch.stack([p.float() for p in parts]).sum(0)
            for algo in algos:
                nnodes = 2 if algo in ("double_ring", "tree") and world >= 4 else 1

                def run(algo=algo, nnodes=nnodes):
                    out = comm.all_reduce(x, algo=algo, nnodes=nnodes)
                    comm.check()
                    torch.testing.assert_close(out.float().cpu(), want, **TOL[dtype])
                    outs = gather_cpu(out)
                    for o in outs[1:]:
                        assert torch.equal(o, outs[0]), "ranks disagree bitwise"
                check(f"all_reduce/{algo}/{dtype}/{n}", run)

            if comm.has_multicast and (n * x.element_size()) % 16 == 0:
                def run_sym():
                    xs = comm.empty(n, dtype=dtype)
                    xs.copy_(x)
                    ys = comm.empty(n, dtype=dtype)
                    comm.all_reduce(xs, out=ys, algo="nvls")
                    comm.check()
                    torch.testing.assert_close(ys.float().cpu(), want, **TOL[dtype])
                    comm.all_reduce(xs, out=xs, algo="nvls")  # in place
                    comm.check()
                    torch.testing.assert_close(xs.float().cpu(), want, **TOL[dtype])
                check(f"all_reduce/nvls-symmetric/{dtype}/{n}", run_sym)

                def run_oneshot_in_place():
                    # every rank reads all inputs through the switch while the others may already be
                    # storing: an output that aliases the symmetric input is served from a staged copy
                    xs = comm.empty(n, dtype=dtype)
                    for _ in range(2):
                        xs.copy_(x)
                        torch.cuda.synchronize()
                        dist.barrier()
                        comm.all_reduce(xs, out=xs, algo="nvls_oneshot")
                        comm.check()
                        torch.testing.assert_close(xs.float().cpu(), want, **TOL[dtype])
                check(f"all_reduce/nvls_oneshot-in-place/{dtype}/{n}", run_oneshot_in_place)

            shard = n
            big = (torch.rand(shard * world, device="cuda", generator=g) * 2 - 1).to(dtype)
            bparts = gather_cpu(big)
            bsum = torch.stack([p.float() for p in bparts]).sum(0)

            def run_rs(nvls=False):
                o = comm.reduce_scatter(big, nvls=nvls)
                comm.check()
                torch.testing.assert_close(o.float().cpu(), bsum[rank * shard:(rank + 1) * shard], **TOL[dtype])
            check(f"reduce_scatter/{dtype}/{n}", run_rs)
            if comm.has_multicast and (shard * x.element_size()) % 16 == 0:
                check(f"reduce_scatter/nvls/{dtype}/{n}", lambda: run_rs(True))

            def run_ag():
                o = comm.all_gather(x)
                comm.check()
                assert torch.equal(o.cpu(), torch.cat(parts))
            check(f"all_gather/{dtype}/{n}", run_ag)
            if comm.has_multicast and (shard * x.element_size()) % 16 == 0:
                def run_ag_nvls():
                    o = comm.empty(shard * world, dtype=dtype)
                    comm.all_gather(x, out=o, nvls=True)
                    comm.check()
                    assert torch.equal(o.cpu(), torch.cat(parts))
                check(f"all_gather/nvls/{dtype}/{n}", run_ag_nvls)

            def run_a2a():
                o = comm.all_to_all(big)
                comm.check()
                want_r = torch.cat([bparts[s][rank * shard:(rank + 1) * shard] for s in range(world)])
                assert torch.equal(o.cpu(), want_r)
            check(f"all_to_all/{dtype}/{n}", run_a2a)

            def run_ex():
                b = x.clone()
                comm.exchange(b, rank ^ 1)
                comm.check()
                assert torch.equal(b.cpu(), parts[rank ^ 1])
            check(f"exchange/{dtype}/{n}", run_ex)

    # fused all-reduce + residual + RMSNorm
    hidden = 4096
    protos = ["ll", "flag", "ll_twoshot"] + (["nvls", "nvls_oneshot"] if comm.has_multicast else [])
    for rows in (1, 8, 64, 256):
        g = torch.Generator(device="cuda").manual_seed(77 + rank + rows)
        xin = (torch.randn(rows, hidden, device="cuda", generator=g) * 0.5).bfloat16()
        g2 = torch.Generator(device="cuda").manual_seed(5)
        res = torch.randn(rows, hidden, device="cuda", generator=g2).bfloat16()
        w = (torch.rand(hidden, device="cuda", generator=g2) + 0.5).bfloat16()
        parts = gather_cpu(xin)
        z = torch.stack([p.float() for p in parts]).sum(0) + res.float().cpu()
        want = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float().cpu()
        for proto in protos:
            def run_fused(proto=proto):
                if proto == "nvls":
                    xi = comm.empty(rows, hidden, dtype=torch.bfloat16)
                    xi.copy_(xin)
                    out = comm.empty(rows, hidden, dtype=torch.bfloat16)
                elif proto == "nvls_oneshot":  # a fresh input buffer per call: consecutive calls never share one
                    xi = comm.empty(rows, hidden, dtype=torch.bfloat16)
                    xi.copy_(xin)
                    out = torch.empty_like(xin)
                else:
                    xi, out = xin, torch.empty_like(xin)
                r = res.clone()
                comm.fused_all_reduce_rmsnorm(xi, w, residual=r, out=out, proto=proto)
                comm.check()
                torch.testing.assert_close(out.float().cpu(), want, **TOL[torch.bfloat16])
                if proto in ("nvls", "ll_twoshot"):  # residual stream stays sharded by row
                    lo = (rows + world - 1) // world * rank
                    hi = min(rows, lo + (rows + world - 1) // world)
                    if hi > lo:
                        torch.testing.assert_close(r[lo:hi].float().cpu(), z[lo:hi], **TOL[torch.bfloat16])
                else:
                    torch.testing.assert_close(r.float().cpu(), z, **TOL[torch.bfloat16])
            check(f"fused_norm/{proto}/{rows}", run_fused)

    # CUDA graph replay of the device-side call counter
    def run_graph():
        x = torch.ones(8192, device="cuda", dtype=torch.bfloat16) * (rank + 1)
        y = torch.empty_like(x)
        comm.all_reduce(x, out=y, algo="oneshot_ll")
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            comm.all_reduce(x, out=y, algo="oneshot_ll")
            comm.all_reduce(y, out=y, algo="twoshot")
        for _ in range(5):
            gr.replay()
        comm.check()
        s = world * (world + 1) / 2
        assert torch.allclose(y.float(), torch.full_like(y, s * world).float()), y[:4]
    check("cuda_graph_replay", run_graph)

    # ---- fused tcgen05 GEMM + collective ----
    def run_fused_gemm():
        import penny_cpp
        M, N, Kfull = 128 * world * 2, 512, 256 * world
        g = torch.Generator(device="cuda").manual_seed(4242)
        a_full = (torch.randn(M, Kfull, device="cuda", generator=g) * 0.5).bfloat16()   # same on all ranks
        w_full = (torch.randn(N, Kfull, device="cuda", generator=g) * 0.5).bfloat16()
        ks = Kfull // world
        a_r, w_r = a_full[:, rank * ks:(rank + 1) * ks].contiguous(), w_full[:, rank * ks:(rank + 1) * ks].contiguous()
        want = a_full.float() @ w_full.float().t()
        rows = M // world
        for _ in range(3):
            out = comm.gemm_reduce_scatter(a_r, w_r)
            assert penny_cpp.gemm_error() == 0
            comm.check()
            torch.testing.assert_close(out.float(), want[rank * rows:(rank + 1) * rows], atol=0.3, rtol=2e-2)
        # all-gather -> GEMM: rows sharded, weight column shard
        nl = N // world if (N // world) % 8 == 0 else N
        w_col = w_full[rank * nl:(rank + 1) * nl] if nl != N else w_full
        a_shard = a_full[rank * rows:(rank + 1) * rows].contiguous()
        for _ in range(3):
            out = comm.all_gather_gemm(a_shard, w_col.contiguous())
            assert penny_cpp.gemm_error() == 0
            comm.check()
            ref_rows = want[:, rank * nl:(rank + 1) * nl] if nl != N else want
            torch.testing.assert_close(out.float(), ref_rows, atol=0.3, rtol=2e-2)
    check("fused_gemm", run_fused_gemm)

    # ---- tensor-parallel decoder vs the same model on one GPU ----
    def run_tp_decode():
        from penny_b200.models.llama_tp import LlamaConfig, LlamaTPDecoder
        cfg = LlamaConfig.tiny()
        if cfg.kv_heads % world:
            cfg.kv_heads, cfg.heads = world, 4 * world
        B, kv = 4, 100
        full = LlamaTPDecoder(cfg, world=1, max_batch=B, max_len=160, use_graph=False, full_init=True)
        full.fill_synthetic_kv(kv)
        protos = ["ll", "flag", "ll_twoshot"] + (["nvls", "nvls_oneshot"] if comm.has_multicast else [])
        for backend, proto in [("penny", p) for p in protos] + [("penny_unfused", "flag"), ("nccl", "flag")]:
            tp = LlamaTPDecoder(cfg, comm=comm, rank=rank, world=world, max_batch=B, max_len=160,
                                backend=backend, proto=proto, use_graph=(backend != "nccl"), full_init=True)
            hk = cfg.kv_heads // world
            for li in range(cfg.layers):
                tp.kcache[li].copy_(full.kcache[li][:, rank * hk:(rank + 1) * hk])
                tp.vcache[li].copy_(full.vcache[li][:, rank * hk:(rank + 1) * hk])
            tp.positions.copy_(full.positions)
            tp.tokens.copy_(full.tokens)
            tp.capture()
            want = full.reference_logits(full.tokens, full.positions, full.kcache, full.vcache)
            tp.step_device()
            comm.check()
            got = tp.logits.float()
            ref_shard = want[:, rank * tp.V:(rank + 1) * tp.V]
            err = (got - ref_shard).abs().max().item()
            assert err < 0.05 * want.std().item() + 0.02, (backend, proto, err)
            chosen = want.gather(1, tp.next_tokens[:, None]).squeeze(1)
            assert torch.all(chosen >= want.max(-1).values - 0.1 * want.std()), (backend, proto)
    check("tp_decode", run_tp_decode)

    # ---- sequence-parallel prefill (fused GEMM + collective in every linear) vs fp32 on one GPU ----
    def run_sp_prefill():
        from penny_b200.models.llama_sp import LlamaSPPrefill
        from penny_b200.models.llama_tp import LlamaConfig
        cfg = LlamaConfig.tiny()
        if cfg.kv_heads % world:
            cfg.kv_heads, cfg.heads = world, 4 * world
        T, L = 256 * world, 2
        g = torch.Generator(device="cuda").manual_seed(77)
        x = torch.randn(T, cfg.hidden, device="cuda", generator=g).bfloat16()       # same on all ranks
        want = LlamaSPPrefill.reference_forward(cfg, x, L, seed=3)
        rows = T // world
        for backend in ("penny", "nccl"):
            m = LlamaSPPrefill(cfg, comm=comm, rank=rank, world=world, tokens=T, layers=L, backend=backend, seed=3)
            for _ in range(2):  # both scratch halves
                got = m.forward(x[rank * rows:(rank + 1) * rows]).float()
                comm.check()
                ref = want[rank * rows:(rank + 1) * rows]
                rel = ((got - ref).norm() / ref.norm()).item()
                assert rel < 3e-2, (backend, rel)
    check("sp_prefill", run_sp_prefill)

    # ---- the reference-style module API on the process-wide communicator ----
    import penny_cpp
    from penny_b200.utils import global_communicator
    gcomm = global_communicator(heap_bytes=256 << 20)

    def run_handle_api():
        n = 1 << 18
        buf = torch.full((n,), float(rank + 1), device="cuda", dtype=torch.float16)
        out = torch.empty_like(buf)
        for algo in (0, 1, 2, 3, 4, 5):
            h = penny_cpp.all_reduce_create(buf, 16, 256, 2 if algo in (4, 5) and world >= 4 else 1, 1, algo)
            penny_cpp.all_reduce_run(h, out)
            penny_cpp.all_reduce_run(h, out)
            penny_cpp.all_reduce_destroy(h)
            gcomm.check()
            assert torch.all(out == world * (world + 1) / 2), (algo, out[:4])
        b = torch.full((n,), float(rank), device="cuda", dtype=torch.float16)
        penny_cpp.nvshmem_register(b)
        penny_cpp.exchange(b, 512, 1024, rank ^ 1)
        penny_cpp.nvshmem_unregister(b)
        gcomm.check()
        assert torch.all(b == float(rank ^ 1))
    check("reference_module_api", run_handle_api)

    # ---- drop-in CustomAllreduce: eager, registered, CUDA-graph capture; on the symmetric-heap
    # kernels (default) and on the pull kernels over IPC-registered buffers ----
    from penny.custom_all_reduce import CustomAllreduce
    gloo = dist.new_group(backend="gloo")
    for backend in ("fast", "pull"):
        os.environ["PENNY_CUSTOM_AR_BACKEND"] = backend
        car = CustomAllreduce(gloo, torch.cuda.current_device())
        os.environ.pop("PENNY_CUSTOM_AR_BACKEND")

        def run_custom(car=car, backend=backend):
            assert not car.disabled and car.fast == (backend == "fast")
            for dtype in (torch.float32, torch.float16, torch.bfloat16):
                for n in (8, 4096, 1 << 18, (1 << 20) + 64):
                    g = torch.Generator(device="cuda").manual_seed(99 + rank + n)
                    x = (torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dtype)
                    parts = gather_cpu(x)
                    want = torch.stack([p.float() for p in parts]).sum(0)
                    if not car.should_custom_ar(x):
                        continue
                    y = car.custom_all_reduce(x)
                    assert car.status()[0] == 0
                    torch.testing.assert_close(y.float().cpu(), want, **TOL[dtype])
                    if n % world == 0 and (n // world * x.element_size()) % 16 == 0:
                        rs = car.custom_reduce_scatter(x)
                        sh = n // world
                        torch.testing.assert_close(rs[:sh].float().cpu(), want[rank * sh:(rank + 1) * sh], **TOL[dtype])
                    if n * world * x.element_size() < car.max_size:
                        ag = car.custom_all_gather(x)
                        assert torch.equal(ag.cpu(), torch.cat(parts))
            assert car.custom_all_reduce(torch.ones(3, device="cuda")) is None  # 12 bytes: not a multiple of 16
        check(f"custom_all_reduce_eager/{backend}", run_custom)

        def run_custom_graph(car=car):
            for n in (4096, 1 << 19):  # flag-in-data lines; the switch or pushes
                x = torch.full((n,), float(rank + 1), device="cuda", dtype=torch.bfloat16)
                with car.capture():
                    car.custom_all_reduce(x)  # warm-up
                    torch.cuda.synchronize()
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr):
                        y = car.custom_all_reduce(x)
                        z = car.custom_all_reduce(y)
                for _ in range(3):
                    gr.replay()
                torch.cuda.synchronize()
                assert car.status()[0] == 0
                s = world * (world + 1) / 2
                assert torch.all(y.float() == s) and torch.all(z.float() == s * world)
        check(f"custom_all_reduce_graph/{backend}", run_custom_graph)
        torch.cuda.synchronize()
        dist.barrier()
        car.close()

    torch.cuda.synchronize()
    dist.barrier()
    all_reports = [None] * world
    dist.all_gather_object(all_reports, report)
    comm.close()
    if rank == 0:
        merged = {"world": world, "multicast": report["multicast"], "describe": report["describe"],
                  "checked": sum(r["checked"] for r in all_reports),
                  "failures": [f"rank{i}: {f}" for i, r in enumerate(all_reports) for f in r["failures"]]}
        with open(out_path, "w") as f:
            json.dump(merged, f, indent=1)
    shutdown()


if __name__ == "__main__":
    main()
