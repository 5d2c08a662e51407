"""Every collective kernel, with all ranks emulated on ONE GPU.

A cooperative launch runs the blocks of all virtual ranks side by side, so the
real cross-rank flag protocols execute (pushes into the other ranks' heaps,
flags, bounded waits) – only the NVLink hop is missing.  The oracle is a plain
PyTorch fp32 sum of the same inputs.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

ALGOS = ["oneshot", "oneshot_ll", "twoshot", "ring_simple", "ring_standard", "double_ring", "tree"]
TOL = {torch.float32: dict(atol=1e-5, rtol=1e-5), torch.bfloat16: dict(atol=6e-2, rtol=2e-2),
       torch.float16: dict(atol=1e-2, rtol=1e-2)}


@pytest.fixture(scope="module")
def comms():
    from penny_b200.parallel.comm import Communicator
    made = {}

    def get(world):
        if world not in made:
            made[world] = Communicator.emulated(world, heap_bytes=192 << 20, timeout_ms=3000)
        return made[world]

    yield get
    for c in made.values():
        c.close()


def make_inputs(world, n, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(1234 + seed)
    return [(torch.rand(n, device="cuda", generator=g, dtype=torch.float32) * 2 - 1).to(dtype) for _ in range(world)]


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_all_reduce(comms, world, algo, dtype):
    comm = comms(world)
    for n in (1, 1023, 4096, 65536, 1 << 20):
        nnodes = 2 if algo in ("double_ring", "tree") and world >= 4 else 1
        ins = make_inputs(world, n, dtype, seed=n)
        want = torch.stack([x.float() for x in ins]).sum(0)
        outs = comm.all_reduce(ins, algo=algo, nnodes=nnodes)
        comm.check()
        for r in range(world):
            torch.testing.assert_close(outs[r].float(), want, **TOL[dtype])
        # every rank must hold bit-identical results
        for r in range(1, world):
            assert torch.equal(outs[r], outs[0])


@pytest.mark.parametrize("world", [2, 8])
def test_all_reduce_repeated_and_in_place(comms, world):
    """Back-to-back calls of different sizes and algorithms reuse the scratch halves."""
    comm = comms(world)
    dtype = torch.bfloat16
    seq = [("oneshot_ll", 2048), ("twoshot", 300000), ("oneshot", 8192), ("ring_standard", 70000),
           ("oneshot_ll", 4096), ("tree", 5000), ("double_ring", 33333), ("twoshot", 64)] * 3
    pending = []
    for i, (algo, n) in enumerate(seq):
        ins = make_inputs(world, n, dtype, seed=i)
        want = torch.stack([x.float() for x in ins]).sum(0)
        outs = comm.all_reduce(ins, out=ins, algo=algo)  # in place, no sync between calls
        pending.append((outs, want))
    comm.check()
    for outs, want in pending:
        for r in range(world):
            torch.testing.assert_close(outs[r].float(), want, **TOL[dtype])


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reduce_scatter_all_gather_all_to_all(comms, world, dtype):
    comm = comms(world)
    for shard in (1, 1023, 4096, 65536):
        n = shard * world
        ins = make_inputs(world, n, dtype, seed=shard)
        want = torch.stack([x.float() for x in ins]).sum(0)
        outs = comm.reduce_scatter(ins)
        comm.check()
        for r in range(world):
            torch.testing.assert_close(outs[r].float(), want[r * shard:(r + 1) * shard], **TOL[dtype])
        shards = make_inputs(world, shard, dtype, seed=shard + 7)
        gathered = comm.all_gather(shards)
        comm.check()
        cat = torch.cat(shards)
        for r in range(world):
            assert torch.equal(gathered[r], cat)
        a2a = comm.all_to_all(ins)
        comm.check()
        for r in range(world):
            want_r = torch.cat([ins[s][r * shard:(r + 1) * shard] for s in range(world)])
            assert torch.equal(a2a[r], want_r)


@pytest.mark.parametrize("world", [2, 8])
def test_direct_output_in_heap(comms, world):
    """Outputs allocated in the symmetric heap are written by the peers directly."""
    comm = comms(world)
    dtype = torch.bfloat16
    shard = 4096
    outs = comm.empty(shard * world, dtype=dtype)
    shards = make_inputs(world, shard, dtype)
    comm.all_gather(shards, out=outs)
    comm.check()
    cat = torch.cat(shards)
    for r in range(world):
        assert torch.equal(outs[r], cat)
    ins = make_inputs(world, shard * world, dtype, seed=3)
    want = torch.stack([x.float() for x in ins]).sum(0)
    comm.all_reduce(ins, out=outs, algo="twoshot")
    comm.check()
    for r in range(world):
        torch.testing.assert_close(outs[r].float(), want, **TOL[dtype])
    comm.all_to_all(ins, out=outs)
    comm.check()
    for r in range(world):
        want_r = torch.cat([ins[s][r * shard:(r + 1) * shard] for s in range(world)])
        assert torch.equal(outs[r], want_r)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_exchange_bit_exact(comms, world):
    comm = comms(world)
    for n in (1023, 1 << 16):
        bufs = make_inputs(world, n, torch.float16, seed=n)
        orig = [b.clone() for b in bufs]
        peers = [r ^ 1 for r in range(world)]
        comm.exchange(bufs, peers)
        # partners change from call to call
        comm.exchange(bufs, [(world - 1 - r) for r in range(world)])
        comm.check()
        for r in range(world):
            src = (world - 1 - r) ^ 1
            assert torch.equal(bufs[r], orig[src])


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("proto", ["ll", "flag", "ll_twoshot"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_all_reduce_rmsnorm(comms, world, proto, dtype):
    comm = comms(world)
    hidden = 4096 if dtype == torch.bfloat16 else 1024
    for rows in (1, 8, 64, 37):
        g = torch.Generator(device="cuda").manual_seed(rows)
        ins = [(torch.randn(rows, hidden, device="cuda", generator=g) * 0.5).to(dtype) for _ in range(world)]
        res = (torch.randn(rows, hidden, device="cuda", generator=g)).to(dtype)
        w = (torch.rand(hidden, device="cuda", generator=g) + 0.5).to(dtype)
        z = torch.stack([x.float() for x in ins]).sum(0) + res.float()
        want = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
        residuals = [res.clone() for _ in range(world)]
        outs, routs = comm.fused_all_reduce_rmsnorm(ins, w, residual=residuals, eps=1e-5, proto=proto)
        comm.check()
        per = -(-rows // world)
        for r in range(world):
            torch.testing.assert_close(outs[r].float(), want, **TOL[dtype])
            if proto == "ll_twoshot":  # rows are sharded over the ranks: a rank keeps the residual of its own rows
                lo, hi = min(rows, r * per), min(rows, (r + 1) * per)
                torch.testing.assert_close(routs[r][lo:hi].float(), z[lo:hi], **TOL[dtype])
            else:
                torch.testing.assert_close(routs[r].float(), z, **TOL[dtype])
            assert torch.equal(outs[r], outs[0])
        # a second call right away: the other scratch half, new line stamps
        outs2, _ = comm.fused_all_reduce_rmsnorm(ins, w, residual=[res.clone() for _ in range(world)], eps=1e-5, proto=proto)
        comm.check()
        assert torch.equal(outs2[0], outs[0])


def test_add_rmsnorm_single_gpu():
    from penny_b200._ext import ops
    for dtype, hidden in ((torch.bfloat16, 4096), (torch.float32, 1000), (torch.float16, 8192)):
        x = torch.randn(33, hidden, device="cuda").to(dtype)
        res = torch.randn(33, hidden, device="cuda").to(dtype)
        w = (torch.rand(hidden, device="cuda") + 0.5).to(dtype)
        out = torch.empty_like(x)
        rout = torch.empty_like(x)
        ops.add_rmsnorm(x, res, w, out, rout, 1e-5)
        z = x.float() + res.float()
        want = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
        torch.testing.assert_close(out.float(), want, **TOL[dtype])
        torch.testing.assert_close(rout.float(), z, **TOL[dtype])


def test_bounded_wait_reports_status(comms):
    """A wait on a flag that nothing sets runs out, records a status and returns."""
    from penny_b200.parallel.comm import PennyTimeoutError
    comm = comms(2)
    comm.set_timeout_ms(200)
    comm.wait_selftest()
    with pytest.raises(PennyTimeoutError) as e:
        comm.check()
    assert e.value.record["code"] == 6
    comm.set_timeout_ms(3000)
    # the communicator is still usable
    ins = make_inputs(2, 4096, torch.float32)
    outs = comm.all_reduce(ins, algo="oneshot")
    comm.check()
    torch.testing.assert_close(outs[0], ins[0] + ins[1])


@pytest.mark.parametrize("world", [2, 4, 8])
def test_reduce_scatter_pipelined(comms, world):
    comm = comms(world)
    for dtype in (torch.float32, torch.bfloat16):
        for shard in (1, 1023, 4096, 300000):
            ins = make_inputs(world, shard * world, dtype, seed=shard)
            total = torch.stack([x.float() for x in ins]).sum(0)
            for _ in range(2):  # both scratch halves
                outs = comm.reduce_scatter(ins, pipelined=True)
                comm.check()
                for r in range(world):
                    torch.testing.assert_close(outs[r].float(), total[r * shard:(r + 1) * shard], **TOL[dtype])


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_to_all_pipelined(comms, world):
    comm = comms(world)
    for dtype in (torch.float32, torch.bfloat16):
        for n in (1, 1023, 4096, 200000):
            ins = make_inputs(world, n * world, dtype, seed=n)
            for _ in range(2):  # both scratch halves
                outs = comm.all_to_all(ins, pipelined=True)
                comm.check()
                for r in range(world):
                    want = torch.cat([ins[s][r * n:(r + 1) * n] for s in range(world)])
                    assert torch.equal(outs[r], want), (world, dtype, n, r)


def test_poisoned_scratch_never_reaches_a_result():
    """debug_poison: every check() overwrites all scratch regions with 0xFF bytes
    (NaN in every float format).  A protocol that consumed scratch it was not sent
    in the current call (a flag satisfied by an older call, a half reused too
    early) would now produce NaNs instead of plausible old numbers."""
    from penny_b200.parallel.comm import Communicator
    world, dtype = 4, torch.bfloat16
    comm = Communicator.emulated(world, heap_bytes=192 << 20, timeout_ms=3000, debug_poison=True)
    try:
        seq = [("twoshot", 300000), ("oneshot_ll", 2048), ("oneshot", 8192), ("ring_standard", 70000),
               ("ring_simple", 5000), ("tree", 5000), ("double_ring", 33333), ("oneshot_ll", 4096), ("twoshot", 64)] * 2
        for i, (algo, n) in enumerate(seq):
            ins = make_inputs(world, n, dtype, seed=100 + i)
            want = torch.stack([x.float() for x in ins]).sum(0)
            outs = comm.all_reduce(ins, algo=algo)
            comm.check()                                   # status, then poison
            for r in range(world):
                assert torch.isfinite(outs[r].float()).all(), (algo, n, r)
                torch.testing.assert_close(outs[r].float(), want, **TOL[dtype])
        n = 4096 * world
        ins = make_inputs(world, n, dtype, seed=7)
        total = torch.stack([x.float() for x in ins]).sum(0)
        for _ in range(2):
            rs = comm.reduce_scatter(ins)
            comm.check()
            ag = comm.all_gather([x[:1024].contiguous() for x in ins])
            comm.check()
            for r in range(world):
                torch.testing.assert_close(rs[r].float(), total[r * 4096:(r + 1) * 4096], **TOL[dtype])
                assert torch.equal(ag[r], torch.cat([x[:1024] for x in ins]))
        w = torch.ones(512, device="cuda", dtype=dtype)
        for proto in ("ll", "flag", "ll_twoshot"):
            xs = [torch.randn(8, 512, device="cuda").to(dtype) for _ in range(world)]
            res = [torch.randn(8, 512, device="cuda").to(dtype) for _ in range(world)]
            full = torch.stack([x.float() for x in xs]).sum(0) + res[0].float()
            res_all = [res[0].clone() for _ in range(world)]
            out, _ = comm.fused_all_reduce_rmsnorm(xs, w, residual=res_all, proto=proto)
            comm.check()
            want = full * torch.rsqrt(full.pow(2).mean(-1, keepdim=True) + 1e-5)
            torch.testing.assert_close(out[0].float(), want, atol=6e-2, rtol=3e-2)
    finally:
        comm.close()


@pytest.mark.parametrize("world", [2, 8])
def test_gemm_push_into_ll_twoshot_fused_norm(comms, world):
    """A row-parallel decode GEMM whose epilogue writes the rows other ranks own straight into their
    flag-in-data receive lines, followed by the all-reduce + RMSNorm that only polls: same result as the
    fp32 oracle and as the unfused path, twice in a row (both scratch halves, new stamps)."""
    from penny_b200._ext import ops
    comm = comms(world)
    hidden, K = 1024, 512
    for rows in (64, 5, 37):
        g = torch.Generator(device="cuda").manual_seed(rows + world)
        xs = [(torch.randn(rows, K, device="cuda", generator=g) * 0.5).bfloat16() for _ in range(world)]
        ws = [(torch.randn(hidden, K, device="cuda", generator=g) * 0.05).bfloat16() for _ in range(world)]
        res = torch.randn(rows, hidden, device="cuda", generator=g).bfloat16()
        w = (torch.rand(hidden, device="cuda", generator=g) + 0.5).bfloat16()
        parts_ref = [(x.float() @ wt.float().t()).bfloat16() for x, wt in zip(xs, ws)]
        z = torch.stack([p.float() for p in parts_ref]).sum(0) + res.float()
        want = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
        targets = [comm.fused_norm_push_target(rows, hidden, view=v) for v in range(world)]
        for rep in range(2):
            parts = [torch.full((rows, hidden), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(world)]
            for v in range(world):
                ops.gemm_decode(xs[v], ws[v], parts[v], False, 0, True, -1, 0, targets[v])
            assert ops.gemm_error() == 0
            outs, routs = comm.fused_all_reduce_rmsnorm(parts, w, residual=[res.clone() for _ in range(world)],
                                                        proto="ll_twoshot", pushed=True)
            comm.check()
            per = -(-rows // world)
            for r in range(world):
                torch.testing.assert_close(outs[r].float(), want, atol=8e-2, rtol=3e-2)
                lo, hi = min(rows, r * per), min(rows, (r + 1) * per)
                torch.testing.assert_close(routs[r][lo:hi].float(), z[lo:hi], atol=8e-2, rtol=3e-2)
                # rows this rank owns were stored locally, the others never touched `part`
                assert torch.isfinite(parts[r][lo:hi].float()).all()
                if lo > 0:
                    assert torch.isnan(parts[r][:lo].float()).all()
