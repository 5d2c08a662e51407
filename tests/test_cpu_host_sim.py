"""The collective bodies that run on the GPU, executed by the host simulator:
rank = free-running thread, block = thread, flags = atomics (csrc/sim/host_sim.cpp).
Several calls run back to back without any synchronisation between ranks other
than the protocol itself, which is what exposes buffer-reuse races."""
import pytest

from penny_b200.parallel import schedule

ALL_REDUCE = ["oneshot", "oneshot_ll", "twoshot", "ring_simple", "ring_standard", "double_ring",
              "tree"]


def grid_for(algo, world, nnodes, routes):
    if algo == "ring_standard":
        return routes * 2
    if algo == "tree":
        return (world // nnodes) * 2
    return 4


@pytest.mark.parametrize("algo", ALL_REDUCE)
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_reduce_protocols(algo, world, dtype):
    # 400000: the pipelined two-shot runs its full 16 pieces per chunk (4 blocks x 8 threads)
    for n in (1, 1023, 4096, 65536):
        for nnodes in ([1] if algo not in ("ring_standard", "double_ring", "tree") else [d for d in (1, 2, 4) if world % d == 0]):
            routes = 2 if algo == "ring_standard" and world > 2 else 1
            failed, err, status = schedule.simulate(algo, dtype, world, grid_for(algo, world, nnodes, routes), 8, n,
                                                    nnodes=nnodes, routes=routes, iters=4, in_place=(n % 2 == 1))
            assert failed == 0, (algo, world, n, nnodes, status)
            assert err <= 1.0, (algo, world, n, nnodes, err)


@pytest.mark.parametrize("op", ["reduce_scatter", "reduce_scatter_pipelined", "all_gather", "all_to_all",
                                "all_to_all_pipelined", "exchange"])
@pytest.mark.parametrize("world", [2, 4, 6, 8])
def test_other_collectives(op, world):
    for dtype in ("float32", "float16", "bfloat16"):
        # 50000 per shard: the pipelined reduce-scatter runs its full 16 chunks (3 blocks x 8 threads)
        for n in (1, 1023, 4096) + ((50000,) if op.endswith("_pipelined") else ()):
            size = n * world if op.startswith("reduce_scatter") else n
            failed, err, status = schedule.simulate(op, dtype, world, 3, 8, size, iters=5)
            assert failed == 0 and err <= 1.0, (op, world, dtype, n, err, status)


def test_one_mb_two_ranks():
    """1,048,576 elements on two ranks, fp32 and bf16."""
    for dtype in ("float32", "bfloat16"):
        for algo in ("twoshot", "ring_standard"):
            failed, err, _ = schedule.simulate(algo, dtype, 2, 4, 16, 1 << 20, iters=1)
            assert failed == 0 and err <= 1.0


@pytest.mark.parametrize("algo", ["oneshot", "oneshot_ll", "twoshot", "ring_standard", "tree", "double_ring",
                                  "reduce_scatter_pipelined", "all_to_all_pipelined"])
def test_missing_rank_times_out_cleanly(algo):
    """Fault injection on the host: rank 1 never joins.  Every other rank must give
    up after the timeout, record who it waited for, and return."""
    world = 4
    nnodes = 2 if algo in ("tree", "double_ring") else 1
    blocks = 3 if algo.endswith("_pipelined") else grid_for(algo, world, nnodes, 1)
    failed, err, status = schedule.simulate(algo, "float32", world, blocks, 8, 4096 * world,
                                            nnodes=nnodes, iters=1, stall_rank=1, timeout_ms=150)
    assert failed >= 1
    assert status[1][0] == 0  # the missing rank ran nothing
    codes = {status[r][0] for r in range(world) if r != 1}
    assert codes <= {0, 1, 2, 3, 4} and codes != {0}
    waited_for = {status[r][2] for r in range(world) if r != 1 and status[r][0] != 0}
    # somebody was directly waiting for the missing rank
    assert 1 in waited_for or algo in ("ring_standard", "double_ring", "tree")


def _sanitizer_run(tmp_path, flags, marker):
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    probe = tmp_path / "probe.cpp"
    probe.write_text("int main() { return 0; }\n")
    if subprocess.run(["g++", *flags, "-o", str(tmp_path / "probe"), str(probe)], capture_output=True).returncode != 0:
        pytest.skip(f"g++ has no runtime for {flags} here")
    exe = tmp_path / "sim_sanitized"
    subprocess.check_call(["g++", "-O1", "-g", "-std=c++17", *flags, "-pthread", "-w", "-o", str(exe),
                           os.path.join(root, "tests", "cpp", "sim_tsan_main.cpp")])
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 report_signal_unsafe=0", ASAN_OPTIONS="detect_leaks=0")
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=900, env=env)
    assert marker not in out.stderr and "runtime error" not in out.stderr, out.stderr[-3000:]
    assert out.returncode == 0 and "sim_tsan ok" in out.stdout, out.stdout[-500:] + out.stderr[-1500:]


def test_protocols_under_thread_sanitizer(tmp_path):
    """Every protocol (fp32 and bf16, sizes 1 / 1023 / 1536, 2 and 4 ranks) with the
    simulator compiled with -fsanitize=thread: ranks and blocks are real threads there,
    so a missing release / acquire between a flag and the data it guards, or a scratch
    slot reused one call too early, shows up as a reported race."""
    _sanitizer_run(tmp_path, ["-fsanitize=thread"], "ThreadSanitizer")


def test_protocols_under_address_sanitizer(tmp_path):
    """The same runs with -fsanitize=address,undefined: the simulated heaps are exactly as
    large as the scratch the launchers ask for, so an index past a slot, a ragged tail read
    as a full vector or a misaligned vector access is reported (the bounds checks that
    compute-sanitizer would do on the device, done on the same code on the CPU)."""
    _sanitizer_run(tmp_path, ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "AddressSanitizer")
