"""The Python-visible surface a user of the reference expects, checked without a GPU."""
import os

import pytest
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

REFERENCE_ENTRY_POINTS = [
    "get_unique_id", "init_with_uid", "exchange", "nvshmem_register", "nvshmem_unregister", "all_reduce_create",
    "all_reduce_run", "all_reduce_destroy", "init_custom_ar", "all_reduce", "reduce_scatter", "all_gather", "dispose",
    "meta_size", "register_buffer", "get_graph_buffer_ipc_meta", "register_graph_buffers",
    "allocate_shared_buffer_and_handle", "open_mem_handle", "free_shared_buffer",
]


def test_extension_imports_without_a_gpu_and_has_every_reference_entry_point():
    import torch  # noqa: F401
    import penny_cpp
    missing = [n for n in REFERENCE_ENTRY_POINTS if not hasattr(penny_cpp, n)]
    assert missing == []
    assert penny_cpp.meta_size() > 0
    uid = penny_cpp.get_unique_id()
    assert isinstance(uid, bytearray) and len(uid) == 32 and uid != penny_cpp.get_unique_id()
    # algorithm ids 0-3 keep the reference's numbering
    assert (penny_cpp.ALGO_RING_STANDARD, penny_cpp.ALGO_RING_SIMPLE, penny_cpp.ALGO_ONESHOT,
            penny_cpp.ALGO_TWOSHOT) == (0, 1, 2, 3)


def test_reference_import_paths():
    from penny.custom_all_reduce import CustomAllreduce, is_weak_contiguous
    from penny.utils import bench_kineto, initialize_distributed  # noqa: F401
    for name in ("capture", "register_graph_buffers", "should_custom_ar", "all_reduce", "custom_all_reduce",
                 "reduce_scatter", "custom_reduce_scatter", "all_gather", "custom_all_gather", "close",
                 "create_shared_buffer", "free_shared_buffer"):
        assert hasattr(CustomAllreduce, name), name
    assert CustomAllreduce._SUPPORTED_WORLD_SIZES == [2, 4, 6, 8]
    import torch
    t = torch.arange(12).reshape(3, 4)
    assert is_weak_contiguous(t) and is_weak_contiguous(t[1:]) and not is_weak_contiguous(t[:, :2])


def test_bootstrap_mesh_between_processes(tmp_path):
    """The native unique-id bootstrap (Unix sockets + fd passing) needs no GPU: two
    processes build the mesh; creating the heap then fails cleanly without CUDA."""
    import subprocess
    code = r'''
import sys, torch
sys.path.insert(0, %r)
import penny_cpp
uid, rank = bytes.fromhex(sys.argv[1]), int(sys.argv[2])
try:
    penny_cpp.comm_create(uid, rank, 2, 1 << 22, 0, False, 2000)
    print("created")
except RuntimeError as e:
    print("error:", str(e)[:60])
''' % ROOT
    import penny_cpp
    uid = bytes(penny_cpp.get_unique_id()).hex()
    procs = [subprocess.Popen([sys.executable, "-c", code, uid, str(r)], stdout=subprocess.PIPE, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    # both ranks met in the bootstrap and then failed on the missing GPU, not on the rendezvous
    for o in outs:
        assert o.startswith("error:") and "bootstrap" not in o, outs


def test_penny_config_env_and_overrides(monkeypatch):
    from penny_b200 import PennyConfig
    for k in ("PENNY_HEAP_BYTES", "PENNY_TIMEOUT_MS", "PENNY_DISABLE_NVLS", "PENNY_HEAP_MODE", "NNODES", "PENNY_ALGO",
              "VLLM_CUSTOM_ALLREDUCE_ALGO", "PENNY_GEMM_PAIR", "PENNY_GEMM_SPLIT_TAIL", "PENNY_DEBUG_POISON"):
        monkeypatch.delenv(k, raising=False)
    d = PennyConfig.from_env()
    assert (d.heap_bytes, d.timeout_ms, d.disable_nvls, d.heap_mode, d.nnodes) == (1 << 30, 10000, False, "auto", 1)
    assert d.gemm_pair and not d.gemm_split_tail and not d.debug_poison and d.algo is None
    monkeypatch.setenv("PENNY_HEAP_BYTES", str(2 << 30))
    monkeypatch.setenv("PENNY_DISABLE_NVLS", "1")
    monkeypatch.setenv("PENNY_ALGO", "twoshot")
    monkeypatch.setenv("NNODES", "2")
    monkeypatch.setenv("PENNY_GEMM_PAIR", "0")
    c = PennyConfig.from_env(timeout_ms=250, heap_mode="ipc")
    assert (c.heap_bytes, c.disable_nvls, c.algo, c.nnodes, c.gemm_pair) == (2 << 30, True, "twoshot", 2, False)
    assert (c.timeout_ms, c.heap_mode) == (250, "ipc")            # keyword overrides win
    assert "timeout_ms=250" in c.describe()
    c.apply_env()
    import os
    assert os.environ["PENNY_TIMEOUT_MS"] == "250" and os.environ["PENNY_HEAP_MODE"] == "ipc"
    with pytest.raises(TypeError):
        PennyConfig.from_env(no_such_field=1)
    with pytest.raises(ValueError):
        PennyConfig.from_env(heap_mode="nvshmem")
    with pytest.raises(ValueError):
        PennyConfig.from_env(vllm_algo="3stage")


def test_custom_allreduce_dispatch_logic(monkeypatch):
    """The host-side decisions of the drop-in CustomAllreduce, with the native calls
    replaced by a recorder: which inputs it serves, staging vs registered buffers,
    the warm-up pass inside capture(), and None as the "use your fallback" answer
    (same contract as the reference, penny/custom_all_reduce.py:214-267)."""
    import torch
    import penny_b200.parallel.custom_all_reduce as car_mod
    calls = []

    class FakeOps:
        def all_reduce(self, ptr, inp, out, reg, size):
            calls.append(("all_reduce", reg, size))

        def reduce_scatter(self, ptr, inp, out, reg, size):
            calls.append(("reduce_scatter", reg, size))

        def all_gather(self, ptr, inp, out, reg, size):
            calls.append(("all_gather", reg, size))

        def get_graph_buffer_ipc_meta(self, ptr):
            raise AssertionError("not reached: the object is disabled when capture() exits in this test")

    monkeypatch.setattr(car_mod, "ops", FakeOps())
    car = car_mod.CustomAllreduce.__new__(car_mod.CustomAllreduce)
    car._IS_CAPTURING, car.disabled, car._ptr, car._comm = False, False, 1234, None
    car.rank, car.world_size, car.fully_connected, car.max_size = 1, 4, True, 1 << 20
    car.buffer_ptrs = [10, 11, 12, 13]

    ok = torch.zeros(4096, dtype=torch.bfloat16)
    assert car.should_custom_ar(ok)
    assert not car.should_custom_ar(torch.zeros(7, dtype=torch.bfloat16))          # not a multiple of 16 bytes
    assert not car.should_custom_ar(torch.zeros(1 << 20, dtype=torch.bfloat16))    # 2 MiB >= max_size
    assert not car.should_custom_ar(torch.zeros(64, 64)[:, ::2])                   # not weakly contiguous
    assert car.should_custom_ar(torch.zeros(64, 64)[8:])                           # a dense tail of a storage is fine
    # dense, 16-byte multiple, but starting 6 bytes into its storage: the kernels' 16-byte vectors would fault
    odd = torch.zeros(4096 + 8, dtype=torch.bfloat16)[3:3 + 4096]
    tail = torch.zeros(4096 + 3, dtype=torch.bfloat16)[3:]
    assert tail.data_ptr() % 16 != 0 and not car.should_custom_ar(tail)
    assert car.custom_all_reduce(tail) is None
    del odd

    # eager: staged through this rank's registered buffer
    out = car.custom_all_reduce(ok)
    assert out is not None and out.shape == ok.shape and calls[-1] == ("all_reduce", 11, 1 << 20)
    assert car.custom_all_reduce(torch.zeros(7, dtype=torch.bfloat16)) is None     # caller falls back
    # inside capture() but not capturing a graph yet (the warm-up run): no communication
    n = len(calls)
    car._IS_CAPTURING = True
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    warm = car.custom_all_gather(ok)
    assert len(calls) == n and warm.numel() == ok.numel() * 4
    # while the graph is being captured: the buffer itself is registered later, no staging copy
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: True)
    car.custom_reduce_scatter(ok)
    assert calls[-1] == ("reduce_scatter", 0, 0)
    car._IS_CAPTURING = False
    # disabled object: every entry point answers None
    car.disabled = True
    assert car.custom_all_reduce(ok) is None and car.custom_all_gather(ok) is None
    car._ptr = 0  # nothing to dispose in __del__


def test_bench_clock_sampler_against_fake_nvml(monkeypatch):
    """bench.py samples SM clocks and throttle reasons during the timed region through
    NVML (read-only queries).  Checked here against a fake NVML: the median clock, the
    decoding of the reason bit mask, and the look-up of the GPU by UUID."""
    import importlib.util
    import time
    import types
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    spec.loader.exec_module(bench)

    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.NVMLError = RuntimeError
    seen = {"uuid": None, "polls": 0}
    fake.nvmlInit = lambda: None

    def by_uuid(u):
        seen["uuid"] = u
        return "handle"
    fake.nvmlDeviceGetHandleByUUID = by_uuid
    fake.nvmlDeviceGetHandleByIndex = lambda i: "handle"
    fake.nvmlDeviceGetMaxClockInfo = lambda h, k: 1965

    def clock(h, k):
        seen["polls"] += 1
        return 1965 if seen["polls"] % 4 else 1700
    fake.nvmlDeviceGetClockInfo = clock
    fake.nvmlDeviceGetCurrentClocksThrottleReasons = lambda h: 0x4 | 0x1    # sw_power_cap | gpu_idle (ignored)
    monkeypatch.setitem(sys.modules, "pynvml", fake)

    s = bench.ClockSampler(3, "abcd-ef").prepare()
    s.start()
    time.sleep(0.08)
    rec = s.stop()
    assert seen["uuid"] == b"GPU-abcd-ef"
    assert rec["source"] == "nvml" and rec["samples"] >= 3
    assert rec["sm_mhz"] == 1965.0 and rec["sm_max_mhz"] == 1965.0
    assert rec["reasons"] == ["sw_power_cap"]
    fake.nvmlDeviceGetCurrentClocksThrottleReasons = lambda h: 0x40 | 0x8
    s2 = bench.ClockSampler(0).prepare()
    s2.start()
    time.sleep(0.03)
    assert s2.stop()["reasons"] == ["hw_slowdown", "hw_thermal_slowdown"]


def test_attention_split_rule_reproduces_the_measured_choices():
    """The split rule of the decode attention is a fit to measurements; the points it was fitted to."""
    from penny_b200.models.llama_tp import LlamaTPDecoder
    f = LlamaTPDecoder.attention_splits
    assert f(64, 2112) == 4       # TP 8, batch 64: 256 CTAs in one wave beat 320 in two (14.7 vs 20.8 us in the step)
    assert f(512, 2112) == 1      # TP 1, batch 64: 512 long CTAs beat 2048 short ones (83.7 vs 92.6 us)
    assert f(8, 2112) >= 8        # a handful of rows: as many splits as still pay their fixed cost
    for items in (1, 3, 64, 100, 512, 4096):
        for kv in (16, 2048, 32768):
            s = f(items, kv)
            assert 1 <= s <= 16
