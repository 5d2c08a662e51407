"""Headline benchmark: Llama-3-8B-shaped tensor-parallel decode, tokens/s.

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 50 --warmup 5

One rank per GPU, TP degree = number of GPUs (strong scaling: the model and the
batch are fixed).  Random-init bf16 weights of the real architecture, a synthetic
2048-token KV cache, batch 64 by default (`--batch` for the other points of the
1/8/64/256 series).  A step is one full decode step: 32 layers, the two fused
all-reduce + residual + RMSNorm kernels per layer, lm_head, arg-max, token
feedback.  `value` is timed on the device with CUDA events around exactly
`--steps` graph replays (barrier + synchronize on both sides, max over ranks);
`e2e` is the same loop through `LlamaTPDecoder.step()` with a pinned-host ->
device copy of the step's tokens and a device -> host read of its result inside
every step.

`--impl reference` runs the unmodified reference (baseline/_ref, NVSHMEM build)
through its own public API – `penny.utils.initialize_distributed` and
`penny.custom_all_reduce.CustomAllreduce` (with CUDA-graph capture, NCCL when it
declines) – under a plain-PyTorch implementation of the same model with fixed
shapes, captured in a CUDA graph as the serving engines do; nothing of this
repository's package is imported on that path.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PUBLISHED_TOKS = None  # the reference publishes no tokens/s figure for this config
MODEL_NAME = "Llama-3-8B-shaped (hidden 4096, 32 layers, 32q/8kv heads, FFN 14336, vocab 128256)"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="penny", choices=["penny", "reference"])
    p.add_argument("--batch", type=int, default=64)
    p.add_argument("--kv-len", type=int, default=2048)
    p.add_argument("--backend", default="penny", choices=["penny", "penny_unfused", "nccl"])
    p.add_argument("--proto", default="auto", choices=["auto", "ll", "ll_twoshot", "flag", "nvls", "nvls_oneshot"])
    p.add_argument("--linears", default="auto", choices=["auto", "penny", "cublas"],
                   help="auto: this library's tcgen05 decode GEMM up to 128 rows, the library GEMM above; penny / cublas force one")
    p.add_argument("--layers", type=int, default=32, help="debug only: anything but 32 is not the named config")
    p.add_argument("--no-graph", action="store_true")
    return p.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons while a region runs.

    Polls NVML from a thread every few milliseconds (a TP-8 timed region can be shorter than one nvidia-smi
    period); falls back to an `nvidia-smi -lms` child when the NVML binding is missing. Read-only queries.
    """
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, gpu_index: int, uuid: str = None):
        self.gpu = gpu_index
        self.uuid = uuid
        self.proc = None
        self.lines = []
        self.nvml = None
        self.sm, self.mx, self.reasons = [], None, set()
        self._stop = threading.Event()

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        if self.uuid:
            u = self.uuid if self.uuid.startswith("GPU-") else "GPU-" + self.uuid
            try:
                return pynvml, pynvml.nvmlDeviceGetHandleByUUID(u.encode())
            except pynvml.NVMLError:
                pass
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu)

    def prepare(self):
        """Opens NVML (tens of milliseconds) so that start() inside the timed region only spawns the thread."""
        try:
            self.nvml, self.handle = self._nvml_handle()
            self.mx = float(self.nvml.nvmlDeviceGetMaxClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
            self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None
        return self

    def start(self):
        if self.nvml is not None:
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _poll_once(self):
        n = self.nvml
        self.sm.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
        try:
            mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
        except Exception:
            mask = 0
        for bit, name in self.BITS.items():
            if mask & bit:
                self.reasons.add(name)

    def _poll(self):
        while True:
            try:
                self._poll_once()
            except Exception:
                return
            if self._stop.wait(0.005):
                return

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self._stop.set()
            self.t.join(timeout=2)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.mx,
                    "reasons": sorted(self.reasons), "samples": len(self.sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


def _gpu_uuid(torch):
    try:
        return str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
    except Exception:
        return None


def run_penny(args):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from penny_b200.models.llama_tp import LlamaConfig, LlamaTPDecoder
    from penny_b200.utils import initialize_distributed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    rank, comm = 0, None
    if world > 1:
        rank, world, comm = initialize_distributed(heap_bytes=1 << 30)
    else:
        torch.cuda.set_device(0)
    cfg = LlamaConfig.llama3_8b()
    cfg.layers = args.layers
    max_len = args.kv_len + args.steps * 2 + args.warmup * 2 + 64
    model = LlamaTPDecoder(cfg, comm=comm, rank=rank, world=world, max_batch=args.batch, max_len=max_len,
                           backend=args.backend, proto=args.proto, use_graph=not args.no_graph, linears=args.linears)

    def ops_pdl_enabled():
        from penny_b200._ext import ops
        return ops.pdl_enabled()
    model.fill_synthetic_kv(args.kv_len)
    model.capture()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-timed loop ----
    for _ in range(args.warmup):
        model.step_device()
    sync_all()
    sampler = ClockSampler(torch.cuda.current_device(), _gpu_uuid(torch)).prepare()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        model.step_device()
        if i == 0:
            sampler.start()  # samples only while the timed steps are in flight
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    if comm is not None:
        comm.check()

    # ---- end to end through the public API: pinned host tokens in, host tokens out ----
    model.fill_synthetic_kv(args.kv_len)
    host_tokens = torch.randint(0, cfg.vocab, (args.batch,), dtype=torch.int64).pin_memory()
    for _ in range(args.warmup):
        host_tokens = model.step(host_tokens).clone().pin_memory()
    sync_all()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = model.step(host_tokens)
        host_tokens.copy_(out)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if comm is not None:
        comm.check()
    if world > 1:
        t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    toks = args.batch * args.steps / (ms * 1e-3)
    e2e_toks = args.batch * args.steps / (e2e_ms * 1e-3)
    if rank == 0:
        print(json.dumps({
            "metric": "TP decode tokens/s (Llama-3-8B-shaped, 2048-token KV cache)", "value": round(toks, 1),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic tokens + synthetic KV cache, random-init weights",
            "impl": "penny_b200",
            "config": {"model": MODEL_NAME if args.layers == 32 else f"DEBUG {args.layers} layers",
                       "global_batch": args.batch, "seq_len": args.kv_len, "parallelism": f"tp{world}",
                       "cuda_graph": not args.no_graph,
                       "l2": "inputs larger than L2 (weights + KV streamed every step)"},
            "impl_detail": {"backend": args.backend, "proto": model.proto, "linears": model.linears,
                            "programmatic_dependent_launch": bool(ops_pdl_enabled()),
                            "streamed_gb_per_gpu_per_step": round(
                                (model.weight_bytes() - model.embed.numel() * 2
                                 + 2 * args.batch * model.Hkv * args.kv_len * 128 * 2 * cfg.layers) / 1e9, 2),
                            "attended_kv_len": args.kv_len + 1},
            "clocks": clocks,
            "e2e": {"value": round(e2e_toks, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / args.steps, 4),
                    "h2d_bytes_per_step": args.batch * 8, "d2h_bytes_per_step": args.batch * 8},
            "gpu_launches": model.kernels_per_step * args.steps,
        }), flush=True)
    _leave(comm, world)


def run_reference(args):
    """Plain PyTorch model + the reference's CustomAllreduce.  Imports nothing of this package."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "penny")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}))
        return
    sys.path = [ref_dir] + [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
    os.environ.setdefault("NNODES", "1")
    os.environ.setdefault("NVSHMEM_REMOTE_TRANSPORT", "none")
    os.environ.setdefault("NVSHMEM_DISABLE_NVLS", "1")  # no multicast binding to tear down at exit
    import math
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus
    rank, car = 0, None
    try:
        if world > 1:
            from penny.utils import initialize_distributed  # the reference's own
            from penny.custom_all_reduce import CustomAllreduce
            initialize_distributed()
            rank = dist.get_rank()
            gloo = dist.new_group(backend="gloo")
            car = CustomAllreduce(gloo, torch.cuda.current_device(), nvshmem_registered=True)
        else:
            torch.cuda.set_device(0)
    except Exception as e:  # noqa: BLE001
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"reference init failed: {str(e)[:160]}"}))
        return
    dev = torch.device("cuda", torch.cuda.current_device())
    dt = torch.bfloat16
    H, D, L, B = 4096, 128, args.layers, args.batch
    Hq, Hkv, Fl, Vl = 32 // world, 8 // world, 14336 // world, 128256 // world
    g = torch.Generator(device=dev).manual_seed(rank + 1)

    def rnd(*s):
        return (torch.randn(*s, device=dev, generator=g, dtype=torch.float32) * 0.02).to(dt)
    embed, lm_head = rnd(128256, H), rnd(Vl, H)
    ones = torch.ones(H, dtype=dt, device=dev)
    layers = [dict(wqkv=rnd((Hq + 2 * Hkv) * D, H), wo=rnd(H, Hq * D), wgu=rnd(2 * Fl, H), wdown=rnd(H, Fl))
              for _ in range(L)]
    max_len = args.kv_len + args.steps + args.warmup + 2  # every phase restarts at kv_len
    kc = [torch.randn(B, Hkv, max_len, D, device=dev, generator=g, dtype=torch.float32).to(dt) for _ in range(L)]
    vc = [torch.randn(B, Hkv, max_len, D, device=dev, generator=g, dtype=torch.float32).to(dt) for _ in range(L)]
    tokens = torch.randint(0, 128256, (B,), device=dev, generator=g)
    next_tokens = torch.zeros_like(tokens)
    inv = 500000.0 ** (-torch.arange(0, D // 2, device=dev, dtype=torch.float32) * 2 / D)
    # Fixed shapes (full-length cache + additive mask, position held in a device
    # tensor) so that the step can be captured in a CUDA graph, the way vLLM /
    # SGLang run decode with the reference's CustomAllreduce.capture().
    pos_t = torch.full((1,), args.kv_len, dtype=torch.int64, device=dev)
    mask = torch.full((1, 1, 1, max_len), float("-inf"), dtype=dt, device=dev)
    mask[..., :args.kv_len] = 0

    served = {"reference_kernel": 0, "nccl_fallback": 0}  # all-reduce calls of the step being traced

    def all_reduce(x):
        if world == 1:
            return x
        out = car.custom_all_reduce(x)
        if out is None:
            served["nccl_fallback"] += 1
            dist.all_reduce(x)
            return x
        served["reference_kernel"] += 1
        return out

    def rope(t, cos, sin):
        a, b = t[..., :D // 2].float(), t[..., D // 2:].float()
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1).to(dt)

    def step():
        res = embed[tokens]
        x = F.rms_norm(res, (H,), ones, 1e-5)
        ang = pos_t.float() * inv
        cos, sin = ang.cos(), ang.sin()
        mask.index_fill_(3, pos_t, 0.0)
        for li, W in enumerate(layers):
            qkv = F.linear(x, W["wqkv"])
            q = rope(qkv[:, :Hq * D].view(B, Hq, D), cos, sin)
            k = rope(qkv[:, Hq * D:(Hq + Hkv) * D].view(B, Hkv, D), cos, sin)
            v = qkv[:, (Hq + Hkv) * D:].view(B, Hkv, D)
            kc[li].index_copy_(2, pos_t, k.unsqueeze(2))
            vc[li].index_copy_(2, pos_t, v.unsqueeze(2))
            att = F.scaled_dot_product_attention(q.unsqueeze(2), kc[li], vc[li], attn_mask=mask, enable_gqa=True)
            o = all_reduce(F.linear(att.reshape(B, Hq * D), W["wo"]))
            res = res + o
            x = F.rms_norm(res, (H,), ones, 1e-5)
            gu = F.linear(x, W["wgu"])
            d = all_reduce(F.linear(F.silu(gu[:, :Fl]) * gu[:, Fl:], W["wdown"]))
            res = res + d
            x = F.rms_norm(res, (H,), ones, 1e-5)
        logits = F.linear(x, lm_head)
        val, idx = logits.float().max(dim=-1)
        if world > 1:
            vals = torch.empty(world, B, dtype=val.dtype, device=dev)
            idxs = torch.empty(world, B, dtype=idx.dtype, device=dev)
            dist.all_gather_into_tensor(vals, val)
            dist.all_gather_into_tensor(idxs, idx + rank * Vl)
            best = vals.argmax(0, keepdim=True)
            idx = idxs.gather(0, best).view(B)
        next_tokens.copy_(idx)
        tokens.copy_(idx)
        pos_t.add_(1)

    def reset():
        pos_t.fill_(args.kv_len)
        mask.fill_(float("-inf"))
        mask[..., :args.kv_len] = 0

    graph, mode = None, "eager"
    try:
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            step()
            step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        served.update(reference_kernel=0, nccl_fallback=0)
        if car is not None:
            with car.capture():
                with torch.cuda.graph(graph):
                    step()
        else:
            with torch.cuda.graph(graph):
                step()
        torch.cuda.synchronize()
        mode = "cuda graph"
    except Exception as e:  # noqa: BLE001
        graph, mode = None, f"eager (graph capture failed: {str(e)[:80]})"
    reset()

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step()

    for _ in range(args.warmup):
        run_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(torch.cuda.current_device(), _gpu_uuid(torch)).prepare()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        run_step()
        if i == 0:
            sampler.start()  # samples only while the timed steps are in flight
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    # end to end: pinned host tokens in, host tokens out, every step
    host_in = torch.randint(0, 128256, (B,), dtype=torch.int64).pin_memory()
    host_out = torch.zeros(B, dtype=torch.int64).pin_memory()
    reset()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tokens.copy_(host_in, non_blocking=True)
        run_step()
        host_out.copy_(next_tokens, non_blocking=True)
        torch.cuda.synchronize()
        host_in.copy_(host_out)
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if world > 1:
        t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    if rank == 0:
        print(json.dumps({
            "metric": "TP decode tokens/s (Llama-3-8B-shaped, 2048-token KV cache)",
            "value": round(B * args.steps / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic tokens + synthetic KV cache, random-init weights", "impl": "reference",
            "config": {"model": MODEL_NAME if L == 32 else f"DEBUG {L} layers", "global_batch": B,
                       "seq_len": args.kv_len, "parallelism": f"tp{world}", "cuda_graph": graph is not None,
                       "l2": "inputs larger than L2 (weights + KV streamed every step)"},
            "impl_detail": {"allreduce": "reference CustomAllreduce (custom_all_reduce under its capture()), "
                                         "torch.distributed NCCL when it returns None",
                            "allreduce_calls_per_step": dict(served), "mode": mode,
                            "model_code": "plain PyTorch (the reference ships no model)",
                            "attended_kv_len": f"{max_len} cache rows under an additive mask "
                                               f"({args.kv_len + 1} of them unmasked in the first timed step)"},
            "clocks": clocks,
            "e2e": {"value": round(B * args.steps / (e2e_ms * 1e-3), 1), "unit": "tokens/s",
                    "ms_per_step": round(e2e_ms / args.steps, 4), "h2d_bytes_per_step": B * 8,
                    "d2h_bytes_per_step": B * 8},
            "gpu_launches": 0,
        }), flush=True)
    _leave(None, world)


def _leave(comm, world):
    """Ends the process without the collective tear-downs of torch.distributed /
    NVSHMEM, which were seen to block for minutes after CUDA graphs containing
    their kernels (the numbers are already printed).  The native communicator IS
    closed first: its heap must be unbound from the NVLS multicast object on every
    rank before any rank's process goes away."""
    import torch
    torch.cuda.synchronize()
    if comm is not None:
        comm.barrier()
        comm.close()
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        import torch.distributed as dist
        try:
            dist.barrier()  # everyone has finished its GPU work
            torch.cuda.synchronize()
        except Exception:  # noqa: BLE001
            pass
        os._exit(0)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_penny(a)
