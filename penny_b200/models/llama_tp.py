"""Llama-3-8B-shaped tensor-parallel decode (random weights, synthetic KV cache).

One decode step for a batch of sequences on `world` GPUs:

    embed -> [ rmsnorm -> qkv GEMM -> (RoPE + KV append + GQA decode attention +
               split merge, ONE kernel) -> o_proj GEMM --(all-reduce + residual +
               rmsnorm, ONE kernel)--> gate/up GEMM with silu*mul in its epilogue
               -> down GEMM --(all-reduce + residual + rmsnorm of the NEXT layer,
               one kernel)--> ] x layers
          -> lm_head shard GEMM -> arg-max (local, then across ranks)

Seven launches per layer, all of them this library's kernels: the linears are
the tcgen05 decode GEMM (`ops.gemm_decode`; `linears="cublas"` swaps in
torch.matmul for comparison), and every kernel is launched with programmatic
stream serialization, so inside the captured CUDA graph a kernel's prologue and
the loads of its constant operands (weights, old KV-cache rows) overlap the
tail of the kernel before it.

Column-parallel qkv / gate-up / lm_head, row-parallel o_proj / down (Megatron
layout); 4 query heads + 1 KV head, 1792 FFN columns and 16032 vocabulary rows
per GPU at TP=8.  The two all-reduces per layer are the fused kernels of this
library (`backend="penny"`), or separate all-reduce + norm kernels
(`"penny_unfused"`), or NCCL + norm (`"nccl"`, the baseline).  The whole step is
captured in a CUDA graph (the collectives keep their call counter in device
memory, so the graph replays correctly).

The reference has no model code: it is used by patching SGLang/vLLM
(extra/sglang.patch, README.md:20-33).  This module is the stand-alone
equivalent of that serving path for the TP-decode benchmark.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .._ext import ops


@dataclass
class LlamaConfig:
    hidden: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    eps: float = 1e-5
    rope_theta: float = 500000.0
    init_std: float = 0.02

    @classmethod
    def llama3_8b(cls):
        return cls()

    @classmethod
    def tiny(cls):
        """Same structure, small enough for unit tests (head_dim stays 128)."""
        return cls(hidden=512, layers=2, heads=8, kv_heads=2, head_dim=128, ffn=1024, vocab=2048)


# world size -> largest batch for which the decode step with proto="ll_twoshot" and the GEMM epilogue
# push was measured faster than with the transport the stand-alone table picks (8 x B200, Llama-3-8B
# shapes, kv 2048: batch 1 2.01 vs 2.21 ms, batch 8 2.13 vs 2.31, batch 64 2.70 vs 2.80-2.88; at
# batch 256 the switch two-shot wins, 5.84 vs 7.39 ms; at 2 GPUs plain "ll" wins, 4.30 vs 4.40 ms).
# 4 GPUs: not measured (no 4-GPU box could be had); the pushed two-shot is taken there because it is
# the best or within 1 % of the best at both 2 and 8 GPUs, while the table-less fallback (the switch
# two-shot) was the slowest transport at both.
PUSHED_STEP_WINS = {4: 128, 8: 128}


class LlamaTPDecoder:
    def __init__(self, cfg: LlamaConfig, comm=None, rank: int = 0, world: int = 1, max_batch: int = 64,
                 max_len: int = 2560, backend: str = "penny", proto: str = "auto", seed: int = 0,
                 use_graph: bool = True, full_init: bool = False, process_group=None, linears: str = "auto",
                 pdl: bool = True):
        assert cfg.heads % world == 0 and cfg.kv_heads % world == 0 and cfg.ffn % world == 0
        assert cfg.vocab % world == 0 and cfg.head_dim == 128 and (cfg.ffn // world) % 64 == 0
        assert backend in ("penny", "penny_unfused", "nccl") and linears in ("auto", "penny", "cublas")
        if linears == "auto":
            # measured (one layer's four linears replayed from a graph, batch 256): this library's decode
            # GEMM is a weight-streaming kernel with a 128-row batch tile, 56.9 vs 34.3 us at TP 8 and 231 vs
            # 119 us at TP 1 against the library GEMM once the problem is compute-bound; up to 128 rows it
            # is level (95 vs 92 us at TP 1, batch 64) and lets the epilogues fuse
            linears = "penny" if max_batch <= 128 else "cublas"
        self.linears, self.pdl = linears, pdl
        if world > 1 and backend != "nccl":
            assert comm is not None, "a Communicator is required for the penny backends"
        self.cfg, self.comm, self.rank, self.world = cfg, comm, rank, world
        self.backend, self.use_graph, self.pg = backend, use_graph, process_group
        self.B, self.max_len = max_batch, max_len
        self.Hq, self.Hkv = cfg.heads // world, cfg.kv_heads // world
        self.F, self.V = cfg.ffn // world, cfg.vocab // world
        self.dev = torch.device("cuda", torch.cuda.current_device())
        dt = torch.bfloat16
        D, H = cfg.head_dim, cfg.hidden
        if proto == "auto":
            # 1. where the row-parallel GEMMs can write into the all-reduce's receive lines and that was
            #    measured to win the whole step (PUSHED_STEP_WINS), the pushed flag-in-data two-shot;
            # 2. else the measured table of the stand-alone fused kernel, when it covers this shape;
            # 3. else flag-in-data lines for a handful of rows, the switch (when bound) or flag barriers
            can_push = (comm is not None and world > 1 and backend == "penny" and linears == "penny"
                        and hasattr(comm, "fused_norm_push_target") and not getattr(comm, "emulated", False))
            if can_push and max_batch <= PUSHED_STEP_WINS.get(world, 0):
                proto = "ll_twoshot"
            elif comm is not None and world > 1 and hasattr(comm, "pick_fused_proto"):
                proto = comm.pick_fused_proto(max_batch, H, dt, alternating_inputs=True)  # self.parts
            elif max_batch <= 16:
                proto = "ll"
            elif comm is not None and getattr(comm, "has_multicast", False):
                proto = "nvls"
            else:
                proto = "flag"
        self.proto = proto
        # flag-in-data two-shot: the o_proj / down GEMMs write the rows other ranks own straight into
        # those ranks' receive lines, the all-reduce kernel only polls, reduces and sends back
        self._push = None
        if (comm is not None and world > 1 and backend == "penny" and proto == "ll_twoshot" and linears == "penny"
                and max_batch <= 128 and hasattr(comm, "fused_norm_push_target")):
            self._push = comm.fused_norm_push_target(max_batch, H)
        self._init_weights(seed, full_init)

        def buf(*shape, dtype=dt, heap=False):
            if heap and comm is not None and world > 1 and backend == "penny" and proto in ("nvls", "nvls_oneshot"):
                return comm.empty(*shape, dtype=dtype)
            return torch.empty(*shape, dtype=dtype, device=self.dev)

        B = max_batch
        self.tokens = torch.zeros(B, dtype=torch.int64, device=self.dev)
        self.positions = torch.zeros(B, dtype=torch.int32, device=self.dev)
        self.residual = buf(B, H)
        self.x = buf(B, H, heap=True)            # normalised activations (multicast target under NVLS)
        self.qkv = buf(B, (self.Hq + 2 * self.Hkv) * D)
        self.attn = buf(B, self.Hq * D)
        # row-parallel partial sums (switch-reduced under NVLS): o_proj and down write different
        # buffers, so consecutive all-reduces never read the same one
        self.parts = [buf(B, H, heap=True), buf(B, H, heap=True)]
        self.part = self.parts[0]
        self.gu = buf(B, 2 * self.F) if linears == "cublas" else None
        self.act = buf(B, self.F)
        self.logits = buf(B, self.V)
        self.max_val = torch.empty(B, dtype=torch.float32, device=self.dev)
        self.max_idx = torch.empty(B, dtype=torch.int64, device=self.dev)
        self.pair = torch.empty(2 * B, dtype=torch.float32, device=self.dev)
        self.argmax_ws = torch.zeros(ops.argmax_workspace_bytes(B), dtype=torch.uint8, device=self.dev)
        self.pairs_all = torch.empty(world * 2 * B, dtype=torch.float32, device=self.dev)
        self.next_tokens = torch.zeros(B, dtype=torch.int64, device=self.dev)
        self.kcache = [torch.zeros(B, self.Hkv, max_len, D, dtype=dt, device=self.dev) for _ in range(cfg.layers)]
        self.vcache = [torch.zeros(B, self.Hkv, max_len, D, dtype=dt, device=self.dev) for _ in range(cfg.layers)]
        self.splits = self.attention_splits(B * self.Hkv, max_len)
        # split partials + self-resetting arrival counters (zero before the first use)
        self.workspace = torch.zeros(ops.decode_attn_fused_workspace_bytes(B, self.Hq, self.Hkv, self.splits),
                                     dtype=torch.uint8, device=self.dev)
        self.scale = 1.0 / math.sqrt(D)
        self._graph = None
        self._host_in = torch.zeros(B, dtype=torch.int64).pin_memory()
        self._host_out = torch.zeros(B, dtype=torch.int64).pin_memory()
        # kernels of this library launched per step (the few torch glue ops excluded)
        chunks = -(-B // 1024)  # the decode GEMM takes up to 1024 rows per launch
        gemms = 4 * chunks if self.linears == "penny" else 0
        per_layer = gemms + 1 + (1 if self.linears == "cublas" else 0)  # + fused attention (+ silu*mul beside cuBLAS)
        norms = 2 * cfg.layers + 1
        if backend == "penny_unfused" and world > 1:
            norms += 2 * cfg.layers  # separate all-reduce kernels
        # + arg-max + sampling tail (+ the all-gather of the ranks' candidates) + LM head
        self.kernels_per_step = (cfg.layers * per_layer + norms + 2 + (1 if world > 1 else 0)
                                 + (chunks if self.linears == "penny" else 0))

    # ------------------------------------------------------------------ weights
    def _init_weights(self, seed: int, full_init: bool):
        cfg, w, r = self.cfg, self.world, self.rank
        D, H = cfg.head_dim, cfg.hidden
        dt = torch.bfloat16
        g = torch.Generator(device=self.dev)

        def rnd(*shape, sub=0):
            # one stream per (tensor, shard): identical for every world size only with full_init
            g.manual_seed(seed * 1000003 + sub)
            return (torch.randn(*shape, device=self.dev, generator=g, dtype=torch.float32) * cfg.init_std).to(dt)

        def col_shard(full_rows, cols, sub):
            """[out, in] weight split along `out` (column-parallel)."""
            if full_init:
                return rnd(full_rows, cols, sub=sub)[r * (full_rows // w):(r + 1) * (full_rows // w)].contiguous()
            return rnd(full_rows // w, cols, sub=sub * 64 + r + 1)

        def row_shard(rows, full_cols, sub):
            """[out, in] weight split along `in` (row-parallel)."""
            if full_init:
                return rnd(rows, full_cols, sub=sub)[:, r * (full_cols // w):(r + 1) * (full_cols // w)].contiguous()
            return rnd(rows, full_cols // w, sub=sub * 64 + r + 1)

        self.embed = rnd(cfg.vocab, H, sub=1)
        self.final_norm = torch.ones(H, dtype=dt, device=self.dev)
        self.lm_head = col_shard(cfg.vocab, H, 2)
        self.layers = []
        for li in range(cfg.layers):
            base = 100 + li * 10
            if full_init:
                q = rnd(cfg.heads * D, H, sub=base)
                k = rnd(cfg.kv_heads * D, H, sub=base + 1)
                v = rnd(cfg.kv_heads * D, H, sub=base + 2)
                hq, hk = cfg.heads // w * D, cfg.kv_heads // w * D
                wqkv = torch.cat([q[r * hq:(r + 1) * hq], k[r * hk:(r + 1) * hk], v[r * hk:(r + 1) * hk]]).contiguous()
                gate = rnd(cfg.ffn, H, sub=base + 4)
                up = rnd(cfg.ffn, H, sub=base + 5)
                f = cfg.ffn // w
                wgu = self.interleave_gate_up(gate[r * f:(r + 1) * f], up[r * f:(r + 1) * f])
            else:
                wqkv = rnd((self.Hq + 2 * self.Hkv) * D, H, sub=base * 64 + r + 1)
                wgu = rnd(2 * self.F, H, sub=(base + 4) * 64 + r + 1)  # random: already "interleaved"
            layer = dict(
                wqkv=wqkv, wo=row_shard(H, cfg.heads * D, base + 3), wgu=wgu, wdown=row_shard(H, cfg.ffn, base + 6),
                norm1=torch.ones(H, dtype=dt, device=self.dev), norm2=torch.ones(H, dtype=dt, device=self.dev))
            if self.linears == "cublas":
                layer["wgu_cat"] = torch.cat(self.split_gate_up(wgu)).contiguous()
            self.layers.append(layer)

    @staticmethod
    def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """[F, H] gate and up -> the layout the fused silu*mul epilogue reads: blocks of 64 gate rows
        followed by the 64 up rows of the same features."""
        F, H = gate.shape
        return torch.stack([gate.reshape(F // 64, 64, H), up.reshape(F // 64, 64, H)], 1).reshape(2 * F, H).contiguous()

    @staticmethod
    def split_gate_up(wgu: torch.Tensor):
        """Inverse of interleave_gate_up: (gate [F, H], up [F, H])."""
        F2, H = wgu.shape
        v = wgu.view(F2 // 128, 2, 64, H)
        return v[:, 0].reshape(F2 // 2, H), v[:, 1].reshape(F2 // 2, H)

    @staticmethod
    def attention_splits(items: int, kv_len: int = 2048, slots: int = 2 * 148, max_splits: int = 16) -> int:
        """KV splits of the decode attention for `items` = batch x KV heads (row, head) pairs.  Two
        CTAs fit an SM, so `slots` run at once and a grid a little larger than that costs a whole
        second wave.  Measured on B200 (TP 8: 320 CTAs took twice as long as 256; TP 1: 2048 short
        CTAs lost 10 % to 512 long ones): a CTA costs its KV positions plus about 200 positions of
        fixed work, a launch costs that times its waves; ties go to fewer splits."""
        best, best_cost = 1, None
        for s in range(1, max_splits + 1):
            waves = -(-items * s // slots)
            cost = waves * (kv_len / s + 200.0)
            if best_cost is None or cost < best_cost * 0.98:
                best, best_cost = s, cost
        return best

    def weight_bytes(self) -> int:
        n = self.embed.numel() + self.lm_head.numel()
        for l in self.layers:
            n += sum(l[k].numel() for k in ("wqkv", "wo", "wgu", "wdown"))  # wgu_cat (cuBLAS mode) is a copy
        return n * 2

    # ------------------------------------------------------------------- state
    def fill_synthetic_kv(self, kv_len: int, seed: int = 1):
        """Random K/V rows for positions [0, kv_len) and random current tokens."""
        assert kv_len < self.max_len
        g = torch.Generator(device=self.dev).manual_seed(seed + 17 * self.rank)
        for li in range(self.cfg.layers):
            for cache in (self.kcache[li], self.vcache[li]):
                cache[:, :, :kv_len].copy_(torch.randn(self.B, self.Hkv, kv_len, self.cfg.head_dim, device=self.dev,
                                                       generator=g, dtype=torch.float32).to(torch.bfloat16))
        self.positions.fill_(kv_len)
        gt = torch.Generator(device=self.dev).manual_seed(seed)
        self.tokens.copy_(torch.randint(0, self.cfg.vocab, (self.B,), device=self.dev, generator=gt))

    # ----------------------------------------------------------------- the step
    def _reduce_norm(self, part, weight):
        """part (partial sums) -> self.x = rmsnorm(sum + residual) * weight; residual updated."""
        if self.world == 1:
            ops.add_rmsnorm(part, self.residual, weight, self.x, self.residual, self.cfg.eps)
        elif self.backend == "penny":
            self.comm.fused_all_reduce_rmsnorm(part, weight, residual=self.residual, out=self.x,
                                               eps=self.cfg.eps, proto=self.proto, pushed=self._push is not None)
        elif self.backend == "penny_unfused":
            self.comm.all_reduce(part, out=part)
            ops.add_rmsnorm(part, self.residual, weight, self.x, self.residual, self.cfg.eps)
        else:
            import torch.distributed as dist
            dist.all_reduce(part, group=self.pg)
            ops.add_rmsnorm(part, self.residual, weight, self.x, self.residual, self.cfg.eps)

    def _linear(self, x, w, out, silu_pairs=False, smem_kb=0, push=None):
        """out = x @ w^T on this library's decode GEMM: one launch (batches above 128 rows run as
        slabs of 128 rows inside it, 1024 rows per launch at most)."""
        B = x.shape[0]
        for r in range(0, B, 1024):
            ops.gemm_decode(x[r:r + 1024], w, out[r:r + 1024], silu_pairs, 0, self.pdl, -1, smem_kb, push)

    def _step_impl(self):
        cfg = self.cfg
        torch.index_select(self.embed, 0, self.tokens, out=self.residual)
        ops.add_rmsnorm(self.residual, None, self.layers[0]["norm1"], self.x, None, cfg.eps)
        for li, L in enumerate(self.layers):
            if self.linears == "penny":
                self._linear(self.x, L["wqkv"], self.qkv)
            else:
                torch.matmul(self.x, L["wqkv"].t(), out=self.qkv)
            ops.decode_attention_fused(self.qkv, self.kcache[li], self.vcache[li], self.positions, self.attn,
                                       self.workspace, self.Hq, self.Hkv, self.splits, self.scale, cfg.rope_theta,
                                       self.pdl)
            if self.linears == "penny":
                self._linear(self.attn, L["wo"], self.parts[0], push=self._push)
            else:
                torch.matmul(self.attn, L["wo"].t(), out=self.parts[0])
            self._reduce_norm(self.parts[0], L["norm2"])
            if self.linears == "penny":
                self._linear(self.x, L["wgu"], self.act, silu_pairs=True)
                self._linear(self.act, L["wdown"], self.parts[1], push=self._push)
            else:
                torch.matmul(self.x, L["wgu_cat"].t(), out=self.gu)
                ops.silu_mul(self.gu, self.act)
                torch.matmul(self.act, L["wdown"].t(), out=self.parts[1])
            nxt = self.layers[li + 1]["norm1"] if li + 1 < cfg.layers else self.final_norm
            self._reduce_norm(self.parts[1], nxt)
        if self.linears == "penny":
            # nothing of the step needs to overlap with the LM head: give it the whole shared memory
            self._linear(self.x, self.lm_head, self.logits, smem_kb=200)
        else:
            torch.matmul(self.x, self.lm_head.t(), out=self.logits)
        # greedy sampling: per-row (value, index) of this rank's vocabulary shard (indices < 2^24, exact
        # in fp32), gathered over the ranks; one kernel then picks the best rank per sequence, feeds the
        # token back (step() overwrites self.tokens with the caller's tokens) and advances the positions
        ops.argmax_rows(self.logits, self.max_val, self.max_idx, self.rank * self.V, self.argmax_ws, self.pair)
        if self.world == 1:
            ops.sample_finish(self.pair, 1, self.next_tokens, self.tokens, self.positions)
        else:
            if self.backend == "nccl":
                import torch.distributed as dist
                dist.all_gather_into_tensor(self.pairs_all, self.pair, group=self.pg)
            else:
                self.comm.all_gather(self.pair, out=self.pairs_all)
            ops.sample_finish(self.pairs_all, self.world, self.next_tokens, self.tokens, self.positions)

    def capture(self):
        """Warm up (cuBLAS handles, scratch growth) and capture the step in a CUDA graph."""
        saved = (self.positions.clone(), self.tokens.clone())
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self._step_impl()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        if self.use_graph:
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._step_impl()
            torch.cuda.synchronize()
        self.positions.copy_(saved[0])
        self.tokens.copy_(saved[1])

    def step_device(self):
        """One decode step on the device buffers: self.tokens -> self.next_tokens."""
        if self._graph is not None:
            self._graph.replay()
        else:
            self._step_impl()

    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """Public decode call: `tokens` is a CPU int64 tensor [batch]; returns the
        next token of every sequence as a CPU tensor.  Host -> device copy of the
        inputs from pinned memory, the step, device -> host read of the result."""
        self._host_in.copy_(tokens)
        self.tokens.copy_(self._host_in, non_blocking=True)
        self.step_device()
        self._host_out.copy_(self.next_tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._host_out

    def decode(self, steps: int) -> torch.Tensor:
        """Autoregressive greedy decode for `steps` tokens; returns [steps, batch] on the device."""
        out = []
        for _ in range(steps):
            self.step_device()
            out.append(self.next_tokens.clone())
        return torch.stack(out)

    # ------------------------------------------------------- fp32 torch oracle
    @torch.no_grad()
    def reference_logits(self, tokens: torch.Tensor, positions: torch.Tensor, kcaches, vcaches):
        """Plain PyTorch fp32 logits of one decode step from FULL (unsharded) state;
        only valid for world == 1 objects (tests build one with full_init=True)."""
        assert self.world == 1
        cfg = self.cfg
        D = cfg.head_dim
        B = tokens.numel()
        res = self.embed[tokens].float()

        def norm(z, w):
            return z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + cfg.eps) * w.float()
        x = norm(res, self.layers[0]["norm1"])
        for li, L in enumerate(self.layers):
            qkv = x.to(torch.bfloat16).float() @ L["wqkv"].float().t()
            q = qkv[:, :cfg.heads * D].view(B, cfg.heads, D)
            k = qkv[:, cfg.heads * D:(cfg.heads + cfg.kv_heads) * D].view(B, cfg.kv_heads, D)
            v = qkv[:, (cfg.heads + cfg.kv_heads) * D:].view(B, cfg.kv_heads, D)
            inv = cfg.rope_theta ** (-torch.arange(0, D // 2, device=self.dev, dtype=torch.float32) * 2 / D)
            ang = positions.float()[:, None] * inv[None]
            cos, sin = ang.cos()[:, None], ang.sin()[:, None]

            def rope(t):
                a, b = t[..., :D // 2], t[..., D // 2:]
                return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
            q, k = rope(q), rope(k)
            outs = []
            for b in range(B):
                p = int(positions[b])
                kk = torch.cat([kcaches[li][b, :, :p].float(), k[b].to(torch.bfloat16).float()[:, None]], 1)
                vv = torch.cat([vcaches[li][b, :, :p].float(), v[b].to(torch.bfloat16).float()[:, None]], 1)
                g = cfg.heads // cfg.kv_heads
                qq = q[b].to(torch.bfloat16).float().view(cfg.kv_heads, g, D)
                s = torch.einsum("hgd,htd->hgt", qq, kk) / math.sqrt(D)
                outs.append(torch.einsum("hgt,htd->hgd", s.softmax(-1), vv).reshape(cfg.heads * D))
            attn = torch.stack(outs)
            res = res.to(torch.bfloat16).float() + (attn.to(torch.bfloat16).float() @ L["wo"].float().t())
            x = norm(res, L["norm2"])
            wg, wu = self.split_gate_up(L["wgu"])
            xb = x.to(torch.bfloat16).float()
            act = torch.nn.functional.silu(xb @ wg.float().t()) * (xb @ wu.float().t())
            res = res.to(torch.bfloat16).float() + (act.to(torch.bfloat16).float() @ L["wdown"].float().t())
            nxt = self.layers[li + 1]["norm1"] if li + 1 < cfg.layers else self.final_norm
            x = norm(res, nxt)
        return x.to(torch.bfloat16).float() @ self.lm_head.float().t()
