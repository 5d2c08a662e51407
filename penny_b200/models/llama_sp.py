"""Llama-3-8B-shaped sequence-parallel prefill (random weights, one sequence of T tokens).

Megatron-style sequence parallelism on top of tensor parallelism: the residual
stream stays sharded along the sequence ([T / world, hidden] per GPU), the
linears are tensor-parallel, and the collective on each side of a linear is
fused INTO the GEMM kernel:

    x_shard -> rmsnorm ------------------(all-gather -> tcgen05 GEMM, one kernel)--> qkv [T, local heads]
            -> RoPE -> causal GQA attention over the local heads
            -> (tcgen05 GEMM -> reduce-scatter, one kernel) o_proj -> + residual -> rmsnorm
            -> (all-gather -> tcgen05 GEMM) gate/up -> silu * mul
            -> (tcgen05 GEMM -> reduce-scatter) down -> + residual

`backend="penny"` uses `Communicator.all_gather_gemm` / `gemm_reduce_scatter`;
`backend="nccl"` is the baseline: NCCL all_gather_into_tensor / reduce_scatter_tensor
around cuBLAS GEMMs.  With `device="cpu"` (and a `CpuCommunicator` over gloo) the
same sharding and layer logic runs on CPU tensors with plain torch ops, which is
how the model's partitioning is tested without a GPU.  The attention itself is not a communication op and goes
to the library kernel behind `torch.nn.functional.scaled_dot_product_attention`
in both backends; norms, RoPE and silu*mul are this library's kernels in both.

Weights are generated in full from the seed and sliced, so every world size
runs the same model and `reference_forward` (fp32, one device) is its oracle.

The reference has no model code and no sequence parallelism; it only offers
the reduce-scatter / all-gather building blocks (custom_all_reduce.py:269-349).
"""
from __future__ import annotations

import math
from typing import Iterator, Optional

import torch
import torch.nn.functional as F_

from .._ext import ops
from .llama_tp import LlamaConfig


def _full_weights(cfg: LlamaConfig, layers: int, seed: int, device) -> Iterator[dict]:
    """Full (unsharded) bf16 weights, one layer at a time, [out, in] like nn.Linear."""
    g = torch.Generator(device=device)
    D, H, Fn = cfg.head_dim, cfg.hidden, cfg.ffn
    for li in range(layers):
        def rnd(*shape, sub):
            g.manual_seed(seed * 1000003 + li * 101 + sub)
            return (torch.randn(*shape, device=device, generator=g, dtype=torch.float32) * cfg.init_std).bfloat16()
        yield {
            "wq": rnd(cfg.heads * D, H, sub=1), "wk": rnd(cfg.kv_heads * D, H, sub=2),
            "wv": rnd(cfg.kv_heads * D, H, sub=3), "wo": rnd(H, cfg.heads * D, sub=4),
            "wg": rnd(Fn, H, sub=5), "wu": rnd(Fn, H, sub=6), "wd": rnd(H, Fn, sub=7),
            "norm1": (1.0 + 0.1 * rnd(H, sub=8).float()).bfloat16(),
            "norm2": (1.0 + 0.1 * rnd(H, sub=9).float()).bfloat16(),
        }


class LlamaSPPrefill:
    """`layers` transformer layers over one sequence of `tokens` tokens, sequence-parallel over `world` GPUs."""

    def __init__(self, cfg: LlamaConfig, comm=None, rank: int = 0, world: int = 1, tokens: int = 4096,
                 layers: Optional[int] = None, backend: str = "penny", seed: int = 0, process_group=None,
                 device: str = "cuda"):
        assert backend in ("penny", "nccl")
        assert cfg.heads % world == 0 and cfg.kv_heads % world == 0 and cfg.ffn % world == 0 and cfg.head_dim == 128
        self.cpu = device == "cpu"
        if self.cpu:
            assert tokens % world == 0
        else:
            assert tokens % (world * 128) == 0, "every rank's sequence shard must be whole 128-row blocks"
        if backend == "penny":
            assert comm is not None, "the fused kernels need a Communicator (use Communicator.emulated(1) on one GPU)"
        self.cfg, self.comm, self.rank, self.world, self.T = cfg, comm, rank, world, tokens
        self.backend, self.pg = backend, process_group
        self.L = cfg.layers if layers is None else layers
        self.Hq, self.Hkv, self.F = cfg.heads // world, cfg.kv_heads // world, cfg.ffn // world
        self.dev = torch.device("cpu") if self.cpu else torch.device("cuda", torch.cuda.current_device())
        D, H, r = cfg.head_dim, cfg.hidden, rank
        self.layers = []
        for w in _full_weights(cfg, self.L, seed, self.dev):
            q = w["wq"][r * self.Hq * D:(r + 1) * self.Hq * D]
            k = w["wk"][r * self.Hkv * D:(r + 1) * self.Hkv * D]
            v = w["wv"][r * self.Hkv * D:(r + 1) * self.Hkv * D]
            self.layers.append({
                "wqkv": torch.cat([q, k, v], 0).contiguous(),
                "wo": w["wo"][:, r * self.Hq * D:(r + 1) * self.Hq * D].contiguous(),
                "wgu": torch.cat([w["wg"][r * self.F:(r + 1) * self.F], w["wu"][r * self.F:(r + 1) * self.F]], 0).contiguous(),
                "wd": w["wd"][:, r * self.F:(r + 1) * self.F].contiguous(),
                "norm1": w["norm1"], "norm2": w["norm2"],
            })
        dt, Ts = torch.bfloat16, tokens // world
        e = lambda *s: torch.empty(*s, dtype=dt, device=self.dev)  # noqa: E731
        self.h = e(Ts, H)                                  # normalised shard, input of the gathered GEMMs
        self.qkv = e(tokens, (self.Hq + 2 * self.Hkv) * D)
        self.attn = e(tokens, self.Hq * D)
        self.part = e(Ts, H)                               # reduce-scattered linear output
        self.gu = e(tokens, 2 * self.F)
        self.act = e(tokens, self.F)
        self.gathered = e(tokens, H) if backend == "nccl" and not self.cpu else None
        self.full = e(tokens, H) if backend == "nccl" and not self.cpu else None
        self.scale = 1.0 / math.sqrt(D)
        # kernels of this library per forward: per layer 2 norms, RoPE, silu*mul and (penny) 4 fused GEMMs
        self.kernels_per_forward = self.L * (4 + (4 if backend == "penny" else 0))

    # ------------------------------------------------------------------ linears
    def _col(self, h_shard: torch.Tensor, w: torch.Tensor, out: torch.Tensor):
        """Column-parallel linear on the gathered sequence: out[T, n] = all_gather(h_shard) @ w^T."""
        if self.backend == "penny" or self.cpu:
            self.comm.all_gather_gemm(h_shard, w, out=out)
        else:
            if self.world > 1:
                torch.distributed.all_gather_into_tensor(self.gathered, h_shard, group=self.pg)
                torch.matmul(self.gathered, w.t(), out=out)
            else:
                torch.matmul(h_shard, w.t(), out=out)

    def _row(self, a: torch.Tensor, w: torch.Tensor, out_shard: torch.Tensor):
        """Row-parallel linear, result summed over ranks and scattered along the sequence."""
        if self.backend == "penny" or self.cpu:
            self.comm.gemm_reduce_scatter(a, w, out=out_shard)
        else:
            if self.world > 1:
                torch.matmul(a, w.t(), out=self.full)
                torch.distributed.reduce_scatter_tensor(out_shard, self.full, group=self.pg)
            else:
                torch.matmul(a, w.t(), out=out_shard)

    # ------------------------------------------- elementwise kernels (torch on CPU)
    def _add_rmsnorm(self, x, residual, weight, out, residual_out):
        if not self.cpu:
            ops.add_rmsnorm(x, residual, weight, out, residual_out, self.cfg.eps)
            return
        z = x.float() if residual is None else x.float() + residual.float()
        if residual_out is not None:
            residual_out.copy_(z.to(residual_out.dtype))      # the norm below uses the unrounded sum, like the kernel
        out.copy_((z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * weight.float()).to(out.dtype))

    def _rope(self):
        cfg, D = self.cfg, self.cfg.head_dim
        if not self.cpu:
            ops.rope_rows(self.qkv, self.Hq, self.Hkv, D, 0, cfg.rope_theta)
            return
        half, nh = D // 2, self.Hq + self.Hkv
        inv = cfg.rope_theta ** (-2.0 * torch.arange(half, dtype=torch.float32) / D)
        ang = torch.arange(self.T, dtype=torch.float32)[:, None] * inv[None]
        cos, sin = ang.cos()[:, None], ang.sin()[:, None]
        v = self.qkv.view(self.T, self.Hq + 2 * self.Hkv, D)
        a, b = v[:, :nh, :half].float(), v[:, :nh, half:].float()
        v[:, :nh, :half] = (a * cos - b * sin).to(v.dtype)
        v[:, :nh, half:] = (b * cos + a * sin).to(v.dtype)

    def _silu_mul(self):
        if not self.cpu:
            ops.silu_mul(self.gu, self.act)
            return
        g, u = self.gu[:, :self.F].float(), self.gu[:, self.F:].float()
        self.act.copy_((F_.silu(g) * u).to(self.act.dtype))

    def _attention(self):
        cfg, D, T = self.cfg, self.cfg.head_dim, self.T
        self._rope()
        q = self.qkv[:, :self.Hq * D].view(T, self.Hq, D).permute(1, 0, 2).unsqueeze(0)
        k = self.qkv[:, self.Hq * D:(self.Hq + self.Hkv) * D].view(T, self.Hkv, D).permute(1, 0, 2).unsqueeze(0)
        v = self.qkv[:, (self.Hq + self.Hkv) * D:].view(T, self.Hkv, D).permute(1, 0, 2).unsqueeze(0)
        o = F_.scaled_dot_product_attention(q, k, v, is_causal=True, scale=self.scale, enable_gqa=True)
        self.attn.view(T, self.Hq, D).copy_(o[0].permute(1, 0, 2))

    # ------------------------------------------------------------------ forward
    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        """x_shard: this rank's [T / world, hidden] rows of the residual stream; returns the same rows after all layers."""
        res = x_shard.clone()
        self._add_rmsnorm(res, None, self.layers[0]["norm1"], self.h, None)
        for li, l in enumerate(self.layers):
            self._col(self.h, l["wqkv"], self.qkv)
            self._attention()
            self._row(self.attn, l["wo"], self.part)
            self._add_rmsnorm(self.part, res, l["norm2"], self.h, res)          # res += o_proj; h = norm(res)
            self._col(self.h, l["wgu"], self.gu)
            self._silu_mul()
            self._row(self.act, l["wd"], self.part)
            if li + 1 < len(self.layers):
                self._add_rmsnorm(self.part, res, self.layers[li + 1]["norm1"], self.h, res)
            else:
                res.add_(self.part)
        return res

    # ------------------------------------------------------------------- oracle
    @staticmethod
    def reference_forward(cfg: LlamaConfig, x: torch.Tensor, layers: int, seed: int = 0) -> torch.Tensor:
        """The same model on one device in fp32 from the full weights: x [T, hidden] -> [T, hidden]."""
        D, T = cfg.head_dim, x.shape[0]
        half = D // 2
        inv = cfg.rope_theta ** (-2.0 * torch.arange(half, device=x.device, dtype=torch.float32) / D)
        ang = torch.arange(T, device=x.device, dtype=torch.float32)[:, None] * inv[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

        def norm(v, w):
            return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * w.float()

        def rope(t):  # [T, heads, D]
            a, b = t[..., :half], t[..., half:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
        res = x.float()
        for w in _full_weights(cfg, layers, seed, x.device):
            h = norm(res, w["norm1"]).bfloat16().float()
            q = rope((h @ w["wq"].float().t()).bfloat16().float().view(T, cfg.heads, D)).bfloat16().float()
            k = rope((h @ w["wk"].float().t()).bfloat16().float().view(T, cfg.kv_heads, D)).bfloat16().float()
            v = (h @ w["wv"].float().t()).bfloat16().float().view(T, cfg.kv_heads, D)
            o = F_.scaled_dot_product_attention(q.permute(1, 0, 2)[None], k.permute(1, 0, 2)[None],
                                                v.permute(1, 0, 2)[None], is_causal=True,
                                                scale=1.0 / math.sqrt(D), enable_gqa=True)[0]
            attn = o.permute(1, 0, 2).reshape(T, cfg.heads * D).bfloat16().float()
            res = (res + (attn @ w["wo"].float().t())).bfloat16().float()
            h = norm(res, w["norm2"]).bfloat16().float()
            act = (F_.silu((h @ w["wg"].float().t()).bfloat16().float()) *
                   (h @ w["wu"].float().t()).bfloat16().float()).bfloat16().float()
            res = (res + (act @ w["wd"].float().t())).bfloat16().float()
        return res
