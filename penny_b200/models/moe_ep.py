"""Mixtral-8x7B-shaped MoE layer with expert parallelism.

Every rank holds `experts / world` experts (SwiGLU FFNs) and its own tokens.
One forward pass:

    router (top-k of softmax-normalised logits)
    -> routing tables (which row goes where; a tiny all-gather of per-expert counts)
    -> dispatch: rows pushed over NVLink straight into the owners' dense
       expert-input buffers                                   (one kernel)
    -> expert FFN on the received rows (tcgen05 GEMMs of this library)
    -> combine: outputs pushed back to their sources and summed with the gate
       weights in the same kernel                             (one kernel)

`backend="nccl"` does the two exchanges with all_to_all_single (padded to equal
splits is not needed: it uses the split-size form) and the weighted sum as a
separate op – the baseline.  Works with a real communicator (one process per
GPU) or an emulated one (all ranks on one GPU: every tensor argument is then a
list).  The reference has no MoE path; its exchange is a pairwise swap
(csrc/exchange.cu).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from .._ext import ops


@dataclass
class MoeConfig:
    hidden: int = 4096
    ffn: int = 14336
    experts: int = 8
    topk: int = 2
    init_std: float = 0.02

    @classmethod
    def mixtral_8x7b(cls):
        return cls()

    @classmethod
    def tiny(cls):
        return cls(hidden=256, ffn=512, experts=8, topk=2)


def route(logits: torch.Tensor, topk: int):
    """Top-k routing: expert ids [T, k] (int32) and gate weights [T, k] (fp32,
    softmax over the selected logits, as Mixtral does).  One kernel for bf16 CUDA logits
    (csrc/moe_routing.cu), torch ops otherwise."""
    if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.is_contiguous() and topk <= 8:
        return ops.moe_route(logits, topk)
    return route_torch(logits, topk)


def route_torch(logits: torch.Tensor, topk: int):
    vals, ids = logits.float().topk(topk, dim=-1)
    return ids.to(torch.int32).contiguous(), torch.softmax(vals, dim=-1).contiguous()


def build_routing(topk_ids: torch.Tensor, experts: int):
    """Sender-side tables for one rank: pairs sorted by expert (stable), per-expert counts.
    One kernel (a counting sort in one thread block) instead of sort + bincount + cumsum."""
    if topk_ids.is_cuda and topk_ids.dtype == torch.int32 and experts <= 256:
        return ops.moe_tables(topk_ids.reshape(-1).contiguous(), experts)
    return build_routing_torch(topk_ids, experts)


def build_routing_torch(topk_ids: torch.Tensor, experts: int):
    flat = topk_ids.reshape(-1).to(torch.int64)
    expert_sorted, order = torch.sort(flat, stable=True)
    counts = torch.bincount(flat, minlength=experts)
    send_off = torch.zeros(experts + 1, dtype=torch.int64, device=flat.device)
    send_off[1:] = counts.cumsum(0)
    return (order.to(torch.int32).contiguous(), expert_sorted.to(torch.int32).contiguous(),
            send_off.to(torch.int32).contiguous(), counts)


def placement_device(counts_all: torch.Tensor):
    """`placement` on the device: counts_all [W, E] int32 (CUDA) -> dst_base [W, E] int32 (stays on
    the device for the dispatch kernel), and - the one host round trip of the layer, because the
    expert GEMMs are launched with host-side shapes - rows_per_rank and per-rank expert ranges."""
    W, E = counts_all.shape
    dst_base, rows, ranges = ops.moe_placement(counts_all.contiguous())
    host = torch.cat([rows, ranges.reshape(-1)]).cpu().tolist()
    rows_per_rank, flat = host[:W], host[W:]
    epr = E // W
    expert_ranges = [[(flat[2 * (d * epr + le)], flat[2 * (d * epr + le) + 1]) for le in range(epr)] for d in range(W)]
    return dst_base, rows_per_rank, expert_ranges


def placement(counts_all: torch.Tensor, world: int):
    """counts_all[s, e] = rows rank s sends to expert e.  Returns
    dst_base[s, e] (row at e's owner where s's rows of e start), rows_per_rank[d]
    and expert_rows[d] = per-local-expert row ranges (start, end) at rank d.
    Rows at an owner are ordered by local expert, then by source rank."""
    W, E = counts_all.shape
    epr = E // world
    dst_base = torch.zeros_like(counts_all)
    rows_per_rank, expert_ranges = [], []
    for d in range(world):
        base = 0
        ranges = []
        for le in range(epr):
            e = d * epr + le
            start = base
            for s in range(W):
                dst_base[s, e] = base
                base += int(counts_all[s, e])
            ranges.append((start, base))
        rows_per_rank.append(base)
        expert_ranges.append(ranges)
    return dst_base, rows_per_rank, expert_ranges


class MoeEPLayer:
    def __init__(self, cfg: MoeConfig, comm, tokens: int, cap_factor: float = 2.0, backend: str = "penny",
                 seed: int = 0, use_own_gemm: bool = True):
        self.cfg, self.comm, self.backend = cfg, comm, backend
        self.world = comm.world_size
        self.views = comm.views
        self.tokens = tokens
        self.epr = cfg.experts // self.world
        assert cfg.experts % self.world == 0
        self.use_own_gemm = use_own_gemm
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        pairs = tokens * cfg.topk
        self.cap_rows = int(cap_factor * pairs) // 8 * 8
        dt = torch.bfloat16
        # symmetric buffers the peers write into
        self.recv = self._as_views(comm.empty(self.cap_rows, cfg.hidden, dtype=dt))
        self.meta = self._as_views(comm.empty(self.cap_rows, dtype=torch.float32))  # int32 payload
        self.meta = [m.view(torch.int32) for m in self.meta]
        self.comb = self._as_views(comm.empty(pairs, cfg.hidden, dtype=dt))
        self.counts_buf = self._as_views(comm.empty(cfg.experts, dtype=torch.float32))
        self.dst_row_of_pair = [torch.zeros(pairs, dtype=torch.int32, device=dev) for _ in range(self.views)]
        # weights: router replicated; experts sharded
        self.ranks = list(range(self.world)) if comm.emulated else [comm.rank]
        g = torch.Generator(device=dev)
        self.router, self.w13, self.w2 = [], [], []
        for r in self.ranks:
            g.manual_seed(seed * 7919 + 1)
            self.router.append((torch.randn(cfg.experts, cfg.hidden, device=dev, generator=g) * cfg.init_std).to(dt))
            w13, w2 = [], []
            for le in range(self.epr):
                g.manual_seed(seed * 7919 + 100 + r * self.epr + le)
                w13.append((torch.randn(2 * cfg.ffn, cfg.hidden, device=dev, generator=g) * cfg.init_std).to(dt))
                w2.append((torch.randn(cfg.hidden, cfg.ffn, device=dev, generator=g) * cfg.init_std).to(dt))
            self.w13.append(w13)
            self.w2.append(w2)

    def _as_views(self, t) -> List[torch.Tensor]:
        return list(t) if isinstance(t, (list, tuple)) else [t]

    def _gemm(self, a, w):
        out = torch.empty(a.shape[0], w.shape[0], dtype=a.dtype, device=a.device)
        if a.shape[0] == 0:
            return out
        if self.use_own_gemm:
            ops.gemm_bf16(a, w, out, 0)
        else:
            torch.matmul(a, w.t(), out=out)
        return out

    def _experts(self, v: int, rows: torch.Tensor, ranges):
        """SwiGLU FFN of this rank's local experts over its received rows."""
        y = torch.empty_like(rows)
        for le, (s, e) in enumerate(ranges):
            if e <= s:
                continue
            h = self._gemm(rows[s:e], self.w13[v][le])
            act = torch.empty(e - s, self.cfg.ffn, dtype=rows.dtype, device=rows.device)
            ops.silu_mul(h, act)
            y[s:e] = self._gemm(act, self.w2[v][le])
        return y

    def forward(self, x):
        """x: [tokens, hidden] (a list with one tensor per virtual rank when emulated)."""
        cfg, comm = self.cfg, self.comm
        xs = self._as_views(x)
        ids, gates, tables = [], [], []
        for v, xv in enumerate(xs):
            i, g = route(torch.matmul(xv, self.router[v].t()), cfg.topk)
            ids.append(i)
            gates.append(g)
            tables.append(build_routing(i, cfg.experts))
            self.counts_buf[v].view(torch.int32).copy_(tables[v][3].to(torch.int32))
        # every rank learns how many rows each rank sends to each expert
        if self.world > 1:
            gathered = comm.all_gather(self.counts_buf if comm.emulated else self.counts_buf[0])
            gathered = self._as_views(gathered)
            counts_dev = gathered[0].view(torch.int32).view(self.world, cfg.experts)
        else:
            counts_dev = tables[0][3].to(torch.int32).view(1, cfg.experts)
        dst_base, rows_per_rank, expert_ranges = placement_device(counts_dev)
        if max(rows_per_rank) > self.cap_rows:
            raise RuntimeError(f"MoE capacity exceeded: {max(rows_per_rank)} rows > {self.cap_rows}")
        dst_base_dev = [dst_base[r].contiguous() for r in self.ranks]
        counts_all = counts_dev.cpu() if self.backend != "penny" else None  # the NCCL baseline wants split sizes
        L = (lambda t: t) if comm.emulated else (lambda t: t[0])
        if self.backend == "penny":
            comm.moe_dispatch(L(xs), L([t[0] for t in tables]), L([t[1] for t in tables]), L([t[2] for t in tables]),
                              L(dst_base_dev), L(self.dst_row_of_pair), L(self.recv), L(self.meta), cfg.topk,
                              cfg.experts)
            ys = []
            for v, r in enumerate(self.ranks):
                ys.append(self._experts(v, self.recv[v][:rows_per_rank[r]], expert_ranges[r]))
            outs = [torch.empty_like(xv) for xv in xs]
            comm.moe_combine(L(ys), L(outs), L([i.reshape(-1).contiguous() for i in ids]),
                             L([g.reshape(-1).contiguous() for g in gates]), L(self.meta), L(self.dst_row_of_pair),
                             L(self.comb), [rows_per_rank[r] for r in self.ranks] if comm.emulated
                             else rows_per_rank[self.ranks[0]], cfg.experts)
            return outs if comm.emulated else outs[0]
        return self._forward_nccl(xs[0], ids[0], gates[0], tables[0], counts_all, rows_per_rank, expert_ranges)

    def _forward_nccl(self, x, ids, gates, table, counts_all, rows_per_rank, expert_ranges):
        """Baseline: the same layer with NCCL all_to_all_single for both exchanges."""
        import torch.distributed as dist
        cfg, r = self.cfg, self.comm.rank
        order, expert_sorted, send_off, _ = table
        send_rows = x[(order.long() // cfg.topk)]
        # per-destination split sizes; received rows arrive ordered by source, then expert
        in_splits = [int(counts_all[r, d * self.epr:(d + 1) * self.epr].sum()) for d in range(self.world)]
        out_splits = [int(counts_all[s, r * self.epr:(r + 1) * self.epr].sum()) for s in range(self.world)]
        recv = torch.empty(sum(out_splits), cfg.hidden, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(recv, send_rows, out_splits, in_splits)
        if self.epr == 1:
            ranges = [(0, recv.shape[0])]
            y = self._experts(0, recv, ranges)
        else:  # regroup by expert
            src_expert = torch.cat([torch.repeat_interleave(torch.arange(self.epr, device=x.device),
                                                            counts_all[s, r * self.epr:(r + 1) * self.epr].to(x.device))
                                    for s in range(self.world)])
            perm = torch.argsort(src_expert, stable=True)
            cnt = torch.bincount(src_expert, minlength=self.epr).tolist()
            ranges, b = [], 0
            for c in cnt:
                ranges.append((b, b + c))
                b += c
            y = torch.empty_like(recv)
            y[perm] = self._experts(0, recv[perm], ranges)
        back = torch.empty_like(send_rows)
        dist.all_to_all_single(back, y, in_splits, out_splits)
        per_pair = torch.empty_like(back)
        per_pair[order.long()] = back
        return (per_pair.view(self.tokens, cfg.topk, cfg.hidden).float() * gates[..., None]).sum(1).to(x.dtype)

    def reference(self, xs: List[torch.Tensor], all_w13, all_w2, router):
        """fp32 PyTorch oracle from FULL expert weights (all_w13[e], all_w2[e])."""
        outs = []
        for x in xs:
            ids, gates = route(torch.matmul(x, router.t()), self.cfg.topk)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for k in range(self.cfg.topk):
                for e in range(self.cfg.experts):
                    sel = (ids[:, k] == e).nonzero().squeeze(1)
                    if sel.numel() == 0:
                        continue
                    h = (x[sel].float() @ all_w13[e].float().t()).to(torch.bfloat16).float()
                    act = (torch.nn.functional.silu(h[:, :self.cfg.ffn]) * h[:, self.cfg.ffn:]).to(torch.bfloat16).float()
                    y = (act @ all_w2[e].float().t()).to(torch.bfloat16).float()
                    out[sel] += gates[sel, k, None] * y
            outs.append(out)
        return outs
