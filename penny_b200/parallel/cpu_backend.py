"""The same collectives on CPU tensors over a torch.distributed (gloo) group.

This backend exists so that the API and the data semantics – shard order = rank
order, fp32 accumulation in rank order, ragged sizes, out-of-place results – can
be exercised with no GPU at all (world_size >= 2 over gloo).  The rings follow
the very schedule the kernels use (penny_b200.parallel.schedule -> csrc/schedule.h),
moved with send/recv; the direct algorithms map onto gloo collectives.
The reference has no CPU path: `custom_ar` is simply False without a GPU
(penny/custom_all_reduce.py:16-21).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import schedule


def _acc_dtype(t: torch.Tensor):
    return torch.float32 if t.dtype in (torch.float16, torch.bfloat16) else t.dtype


class CpuCommunicator:
    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.emulated = False
        self.has_multicast = False

    def _global(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    # -------------------------------------------------------------- all-reduce
    def all_reduce(self, inp: torch.Tensor, out: Optional[torch.Tensor] = None, algo: str = "auto",
                   nnodes: int = 1, routes: int = 0, **_):
        flat = inp.reshape(-1)
        if algo in ("ring_standard", "ring", "double_ring"):
            res = self._ring_all_reduce(flat, nnodes if algo != "double_ring" else 1)
        elif algo in ("ring_simple",):
            res = self._chain_all_reduce(flat)
        else:  # one-shot / two-shot / tree / nvls: gather everything, add in rank order
            parts = [torch.empty_like(flat) for _ in range(self.world_size)]
            dist.all_gather(parts, flat.contiguous(), group=self.group)
            acc = torch.zeros(flat.shape, dtype=_acc_dtype(flat))
            for p in parts:
                acc += p.to(acc.dtype)
            res = acc.to(inp.dtype)
        res = res.reshape(inp.shape)
        if out is None:
            return res
        out.copy_(res)
        return out

    def _sendrecv(self, send: torch.Tensor, dst: int, recv: torch.Tensor, src: int):
        ops = [dist.P2POp(dist.isend, send.contiguous(), self._global(dst), self.group),
               dist.P2POp(dist.irecv, recv, self._global(src), self.group)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()

    def _ring_all_reduce(self, flat: torch.Tensor, nnodes: int):
        n = self.world_size
        order = schedule.ring_order(n, nnodes, 0)
        pos = order.index(self.rank)
        nxt, prv = order[(pos + 1) % n], order[(pos - 1) % n]
        total = flat.numel()
        work = flat.clone()
        spans = [schedule.split_span(total, n, i) for i in range(n)]
        for step in range(2 * (n - 1)):
            sc, rc, reduce = schedule.ring_step_chunks(n, pos, step)
            sb, se = spans[sc]
            rb, re = spans[rc]
            recv = torch.empty(re - rb, dtype=flat.dtype)
            self._sendrecv(work[sb:se], nxt, recv, prv)
            if reduce:  # two values added in fp32, rounded once per hop
                work[rb:re] = (work[rb:re].to(_acc_dtype(flat)) + recv.to(_acc_dtype(flat))).to(flat.dtype)
            else:
                work[rb:re] = recv
        return work

    def _chain_all_reduce(self, flat: torch.Tensor):
        n, r = self.world_size, self.rank
        work = flat.clone()
        if r > 0:
            recv = torch.empty_like(work)
            dist.recv(recv, self._global(r - 1), group=self.group)
            work = (work.to(_acc_dtype(flat)) + recv.to(_acc_dtype(flat))).to(flat.dtype)
        if r < n - 1:
            dist.send(work, self._global(r + 1), group=self.group)
        # the result travels N-1 -> 0 -> 1 -> ... -> N-2
        if r == n - 1:
            dist.send(work, self._global(0), group=self.group)
        else:
            dist.recv(work, self._global((r - 1) % n), group=self.group)
            if r < n - 2:
                dist.send(work, self._global(r + 1), group=self.group)
        return work

    # ------------------------------------------------------- the other collectives
    def all_gather(self, inp: torch.Tensor, out: Optional[torch.Tensor] = None, **_):
        flat = inp.reshape(-1).contiguous()
        parts = [torch.empty_like(flat) for _ in range(self.world_size)]
        dist.all_gather(parts, flat, group=self.group)
        res = torch.cat(parts)
        if out is None:
            return res
        out.reshape(-1).copy_(res)
        return out

    def reduce_scatter(self, inp: torch.Tensor, out: Optional[torch.Tensor] = None, **_):
        flat = inp.reshape(-1)
        if flat.numel() % self.world_size:
            raise ValueError("reduce_scatter needs a multiple of the world size")
        shard = flat.numel() // self.world_size
        parts = [torch.empty_like(flat) for _ in range(self.world_size)]
        dist.all_gather(parts, flat.contiguous(), group=self.group)
        acc = torch.zeros(shard, dtype=_acc_dtype(flat))
        for p in parts:
            acc += p[self.rank * shard:(self.rank + 1) * shard].to(acc.dtype)
        res = acc.to(inp.dtype)
        if out is None:
            return res
        out.reshape(-1)[:shard].copy_(res)
        return out

    def all_to_all(self, inp: torch.Tensor, out: Optional[torch.Tensor] = None, **_):
        flat = inp.reshape(-1).contiguous()
        chunk = flat.numel() // self.world_size
        ins = list(flat.split(chunk))
        outs = [torch.empty(chunk, dtype=flat.dtype) for _ in range(self.world_size)]
        # gloo has no all_to_all: pairwise send/recv
        ops = []
        for p in range(self.world_size):
            if p == self.rank:
                outs[p].copy_(ins[p])
                continue
            ops.append(dist.P2POp(dist.isend, ins[p].contiguous(), self._global(p), self.group))
            ops.append(dist.P2POp(dist.irecv, outs[p], self._global(p), self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        res = torch.cat(outs)
        if out is None:
            return res
        out.reshape(-1).copy_(res)
        return out

    def exchange(self, buf: torch.Tensor, peer: int, **_):
        if peer == self.rank:
            return buf
        recv = torch.empty_like(buf)
        self._sendrecv(buf, peer, recv, peer)
        buf.copy_(recv)
        return buf

    def fused_all_reduce_rmsnorm(self, inp, weight, residual=None, out=None, residual_out=None, eps=1e-5, **_):
        z = self.all_reduce(inp).float()
        if residual is not None:
            z = z + residual.float()
        normed = (z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(inp.dtype)
        znew = z.to(inp.dtype)
        if out is not None:
            out.copy_(normed)
            normed = out
        if residual_out is not None:
            residual_out.copy_(znew)
            znew = residual_out
        elif residual is not None:
            residual.copy_(znew)
            znew = residual
        return normed, znew

    # ------------------------------------------ sequence-parallel linears (semantics)
    def gemm_reduce_scatter(self, a: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None):
        """out[M / world, N] = this rank's row shard of sum_r a_r[M, K_r] @ weight_r[N, K_r]^T
        (the GPU path fuses the GEMM and the reduce-scatter into one tcgen05 kernel)."""
        M = a.shape[0]
        if M % self.world_size:
            raise ValueError("gemm_reduce_scatter needs M to be a multiple of the world size")
        partial = (a.float() @ weight.float().t()).to(a.dtype)      # what each rank's GEMM epilogue emits
        shard = self.reduce_scatter(partial).reshape(M // self.world_size, weight.shape[0])
        if out is None:
            return shard
        out.copy_(shard)
        return out

    def all_gather_gemm(self, a_shard: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None, **_):
        """out[M, N] = all_gather(a_shard)[M, K] @ weight[N, K]^T."""
        full = self.all_gather(a_shard).reshape(a_shard.shape[0] * self.world_size, a_shard.shape[1])
        res = (full.float() @ weight.float().t()).to(a_shard.dtype)
        if out is None:
            return res
        out.copy_(res)
        return out

    def empty(self, *shape, dtype=torch.float32):
        """Counterpart of the symmetric-heap allocation: plain CPU memory here."""
        return torch.empty(*shape, dtype=dtype)

    def poison_scratch(self):
        return None

    def barrier(self):
        dist.barrier(group=self.group)

    def check(self):
        return None

    def close(self):
        return None
