"""Functional API: the collectives and fused ops on whichever backend the process has.

    import penny_b200.ops as P
    P.init()                       # after torch.distributed is up (torchrun)
    y = P.all_reduce(x)            # auto-selected algorithm
    y = P.all_reduce(x, algo="nvls")
    out, res = P.all_reduce_rmsnorm(partial, weight, residual)

With a GPU the calls go to the native communicator (symmetric heap + peer-memory
kernels); without one they go to the gloo backend with the same semantics, which
is what the CPU test tier runs.  The reference exposes the same operations as
methods of algorithm objects (csrc/common.h:89-118) and of CustomAllreduce.
"""
from __future__ import annotations

from typing import Optional

import torch

_BACKEND = None


def init(group=None, heap_bytes: Optional[int] = None, force_cpu: bool = False):
    """Creates the process-wide backend over `group` (default group if None)."""
    global _BACKEND
    if _BACKEND is not None:
        return _BACKEND
    if torch.cuda.is_available() and not force_cpu:
        if group is None:
            from ..utils import global_communicator
            _BACKEND = global_communicator(heap_bytes=heap_bytes)
        else:
            from ..parallel.comm import Communicator
            _BACKEND = Communicator.create(group, heap_bytes=heap_bytes)
    else:
        from ..parallel.cpu_backend import CpuCommunicator
        _BACKEND = CpuCommunicator(group)
    return _BACKEND


def backend():
    if _BACKEND is None:
        raise RuntimeError("penny_b200.ops.init() has not been called")
    return _BACKEND


def shutdown():
    global _BACKEND
    if _BACKEND is not None:
        _BACKEND.close()
        _BACKEND = None


def all_reduce(x, out=None, algo="auto", **kw):
    return backend().all_reduce(x, out=out, algo=algo, **kw)


def all_gather(x, out=None, **kw):
    return backend().all_gather(x, out=out, **kw)


def reduce_scatter(x, out=None, **kw):
    return backend().reduce_scatter(x, out=out, **kw)


def all_to_all(x, out=None, **kw):
    return backend().all_to_all(x, out=out, **kw)


def exchange(buf, peer, **kw):
    return backend().exchange(buf, peer, **kw)


def all_reduce_rmsnorm(x, weight, residual=None, out=None, eps: float = 1e-5, proto: str = "ll", **kw):
    """(rmsnorm(all_reduce(x) + residual) * weight, all_reduce(x) + residual)."""
    return backend().fused_all_reduce_rmsnorm(x, weight, residual=residual, out=out, eps=eps, proto=proto, **kw)


def gemm_reduce_scatter(a, weight, out=None):
    return backend().gemm_reduce_scatter(a, weight, out=out)


def all_gather_gemm(a_shard, weight, out=None, **kw):
    return backend().all_gather_gemm(a_shard, weight, out=out, **kw)


def empty(*shape, dtype=torch.bfloat16):
    """A tensor in the symmetric heap (peers and the NVSwitch can address it)."""
    return backend().empty(*shape, dtype=dtype)
