"""Drop-in ``CustomAllreduce`` for vLLM / SGLang tensor-parallel workers.

Constructor arguments, attributes and methods follow the reference class
(penny/custom_all_reduce.py:38-392): ``capture()``, ``register_graph_buffers``,
``should_custom_ar``, ``all_reduce / custom_all_reduce``, ``reduce_scatter /
custom_reduce_scatter``, ``all_gather / custom_all_gather``, ``close``, and the
static ``create_shared_buffer / free_shared_buffer``.  What differs:

* no NVSHMEM bootstrap (``nvshmem_registered`` / ``symm_mem_enabled`` are
  accepted and ignored) and ``NNODES`` is optional (default 1: one box);
* on one box the three collectives run on the symmetric-heap communicator's
  kernels, chosen per message size from the measured table: flag-in-data
  pushes for the smallest messages, the switch reduction (NVLS) or pushes
  above.  Those kernels read their input where it is - the owner pushes, or
  the host stages it into the heap - so nothing has to be registered, in eager
  mode or under ``capture()``, and the eager path needs no staging copy;
* the pull kernels with bounded waits (csrc/custom_all_reduce.cu), which read
  the peers' IPC-registered buffers like the reference's, remain: they serve
  ``all_reduce(..., registered=True)`` on buffers registered through raw IPC
  pointers, multi-node groups, and everything when
  ``PENNY_CUSTOM_AR_BACKEND=pull``;
* P2P capability is really checked (the reference's ``_can_p2p`` returns True
  unconditionally, :23-30);
* ``fused_all_reduce_rmsnorm`` – all-reduce + residual add + RMSNorm in one
  kernel through the symmetric-heap communicator – is offered on top.
"""
from __future__ import annotations

import logging
import os
from contextlib import contextmanager
from typing import List, Optional, Union

import torch
import torch.distributed as dist
from torch.distributed import ProcessGroup

from .._ext import ops

logger = logging.getLogger(__name__)
nnodes = int(os.getenv("NNODES", "1"))

try:
    ops.meta_size()
    custom_ar = True
except Exception:  # pragma: no cover - extension without the custom-AR family
    custom_ar = False


def _can_p2p(rank: int, world_size: int) -> bool:
    for i in range(world_size):
        if i == rank:
            continue
        if not torch.cuda.can_device_access_peer(rank, i):
            return False
    return True


def is_weak_contiguous(inp: torch.Tensor) -> bool:
    return inp.is_contiguous() or (inp.untyped_storage().nbytes() - inp.storage_offset() * inp.element_size()
                                   == inp.numel() * inp.element_size())


class CustomAllreduce:
    _SUPPORTED_WORLD_SIZES = [2, 4, 6, 8]

    def __init__(self, group: ProcessGroup, device: Union[int, str, torch.device], max_size=8192 * 1024,
                 symm_mem_enabled=False, nvshmem_registered=False) -> None:
        """group: a non-NCCL (gloo) process group whose ranks are the GPUs of one
        box; device: this rank's GPU; max_size: largest message (bytes) served."""
        self._IS_CAPTURING = False
        self.disabled = True
        self._ptr = 0
        self._comm = None
        self._own_comm = False
        self._fast_cache = {}
        if not custom_ar or not torch.cuda.is_available():
            logger.info("Custom allreduce is disabled because of missing custom allreduce library or GPU")
            return
        self.group = group
        assert dist.get_backend(group) != dist.Backend.NCCL, (
            "CustomAllreduce should be attached to a non-NCCL group.")
        rank = dist.get_rank(group=self.group)
        world_size = dist.get_world_size(group=self.group) // nnodes
        if world_size == 1:
            return
        if world_size not in CustomAllreduce._SUPPORTED_WORLD_SIZES:
            logger.warning("Custom allreduce is disabled due to an unsupported world size: %d. "
                           "Supported world sizes: %s.", world_size, str(CustomAllreduce._SUPPORTED_WORLD_SIZES))
            return
        if isinstance(device, int):
            device = torch.device(f"cuda:{device}")
        elif isinstance(device, str):
            device = torch.device(device)
        assert isinstance(device, torch.device)
        self.device = device
        if torch.cuda.device_count() >= world_size and not _can_p2p(rank % world_size, world_size):
            logger.warning("Custom allreduce is disabled because the GPUs lack peer-to-peer access.")
            return
        self.disabled = False
        # metadata (flags + 2-stage scratch) and the eager-mode staging buffer, both IPC-shared
        self.meta_ptrs = self.create_shared_buffer(ops.meta_size() + max_size, group=group, uncached=True)
        self.buffer_ptrs = self.create_shared_buffer(max_size, group=group)
        # pointer tuples of registered buffers: 64 B each, 8 MiB holds 131072 of them
        self.rank_data = torch.empty(8 * 1024 * 1024, dtype=torch.uint8, device=self.device)
        self.max_size = max_size
        self.rank = rank % world_size
        self.world_size = world_size
        self.fully_connected = True
        self._ptr = ops.init_custom_ar(self.meta_ptrs, self.rank_data, self.rank, self.fully_connected)
        ops.register_buffer(self._ptr, self.buffer_ptrs)
        # the fast path: a symmetric-heap communicator over the same ranks (one box only)
        if nnodes == 1 and os.environ.get("PENNY_CUSTOM_AR_BACKEND", "fast") != "pull":
            try:
                from .comm import Communicator
                heap = max(256 << 20, 24 * int(max_size))
                self._comm = Communicator.create(group, heap_bytes=heap)
                self._own_comm = True
            except Exception as e:  # noqa: BLE001
                logger.warning("CustomAllreduce: no symmetric-heap communicator (%s); using the pull kernels", e)
                self._comm = None

    # ----------------------------------------------------------- graph capture
    @contextmanager
    def capture(self):
        """Buffers first seen while a CUDA graph is being captured are registered
        with the peers when the context exits."""
        try:
            self._IS_CAPTURING = True
            yield
        finally:
            self._IS_CAPTURING = False
            if not self.disabled:
                self.register_graph_buffers()

    def register_graph_buffers(self):
        handle, offset = ops.get_graph_buffer_ipc_meta(self._ptr)
        world_size = dist.get_world_size(group=self.group)
        local_size = world_size // nnodes
        rank = dist.get_rank(group=self.group)
        all_data = [[None, None] for _ in range(world_size)]
        all_data[rank] = [handle, offset]
        ranks = sorted(dist.get_process_group_ranks(group=self.group))
        off = (rank // local_size) * local_size
        # broadcast_object_list instead of all_gather_object: the latter breaks
        # under gloo in inference mode
        for i, r in enumerate(ranks):
            dist.broadcast_object_list(all_data[i], src=r, group=self.group, device="cpu")
        handles = [d[0] for d in all_data[off:off + local_size]]
        offsets = [d[1] for d in all_data[off:off + local_size]]
        ops.register_graph_buffers(self._ptr, handles, offsets)

    # ------------------------------------------------------------- dispatching
    def should_custom_ar(self, inp: torch.Tensor) -> bool:
        if self.disabled:
            return False
        inp_size = inp.numel() * inp.element_size()
        if inp_size % 16 != 0:
            return False
        if not is_weak_contiguous(inp):
            return False
        # the kernels move 16-byte vectors: a dense slice that starts off a 16-byte
        # boundary (buf[3:] of a bf16 tensor) goes to the caller's fallback
        if inp.data_ptr() % 16 != 0:
            return False
        if self.world_size == 2 or self.fully_connected:
            return inp_size < self.max_size
        return False

    def _run(self, fn, inp, out, registered):
        if registered:
            fn(self._ptr, inp, out, 0, 0)
        else:
            fn(self._ptr, inp, out, self.buffer_ptrs[self.rank], self.max_size)
        return out

    @property
    def fast(self) -> bool:
        """True when the collectives run on the symmetric-heap communicator's kernels."""
        return self._comm is not None and not self.disabled

    def _dispatch(self, fast, eager, input, out, warmup_result):
        if self.disabled or not self.should_custom_ar(input):
            return None
        if self.fast:
            # nothing to register and nothing to stage: the same call in eager mode, while
            # warming up for a capture and inside the capture
            return fast(input, out)
        if self._IS_CAPTURING:
            if torch.cuda.is_current_stream_capturing():
                return eager(input, out=out, registered=True)
            # warm-up before capture: mimic the allocation, communicate nothing
            return warmup_result()
        return eager(input, out=out, registered=False)

    def all_reduce(self, inp: torch.Tensor, *, out: torch.Tensor = None, registered: bool = False):
        """Out-of-place all-reduce on the pull kernels.  registered=False copies the input into
        the pre-registered staging buffer first; registered=True reads `inp` through the IPC
        registration made by register_buffer / register_graph_buffers."""
        if out is None:
            out = torch.empty_like(inp)
        return self._run(ops.all_reduce, inp, out, registered)

    # The fast path goes straight to the extension: the tensors of a serving engine are ordinary
    # (non-heap) memory, so the memory class is known, and the table lookup is remembered per size.
    def _fast_all_reduce(self, inp, out):
        if out is None:
            out = torch.empty_like(inp)
        ops.comm_all_reduce(self._comm._h, [inp.view(-1)], [out.view(-1)], -1, 0, 0, 1, 0, False, False)
        return out

    def custom_all_reduce(self, input: torch.Tensor, out=None) -> Optional[torch.Tensor]:
        """All-reduce with CUDA-graph support; None means "use your fallback"."""
        return self._dispatch(self._fast_all_reduce, self.all_reduce, input, out, lambda: torch.empty_like(input))

    def reduce_scatter(self, inp: torch.Tensor, *, out: torch.Tensor = None, registered: bool = False):
        """Out-of-place reduce-scatter on the pull kernels; the shard lands in out[: numel // world]."""
        if out is None:
            out = torch.empty_like(inp)
        return self._run(ops.reduce_scatter, inp, out, registered)

    def _fast_algo(self, op, nbytes, dtype, allowed):
        key = (op, nbytes, dtype)
        algo = self._fast_cache.get(key)
        if algo is None:
            algo = self._comm._pick(op, nbytes, dtype, False) or "push"
            if algo not in allowed:
                algo = "push"
            self._fast_cache[key] = algo
        return algo

    def _fast_reduce_scatter(self, inp, out):
        if out is None:
            out = torch.empty_like(inp)
        shard = inp.numel() // self.world_size
        nbytes = shard * inp.element_size()
        algo = self._fast_algo("reduce_scatter", nbytes, inp.dtype,
                               ("push", "pipelined", "nvls") if nbytes % 16 == 0 and self._comm.has_multicast
                               else ("push", "pipelined"))
        ops.comm_reduce_scatter(self._comm._h, [inp.view(-1)], [out.view(-1)[:shard]], algo == "nvls", 0, 0, False,
                                algo == "pipelined")
        return out

    def custom_reduce_scatter(self, input: torch.Tensor, out=None) -> Optional[torch.Tensor]:
        if not self.disabled and input.numel() % self.world_size != 0:
            return None
        return self._dispatch(self._fast_reduce_scatter, self.reduce_scatter, input, out,
                              lambda: torch.empty_like(input))

    def all_gather(self, inp: torch.Tensor, *, out: torch.Tensor = None, registered: bool = False):
        if out is None:
            out = torch.empty(inp.numel() * self.world_size, dtype=inp.dtype, device=inp.device)
        return self._run(ops.all_gather, inp, out, registered)

    def _fast_all_gather(self, inp, out):
        n = inp.numel()
        if out is None:
            out = torch.empty(n * self.world_size, dtype=inp.dtype, device=inp.device)
        # the multicast all-gather needs an output in the heap: ordinary outputs take the pushes
        ops.comm_all_gather(self._comm._h, [inp.view(-1)], [out.view(-1)[:n * self.world_size]], False, 0, 0, False)
        return out

    def custom_all_gather(self, input: torch.Tensor, out=None) -> Optional[torch.Tensor]:
        # the gathered result, not the shard, has to fit the staging buffer's peers
        def warm():
            if out is None:
                return torch.empty(input.numel() * self.world_size, dtype=input.dtype, device=input.device)
            return out
        return self._dispatch(self._fast_all_gather, self.all_gather, input, out, warm)

    # ------------------------------------------------------------------- fused
    def attach_communicator(self, comm):
        """Uses `comm` (a symmetric-heap communicator over the same ranks) instead of the one
        made by the constructor, e.g. to share one heap with the rest of the engine."""
        if self._own_comm and self._comm is not None:
            self._comm.close()
        self._comm = comm
        self._own_comm = False

    def fused_all_reduce_rmsnorm(self, input: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor,
                                 eps: float = 1e-5, proto: str = "ll"):
        """rmsnorm(all_reduce(input) + residual) in one kernel; residual is updated
        in place.  Needs attach_communicator (or penny_b200.utils.global_communicator)."""
        comm = self._comm
        if comm is None:
            from ..utils import global_communicator
            comm = self._comm = global_communicator()
        out, _ = comm.fused_all_reduce_rmsnorm(input, weight, residual=residual, eps=eps, proto=proto)
        return out

    # ----------------------------------------------------------------- teardown
    def status(self, clear: bool = True) -> List[int]:
        """Status words of the last device-side timeout ([0] == 0: none), of the fast path's
        communicator when that is in use, else of the pull kernels."""
        if self.fast:
            rec = self._comm.status(0, clear)
            if rec["code"] != 0:
                return [rec["code"], rec["rank"], rec["peer"], rec["block"], 0, 0, 0, 0]
        return list(ops.custom_ar_status(self._ptr, clear)) if self._ptr else [0] * 8

    def close(self):
        if self._own_comm and self._comm is not None:
            try:
                torch.cuda.synchronize()
                self._comm.close()
            finally:
                self._comm, self._own_comm = None, False
        if not self.disabled and self._ptr:
            if ops is not None:
                ops.dispose(self._ptr)
            self._ptr = 0
            self.free_shared_buffer(self.meta_ptrs, rank=self.rank)
            self.free_shared_buffer(self.buffer_ptrs, rank=self.rank)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def create_shared_buffer(size_in_bytes: int, group: Optional[ProcessGroup] = None,
                             uncached: Optional[bool] = False) -> List[int]:
        pointer, handle = ops.allocate_shared_buffer_and_handle(size_in_bytes)
        world_size = dist.get_world_size(group=group)
        local_size = world_size // nnodes
        rank = dist.get_rank(group=group)
        local_rank = rank % local_size
        handles = [None] * world_size
        dist.all_gather_object(handles, handle, group=group)
        off = (rank // local_size) * local_size
        handles = handles[off:off + local_size]
        pointers: List[int] = []
        for i, h in enumerate(handles):
            if i == local_rank:
                pointers.append(pointer)
            else:
                pointers.append(ops.open_mem_handle(h))
        return pointers

    @staticmethod
    def free_shared_buffer(pointers: List[int], group: Optional[ProcessGroup] = None,
                           rank: Optional[int] = None) -> None:
        if rank is None:
            rank = dist.get_rank(group=group)
        if ops is not None:
            ops.free_shared_buffer(pointers[rank])
