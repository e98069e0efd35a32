"""Tensor-in / tensor-out collectives addressed by ``ParallelMode``.

Parity: cubework/distributed/collective.py:6-97 — ``all_gather(t, dim, mode, async_op)``,
``reduce_scatter(t, dim, mode, op, async_op)``, ``all_reduce``, ``broadcast``, ``reduce``; every call
short-circuits on a group of one, uses the gloo twin for host tensors and returns ``(out, work)``
when ``async_op`` is set.

Differences: communication accounting is built in (each call reports its algorithm bytes and a pair
of stream events to the active :class:`~cubework_b200.utils.profiling.CommProfiler`, so profiling
needs neither monkey-patching nor a host synchronisation per call).  Every function here is a
``torch.distributed`` (NCCL / gloo) call; the collectives that follow or precede a GEMM do not come
through this module on CUDA but run inside the GEMM kernel (:mod:`cubework_b200.parallel.fused`).
``STATS`` counts calls and payload bytes per kind, so a caller can verify what still goes through
the library on a hot path.
"""
from typing import Optional

import torch
import torch.distributed as dist
from torch.distributed import ReduceOp

from .mesh import ParallelMode

_profiler = None  # set by CommProfiler.start()
STATS = {}        # kind -> [calls, payload bytes] issued by this process through the wrappers below


def _tally(kind, tensor):
    rec = STATS.setdefault(kind, [0, 0])
    rec[0] += 1
    rec[1] += tensor.numel() * tensor.element_size()


def stats_snapshot():
    return {k: tuple(v) for k, v in STATS.items()}


def _set_profiler(p):
    global _profiler
    _profiler = p


class _Ticket:
    """Marks one collective for the profiler; ``close()`` when the data has landed."""
    __slots__ = ("prof", "rec")

    def __init__(self, kind, nbytes, tensor):
        self.prof = _profiler
        self.rec = self.prof._open(kind, nbytes, tensor) if self.prof is not None else None

    def close(self):
        if self.rec is not None:
            self.prof._close(self.rec)
            self.rec = None


class _Work:
    """Async handle that also closes the profiler ticket on ``wait``."""

    def __init__(self, work, ticket):
        self.work = work
        self.ticket = ticket

    def wait(self):
        if self.work is not None:
            self.work.wait()
        self.ticket.close()

    def is_completed(self):
        return self.work is None or self.work.is_completed()


def _finish(out, work, ticket, async_op):
    if async_op:
        return out, _Work(work, ticket)
    ticket.close()
    return out


def _nbytes(t):
    return t.numel() * t.element_size()


def all_gather(tensor: torch.Tensor, dim: int, parallel_mode: ParallelMode, async_op: bool = False):
    n = parallel_mode.world_size
    if n == 1:
        return (tensor, None) if async_op else tensor
    dim = dim % tensor.dim()
    src = tensor.contiguous() if dim == 0 else tensor.transpose(0, dim).contiguous()
    out = src.new_empty((n * src.shape[0], ) + tuple(src.shape[1:]))
    _tally("all_gather", out)
    ticket = _Ticket("all_gather", _nbytes(out) * (n - 1) // n, tensor)
    work = dist.all_gather_into_tensor(out, src, group=parallel_mode.group_for(tensor), async_op=async_op)
    if dim != 0:
        out = out.transpose(0, dim)  # stays a view; consumers call .contiguous() when they need it
    return _finish(out, work, ticket, async_op)


def reduce_scatter(tensor: torch.Tensor,
                   dim: int,
                   parallel_mode: ParallelMode,
                   op: ReduceOp = ReduceOp.SUM,
                   async_op: bool = False):
    n = parallel_mode.world_size
    if n == 1:
        return (tensor, None) if async_op else tensor
    dim = dim % tensor.dim()
    assert tensor.shape[dim] % n == 0, f"dim {dim} of {tuple(tensor.shape)} is not divisible by {n}"
    src = tensor.contiguous() if dim == 0 else tensor.transpose(0, dim).contiguous()
    out = src.new_empty((src.shape[0] // n, ) + tuple(src.shape[1:]))
    _tally("reduce_scatter", src)
    ticket = _Ticket("reduce_scatter", _nbytes(src) * (n - 1) // n, tensor)
    group = parallel_mode.group_for(tensor)
    if tensor.device.type == "cpu":
        # gloo has no reduce_scatter: reduce the whole buffer and keep this rank's slice
        tmp = src.clone()
        work = dist.all_reduce(tmp, op=op, group=group, async_op=False)
        out.copy_(tmp.chunk(n, 0)[parallel_mode.local_rank])
        work = None
    else:
        work = dist.reduce_scatter_tensor(out, src, op=op, group=group, async_op=async_op)
    if dim != 0:
        out = out.transpose(0, dim)
    return _finish(out, work, ticket, async_op)


def all_reduce(tensor: torch.Tensor,
               parallel_mode: ParallelMode,
               op: ReduceOp = ReduceOp.SUM,
               async_op: bool = False):
    n = parallel_mode.world_size
    if n == 1:
        return (tensor, None) if async_op else tensor
    out = tensor.contiguous()
    _tally("all_reduce", out)
    ticket = _Ticket("all_reduce", _nbytes(out) * 2 * (n - 1) // n, tensor)
    work = dist.all_reduce(out, op=op, group=parallel_mode.group_for(tensor), async_op=async_op)
    return _finish(out, work, ticket, async_op)


def broadcast(tensor: torch.Tensor, src: int, parallel_mode: ParallelMode, async_op: bool = False):
    """``src`` is a *global* rank (use ``mode.rank_by_idx``), as in the reference."""
    if parallel_mode.world_size == 1:
        return (tensor, None) if async_op else tensor
    out = tensor.contiguous()
    _tally("broadcast", out)
    ticket = _Ticket("broadcast", _nbytes(out), tensor)
    work = dist.broadcast(out, src=src, group=parallel_mode.group_for(tensor), async_op=async_op)
    return _finish(out, work, ticket, async_op)


def reduce(tensor: torch.Tensor,
           dst: int,
           parallel_mode: ParallelMode,
           op: ReduceOp = ReduceOp.SUM,
           async_op: bool = False):
    if parallel_mode.world_size == 1:
        return (tensor, None) if async_op else tensor
    out = tensor.contiguous()
    _tally("reduce", out)
    ticket = _Ticket("reduce", _nbytes(out), tensor)
    work = dist.reduce(out, dst=dst, op=op, group=parallel_mode.group_for(tensor), async_op=async_op)
    return _finish(out, work, ticket, async_op)


def barrier(parallel_mode: Optional[ParallelMode] = None, device=None):
    if parallel_mode is None:
        dist.barrier()
    elif parallel_mode.world_size > 1:
        g = parallel_mode.group if (device is not None and torch.device(device).type == "cuda") else \
            parallel_mode.cpu_group
        dist.barrier(group=g)
