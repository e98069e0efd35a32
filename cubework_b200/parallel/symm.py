"""Symmetric (peer-mapped) device workspaces and the fused compute+collective launches on them.

One workspace per process group: a buffer of the same size on every rank of the group, each rank
holding every peer's device pointer to it, plus a flag area for arrival counters and an error word.
The buffers are exchanged as CUDA IPC handles over the group's host (gloo) twin, so the mapping
needs nothing beyond ``torch.distributed``.  Kernels in ``ops/csrc/fused_gemm_sm100.cu`` store
partial output tiles straight into the owner's workspace and bump its arrival counter; reducer CTAs
of the same launch sum the partials and write the result to every rank that needs it.

The reference has no counterpart: it issues a cuBLAS GEMM and then a blocking NCCL collective
(cubework/distributed/collective.py:6-97).
"""
import os

import torch

_WORKSPACES = {}
# CUBEWORK_B200_FUSED: "1" always use the fused GEMM+collective kernels, "0" never (cuBLAS-free GEMM followed by NCCL),
# "auto" (default) use them where the local product is large enough to hide the exchange behind it.
_POLICY = os.environ.get("CUBEWORK_B200_FUSED", "auto")
_DISABLED = _POLICY == "0"


def prefer_fused(M, N, K, n) -> bool:
    """Peer-to-peer two-shot exchange overlapped with the product vs. product followed by an NVLS all-reduce.

    Measured on B200 (GPT-2 XL shapes and the 16384 x K x N microbenchmark): the fused kernel wins or ties when
    the product takes clearly longer than its exchange (about 1.5x); when the exchange dominates (8-way sharding
    of a 1600-wide layer) the in-switch reduction NCCL uses moves half the bytes and wins."""
    if _DISABLED:
        return False
    if _POLICY == "1":
        return True
    t_gemm = 2.0 * M * N * K / 1.3e15
    t_link = 2.0 * (n - 1) / n * M * N * 2 / 650e9
    return t_gemm >= 1.5 * t_link


def prefer_fused_gather_scatter(M, N, K) -> bool:
    """The gather / reduce-scatter fused kernel is used for products large enough that the exchange can hide
    behind them (tens of microseconds of tensor-core time); tiny products are launch-latency bound either way."""
    if _DISABLED:
        return False
    if _POLICY == "1":
        return True
    return 2.0 * M * N * K >= _GGS_MIN_FLOPS


_GGS_MIN_FLOPS = float(os.environ.get("CUBEWORK_B200_FUSED_MIN_GFLOP", "20")) * 1e9


_HAS_FUSED = None


def available() -> bool:
    global _HAS_FUSED
    if _DISABLED:
        return False
    if _HAS_FUSED is None:
        from ..ops import ext
        _HAS_FUSED = torch.cuda.is_available() and ext.has("fused")
    return _HAS_FUSED


def release_all():
    for ws in list(_WORKSPACES.values()):
        try:
            ws.close()
        except Exception:
            pass
    _WORKSPACES.clear()


def invalidate_all():
    """Forget every workspace without touching the device (after a reported device-side timeout the epochs of
    the ranks may disagree).  The regions are re-created, with fresh flags, at the next fused call - which is
    collective, so every rank of a group has to get here (each one's status check fails the same way, or the job
    is torn down).  The old allocations are released at process exit."""
    _WORKSPACES.clear()


def fused_gather_gemm_reduce(a, b, trans_a, trans_b, gather_a, gather_b, scatter, reduce, bias, out_dtype,
                             keep_gathered, act=None, pre_act_out=False):
    """Returns None when the pattern/shape is not covered, so the caller composes it from parts."""
    from . import symm_impl
    return symm_impl.dispatch(a, b, trans_a, trans_b, gather_a, gather_b, scatter, reduce, bias, out_dtype,
                              keep_gathered, act, pre_act_out)
