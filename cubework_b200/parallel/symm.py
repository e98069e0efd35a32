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
_DISABLED = os.environ.get("CUBEWORK_B200_FUSED", "1") == "0"


def available() -> bool:
    if _DISABLED or not torch.cuda.is_available():
        return False
    from ..ops import ext
    return ext.has("fused")


def release_all():
    for ws in list(_WORKSPACES.values()):
        try:
            ws.close()
        except Exception:
            pass
    _WORKSPACES.clear()


def fused_gather_gemm_reduce(a, b, trans_a, trans_b, gather_a, gather_b, scatter, reduce, bias, out_dtype,
                             keep_gathered):
    """Returns None when the pattern/shape is not covered, so the caller composes it from parts."""
    from . import symm_impl
    return symm_impl.dispatch(a, b, trans_a, trans_b, gather_a, gather_b, scatter, reduce, bias, out_dtype,
                              keep_gathered)
