"""The one communication pattern behind every parallel matmul of the three modes:

    gather an operand along one grid axis  ->  GEMM  ->  reduce(-scatter) the result along another

* 1D row forward / column backward: ``GEMM -> all-reduce``            (parallel_1d/module.py:263-346)
* 2D SUMMA ``AB``:  ``gather_K(A, row) x gather_K(B, col) -> GEMM``    (parallel_2d/_operation.py:15-80)
* 2D SUMMA ``ABT``: ``gather_N(B, col) -> GEMM -> reduce-scatter_N(row)`` (_operation.py:94-160)
* 2D SUMMA ``ATB``: ``gather_K(A, row) -> GEMM -> reduce-scatter_K(col)`` (_operation.py:174-239)
* 3D: ``gather_M(X, input) x gather_N(W, weight) -> GEMM -> reduce-scatter_M(output)``
  (parallel_3d/_operation.py:12-68)

:func:`gather_gemm_reduce` expresses all of them.  For CUDA bf16/fp16 operands it runs the fused
sm_100a kernels of :mod:`cubework_b200.ops.ext` (tcgen05 tiles whose epilogue pushes partial tiles
into the owners' peer memory, and whose operand loads wait on per-panel arrival flags); on the host,
in fp32, or when a shape does not fit the symmetric workspace it composes the collective wrappers
with the local GEMM, which is also the oracle the fused kernels are tested against.
"""
from typing import Optional, Tuple

import torch

from .. import ops
from . import symm
from .collective import all_gather, all_reduce, reduce_scatter
from .mesh import ParallelMode

Spec = Optional[Tuple[ParallelMode, int]]   # (group, dim of the *stored* 2-D operand / result)


def _live(spec):
    return spec is not None and spec[0].world_size > 1


def gather_gemm_reduce(a: torch.Tensor, b: torch.Tensor, trans_a: bool = False, trans_b: bool = False, *,
                       gather_a: Spec = None, gather_b: Spec = None, scatter: Spec = None,
                       reduce: Optional[ParallelMode] = None, bias: Optional[torch.Tensor] = None,
                       out_dtype: Optional[torch.dtype] = None, keep_gathered=False, act: Optional[str] = None,
                       pre_act_out: bool = False):
    """``C = act( reduce( op(gather(a)) @ op(gather(b)) ) + bias )``.

    ``gather_a/gather_b = (mode, dim)`` all-gather the stored operand along ``dim`` over ``mode``;
    ``scatter = (mode, dim)`` reduce-scatters the product along ``dim``; ``reduce = mode`` all-reduces
    it instead.  ``bias`` is added after the reduction, then the activation (``"gelu"`` / ``"relu"``).
    Returns ``C``, followed by the value before the activation when ``pre_act_out`` is set, followed by
    the gathered operands ``a_full, b_full`` when ``keep_gathered`` is set (the backward of the 3D and
    of the row-sharded 1D linears reuses them).  ``keep_gathered="view"`` allows the gathered operands
    to be views of the communication workspace that are only valid until the next fused call on the
    same group: for consumers that run next on the same stream.
    """
    assert not (scatter is not None and reduce is not None)
    out_dtype = out_dtype or a.dtype
    if ops.use_kernels(a) and symm.available():
        res = symm.fused_gather_gemm_reduce(a, b, trans_a, trans_b, gather_a, gather_b, scatter, reduce, bias,
                                            out_dtype, keep_gathered, act, pre_act_out)
        if res is not None:
            return res
    a_full = all_gather(a, gather_a[1], gather_a[0]).contiguous() if _live(gather_a) else a
    b_full = all_gather(b, gather_b[1], gather_b[0]).contiguous() if _live(gather_b) else b
    needs_comm = _live(scatter) or (reduce is not None and reduce.world_size > 1)
    z = None
    if not needs_comm:
        c = ops.gemm(a_full, b_full, trans_a, trans_b, bias=bias, act=act, out_dtype=out_dtype,
                     pre_act_out=pre_act_out)
        if pre_act_out:
            c, z = c
    else:
        c = ops.gemm(a_full, b_full, trans_a, trans_b, out_dtype=out_dtype)
        if _live(scatter):
            c = reduce_scatter(c, scatter[1], scatter[0]).contiguous()
        else:
            c = all_reduce(c, reduce)
        if bias is not None:
            c = c + bias.to(c.dtype)
        if pre_act_out:
            z = c
        if act is not None:
            c = ops._act(c, act)
    res = (c, z) if pre_act_out else (c, )
    if keep_gathered:
        res = res + (a_full, b_full)
    return res if len(res) > 1 else res[0]


def gemm_all_reduce(a, b, trans_a, trans_b, mode, bias=None, out_dtype=None):
    return gather_gemm_reduce(a, b, trans_a, trans_b, reduce=mode, bias=bias, out_dtype=out_dtype)


def gemm_all_reduce_async(a, b, trans_a, trans_b, mode, out_dtype=None):
    """``(C, work)``: like :func:`gemm_all_reduce`, but when the fused kernel is not used the all-reduce is
    started asynchronously and ``work.wait()`` must be called before ``C`` is read - the caller runs an
    independent GEMM (the weight gradient) in between.  ``work`` is None when nothing is pending."""
    out_dtype = out_dtype or a.dtype
    if ops.use_kernels(a) and symm.available():
        res = symm.fused_gather_gemm_reduce(a, b, trans_a, trans_b, None, None, None, mode, None, out_dtype, False)
        if res is not None:
            return res, None
    c = ops.gemm(a, b, trans_a, trans_b, out_dtype=out_dtype)
    if mode.world_size > 1:
        return all_reduce(c, mode, async_op=True)
    return c, None


def gemm_reduce_scatter_async(a, b, trans_a, trans_b, scatter: Spec, out_dtype=None):
    """``(C, work)`` with ``C = reduce-scatter(op(a) @ op(b))``.  The fused kernel does both at once (``work`` is
    None); otherwise the product is followed by an asynchronous reduce-scatter and ``work.wait()`` must be called
    before ``C`` is read, so the caller can overlap it with its next product."""
    out_dtype = out_dtype or a.dtype
    if not _live(scatter):
        return ops.gemm(a, b, trans_a, trans_b, out_dtype=out_dtype), None
    if ops.use_kernels(a) and symm.available():
        res = symm.fused_gather_gemm_reduce(a, b, trans_a, trans_b, None, None, scatter, None, None, out_dtype, False)
        if res is not None:
            return res, None
    c = ops.gemm(a, b, trans_a, trans_b, out_dtype=out_dtype)
    return reduce_scatter(c, scatter[1], scatter[0], async_op=True)
