"""1D (Megatron-style) tensor-parallel autograd functions.

Parity: cubework/module/parallel_1d/_utils.py:26-126 — ``reduce_grad`` (identity fwd / all-reduce
bwd), ``reduce_input`` (all-reduce fwd / identity bwd), ``split_forward_gather_backward``,
``gather_forward_split_backward``, ``set/get_parallel_input``.

In addition :func:`linear_1d` is the whole column / row linear as ONE autograd function, so that on
CUDA the GEMM and the all-reduce that follows it (row forward, column backward) run as a single fused
kernel over peer memory (:mod:`cubework_b200.parallel.fused`) instead of cuBLAS followed by NCCL
(parallel_1d/module.py:263-278, 331-346 in the reference).
"""
import torch

from .. import ops
from ..global_vars import env
from . import fused
from .collective import all_gather, all_reduce, reduce_scatter


_RECOMPUTING = [0]


class recomputing:
    """Context in which a checkpointed block is re-run for its gradients (set by the models' checkpoint wrapper)."""

    def __enter__(self):
        _RECOMPUTING[0] += 1

    def __exit__(self, *exc):
        _RECOMPUTING[0] -= 1


def skip_product(module) -> bool:
    """True when ``module``'s output is not needed: it is the last linear of a block that is being re-run."""
    return _RECOMPUTING[0] > 0 and getattr(module, "output_unused_in_recompute", False)


def set_parallel_input(input_parallel: bool):
    env.parallel_input_1d = input_parallel


def get_parallel_input():
    return env.parallel_input_1d


def _split(x, mode, dim):
    n = mode.world_size
    if n == 1:
        return x
    assert x.size(dim) % n == 0, f"dim {dim} of {tuple(x.shape)} is not divisible by {n}"
    return torch.chunk(x, n, dim=dim)[mode.local_rank].contiguous()


class _ReduceGrad(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, mode):
        ctx.mode = mode
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return all_reduce(g.contiguous().clone(), ctx.mode), None


class _ReduceInput(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, mode):
        return all_reduce(x.contiguous().clone(), mode)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _SplitForwardGatherBackward(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, mode, dim):
        ctx.mode, ctx.dim = mode, dim
        return _split(x, mode, dim)

    @staticmethod
    def backward(ctx, g):
        return all_gather(g.contiguous(), ctx.dim, ctx.mode).contiguous(), None, None


class _GatherForwardSplitBackward(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, mode, dim):
        ctx.mode, ctx.dim = mode, dim
        return all_gather(x.contiguous(), dim, mode).contiguous()

    @staticmethod
    def backward(ctx, g):
        return _split(g, ctx.mode, ctx.dim), None, None


def reduce_grad(x, mode):
    return _ReduceGrad.apply(x, mode)


def reduce_input(x, mode):
    return _ReduceInput.apply(x, mode)


def split_forward_gather_backward(x, mode, dim):
    return _SplitForwardGatherBackward.apply(x, mode, dim)


def gather_forward_split_backward(x, mode, dim):
    return _GatherForwardSplitBackward.apply(x, mode, dim)


class _Linear1D(torch.autograd.Function):
    """``y = act(x @ w.T (+ b))`` with the all-reduce of either direction fused into its GEMM.

    ``reduce_fwd``: sum ``y`` over the group (row-parallel; bias added once, after the sum).
    ``reduce_bwd``: sum ``dx`` over the group (column-parallel, replicated input).
    """

    @staticmethod
    def forward(ctx, x, w, b, mode, reduce_fwd, reduce_bwd, act, skip=False):
        cd = ops.compute_dtype(x)
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != cd:
            x2 = x2.to(cd)
        x2 = x2.contiguous()
        wc = ops.shadow(w, cd)
        z = None
        if skip and act is None:
            # re-run of a checkpointed block whose output nobody reads: the backward below needs x and w only
            y = x2.new_empty((x2.shape[0], w.shape[0]))
        elif reduce_fwd and mode.world_size > 1:
            assert act is None
            y = fused.gemm_all_reduce(x2, wc, False, True, mode, bias=b)
        elif act is not None:
            y, z = ops.gemm(x2, wc, trans_b=True, bias=b, act=act, pre_act_out=True)
        else:
            y = ops.gemm(x2, wc, trans_b=True, bias=b)
        ctx.save_for_backward(x2, w, z if z is not None else x2.new_empty(0))
        ctx.mode, ctx.reduce_bwd, ctx.act, ctx.cd = mode, reduce_bwd, act, cd
        ctx.has_bias = b is not None
        ctx.bias_dtype = b.dtype if b is not None else None
        ctx.x_dtype, ctx.x_shape = x.dtype, x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, z = ctx.saved_tensors
        cd = ctx.cd
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != cd:
            dy2 = dy2.to(cd)
        dy2 = dy2.contiguous()
        db = None
        if ctx.act is not None:
            dy2, db = ops.act_backward(dy2, z, ctx.act, ctx.has_bias and ctx.needs_input_grad[2])
        elif ctx.has_bias and ctx.needs_input_grad[2]:
            db = ops.column_sum(dy2)
        if db is not None:
            db = db.to(ctx.bias_dtype)
        dx = None
        pending = None
        if ctx.needs_input_grad[0]:
            wc = ops.shadow(w, cd)
            if ctx.reduce_bwd and ctx.mode.world_size > 1:
                # fused GEMM+all-reduce, or GEMM + an all-reduce that runs behind the weight-gradient GEMM below
                dx, pending = fused.gemm_all_reduce_async(dy2, wc, False, False, ctx.mode)
            else:
                dx = ops.gemm(dy2, wc)
        dw = None
        if ctx.needs_input_grad[1]:
            dw = ops.gemm(dy2, x2, trans_a=True, out_dtype=w.dtype)
        if pending is not None:
            pending.wait()
        if dx is not None:
            dx = dx.view(ctx.x_shape)
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        return dx, dw, db, None, None, None, None, None


def linear_1d(x, w, b, mode, reduce_fwd=False, reduce_bwd=False, act=None, skip=False):
    return _Linear1D.apply(x, w, b, mode, reduce_fwd, reduce_bwd, act, skip)


class _Linear1DRows(torch.autograd.Function):
    """Column / row linear whose replicated side is kept *sharded along the rows* (tokens) instead.

    ``kind="gather"`` (column-parallel): ``x`` is this rank's block of rows ``[M/n, in]``;
    ``y = act(all-gather_rows(x) @ w.T + b)`` is ``[M, out/n]``.  Backward: ``dx = reduce-scatter_rows(dy @ w)``,
    ``dw = dy.T @ x_full`` with the gathered input kept from the forward.
    ``kind="scatter"`` (row-parallel): ``x`` is ``[M, in/n]``; ``y = reduce-scatter_rows(x @ w.T) + b`` is
    ``[M/n, out]``.  Backward: ``dx = all-gather_rows(dy) @ w``, ``dw = dy_full.T @ x``; the bias gradient is the
    column sum of this rank's rows only, i.e. a partial sum over the group (see ``mark_partial_grad``).

    Together they replace the all-reduce of a column/row pair (parallel_1d/module.py:263-278, 331-346 in the
    reference) by an all-gather in front of the first GEMM and a reduce-scatter behind the second, so everything
    between two such pairs (layer norm, residual, dropout) runs on ``1/n`` of the rows.  On CUDA each collective
    runs inside its GEMM kernel (:func:`cubework_b200.parallel.fused.gather_gemm_reduce`).
    """

    @staticmethod
    def forward(ctx, x, w, b, mode, kind, act, skip=False):
        cd = ops.compute_dtype(x)
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != cd:
            x2 = x2.to(cd)
        x2 = x2.contiguous()
        wc = ops.shadow(w, cd)
        n = mode.world_size
        z = None
        if kind == "gather":
            res = fused.gather_gemm_reduce(x2, wc, False, True, gather_a=(mode, 0), bias=b, act=act,
                                           pre_act_out=act is not None, keep_gathered=True)
            if act is not None:
                y, z, x_keep, _ = res
            else:
                y, x_keep, _ = res
            lead = (x.shape[0] * n, ) + tuple(x.shape[1:-1])
        else:
            assert act is None, "the activation belongs to the column-parallel linear of the pair"
            if skip:    # re-run of a checkpointed block whose output nobody reads (every rank skips alike)
                y = x2.new_empty((x2.shape[0] // n, w.shape[0]))
            else:
                y = fused.gather_gemm_reduce(x2, wc, False, True, scatter=(mode, 0), bias=b)
            x_keep = x2
            assert x.shape[0] % n == 0, f"leading dimension {x.shape[0]} is not divisible by the group size {n}"
            lead = (x.shape[0] // n, ) + tuple(x.shape[1:-1])
        ctx.save_for_backward(x_keep, w, z if z is not None else x2.new_empty(0))
        ctx.mode, ctx.kind, ctx.act, ctx.cd = mode, kind, act, cd
        ctx.has_bias = b is not None
        ctx.bias_dtype = b.dtype if b is not None else None
        ctx.x_dtype, ctx.x_shape = x.dtype, x.shape
        return y.view(*lead, w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x_keep, w, z = ctx.saved_tensors
        cd, mode = ctx.cd, ctx.mode
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != cd:
            dy2 = dy2.to(cd)
        dy2 = dy2.contiguous()
        want_db = ctx.has_bias and ctx.needs_input_grad[2]
        db = None
        if ctx.act is not None:
            dy2, db = ops.act_backward(dy2, z, ctx.act, want_db)
        elif want_db:
            db = ops.column_sum(dy2)
        if db is not None:
            db = db.to(ctx.bias_dtype)
        wc = ops.shadow(w, cd)
        dx = dw = None
        if ctx.kind == "gather":
            pending = None
            if ctx.needs_input_grad[0]:
                dx, pending = fused.gemm_reduce_scatter_async(dy2, wc, False, False, (mode, 0))
            if ctx.needs_input_grad[1]:
                dw = ops.gemm(dy2, x_keep, trans_a=True, out_dtype=w.dtype)
            if pending is not None:
                pending.wait()
        else:
            # the gathered dy is consumed by the weight-gradient product right behind this call
            dx, dy_full, _ = fused.gather_gemm_reduce(dy2, wc, False, False, gather_a=(mode, 0), keep_gathered="view")
            if ctx.needs_input_grad[1]:
                dw = ops.gemm(dy_full, x_keep, trans_a=True, out_dtype=w.dtype)
            if not ctx.needs_input_grad[0]:
                dx = None
        if dx is not None:
            dx = dx.view(ctx.x_shape)
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
        return dx, dw, db, None, None, None, None


def linear_1d_rows(x, w, b, mode, kind, act=None, skip=False):
    """See :class:`_Linear1DRows`; with a group of one this is the plain linear."""
    if mode.world_size == 1:
        return _Linear1D.apply(x, w, b, mode, False, False, act, skip)
    return _Linear1DRows.apply(x, w, b, mode, kind, act, skip)


class _ScatterRows(torch.autograd.Function):
    """This rank's block of the leading dimension forward, all-gather of the gradient backward."""

    @staticmethod
    def forward(ctx, x, mode):
        ctx.mode = mode
        return _split(x, mode, 0)

    @staticmethod
    def backward(ctx, g):
        return all_gather(g.contiguous(), 0, ctx.mode).contiguous(), None


class _GatherRows(torch.autograd.Function):
    """All-gather along the leading dimension forward; backward keeps this rank's block of the gradient (every
    rank holds the same full gradient behind a replicated computation)."""

    @staticmethod
    def forward(ctx, x, mode):
        ctx.mode = mode
        return all_gather(x.contiguous(), 0, mode).contiguous()

    @staticmethod
    def backward(ctx, g):
        return _split(g, ctx.mode, 0), None


class _ReduceScatterRows(torch.autograd.Function):
    """Sum over the group and keep this rank's block of the leading dimension; all-gather backward."""

    @staticmethod
    def forward(ctx, x, mode):
        ctx.mode = mode
        return reduce_scatter(x.contiguous(), 0, mode).contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather(g.contiguous(), 0, ctx.mode).contiguous(), None


def scatter_rows(x, mode):
    return x if mode.world_size == 1 else _ScatterRows.apply(x, mode)


def gather_rows(x, mode):
    return x if mode.world_size == 1 else _GatherRows.apply(x, mode)


def reduce_scatter_rows(x, mode):
    return x if mode.world_size == 1 else _ReduceScatterRows.apply(x, mode)


# ---------------------------------------------------------------------------------------------------------------
# parameters whose gradient is a partial sum over the 1D group
# ---------------------------------------------------------------------------------------------------------------
PARTIAL_GRAD = "partial_grad_1d"


def mark_partial_grad(param):
    """A replicated parameter applied to row-sharded activations (layer-norm scale and shift, the bias of a row
    linear, a position table) sees only this rank's rows, so its gradient is a partial sum; it is completed by
    :func:`reduce_partial_grads` after the backward pass."""
    setattr(param, PARTIAL_GRAD, True)


def reduce_partial_grads(params):
    """One all-reduce over the 1D group of the gradients of all marked parameters (flattened into one buffer)."""
    from .mesh import pm
    mode = pm.PARALLEL_1D
    if not mode.is_initialized() or mode.world_size == 1:
        return
    todo = [p for p in params if getattr(p, PARTIAL_GRAD, False) and p.grad is not None]
    if not todo:
        return
    flat = torch.cat([p.grad.detach().reshape(-1).float() for p in todo])
    flat = all_reduce(flat, mode)
    off = 0
    for p in todo:
        k = p.grad.numel()
        p.grad.detach().copy_(flat[off:off + k].view_as(p.grad))
        off += k
