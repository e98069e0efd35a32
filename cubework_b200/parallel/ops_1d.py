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
from .collective import all_gather, all_reduce


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
    def forward(ctx, x, w, b, mode, reduce_fwd, reduce_bwd, act):
        cd = ops.compute_dtype(x)
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != cd:
            x2 = x2.to(cd)
        x2 = x2.contiguous()
        wc = ops.shadow(w, cd)
        z = None
        if reduce_fwd and mode.world_size > 1:
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
        return dx, dw, db, None, None, None, None


def linear_1d(x, w, b, mode, reduce_fwd=False, reduce_bwd=False, act=None):
    return _Linear1D.apply(x, w, b, mode, reduce_fwd, reduce_bwd, act)
