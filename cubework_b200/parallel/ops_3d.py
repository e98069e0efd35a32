"""3D (cube) tensor-parallel autograd functions on a ``d x d x d`` grid.

Parity: cubework/module/parallel_3d/_operation.py:12-339 and _utils.py:12-184 — ``linear_3d``,
``classifier_3d``, ``vocab_parallel_classifier_3d``, ``layernorm_3d``, ``all_gather_weight_3d``,
``reduce_scatter_tensor_3d``, ``reduce_tensor_3d``, ``reduce_by_batch_3d``, ``split_batch_3d``,
``swap_in_out_group`` and the group getters that resolve the *current* role names stored in ``env``.

In-TP rank ``r = i + d*(j + d*k)``: the INPUT group varies ``j``, WEIGHT varies ``i``, OUTPUT varies
``k`` (distributed/utils.py:251-400).  A linear layer is

    ``Y = reduce-scatter_M(output)( gather_M(X, input) @ gather_N(W, weight) ) + b``

which is one :func:`~cubework_b200.parallel.fused.gather_gemm_reduce` call; its backward gathers
``dY`` once over the output group and issues two more such calls (``dW`` reduce-scattered over the
weight group, ``dX`` over the input group).

Differences from the reference: parameter-gradient reductions are started asynchronously and awaited
before ``backward`` returns (overlapping the ``dX`` product) instead of returning zeros to autograd
and patching the gradient in a hook (module/utils.py:38-92); ``classifier_3d`` reduces its weight
gradient to *every* rank that holds that shard, so no per-forward re-broadcast from the cube diagonal
is needed (_operation.py:105-150 keeps the gradient on ``j == k`` ranks only).
"""
import torch

from .. import ops
from ..global_vars import env
from .collective import all_gather, all_reduce, reduce_scatter
from .fused import gather_gemm_reduce, gemm_reduce_scatter_async
from .functional import as_compute
from .mesh import ParallelMode, pm
from .ops_2d import _GatherParam, _ReduceByBatch, _ReduceScatterTensor, _ReduceTensor, layer_norm_sharded


def get_depth_from_env() -> int:
    d = env.depth_3d
    assert d and d > 0, "DEPTH must be greater than zero"
    return d


def get_input_parallel_mode() -> ParallelMode:
    return pm.get(env.input_group_3d)


def get_weight_parallel_mode() -> ParallelMode:
    return pm.get(env.weight_group_3d)


def get_output_parallel_mode() -> ParallelMode:
    return pm.get(env.output_group_3d)


def get_input_x_weight_parallel_mode() -> ParallelMode:
    return pm.get(env.input_x_weight_group_3d)


def get_output_x_weight_parallel_mode() -> ParallelMode:
    return pm.get(env.output_x_weight_group_3d)


def swap_in_out_group():
    env.swap_in_out_3d()


def split_batch_3d(tensor, dim: int = 0, input_parallel_mode=None, weight_parallel_mode=None):
    """Batch slice of this rank: first by weight-group rank, then by input-group rank."""
    if tensor.size(dim) <= 1:
        return tensor
    wm = weight_parallel_mode or get_weight_parallel_mode()
    im = input_parallel_mode or get_input_parallel_mode()
    out = torch.chunk(tensor, wm.world_size, dim=dim)[wm.local_rank]
    out = torch.chunk(out, im.world_size, dim=dim)[im.local_rank]
    return out.contiguous()


def reduce_tensor_3d(tensor, parallel_mode):
    return _ReduceTensor.apply(tensor, parallel_mode)


def all_gather_weight_3d(tensor, dim, parallel_mode):
    return _GatherParam.apply(tensor, dim, parallel_mode)


def reduce_scatter_tensor_3d(tensor, dim, parallel_mode):
    return _ReduceScatterTensor.apply(tensor, dim, parallel_mode)


def reduce_by_batch_3d(tensor, input_parallel_mode=None, weight_parallel_mode=None, reduce_mean: bool = False):
    im = input_parallel_mode or get_input_parallel_mode()
    wm = weight_parallel_mode or get_weight_parallel_mode()
    return _ReduceByBatch.apply(tensor, (im, wm), reduce_mean)


class _Linear3D(torch.autograd.Function):
    """``w_is_out_in`` False: W ``[in/d, out/d^2]`` (Linear3D).  True: W ``[out/d^2, in/d]``
    (vocab-parallel classifier, where the weight can be the tied embedding table)."""

    @staticmethod
    def forward(ctx, x, w, bias, im, wm, om, w_is_out_in):
        cd = ops.compute_dtype(x)
        x2 = as_compute(x.reshape(-1, x.shape[-1]), cd)
        wc = ops.shadow(w, cd)
        y, x_full, w_full = gather_gemm_reduce(x2, wc, trans_b=w_is_out_in, gather_a=(im, 0),
                                               gather_b=(wm, 0 if w_is_out_in else 1), scatter=(om, 0),
                                               bias=bias, keep_gathered=True)
        ctx.save_for_backward(x_full, w_full)
        ctx.cfg = (cd, im, wm, om, w_is_out_in, x.shape, x.dtype, w.dtype,
                   bias.dtype if bias is not None else None)
        return y.reshape(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x_full, w_full = ctx.saved_tensors
        cd, im, wm, om, w_is_out_in, x_shape, x_dtype, w_dtype, b_dtype = ctx.cfg
        dy2 = as_compute(dy.reshape(-1, dy.shape[-1]), cd)
        dy_full = all_gather(dy2, 0, om).contiguous()
        dw = db = dx = None
        works = []
        if ctx.needs_input_grad[1]:
            if w_is_out_in:   # dW = dY^T X  [out/d, in/d] -> scatter rows over the weight group
                dw, wk = gemm_reduce_scatter_async(dy_full, x_full, True, False, (wm, 0), out_dtype=w_dtype)
            else:             # dW = X^T dY  [in/d, out/d] -> scatter columns over the weight group
                dw, wk = gemm_reduce_scatter_async(x_full, dy_full, True, False, (wm, 1), out_dtype=w_dtype)
            works.append(wk)
        if b_dtype is not None and ctx.needs_input_grad[2]:
            db, wk = all_reduce(ops.column_sum(dy_full).to(b_dtype), wm, async_op=True)
            works.append(wk)
        if ctx.needs_input_grad[0]:
            dx = gather_gemm_reduce(dy_full, w_full, trans_b=not w_is_out_in, scatter=(im, 0)).reshape(x_shape)
            if dx.dtype != x_dtype:
                dx = dx.to(x_dtype)
        for wk in works:
            if wk is not None:
                wk.wait()
        if dw is not None:
            dw = dw.contiguous()
        return dx, dw, db, None, None, None, None


def linear_3d(input_, weight, bias, input_parallel_mode, weight_parallel_mode, output_parallel_mode):
    return _Linear3D.apply(input_, weight, bias, input_parallel_mode, weight_parallel_mode, output_parallel_mode,
                           False)


def vocab_parallel_classifier_3d(input_, weight, bias, input_parallel_mode, weight_parallel_mode,
                                 output_parallel_mode):
    return _Linear3D.apply(input_, weight, bias, input_parallel_mode, weight_parallel_mode, output_parallel_mode,
                           True)


class _Classifier3D(torch.autograd.Function):
    """``logits = all-reduce(output)(X @ W^T) + b`` with W ``[C, H/d]`` (hidden shard = output rank).

    ``reduce_weight_grad`` is False for a tied weight whose owner already sums its gradient over the
    input x weight plane."""

    @staticmethod
    def forward(ctx, x, w, bias, om, ixw, reduce_weight_grad):
        cd = ops.compute_dtype(x)
        x2 = as_compute(x.reshape(-1, x.shape[-1]), cd)
        y = gather_gemm_reduce(x2, ops.shadow(w, cd), trans_b=True, reduce=om, bias=bias)
        ctx.save_for_backward(x2, w)
        ctx.cfg = (cd, om, ixw, reduce_weight_grad, x.shape, x.dtype, bias.dtype if bias is not None else None)
        return y.reshape(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        cd, om, ixw, reduce_weight_grad, x_shape, x_dtype, b_dtype = ctx.cfg
        dy2 = as_compute(dy.reshape(-1, dy.shape[-1]), cd)
        dw = db = dx = None
        works = []
        if ctx.needs_input_grad[1]:
            dw = ops.gemm(dy2, x2, trans_a=True, out_dtype=w.dtype)
            if reduce_weight_grad:
                dw, wk = all_reduce(dw, ixw, async_op=True)
                works.append(wk)
        if b_dtype is not None and ctx.needs_input_grad[2]:
            db, wk = all_reduce(ops.column_sum(dy2).to(b_dtype), ixw, async_op=True)
            works.append(wk)
        if ctx.needs_input_grad[0]:
            dx = ops.gemm(dy2, ops.shadow(w, cd)).reshape(x_shape)
            if dx.dtype != x_dtype:
                dx = dx.to(x_dtype)
        for wk in works:
            if wk is not None:
                wk.wait()
        return dx, dw, db, None, None, None


def classifier_3d(input_, weight, bias, input_parallel_mode, weight_parallel_mode, output_parallel_mode,
                  input_x_weight_parallel_mode=None, reduce_weight_grad=True):
    ixw = input_x_weight_parallel_mode or get_input_x_weight_parallel_mode()
    return _Classifier3D.apply(input_, weight, bias, output_parallel_mode, ixw, reduce_weight_grad)


def layernorm_3d(input_, weight, bias, normalized_shape, eps, input_parallel_mode, weight_parallel_mode,
                 output_parallel_mode, input_x_weight_parallel_mode):
    return layer_norm_sharded(input_, weight, bias, eps, normalized_shape, output_parallel_mode,
                              grad_modes=(input_x_weight_parallel_mode, ))
