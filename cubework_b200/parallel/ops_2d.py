"""2D (SUMMA) tensor-parallel autograd functions.

Parity: cubework/module/parallel_2d/_operation.py:15-439 and _utils.py:12-101 — ``summa_AB``,
``summa_ABT``, ``summa_ATB``, ``add_bias_2d``, ``layernorm_2d`` (here :func:`layer_norm_sharded`),
``classifier_2d``, ``all_gather_tensor_2d``, ``reduce_scatter_tensor_2d``, ``reduce_tensor_2d``,
``reduce_by_batch_2d``, ``split_batch_2d``.

Grid convention (distributed/utils.py:189-248): rank ``(i, j)`` = (grid row, grid column);
``PARALLEL_2D_COL`` spans a column (its local rank is ``i``), ``PARALLEL_2D_ROW`` spans a row (local
rank ``j``).

Instead of the reference's ``q`` rounds of (broadcast, broadcast, addmm) each product is one
``gather -> GEMM -> reduce-scatter`` call (:func:`cubework_b200.parallel.fused.gather_gemm_reduce`):

* ``AB``  : ``C_ij = sum_t A_it B_tj``    = gather A along K over the row, B along K down the column
* ``ABT`` : ``C_it = sum_j A_ij B_tj^T``  = gather B along N down the column, reduce-scatter N over the row
* ``ATB`` : ``C_tj = sum_i A_it^T B_ij``  = gather A along K over the row, reduce-scatter K down the column
"""
import torch
import torch.nn as nn

from .. import ops
from ..global_vars import env
from .collective import all_gather, all_reduce, reduce_scatter
from .fused import gather_gemm_reduce
from .functional import as_compute
from .mesh import pm


def assert_summa_initialization():
    assert pm.PARALLEL_2D_COL.is_initialized() and pm.PARALLEL_2D_ROW.is_initialized(), \
        "Both PARALLEL_2D_COL and PARALLEL_2D_ROW must be initialized by the processor."


def get_summa_dim_from_env() -> int:
    q = env.summa_dim
    assert q and q > 0, "SUMMA_DIM must be larger than zero"
    return q


def _prep(t, cd):
    """2-D low-precision operand: the cached shadow of a parameter, a cast of an activation."""
    if isinstance(t, nn.Parameter):
        return ops.shadow(t, cd)
    return as_compute(t.reshape(-1, t.shape[-1]), cd)


def _summa(kind, a, b, row, col, out_dtype=None):
    if kind == "AB":
        return gather_gemm_reduce(a, b, gather_a=(row, 1), gather_b=(col, 0), out_dtype=out_dtype)
    if kind == "ABT":
        return gather_gemm_reduce(a, b, trans_b=True, gather_b=(col, 0), scatter=(row, 1), out_dtype=out_dtype)
    if kind == "ATB":
        return gather_gemm_reduce(a, b, trans_a=True, gather_a=(row, 1), scatter=(col, 0), out_dtype=out_dtype)
    raise ValueError(kind)


# kind -> ((kind of dA, its operands), (kind of dB, its operands)), "g" being dC
_BWD = {
    "AB": (("ABT", "g", "b"), ("ATB", "a", "g")),
    "ABT": (("AB", "g", "b"), ("ATB", "g", "a")),
    "ATB": (("ABT", "b", "g"), ("AB", "a", "g")),
}


class _Summa(torch.autograd.Function):

    @staticmethod
    def forward(ctx, a, b, kind, out_shape, row, col):
        cd = ops.compute_dtype(a)
        a2, b2 = _prep(a, cd), _prep(b, cd)
        c = _summa(kind, a2, b2, row, col)
        # parameters are saved as themselves (their shadow is persistent), activations as the cast copy
        ctx.save_for_backward(a if isinstance(a, nn.Parameter) else a2, b if isinstance(b, nn.Parameter) else b2)
        ctx.cfg = (kind, cd, row, col, a.shape, b.shape, a.dtype, b.dtype)
        return c.reshape(out_shape)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        kind, cd, row, col, a_shape, b_shape, a_dtype, b_dtype = ctx.cfg
        t = {"a": _prep(a, cd), "b": _prep(b, cd), "g": as_compute(g.reshape(-1, g.shape[-1]), cd)}
        (ka, xa, ya), (kb, xb, yb) = _BWD[kind]
        da = db = None
        if ctx.needs_input_grad[0]:
            da = _summa(ka, t[xa], t[ya], row, col, out_dtype=a_dtype).reshape(a_shape)
        if ctx.needs_input_grad[1]:
            db = _summa(kb, t[xb], t[yb], row, col, out_dtype=b_dtype).reshape(b_shape)
        return da, db, None, None, None, None


def summa_AB(A, B, summa_dim, out_shape, row_parallel_mode, col_parallel_mode):
    return _Summa.apply(A, B, "AB", out_shape, row_parallel_mode, col_parallel_mode)


def summa_ABT(A, B, summa_dim, out_shape, row_parallel_mode, col_parallel_mode):
    return _Summa.apply(A, B, "ABT", out_shape, row_parallel_mode, col_parallel_mode)


def summa_ATB(A, B, summa_dim, out_shape, row_parallel_mode, col_parallel_mode):
    return _Summa.apply(A, B, "ATB", out_shape, row_parallel_mode, col_parallel_mode)


class _GatherParam(torch.autograd.Function):
    """All-gather a sharded parameter / tensor along ``dim`` (fwd) and reduce-scatter its gradient."""

    @staticmethod
    def forward(ctx, t, dim, mode):
        ctx.dim, ctx.mode = dim, mode
        return all_gather(t.contiguous(), dim, mode).contiguous()

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter(g.contiguous(), ctx.dim, ctx.mode).contiguous(), None, None


class _ReduceScatterTensor(torch.autograd.Function):

    @staticmethod
    def forward(ctx, t, dim, mode):
        ctx.dim, ctx.mode = dim, mode
        return reduce_scatter(t.contiguous(), dim, mode).contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather(g.contiguous(), ctx.dim, ctx.mode).contiguous(), None, None


class _ReduceTensor(torch.autograd.Function):

    @staticmethod
    def forward(ctx, t, mode):
        return all_reduce(t.contiguous().clone(), mode)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _ReduceByBatch(torch.autograd.Function):
    """Sum (or mean) of a per-batch-shard value over the groups that split the batch."""

    @staticmethod
    def forward(ctx, t, modes, reduce_mean):
        out = t.float().contiguous().clone()
        factor = 1
        for m in modes:
            out = all_reduce(out, m)
            factor *= m.world_size
        ctx.factor = factor if reduce_mean else 1
        if reduce_mean:
            out = out / factor
        return out.to(t.dtype) if t.is_floating_point() else out

    @staticmethod
    def backward(ctx, g):
        return g / ctx.factor, None, None


def all_gather_tensor_2d(tensor, dim, parallel_mode):
    return _GatherParam.apply(tensor, dim, parallel_mode)


def reduce_scatter_tensor_2d(tensor, dim, parallel_mode):
    return _ReduceScatterTensor.apply(tensor, dim, parallel_mode)


def reduce_tensor_2d(tensor, parallel_mode):
    return _ReduceTensor.apply(tensor, parallel_mode)


def reduce_by_batch_2d(tensor, reduce_mean: bool = False):
    return _ReduceByBatch.apply(tensor, (pm.PARALLEL_2D_COL, ), reduce_mean)


def split_batch_2d(tensor, dim: int = 0):
    """This grid row's slice of the batch dimension."""
    mode = pm.PARALLEL_2D_COL
    if tensor.size(dim) <= 1 or mode.world_size == 1:
        return tensor
    return torch.chunk(tensor, mode.world_size, dim=dim)[mode.local_rank].contiguous()


class _AddBias2D(torch.autograd.Function):
    """``y + gather_col(bias)``; with ``skip_bias_add`` only the gathered bias is produced."""

    @staticmethod
    def forward(ctx, x, bias, row, col, skip_bias_add):
        full = all_gather(bias.contiguous(), -1, col).contiguous()
        ctx.col, ctx.skip, ctx.b_dtype = col, skip_bias_add, bias.dtype
        if skip_bias_add:
            return full
        return x + full.to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        if ctx.skip:
            gb = g.float().reshape(-1, g.shape[-1]).sum(0) if g.dim() > 1 else g.float()
            return None, reduce_scatter(gb.contiguous(), -1, ctx.col).to(ctx.b_dtype), None, None, None
        gb = ops.column_sum(g.reshape(-1, g.shape[-1]).contiguous())
        return g, reduce_scatter(gb, -1, ctx.col).to(ctx.b_dtype), None, None, None


def add_bias_2d(input_, bias, row_parallel_mode, col_parallel_mode, skip_bias_add):
    return _AddBias2D.apply(input_, bias, row_parallel_mode, col_parallel_mode, skip_bias_add)


class _LayerNormSharded(torch.autograd.Function):
    """Layer norm whose hidden dimension is split over ``stat_mode``.

    One exchange of per-row ``(sum x, sum x^2)`` forward and of ``(sum g, sum g*xhat)`` backward
    (the reference issues two all-reduces each way: parallel_2d/module.py:142-171,
    _operation.py:330-347; parallel_3d/_operation.py:273-281, 293-313).  ``gamma``/``beta`` arrive
    already at the local hidden width; ``grad_modes`` are the groups over which their gradients must
    be summed afterwards (the ranks that hold other rows of the batch), reduced asynchronously.
    """

    @staticmethod
    def forward(ctx, x, gamma, beta, eps, hidden, stat_mode, grad_modes):
        cd = ops.compute_dtype(x)
        x2 = as_compute(x.reshape(-1, x.shape[-1]), cd)
        mom = ops.row_moments(x2)
        mom = all_reduce(mom, stat_mode)
        mean = mom[:, 0] / hidden
        var = (mom[:, 1] / hidden - mean * mean).clamp_min(0.0)
        rstd = torch.rsqrt(var + eps)
        y = ops.norm_apply(x2, mean, rstd, gamma, beta)
        ctx.save_for_backward(x2, mean, rstd, gamma)
        ctx.cfg = (hidden, stat_mode, grad_modes, x.dtype, gamma.dtype)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, mean, rstd, gamma = ctx.saved_tensors
        hidden, stat_mode, grad_modes, x_dtype, p_dtype = ctx.cfg
        dy2 = as_compute(dy.reshape(-1, dy.shape[-1]), x2.dtype)
        part, dgamma, dbeta = ops.norm_bwd_partials(dy2, x2, mean, rstd, gamma)
        # parameter gradients are summed over the other batch shards while the dx pass runs
        dgb = torch.stack([dgamma, dbeta]).to(p_dtype)
        works = []
        for m in grad_modes:
            if m.world_size > 1:
                dgb, w = all_reduce(dgb, m, async_op=True)
                works.append(w)
        part = all_reduce(part, stat_mode)
        dx = ops.norm_bwd_apply(dy2, x2, mean, rstd, gamma, part, hidden).view(dy.shape)
        if dx.dtype != x_dtype:
            dx = dx.to(x_dtype)
        for w in works:
            w.wait()
        return dx, dgb[0], dgb[1], None, None, None, None


def layer_norm_sharded(x, gamma, beta, eps, hidden, stat_mode, grad_modes=()):
    return _LayerNormSharded.apply(x, gamma, beta, eps, hidden, stat_mode, tuple(grad_modes))


class _Classifier2D(torch.autograd.Function):
    """``logits = all-reduce_row(A @ gather_col(W)^T) + b`` with W ``[C, H/q^2]``."""

    @staticmethod
    def forward(ctx, a, w, bias, out_shape, row, col):
        cd = ops.compute_dtype(a)
        a2 = as_compute(a.reshape(-1, a.shape[-1]), cd)
        wc = ops.shadow(w, cd)
        c, _, w_full = gather_gemm_reduce(a2, wc, trans_b=True, gather_b=(col, 1), reduce=row, bias=bias,
                                          keep_gathered=True)
        ctx.save_for_backward(a2, w_full)
        ctx.cfg = (cd, row, col, a.shape, a.dtype, w.dtype, bias.dtype if bias is not None else None)
        return c.reshape(out_shape)

    @staticmethod
    def backward(ctx, g):
        a2, w_full = ctx.saved_tensors
        cd, row, col, a_shape, a_dtype, w_dtype, b_dtype = ctx.cfg
        g2 = as_compute(g.reshape(-1, g.shape[-1]), cd)
        da = ops.gemm(g2, w_full).reshape(a_shape)
        if da.dtype != a_dtype:
            da = da.to(a_dtype)
        dw = gather_gemm_reduce(g2, a2, trans_a=True, scatter=(col, 1), out_dtype=w_dtype)
        db = None
        if b_dtype is not None:
            db = all_reduce(ops.column_sum(g2), col).to(b_dtype)
        return da, dw, db, None, None, None


def classifier_2d(A, B, bias, summa_dim, out_shape, row_parallel_mode, col_parallel_mode):
    return _Classifier2D.apply(A, B, bias, out_shape, row_parallel_mode, col_parallel_mode)
