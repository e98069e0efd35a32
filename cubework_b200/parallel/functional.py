"""Mode-independent autograd functions built on the hot-op kernels (``cubework_b200.ops``):
local layer norm, masked embedding lookup, local linear, and the dtype plumbing they share.

Reference call sites replaced: ``nn.LayerNorm`` in LayerNorm1D (parallel_1d/module.py:72-87),
``F.embedding`` + mask/zero in the vocab-parallel embeddings (parallel_1d/module.py:441-455),
``F.linear`` in the classifiers.
"""
import torch

from .. import ops


def as_compute(x2d, cd):
    if x2d.dtype != cd:
        x2d = x2d.to(cd)
    return x2d.contiguous()


class _LayerNorm(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        cd = ops.compute_dtype(x)
        x2 = as_compute(x.reshape(-1, x.shape[-1]), cd)
        y, mean, rstd = ops.layer_norm_fwd(x2, gamma, beta, eps)
        ctx.save_for_backward(x2, mean, rstd, gamma)
        ctx.x_dtype, ctx.p_dtype = x.dtype, gamma.dtype
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, mean, rstd, gamma = ctx.saved_tensors
        dy2 = as_compute(dy.reshape(-1, dy.shape[-1]), x2.dtype)
        dx, dg, db = ops.layer_norm_bwd(dy2, x2, mean, rstd, gamma)
        dx = dx.view(dy.shape)
        if dx.dtype != ctx.x_dtype:
            dx = dx.to(ctx.x_dtype)
        return dx, dg.to(ctx.p_dtype), db.to(ctx.p_dtype), None


class _AddLayerNorm(torch.autograd.Function):
    """``s = x + r`` and ``y = LN(s)`` in one pass; returns ``(s, y)``.  Backward: the gradient of ``s`` is the layer
    norm's input gradient plus whatever reaches ``s`` directly (the residual path), again in one pass; ``x`` and ``r``
    both receive it.  Replaces the separate residual add in front of every norm (benchmark/gpt2/gpt2.py:179-186)."""

    @staticmethod
    def forward(ctx, x, r, gamma, beta, eps):
        cd = ops.compute_dtype(x)
        x2 = as_compute(x.reshape(-1, x.shape[-1]), cd)
        r2 = as_compute(r.reshape(-1, r.shape[-1]), cd)
        y, mean, rstd, total = ops.layer_norm_fwd(x2, gamma, beta, eps, residual=r2)
        ctx.save_for_backward(total, mean, rstd, gamma)
        ctx.x_dtype, ctx.r_dtype, ctx.p_dtype = x.dtype, r.dtype, gamma.dtype
        return total.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, ds, dy):
        total, mean, rstd, gamma = ctx.saved_tensors
        dy2 = as_compute(dy.reshape(-1, dy.shape[-1]), total.dtype)
        ds2 = as_compute(ds.reshape(-1, ds.shape[-1]), total.dtype)
        dx, dg, db = ops.layer_norm_bwd(dy2, total, mean, rstd, gamma, dres=ds2)
        dx = dx.view(dy.shape)
        gx = dx if dx.dtype == ctx.x_dtype else dx.to(ctx.x_dtype)
        gr = dx if dx.dtype == ctx.r_dtype else dx.to(ctx.r_dtype)
        return gx, gr, dg.to(ctx.p_dtype), db.to(ctx.p_dtype), None


def layer_norm(x, gamma, beta, eps):
    return _LayerNorm.apply(x, gamma, beta, eps)


def add_layer_norm(x, r, gamma, beta, eps):
    """``(x + r, LN(x + r))``."""
    return _AddLayerNorm.apply(x, r, gamma, beta, eps)


class _MaskedEmbedding(torch.autograd.Function):
    """Lookup in a vocabulary shard that starts at ``vocab_start``; foreign ids give zero rows."""

    @staticmethod
    def forward(ctx, ids, weight, vocab_start, out_dtype):
        ctx.save_for_backward(ids)
        ctx.vocab_start, ctx.rows, ctx.w_dtype = vocab_start, weight.shape[0], weight.dtype
        return ops.embedding_fwd(ids, weight.detach(), vocab_start, out_dtype)

    @staticmethod
    def backward(ctx, dout):
        (ids, ) = ctx.saved_tensors
        dw = ops.embedding_bwd(dout.contiguous(), ids, ctx.vocab_start, ctx.rows, ctx.w_dtype)
        return None, dw, None, None


def masked_embedding(ids, weight, vocab_start=0, out_dtype=None):
    if out_dtype is None:
        out_dtype = ops.compute_dtype(weight)
    return _MaskedEmbedding.apply(ids, weight, vocab_start, out_dtype)


class _LocalLinear(torch.autograd.Function):
    """``y = act(x @ op(w) + b)`` on this rank only; ``w_is_out_in`` selects ``[out,in]`` vs ``[in,out]``."""

    @staticmethod
    def forward(ctx, x, w, b, w_is_out_in, act):
        cd = ops.compute_dtype(x)
        x2 = as_compute(x.reshape(-1, x.shape[-1]), cd)
        wc = ops.shadow(w, cd)
        z = None
        if act is not None:
            y, z = ops.gemm(x2, wc, trans_b=w_is_out_in, bias=b, act=act, pre_act_out=True)
        else:
            y = ops.gemm(x2, wc, trans_b=w_is_out_in, bias=b)
        ctx.save_for_backward(x2, w, z if z is not None else x2.new_empty(0))
        ctx.cfg = (cd, w_is_out_in, act, b is not None, b.dtype if b is not None else None, x.dtype, x.shape)
        return y.view(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x2, w, z = ctx.saved_tensors
        cd, w_is_out_in, act, has_b, b_dtype, x_dtype, x_shape = ctx.cfg
        dy2 = as_compute(dy.reshape(-1, dy.shape[-1]), cd)
        db = None
        if act is not None:
            dy2, db = ops.act_backward(dy2, z, act, has_b)
        elif has_b:
            db = ops.column_sum(dy2)
        if db is not None:
            db = db.to(b_dtype)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = ops.gemm(dy2, ops.shadow(w, cd), trans_b=not w_is_out_in).view(x_shape)
            if dx.dtype != x_dtype:
                dx = dx.to(x_dtype)
        if ctx.needs_input_grad[1]:
            if w_is_out_in:
                dw = ops.gemm(dy2, x2, trans_a=True, out_dtype=w.dtype)
            else:
                dw = ops.gemm(x2, dy2, trans_a=True, out_dtype=w.dtype)
        return dx, dw, db, None, None


def local_linear(x, w, b=None, w_is_out_in=True, act=None):
    return _LocalLinear.apply(x, w, b, w_is_out_in, act)
