"""Hot-op entry points.

Each function has two implementations: the hand-written sm_100a kernel (``cubework_b200/ops/csrc``,
loaded by :mod:`cubework_b200.ops.ext`) used for CUDA tensors in bf16/fp16, and a plain PyTorch
formulation used for host tensors and for fp32 (it is also the numerical oracle of the kernel
tests).  There is no silent fallback on a GPU: if a CUDA bf16 tensor arrives and the extension cannot
be loaded, the call raises.

The ops replace these reference call sites: ``F.linear`` / ``torch.matmul`` / ``addmm`` in
cubework/module/parallel_{1d,2d,3d}; ``nn.LayerNorm`` (parallel_1d/module.py:72-87) and the 2D/3D
layer-norm Functions; ``F.gelu``/``ReLU`` after ``dense_1`` (benchmark/gpt2/gpt2.py:116-117); the
unfused attention (gpt2.py:75-91, vit.py:81-89, opt.py:87-128); the vocab-parallel cross-entropy
(module/loss/loss_1d.py:14-79); ``torch.optim.AdamW``/``SGD`` (gpt2.py:440, opt.py:623).
"""
import math
import os
from typing import List, Optional

import torch
import torch.nn.functional as F

from . import ext

_LOWP = (torch.bfloat16, torch.float16)


def kernels_enabled() -> bool:
    return os.environ.get("CUBEWORK_B200_KERNELS", "1") != "0"


def use_kernels(t: torch.Tensor) -> bool:
    """True when ``t`` should go through the sm_100a kernels (CUDA + 16-bit float)."""
    if not (t.is_cuda and t.dtype in _LOWP and kernels_enabled()):
        return False
    ext.require()
    return True


def compute_dtype(t: torch.Tensor) -> torch.dtype:
    """Autocast dtype when autocast is on for the tensor's device, else the tensor's own dtype."""
    dev = t.device.type
    if torch.is_autocast_enabled(dev):
        return torch.get_autocast_dtype(dev)
    return t.dtype


# ---------------------------------------------------------------------------------------------------
# low-precision shadows of fp32 master parameters
# ---------------------------------------------------------------------------------------------------
class _Shadow:
    __slots__ = ("tensor", "version")


_SHADOWS = {}


def shadow(param: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``param`` in ``dtype``; cached until the parameter changes (the fused optimizers refresh it
    inside their update kernel, so in steady state no cast kernel runs)."""
    if param.dtype == dtype:
        return param.detach()
    key = (id(param), dtype)
    s = _SHADOWS.get(key)
    base = param.detach()
    if s is None or s.tensor.shape != base.shape or s.tensor.device != base.device:
        s = _Shadow()
        s.tensor = base.to(dtype)
        s.version = param._version
        _SHADOWS[key] = s
        _register_shadow_finalizer(param, key)
    elif s.version != param._version:
        s.tensor.copy_(base)
        s.version = param._version
    return s.tensor


def drop_shadow(param: torch.Tensor):
    """Forget the cached low-precision copies of ``param`` (its storage was replaced, or is about to be freed)."""
    for key in [k for k in _SHADOWS if k[0] == id(param)]:
        _SHADOWS.pop(key, None)


def peek_shadow(param: torch.Tensor, dtype: torch.dtype):
    s = _SHADOWS.get((id(param), dtype))
    return s


def _register_shadow_finalizer(param, key):
    import weakref
    try:
        weakref.finalize(param, _SHADOWS.pop, key, None)
    except TypeError:
        pass


# ---------------------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------------------
def _act(x, act):
    if act is None:
        return x
    if act == "gelu":
        return F.gelu(x)
    if act == "relu":
        return F.relu(x)
    raise ValueError(act)


def gemm(a: torch.Tensor,
         b: torch.Tensor,
         trans_a: bool = False,
         trans_b: bool = False,
         bias: Optional[torch.Tensor] = None,
         act: Optional[str] = None,
         out_dtype: Optional[torch.dtype] = None,
         pre_act_out: bool = False):
    """``C = act(op(A) @ op(B) + bias)`` for 2-D operands; ``op`` transposes when the flag is set.

    ``bias`` broadcasts along rows (one value per output column).  With ``pre_act_out`` the value
    before the activation is returned as a second tensor (needed by the activation's backward).
    No autograd: callers are ``autograd.Function`` bodies.
    """
    assert a.dim() == 2 and b.dim() == 2
    out_dtype = out_dtype or a.dtype
    if use_kernels(a) and b.dtype == a.dtype:
        return ext.gemm(a, b, trans_a, trans_b, bias, act, out_dtype, pre_act_out)
    A = a.t() if trans_a else a
    B = b.t() if trans_b else b
    if A.dtype in _LOWP and A.device.type == "cpu":
        z = (A.float() @ B.float())
    else:
        z = A @ B
    if bias is not None:
        z = z + bias.to(z.dtype)
    y = _act(z, act)
    if pre_act_out:
        return y.to(out_dtype), z.to(out_dtype)
    return y.to(out_dtype)


def act_backward(dy: torch.Tensor, z: torch.Tensor, act: str, want_bias_grad: bool = False):
    """``dz = dy * act'(z)`` and optionally ``db = dz.sum(0)`` (fp32) in one pass."""
    if use_kernels(dy):
        return ext.act_backward(dy, z, act, want_bias_grad)
    zf = z.float()
    if act == "gelu":
        cdf = 0.5 * (1.0 + torch.erf(zf / math.sqrt(2.0)))
        pdf = torch.exp(-0.5 * zf * zf) / math.sqrt(2.0 * math.pi)
        dz = dy.float() * (cdf + zf * pdf)
    elif act == "relu":
        dz = dy.float() * (zf > 0).float()
    else:
        raise ValueError(act)
    db = dz.sum(0) if want_bias_grad else None
    return dz.to(dy.dtype), db


def column_sum(x: torch.Tensor) -> torch.Tensor:
    """fp32 sum over rows of a 2-D tensor (bias gradients)."""
    if use_kernels(x):
        return ext.column_sum(x)
    return x.float().sum(0)


# ---------------------------------------------------------------------------------------------------
# LayerNorm (local statistics; the 2D/3D layers pass partial sums through a collective in between)
# ---------------------------------------------------------------------------------------------------
def layer_norm_fwd(x2d, gamma, beta, eps, residual=None):
    """Returns ``(y, mean, rstd)``; statistics in fp32.  With ``residual`` the norm is that of ``x + residual``
    (rounded to the tensors' dtype) and the sum is returned as a fourth value."""
    if use_kernels(x2d):
        return ext.layer_norm_fwd(x2d, gamma, beta, eps, residual)
    if residual is not None:
        total = x2d + residual
        return layer_norm_fwd(total, gamma, beta, eps) + (total, )
    xf = x2d.float()
    mean = xf.mean(-1)
    var = xf.var(-1, unbiased=False)
    rstd = torch.rsqrt(var + eps)
    y = (xf - mean[:, None]) * rstd[:, None] * gamma.float() + beta.float()
    return y.to(x2d.dtype), mean, rstd


def layer_norm_bwd(dy2d, x2d, mean, rstd, gamma, dres=None):
    """Returns ``(dx, dgamma, dbeta)``; parameter gradients in fp32.  ``dres`` (a gradient that reaches the
    normalised tensor by another path, e.g. the residual connection) is added to ``dx``."""
    if use_kernels(x2d):
        return ext.layer_norm_bwd(dy2d, x2d, mean, rstd, gamma, dres)
    if dres is not None:
        dx, dg, db = layer_norm_bwd(dy2d, x2d, mean, rstd, gamma)
        return dx + dres.to(dx.dtype), dg, db
    xf, dyf = x2d.float(), dy2d.float()
    xhat = (xf - mean[:, None]) * rstd[:, None]
    dgamma = (dyf * xhat).sum(0)
    dbeta = dyf.sum(0)
    g = dyf * gamma.float()
    dx = (g - g.mean(-1, keepdim=True) - xhat * (g * xhat).mean(-1, keepdim=True)) * rstd[:, None]
    return dx.to(x2d.dtype), dgamma, dbeta


def row_moments(x2d):
    """Per-row ``[sum(x), sum(x*x)]`` as an fp32 ``[rows, 2]`` tensor (sharded layer norm, pass 1)."""
    if use_kernels(x2d):
        return ext.row_moments(x2d)
    xf = x2d.float()
    return torch.stack([xf.sum(-1), (xf * xf).sum(-1)], dim=-1)


def norm_apply(x2d, mean, rstd, gamma, beta):
    """``(x - mean) * rstd * gamma + beta`` with externally supplied statistics (pass 2)."""
    if use_kernels(x2d):
        return ext.norm_apply(x2d, mean, rstd, gamma, beta)
    y = (x2d.float() - mean[:, None]) * rstd[:, None]
    if gamma is not None:
        y = y * gamma.float() + beta.float()
    return y.to(x2d.dtype)


def norm_bwd_partials(dy2d, x2d, mean, rstd, gamma):
    """Per-row ``[sum(g), sum(g*xhat)]`` with ``g = dy*gamma`` (fp32 ``[rows,2]``) plus the local
    ``dgamma``/``dbeta`` column sums (sharded layer norm backward, pass 1)."""
    if use_kernels(x2d):
        return ext.norm_bwd_partials(dy2d, x2d, mean, rstd, gamma)
    xhat = (x2d.float() - mean[:, None]) * rstd[:, None]
    dyf = dy2d.float()
    g = dyf * gamma.float() if gamma is not None else dyf
    part = torch.stack([g.sum(-1), (g * xhat).sum(-1)], dim=-1)
    return part, (dyf * xhat).sum(0), dyf.sum(0)


def norm_bwd_apply(dy2d, x2d, mean, rstd, gamma, sums, hidden):
    """``dx = (g - sums[:,0]/H - xhat*sums[:,1]/H) * rstd`` (pass 2)."""
    if use_kernels(x2d):
        return ext.norm_bwd_apply(dy2d, x2d, mean, rstd, gamma, sums, hidden)
    xhat = (x2d.float() - mean[:, None]) * rstd[:, None]
    g = dy2d.float() * gamma.float() if gamma is not None else dy2d.float()
    dx = (g - sums[:, 0:1] / hidden - xhat * sums[:, 1:2] / hidden) * rstd[:, None]
    return dx.to(x2d.dtype)


# ---------------------------------------------------------------------------------------------------
# vocab-parallel softmax cross-entropy (local pieces; the caller exchanges the [rows,3] statistics)
# ---------------------------------------------------------------------------------------------------
def ce_local_stats(logits2d, targets, vocab_start):
    """fp32 ``[rows, 3]`` = (row max, sum exp(x - max), target logit or 0 if the target is not local)."""
    if use_kernels(logits2d):
        return ext.ce_local_stats(logits2d, targets, vocab_start)
    lf = logits2d.float()
    mx = lf.max(-1).values
    se = torch.exp(lf - mx[:, None]).sum(-1)
    local = targets - vocab_start
    ok = (local >= 0) & (local < logits2d.shape[-1])
    idx = local.clamp(0, logits2d.shape[-1] - 1)
    tl = torch.where(ok, lf.gather(-1, idx[:, None]).squeeze(-1), torch.zeros_like(mx))
    return torch.stack([mx, se, tl], dim=-1)


def ce_grad(logits2d, targets, vocab_start, gmax, gsum, grad_scale, inplace=False):
    """``(softmax - onehot_local) * grad_scale[row]`` in the logits' dtype, from the global max / sum."""
    if use_kernels(logits2d):
        return ext.ce_grad(logits2d, targets, vocab_start, gmax, gsum, grad_scale, inplace)
    lf = logits2d.float()
    p = torch.exp(lf - gmax[:, None]) / gsum[:, None]
    local = targets - vocab_start
    ok = (local >= 0) & (local < logits2d.shape[-1])
    idx = local.clamp(0, logits2d.shape[-1] - 1)
    p.scatter_add_(-1, idx[:, None], -ok.float()[:, None])
    return (p * grad_scale[:, None]).to(logits2d.dtype)


# ---------------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------------
def attention_reference(q, k, v, causal, key_bias=None, scale=None):
    """Plain softmax(QK^T*scale + mask)V in fp32; ``q,k,v`` are ``[B, heads, T, dh]``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if causal:
        T, S = s.shape[-2], s.shape[-1]
        m = torch.ones(T, S, dtype=torch.bool, device=s.device).tril(S - T)
        s = s.masked_fill(~m, float("-inf"))
    if key_bias is not None:
        s = s + key_bias.float()[:, None, None, :]
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, v.float()).to(q.dtype)


class _AttentionFn(torch.autograd.Function):
    """Fused attention over a packed ``[B, T, heads, 3*dh]`` QKV tensor (per-head q|k|v layout)."""

    @staticmethod
    def forward(ctx, qkv, causal, key_bias, scale):
        out, (lse, packed) = ext.attention_fwd(qkv, causal, key_bias, scale)
        empty = qkv.new_empty(0)
        # `packed` is the padded, TMA-aligned copy of QKV that odd head dims need; keep it for the backward
        ctx.save_for_backward(qkv, out, lse, key_bias if key_bias is not None else empty,
                              packed if packed is not None else empty)
        ctx.causal, ctx.scale, ctx.has_bias, ctx.has_packed = causal, scale, key_bias is not None, packed is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, kb, packed = ctx.saved_tensors
        dqkv = ext.attention_bwd(dout.contiguous(), qkv, out, (lse, packed if ctx.has_packed else None), ctx.causal,
                                 kb if ctx.has_bias else None, ctx.scale)
        return dqkv, None, None, None


def attention_packed(qkv: torch.Tensor, causal: bool, key_bias: Optional[torch.Tensor] = None,
                     scale: Optional[float] = None) -> torch.Tensor:
    """Self-attention on packed QKV ``[B, T, heads, 3*dh]`` -> ``[B, T, heads*dh]``.

    ``key_bias`` is an additive ``[B, T]`` mask over key positions (0 keep / large negative drop).
    """
    B, T, H, D3 = qkv.shape
    dh = D3 // 3
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    if use_kernels(qkv):
        return _AttentionFn.apply(qkv.contiguous(), causal, key_bias, scale).view(B, T, H * dh)
    q, k, v = qkv.permute(0, 2, 1, 3).chunk(3, dim=-1)
    o = attention_reference(q, k, v, causal, key_bias, scale)
    return o.transpose(1, 2).reshape(B, T, H * dh)


def attention_with_prob_dropout(qkv: torch.Tensor, causal: bool, key_bias: Optional[torch.Tensor], dropout,
                                scale: Optional[float] = None) -> torch.Tensor:
    """Self-attention with ``dropout`` (a module) applied to the probabilities: the materialised formulation
    ``softmax(QK^T * scale + mask) -> dropout -> @ V`` on packed QKV ``[B, T, heads, 3*dh]`` (autograd by PyTorch).
    The softmax runs in fp32; the two batched products run in the tensor's dtype."""
    B, T, H, D3 = qkv.shape
    dh = D3 // 3
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    q, k, v = qkv.permute(0, 2, 1, 3).chunk(3, dim=-1)
    s = torch.matmul(q, k.transpose(-1, -2)).float() * scale
    if causal:
        keep = torch.ones(T, T, dtype=torch.bool, device=s.device).tril()
        s = s.masked_fill(~keep, float("-inf"))
    if key_bias is not None:
        s = s + key_bias.float()[:, None, None, :]
    p = dropout(torch.softmax(s, dim=-1).to(qkv.dtype))
    return torch.matmul(p, v).transpose(1, 2).reshape(B, T, H * dh)


# ---------------------------------------------------------------------------------------------------
# embedding
# ---------------------------------------------------------------------------------------------------
def embedding_fwd(ids, weight, vocab_start, out_dtype):
    """Rows ``weight[ids - vocab_start]``; ids outside the local range give zero rows."""
    if weight.is_cuda and kernels_enabled() and out_dtype in _LOWP:
        ext.require()
        return ext.embedding_fwd(ids, weight, vocab_start, out_dtype)
    local = ids - vocab_start
    ok = (local >= 0) & (local < weight.shape[0])
    out = F.embedding(local.clamp(0, weight.shape[0] - 1), weight)
    out = out * ok.unsqueeze(-1).to(out.dtype)
    return out.to(out_dtype)


def embedding_bwd(dout, ids, vocab_start, num_rows, grad_dtype):
    """Scatter-add of ``dout`` rows into a ``[num_rows, H]`` gradient (ids outside the range skipped)."""
    if dout.is_cuda and kernels_enabled() and dout.dtype in _LOWP:
        ext.require()
        return ext.embedding_bwd(dout, ids, vocab_start, num_rows, grad_dtype)
    H = dout.shape[-1]
    local = (ids - vocab_start).reshape(-1)
    ok = (local >= 0) & (local < num_rows)
    g = torch.zeros(num_rows, H, dtype=torch.float32, device=dout.device)
    g.index_add_(0, local[ok], dout.reshape(-1, H)[ok].float())
    return g.to(grad_dtype)


# ---------------------------------------------------------------------------------------------------
# multi-tensor helpers for the optimizer and gradient clipping
# ---------------------------------------------------------------------------------------------------
def grad_norm_pow(params: List[torch.Tensor], weights: List[float], norm_type: float) -> torch.Tensor:
    """fp32 ``[1]`` tensor ``sum_i weights[i] * sum(|grad_i|^norm_type)``."""
    grads = [p.grad.detach() for p in params]
    if grads and grads[0].is_cuda and kernels_enabled() and norm_type == 2.0:
        ext.require()
        return ext.multi_sumsq(grads, weights)
    dev = grads[0].device
    acc = torch.zeros(1, dtype=torch.float32, device=dev)
    for g, w in zip(grads, weights):
        acc += w * g.float().abs().pow(norm_type).sum()
    return acc


def scale_grads(params: List[torch.Tensor], coef: torch.Tensor):
    """``grad *= coef`` for every parameter; ``coef`` is a one-element tensor (no host sync)."""
    grads = [p.grad.detach() for p in params]
    if grads and grads[0].is_cuda and kernels_enabled():
        ext.require()
        ext.multi_scale(grads, coef.float().reshape(1))
        return
    for g in grads:
        g.mul_(coef.to(g.device, g.dtype).reshape(()))
