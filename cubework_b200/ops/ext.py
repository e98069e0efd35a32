"""Loader and thin Python wrappers of the sm_100a extension (``cubework_b200_C.so``, built in-tree by
:mod:`cubework_b200.ops.build`).  ``require()`` raises when the library cannot be loaded: CUDA tensors
never fall back silently to a library path."""
import importlib.util
import os
import warnings

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "cubework_b200_C.so")
_mod = None
_err = None
_warned = set()
_launches = 0   # kernels of this package launched so far (bench.py reports the count inside its timed region)


def launch_count():
    return _launches


def _count(n=1):
    global _launches
    _launches += n


def _load():
    global _mod, _err
    if _mod is not None or _err is not None:
        return
    try:
        if not os.path.exists(_SO):
            if not torch.cuda.is_available():
                raise FileNotFoundError(_SO)
            from . import build as _b
            _b.build()
        spec = importlib.util.spec_from_file_location("cubework_b200_C", _SO)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
    except Exception as e:  # noqa: BLE001
        _err = e


def loaded():
    _load()
    return _mod is not None


def require():
    _load()
    if _mod is None:
        raise RuntimeError(f"cubework_b200 CUDA extension is not available ({_err!r}); build it with "
                           f"`python -m cubework_b200.ops.build`")
    return _mod


def has(feature: str) -> bool:
    if not loaded():
        return False
    return {"fused": hasattr(_mod, "fused_gemm_all_reduce"), "attention": hasattr(_mod, "attention_ready") and
            _mod.attention_ready()}.get(feature, False)


def _warn_once(key, msg):
    if key not in _warned:
        _warned.add(key)
        warnings.warn(msg)


def check_status(clear=True):
    """Raises if any kernel recorded a bounded-wait failure since the last check."""
    code, detail, count = require().read_status(clear)
    if code != 0:
        names = {1: "TMA stage never arrived", 2: "MMA never released a stage", 3: "accumulator never completed",
                 4: "epilogue never drained an accumulator", 5: "peer flag never written", 6: "grid barrier timeout",
                 7: "attention barrier timeout"}
        raise RuntimeError(f"device-side wait timed out: {names.get(code, code)} (detail={detail}, events={count})")


# --------------------------------------------------------------------------------------------------------
def _gemm_ok(a, b, trans_a, trans_b):
    """TMA needs 16-byte aligned bases and leading dimensions that are multiples of 8 elements."""
    return (a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0)


def gemm(a, b, trans_a, trans_b, bias, act, out_dtype, pre_act_out):
    a = a.contiguous()
    b = b.contiguous()
    out_f32 = out_dtype == torch.float32
    if not _gemm_ok(a, b, trans_a, trans_b) or (not out_f32 and out_dtype != a.dtype):
        _warn_once(("gemm", tuple(a.shape), tuple(b.shape)),
                   f"GEMM operands {tuple(a.shape)} x {tuple(b.shape)} are not TMA-compatible; using torch.matmul")
        A = a.t() if trans_a else a
        B = b.t() if trans_b else b
        z = A @ B
        if bias is not None:
            z = z + bias.to(z.dtype)
        y = torch.nn.functional.gelu(z) if act == "gelu" else torch.relu(z) if act == "relu" else z
        return (y.to(out_dtype), z.to(out_dtype)) if pre_act_out else y.to(out_dtype)
    _count(1)
    out, z = require().gemm(a, b, bool(trans_a), bool(trans_b), bias, act or "", out_f32, bool(pre_act_out))
    return (out, z) if pre_act_out else out


def act_backward(dy, z, act, want_bias_grad):
    code = {"gelu": 1, "relu": 2}[act]
    if dy.shape[1] % 8 != 0:
        zf = z.float()
        if act == "gelu":
            dz = dy.float() * (0.5 * (1 + torch.erf(zf * 0.7071067811865476)) +
                               zf * torch.exp(-0.5 * zf * zf) * 0.3989422804014327)
        else:
            dz = dy.float() * (zf > 0)
        dz = dz.to(dy.dtype)
        return dz, (dz.float().sum(0) if want_bias_grad else None)
    _count(2 if want_bias_grad else 1)
    dz, db = require().act_backward(dy.contiguous(), z.contiguous(), code, True, bool(want_bias_grad))
    return dz, (db if want_bias_grad else None)


def column_sum(x):
    if x.shape[1] % 8 != 0:
        return x.float().sum(0)
    _count(2)
    return require().act_backward(x.contiguous(), None, 0, False, True)[1]


def _f32(t):
    return t if (t is None or (t.dtype == torch.float32 and t.is_contiguous())) else t.float().contiguous()


def _norm_ok(x):
    return x.shape[1] % 8 == 0 and x.shape[1] <= 16384


def layer_norm_fwd(x, gamma, beta, eps):
    if not _norm_ok(x):
        xf = x.float()
        mean, var = xf.mean(-1), xf.var(-1, unbiased=False)
        rstd = torch.rsqrt(var + eps)
        return (((xf - mean[:, None]) * rstd[:, None]) * gamma.float() + beta.float()).to(x.dtype), mean, rstd
    _count(1)
    return tuple(require().layer_norm_fwd(x.contiguous(), _f32(gamma), _f32(beta), float(eps)))


def layer_norm_bwd(dy, x, mean, rstd, gamma):
    if not _norm_ok(x):
        xf, dyf = x.float(), dy.float()
        xhat = (xf - mean[:, None]) * rstd[:, None]
        g = dyf * gamma.float()
        dx = (g - g.mean(-1, keepdim=True) - xhat * (g * xhat).mean(-1, keepdim=True)) * rstd[:, None]
        return dx.to(x.dtype), (dyf * xhat).sum(0), dyf.sum(0)
    _count(2)
    return tuple(require().layer_norm_bwd(dy.contiguous(), x, mean, rstd, _f32(gamma)))


def row_moments(x):
    if not _norm_ok(x):
        xf = x.float()
        return torch.stack([xf.sum(-1), (xf * xf).sum(-1)], -1)
    _count(1)
    return require().row_moments(x.contiguous())


def norm_apply(x, mean, rstd, gamma, beta):
    if not _norm_ok(x):
        y = (x.float() - mean[:, None]) * rstd[:, None]
        if gamma is not None:
            y = y * gamma.float() + beta.float()
        return y.to(x.dtype)
    _count(1)
    return require().norm_apply(x.contiguous(), mean.contiguous(), rstd.contiguous(), _f32(gamma), _f32(beta))


def norm_bwd_partials(dy, x, mean, rstd, gamma):
    if not _norm_ok(x):
        xhat = (x.float() - mean[:, None]) * rstd[:, None]
        dyf = dy.float()
        g = dyf * gamma.float() if gamma is not None else dyf
        return torch.stack([g.sum(-1), (g * xhat).sum(-1)], -1), (dyf * xhat).sum(0), dyf.sum(0)
    _count(2)
    return tuple(require().norm_bwd_partials(dy.contiguous(), x, mean.contiguous(), rstd.contiguous(), _f32(gamma)))


def norm_bwd_apply(dy, x, mean, rstd, gamma, sums, hidden):
    if not _norm_ok(x):
        xhat = (x.float() - mean[:, None]) * rstd[:, None]
        g = dy.float() * gamma.float() if gamma is not None else dy.float()
        return ((g - sums[:, 0:1] / hidden - xhat * sums[:, 1:2] / hidden) * rstd[:, None]).to(x.dtype)
    _count(1)
    return require().norm_bwd_apply(dy.contiguous(), x, mean.contiguous(), rstd.contiguous(), _f32(gamma),
                                    sums.contiguous(), float(hidden))


def ce_local_stats(logits, targets, vocab_start):
    _count(1)
    return require().ce_local_stats(logits.contiguous(), targets.contiguous(), int(vocab_start))


def ce_grad(logits, targets, vocab_start, gmax, gsum, grad_scale, inplace=False):
    _count(1)
    return require().ce_grad(logits.contiguous(), targets.contiguous(), int(vocab_start), gmax.contiguous(),
                             gsum.contiguous(), grad_scale.contiguous(), bool(inplace))


def embedding_fwd(ids, weight, vocab_start, out_dtype):
    _count(1)
    return require().embedding_fwd(ids, weight.contiguous(), int(vocab_start), out_dtype)


def embedding_bwd(dout, ids, vocab_start, num_rows, grad_dtype):
    _count(1)
    return require().embedding_bwd(dout.contiguous(), ids, int(vocab_start), int(num_rows)).to(grad_dtype)


def multi_sumsq(grads, weights):
    _count((len(grads) + 23) // 24)
    return require().multi_sumsq([g.contiguous() for g in grads], [float(w) for w in weights])


def multi_scale(grads, coef):
    _count((len(grads) + 23) // 24)
    require().multi_scale(grads, coef)


def multi_adamw(params, grads, exp_avg, exp_avg_sq, shadows, lr, beta1, beta2, eps, wd, step, grad_scale):
    _count((len(params) + 23) // 24)
    require().multi_adamw(params, grads, exp_avg, exp_avg_sq, shadows, float(lr), float(beta1), float(beta2),
                          float(eps), float(wd), int(step), grad_scale)


def multi_sgd(params, grads, bufs, shadows, lr, momentum, wd, first, grad_scale):
    _count((len(params) + 23) // 24)
    require().multi_sgd(params, grads, bufs, shadows, float(lr), float(momentum), float(wd), bool(first), grad_scale)


ATTN_TRACE = None   # optional int64 [2, 4096, 2] CUDA tensor: event stamps of CTA 0 of the next attention forward launches


def attention_fwd(qkv, causal, key_bias, scale):
    m = require()
    out, lse, packed = m.attention_fwd(qkv, bool(causal), key_bias, float(scale), m.status_device_ptr(), ATTN_TRACE)
    _count(1 if packed is None else 2)
    return out, (lse, packed)


def attention_bwd(dout, qkv, out, lse, causal, key_bias, scale):
    m = require()
    lse, packed = lse
    _count(3 if packed is None else 4)
    return m.attention_bwd(dout, qkv, out, lse, bool(causal), key_bias, float(scale), m.status_device_ptr(), packed,
                           ATTN_TRACE)
