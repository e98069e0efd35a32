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
# TMA reads need 16-byte aligned bases and row pitches: operands whose last dimension is not a multiple of eight
# 16-bit elements are zero-padded (a copy) rather than handed to a library GEMM; the result is cut back.
def _pad_cols(t, mult=8):
    extra = (-t.shape[1]) % mult
    return torch.nn.functional.pad(t, (0, extra)) if extra else t


def _pad_rows(t, rows):
    return torch.nn.functional.pad(t, (0, 0, 0, rows - t.shape[0])) if rows != t.shape[0] else t


def _tma_ready(t):
    t = t.contiguous()
    return t if t.data_ptr() % 16 == 0 else t.clone()


def gemm(a, b, trans_a, trans_b, bias, act, out_dtype, pre_act_out):
    out_f32 = out_dtype == torch.float32
    if not out_f32 and out_dtype != a.dtype:
        raise ValueError(f"GEMM output dtype must be float32 or the operands' dtype ({a.dtype}), got {out_dtype}")
    M = a.shape[1] if trans_a else a.shape[0]
    N = b.shape[0] if trans_b else b.shape[1]
    if a.shape[1] % 8 or b.shape[1] % 8:
        a, b = _pad_cols(a), _pad_cols(b)           # pads K (K-major operand) or M / N (MN-major operand) with zeros
        ka = a.shape[0] if trans_a else a.shape[1]
        kb = b.shape[1] if trans_b else b.shape[0]
        k = max(ka, kb)                             # the other operand follows a padded K with zero rows / columns
        if ka != k:
            a = _pad_rows(a, k) if trans_a else torch.nn.functional.pad(a, (0, k - ka))
        if kb != k:
            b = torch.nn.functional.pad(b, (0, k - kb)) if trans_b else _pad_rows(b, k)
        n_pad = b.shape[0] if trans_b else b.shape[1]
        if bias is not None and n_pad != N:
            bias = torch.nn.functional.pad(bias, (0, n_pad - N))
    a, b = _tma_ready(a), _tma_ready(b)
    _count(1)
    out, z = require().gemm(a, b, bool(trans_a), bool(trans_b), bias, act or "", out_f32, bool(pre_act_out))
    if out.shape[0] != M or out.shape[1] != N:
        out = out[:M, :N].contiguous()
        z = z[:M, :N].contiguous() if pre_act_out else z
    return (out, z) if pre_act_out else out


def act_backward(dy, z, act, want_bias_grad):
    code = {"gelu": 1, "relu": 2}[act]
    n = dy.shape[1]
    if n % 8:
        dy, z = _pad_cols(dy), _pad_cols(z)
    _count(2 if want_bias_grad else 1)
    dz, db = require().act_backward(dy.contiguous(), z.contiguous(), code, True, bool(want_bias_grad))
    if dz.shape[1] != n:
        dz = dz[:, :n].contiguous()
        db = db[:n].contiguous() if want_bias_grad else db
    return dz, (db if want_bias_grad else None)


def column_sum(x):
    n = x.shape[1]
    _count(2)
    s = require().act_backward(_pad_cols(x).contiguous(), None, 0, False, True)[1]
    return s[:n].contiguous() if s.shape[0] != n else s


def _f32(t):
    return t if (t is None or (t.dtype == torch.float32 and t.is_contiguous())) else t.float().contiguous()


def _norm_ok(x):
    """The layer-norm kernels read rows in 16-byte pieces and keep one row per CTA in registers."""
    if x.shape[1] % 8 == 0 and x.shape[1] <= 16384:
        return True
    raise ValueError(f"the layer-norm kernels need a hidden size that is a multiple of 8 and at most 16384, got "
                     f"{x.shape[1]} (run this shape in fp32, which takes the PyTorch formulation)")


def layer_norm_fwd(x, gamma, beta, eps, residual=None):
    """``(y, mean, rstd)``, or ``(y, mean, rstd, x + residual)`` when a residual is given (added in the same kernel)."""
    _norm_ok(x)
    _count(1)
    y, mean, rstd, total = require().layer_norm_fwd_res(x.contiguous(), None if residual is None else residual.contiguous(),
                                                        _f32(gamma), _f32(beta), float(eps))
    return (y, mean, rstd) if residual is None else (y, mean, rstd, total)


def layer_norm_bwd(dy, x, mean, rstd, gamma, dres=None):
    """``(dx, dgamma, dbeta)``; ``dres`` (optional) is added to ``dx`` in the same kernel."""
    _norm_ok(x)
    _count(2)
    return tuple(require().layer_norm_bwd_res(dy.contiguous(), x, mean, rstd, _f32(gamma),
                                              None if dres is None else dres.contiguous()))


def row_moments(x):
    _norm_ok(x)
    _count(1)
    return require().row_moments(x.contiguous())


def norm_apply(x, mean, rstd, gamma, beta):
    _norm_ok(x)
    _count(1)
    return require().norm_apply(x.contiguous(), mean.contiguous(), rstd.contiguous(), _f32(gamma), _f32(beta))


def norm_bwd_partials(dy, x, mean, rstd, gamma):
    _norm_ok(x)
    _count(2)
    return tuple(require().norm_bwd_partials(dy.contiguous(), x, mean.contiguous(), rstd.contiguous(), _f32(gamma)))


def norm_bwd_apply(dy, x, mean, rstd, gamma, sums, hidden):
    _norm_ok(x)
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
