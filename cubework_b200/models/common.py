"""Pieces shared by the GPT-2 / OPT / ViT model families: the self-attention core over a packed QKV
projection, the transformer MLP, activation checkpointing and the data-parallel wrapper choice."""
import math

import torch
import torch.nn as nn

from .. import module as cube_nn
from .. import ops


class SelfAttention(nn.Module):
    """QKV projection -> fused attention -> output projection.

    The QKV weight uses the per-head ``[q | k | v]`` output ordering of the reference models
    (benchmark/gpt2/gpt2.py:66-96, vit/vit.py:74-89, opt/opt.py:70-128), so any contiguous shard of
    its output features holds whole heads and the local head count follows from the local width.
    Scores never reach HBM: the attention itself is one flash-style kernel.

    Dropout on the attention probabilities (``attention_dropout``; reference gpt2.py:62,84-86, vit.py:63,84,
    opt.py:141) is applied in training mode by the materialised formulation of the reference - scores, softmax,
    :class:`cubework_b200.module.Dropout` (per-rank TENSOR stream in 2D / 3D), product with V - because the fused
    kernel has no random-number path; with ``attention_dropout == 0`` or in evaluation mode the fused kernel runs.
    """

    def __init__(self, hidden_size, num_heads, attention_dropout=0.0, dropout=0.0, bias=True, causal=False,
                 qkv_kw=None, out_kw=None, out_bias=True, sequence_parallel=False):
        super().__init__()
        self.head_dim = hidden_size // num_heads
        self.causal = causal
        sp = dict(sequence_parallel=sequence_parallel)
        self.query_key_value = cube_nn.Linear(hidden_size, 3 * hidden_size, bias=bias, **sp, **(qkv_kw or {}))
        self.attention_dropout_p = attention_dropout
        self.dense = cube_nn.Linear(hidden_size, hidden_size, bias=out_bias, **sp, **(out_kw or {}))
        self.dropout = cube_nn.Dropout(dropout, **sp)
        # heads are sharded in every mode, so the probabilities differ per rank: per-rank random stream
        self.attention_dropout = cube_nn.Dropout(attention_dropout, sequence_parallel=True)

    def forward(self, x, key_bias=None):
        qkv = self.query_key_value(x)
        b, t, w = qkv.shape
        heads = w // (3 * self.head_dim)
        qkv = qkv.view(b, t, heads, 3 * self.head_dim)
        if self.attention_dropout_p > 0.0 and self.training:
            ctx = ops.attention_with_prob_dropout(qkv, self.causal, key_bias, self.attention_dropout)
        else:
            ctx = ops.attention_packed(qkv, self.causal, key_bias)
        return self.dropout(self.dense(ctx))


class MLP(nn.Module):

    def __init__(self, hidden_size, intermediate_size, activation="gelu", dropout=0.0, bias=True, kw1=None,
                 kw2=None, inner_dropout=0.0, sequence_parallel=False):
        super().__init__()
        sp = dict(sequence_parallel=sequence_parallel)
        self.dense_1 = cube_nn.Linear(hidden_size, intermediate_size, bias=bias, activation=activation, **sp,
                                      **(kw1 or {}))
        self.inner_dropout = cube_nn.Dropout(inner_dropout)
        self.dense_2 = cube_nn.Linear(intermediate_size, hidden_size, bias=bias, **sp, **(kw2 or {}))
        self.dropout = cube_nn.Dropout(dropout, **sp)

    def forward(self, x):
        return self.dropout(self.dense_2(self.inner_dropout(self.dense_1(x))))


class _Recompute(torch.autograd.Function):
    """Activation checkpointing of one block (reference: ``torch.utils.checkpoint`` per block, gpt2.py:190-194,
    opt.py:221-224, vit.py:201-205): the forward keeps only the block's inputs, the backward re-runs the block.

    Two things the library routine does not do: the random streams of every process-group kind
    (``with seed(mode)`` regions, e.g. dropout on sharded activations) are rewound together with the default
    generators, so the re-run draws the same masks; and while the block is re-run
    :func:`cubework_b200.parallel.ops_1d.recomputing` is set, which lets the block's last linear layer skip its
    product and collective - nothing in the backward reads the block's output.
    """

    @staticmethod
    def forward(ctx, fn, *args):
        from ..utils.checkpoint import _rng_states
        ctx.fn = fn
        ctx.rng = _rng_states()
        ctx.autocast = {dev: (torch.is_autocast_enabled(dev), torch.get_autocast_dtype(dev)) for dev in ("cuda", "cpu")}
        ctx.is_tensor = [torch.is_tensor(a) for a in args]
        ctx.consts = [None if t else a for a, t in zip(args, ctx.is_tensor)]
        ctx.save_for_backward(*[a for a in args if torch.is_tensor(a)])
        with torch.no_grad():
            return fn(*args)

    @staticmethod
    def backward(ctx, *grads):
        from ..parallel import ops_1d
        from ..utils.checkpoint import _rng_states, _set_rng_states
        saved = iter(ctx.saved_tensors)
        args = []
        for t, c in zip(ctx.is_tensor, ctx.consts):
            if t:
                a = next(saved).detach()
                a.requires_grad_(a.is_floating_point())
                args.append(a)
            else:
                args.append(c)
        now = _rng_states()
        _set_rng_states(ctx.rng)
        try:
            with torch.enable_grad(), torch.autocast("cuda", dtype=ctx.autocast["cuda"][1], enabled=ctx.autocast["cuda"][0]), \
                    torch.autocast("cpu", dtype=ctx.autocast["cpu"][1], enabled=ctx.autocast["cpu"][0]), \
                    ops_1d.recomputing():
                out = ctx.fn(*args)
        finally:
            _set_rng_states(now)
        outs = out if isinstance(out, (tuple, list)) else (out, )
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, ) + tuple(a.grad if (torch.is_tensor(a) and a.requires_grad) else None for a in args)


def maybe_checkpoint(fn, enabled, *args):
    if enabled and torch.is_grad_enabled() and any(torch.is_tensor(a) and a.requires_grad for a in args):
        return _Recompute.apply(fn, *args)
    return fn(*args)


def mark_block_output(linear):
    """Declare that the output of ``linear`` (a façade ``Linear``) only leaves its checkpointed block through
    value-free operations (dropout, residual add), so a re-run of the block for its gradients may skip the product."""
    inner = getattr(linear, "linear", linear)
    inner.output_unused_in_recompute = True


def key_bias_from_mask(attention_mask, dtype=torch.float32):
    """``[B, T]`` mask of 1 (keep) / 0 (pad) -> additive bias over key positions, or None."""
    if attention_mask is None:
        return None
    m = cube_nn.partition_batch(attention_mask.view(attention_mask.shape[0], -1))
    return (1.0 - m.to(dtype)) * -10000.0


def normal_init(std):
    return cube_nn.init.normal_(std=std)
