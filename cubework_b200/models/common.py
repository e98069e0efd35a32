"""Pieces shared by the GPT-2 / OPT / ViT model families: the self-attention core over a packed QKV
projection, the transformer MLP, activation checkpointing and the data-parallel wrapper choice."""
import math

import torch
import torch.nn as nn
import torch.utils.checkpoint as ckpt

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


def maybe_checkpoint(fn, enabled, *args):
    if enabled and torch.is_grad_enabled():
        return ckpt.checkpoint(fn, *args, use_reentrant=False)
    return fn(*args)


def key_bias_from_mask(attention_mask, dtype=torch.float32):
    """``[B, T]`` mask of 1 (keep) / 0 (pad) -> additive bias over key positions, or None."""
    if attention_mask is None:
        return None
    m = cube_nn.partition_batch(attention_mask.view(attention_mask.shape[0], -1))
    return (1.0 - m.to(dtype)) * -10000.0


def normal_init(std):
    return cube_nn.init.normal_(std=std)
