"""1D tensor-parallel layers.

Parity: cubework/module/parallel_1d/module.py:25-515 — ``Linear1D`` (column when the incoming
activation is replicated, row when it is sharded; decided from ``env.parallel_input_1d`` at
construction, :38-58), ``Linear1D_Col`` (W ``[out/n, in]``, b ``[out/n]``), ``Linear1D_Row``
(W ``[out, in/n]``, b ``[out]`` broadcast from group rank 0), ``LayerNorm1D``, ``Classifier1D``
(W ``[C, in/n]``), ``VocabParallelClassifier1D`` (W ``[C/n, in]``), ``Embedding1D`` (W ``[V, H/n]`` +
all-gather), ``VocabParallelEmbedding1D`` (W ``[V/n, H]``, masked lookup + all-reduce),
``Dropout1D``, ``PatchEmbedding1D`` (replicated).

The forward passes call :func:`~cubework_b200.parallel.ops_1d.linear_1d`, so GEMM and all-reduce
are one kernel on CUDA.  ``activation=`` fuses bias + GELU/ReLU into the column GEMM's epilogue.

Extension (no counterpart in the reference): ``sequence_parallel=True`` keeps the activations *between*
column/row pairs sharded along their leading dimension (rows of tokens) instead of replicated.  A column
linear then starts with an all-gather of rows and a row linear ends with a reduce-scatter of rows - the same
bytes on the wire as the all-reduce they replace - and layer norm, residual adds and dropout in between
touch ``1/n`` of the rows.  The default (``False``) keeps the reference's replicated semantics.
"""
import math
from typing import Callable

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn import Parameter

from ..global_vars import env
from ..utils.common import seed
from . import init
from .collective import broadcast
from .common import set_tensor_parallel_attribute_by_partition as _stamp
from .functional import add_layer_norm, layer_norm, masked_embedding
from .mesh import pm
from .ops_1d import (gather_forward_split_backward, get_parallel_input, linear_1d, linear_1d_rows,
                     mark_partial_grad, reduce_input, reduce_scatter_rows, set_parallel_input, skip_product,
                     split_forward_gather_backward)
from .std import PatchEmbeddingSTD

_W_INIT = init.kaiming_uniform_(a=math.sqrt(5))
_B_INIT = init.xavier_uniform_(a=1, scale=1)


def _div(a, n, what):
    if a % n != 0:
        raise ValueError(f"{what} ({a}) is not divisible by the 1D group size ({n})")
    return a // n


class Linear1D_Col(nn.Module):
    """``Y_local = X W_local^T + b_local``; input replicated, output sharded on the last dim."""

    def __init__(self, in_features, out_features, bias=True, gather_output=False, skip_bias_add=False,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT, activation=None,
                 sequence_parallel=False):
        super().__init__()
        if skip_bias_add and not bias:
            raise ValueError("cannot skip bias addition if bias is None")
        self.in_features, self.out_features = in_features, out_features
        self.gather_output, self.skip_bias_add, self.activation = gather_output, skip_bias_add, activation
        self.sequence_parallel = sequence_parallel
        n = pm.PARALLEL_1D.world_size
        self.out_features_per_partition = _div(out_features, n, "out_features")
        self.weight = Parameter(torch.empty(self.out_features_per_partition, in_features))
        self.bias = Parameter(torch.empty(self.out_features_per_partition)) if bias else None
        with seed(pm.PARALLEL_1D):
            weight_initializer(self.weight, fan_in=in_features, fan_out=out_features)
            if bias:
                bias_initializer(self.bias, fan_in=in_features)
        _stamp(self.weight, n, [(0, "PARALLEL_1D")])
        if bias:
            _stamp(self.bias, n, [(0, "PARALLEL_1D")])
        set_parallel_input(True)

    def forward(self, x):
        b = None if self.skip_bias_add else self.bias
        if self.sequence_parallel:      # x holds this rank's rows; the output has all rows
            y = linear_1d_rows(x, self.weight, b, pm.PARALLEL_1D, "gather", act=self.activation)
        else:
            y = linear_1d(x, self.weight, b, pm.PARALLEL_1D, reduce_bwd=True, act=self.activation)
        if self.gather_output:
            y = gather_forward_split_backward(y, pm.PARALLEL_1D, dim=-1)
        return (y, self.bias) if self.skip_bias_add else y


class Linear1D_Row(nn.Module):
    """``Y = sum_ranks(X_local W_local^T) + b``; input sharded on the last dim, output replicated."""

    def __init__(self, in_features, out_features, bias=True, parallel_input=True, skip_bias_add=False,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT,
                 sequence_parallel=False):
        super().__init__()
        if skip_bias_add and not bias:
            raise ValueError("cannot skip bias addition if bias is None")
        self.in_features, self.out_features = in_features, out_features
        self.parallel_input, self.skip_bias_add = parallel_input, skip_bias_add
        self.sequence_parallel = sequence_parallel
        n = pm.PARALLEL_1D.world_size
        self.input_size_per_partition = _div(in_features, n, "in_features")
        self.weight = Parameter(torch.empty(out_features, self.input_size_per_partition))
        self.bias = Parameter(torch.empty(out_features)) if bias else None
        with seed(pm.PARALLEL_1D):
            weight_initializer(self.weight, fan_in=in_features, fan_out=out_features)
            if bias:
                bias_initializer(self.bias, fan_in=in_features)
        if bias:
            with torch.no_grad():
                broadcast(self.bias.data, pm.PARALLEL_1D.rank_by_idx(0), pm.PARALLEL_1D)
            if sequence_parallel:       # added to this rank's rows only
                mark_partial_grad(self.bias)
        _stamp(self.weight, n, [(-1, "PARALLEL_1D")])
        set_parallel_input(False)

    def forward(self, x):
        if not self.parallel_input:
            x = split_forward_gather_backward(x, pm.PARALLEL_1D, dim=-1)
        b = None if self.skip_bias_add else self.bias
        skip = skip_product(self)
        if self.sequence_parallel:      # the output keeps this rank's rows of the sum
            y = linear_1d_rows(x, self.weight, b, pm.PARALLEL_1D, "scatter", skip=skip)
        else:
            y = linear_1d(x, self.weight, b, pm.PARALLEL_1D, reduce_fwd=True, skip=skip)
        return (y, self.bias) if self.skip_bias_add else y


class Linear1D(nn.Module):

    def __init__(self, in_features, out_features, bias=True, gather_output=False, skip_bias_add=False,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT, activation=None,
                 sequence_parallel=False):
        super().__init__()
        parallel_input = get_parallel_input()
        if not parallel_input:
            self.linear = Linear1D_Col(in_features, out_features, bias=bias, gather_output=gather_output,
                                       skip_bias_add=skip_bias_add, weight_initializer=weight_initializer,
                                       bias_initializer=bias_initializer, activation=activation,
                                       sequence_parallel=sequence_parallel)
        else:
            if activation is not None:
                raise ValueError("a fused activation needs a column-parallel (replicated-input) linear")
            self.linear = Linear1D_Row(in_features, out_features, bias=bias, parallel_input=parallel_input,
                                       skip_bias_add=skip_bias_add, weight_initializer=weight_initializer,
                                       bias_initializer=bias_initializer, sequence_parallel=sequence_parallel)

    def forward(self, *args, **kwargs):
        return self.linear(*args, **kwargs)

    weight = property(lambda self: self.linear.weight)
    bias = property(lambda self: self.linear.bias)


class LayerNorm1D(nn.Module):
    """Replicated layer norm (activations between 1D blocks are replicated).  With ``sequence_parallel`` it is
    applied to this rank's rows only and its parameter gradients are completed over the group afterwards."""

    def __init__(self, normalized_shape: int, eps=1e-05, sequence_parallel=False):
        super().__init__()
        self.normalized_shape, self.eps = normalized_shape, eps
        self.weight = Parameter(torch.ones(normalized_shape))
        self.bias = Parameter(torch.zeros(normalized_shape))
        if sequence_parallel:
            mark_partial_grad(self.weight)
            mark_partial_grad(self.bias)

    def forward(self, x, residual=None):
        """``LN(x)``; with ``residual``: ``(x + residual, LN(x + residual))`` from one kernel."""
        if residual is not None:
            return add_layer_norm(x, residual, self.weight, self.bias, self.eps)
        return layer_norm(x, self.weight, self.bias, self.eps)


class Classifier1D(nn.Module):
    """``logits = sum_ranks(X_local W_local^T) + b`` with W ``[C, in/n]`` (optionally a tied weight)."""

    def __init__(self, in_features, num_classes, weight: Parameter = None, bias=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT):
        super().__init__()
        self.in_features, self.num_classes = in_features, num_classes
        self.parallel_input = get_parallel_input()
        n = pm.PARALLEL_1D.world_size
        self.input_size_per_partition = _div(in_features, n, "in_features")
        self.has_weight = weight is None
        self.weight = weight if weight is not None else Parameter(
            torch.empty(num_classes, self.input_size_per_partition))
        self.bias = Parameter(torch.empty(num_classes)) if bias else None
        with seed(pm.PARALLEL_1D):
            if self.has_weight:
                weight_initializer(self.weight, fan_in=in_features, fan_out=num_classes)
            if bias:
                bias_initializer(self.bias, fan_in=in_features)
        if bias:
            with torch.no_grad():
                broadcast(self.bias.data, pm.PARALLEL_1D.rank_by_idx(0), pm.PARALLEL_1D)
        if self.has_weight:
            _stamp(self.weight, pm.TENSOR.world_size, [(-1, "PARALLEL_1D")])
        set_parallel_input(False)
        env.vocab_parallel = False

    def forward(self, x):
        if not self.parallel_input:
            x = split_forward_gather_backward(x, pm.PARALLEL_1D, dim=-1)
        return linear_1d(x, self.weight, self.bias, pm.PARALLEL_1D, reduce_fwd=True)


class VocabParallelClassifier1D(nn.Module):
    """``logits_local = X W_local^T + b_local`` with W ``[C/n, in]``; output sharded over classes."""

    def __init__(self, in_features, num_classes, weight: Parameter = None, bias=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT,
                 sequence_parallel=False):
        super().__init__()
        self.in_features, self.num_classes = in_features, num_classes
        self.parallel_input = get_parallel_input()
        self.sequence_parallel = sequence_parallel
        n = pm.PARALLEL_1D.world_size
        self.num_classes_per_partition = _div(num_classes, n, "num_classes")
        self.has_weight = weight is None
        self.weight = weight if weight is not None else Parameter(
            torch.empty(self.num_classes_per_partition, in_features))
        self.bias = Parameter(torch.empty(self.num_classes_per_partition)) if bias else None
        with seed(pm.PARALLEL_1D):
            if self.has_weight:
                weight_initializer(self.weight, fan_in=in_features, fan_out=num_classes)
            if bias:
                bias_initializer(self.bias, fan_in=in_features)
        if self.has_weight:
            _stamp(self.weight, n, [(0, "PARALLEL_1D")])
        if bias:
            _stamp(self.bias, n, [(0, "PARALLEL_1D")])
        set_parallel_input(False)
        env.vocab_parallel = True

    def forward(self, x):
        if self.sequence_parallel:      # x holds this rank's rows; the logits cover all rows, local classes
            return linear_1d_rows(x, self.weight, self.bias, pm.PARALLEL_1D, "gather")
        return linear_1d(x, self.weight, self.bias, pm.PARALLEL_1D, reduce_bwd=True)


class Embedding1D(nn.Module):
    """Hidden-sharded table W ``[V, H/n]``; the lookups are all-gathered on the last dim."""

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None,
                 weight_initializer: Callable = init.normal_(), *args, **kwargs):
        super().__init__()
        self.num_embeddings, self.embed_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        n = pm.PARALLEL_1D.world_size
        self.weight = Parameter(torch.empty(num_embeddings, _div(embedding_dim, n, "embedding_dim")))
        with seed(pm.PARALLEL_1D):
            weight_initializer(self.weight, fan_in=num_embeddings, fan_out=embedding_dim)
            if padding_idx is not None:
                with torch.no_grad():
                    self.weight[padding_idx].fill_(0)
        _stamp(self.weight, n, [(-1, "PARALLEL_1D")])
        set_parallel_input(False)

    def forward(self, ids):
        out = masked_embedding(ids, self.weight, 0)
        return gather_forward_split_backward(out, pm.PARALLEL_1D, dim=-1)


class VocabParallelEmbedding1D(nn.Module):
    """Vocabulary-sharded table W ``[V/n, H]``; foreign ids give zeros, then an all-reduce."""

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None,
                 weight_initializer: Callable = init.normal_(), sequence_parallel=False, *args, **kwargs):
        super().__init__()
        self.num_embeddings, self.embed_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.sequence_parallel = sequence_parallel
        n, r = pm.PARALLEL_1D.world_size, pm.PARALLEL_1D.local_rank
        self.num_embeddings_per_partition = _div(num_embeddings, n, "num_embeddings")
        self.vocab_start_index = r * self.num_embeddings_per_partition
        self.vocab_end_index = self.vocab_start_index + self.num_embeddings_per_partition
        self.weight = Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim))
        with seed(pm.PARALLEL_1D):
            weight_initializer(self.weight, fan_in=num_embeddings, fan_out=embedding_dim)
            if padding_idx is not None and self.vocab_start_index <= padding_idx < self.vocab_end_index:
                with torch.no_grad():
                    self.weight[padding_idx - self.vocab_start_index].fill_(0)
        _stamp(self.weight, n, [(0, "PARALLEL_1D")])
        set_parallel_input(False)
        env.vocab_parallel = True

    def forward(self, ids):
        out = masked_embedding(ids, self.weight, self.vocab_start_index)
        if self.sequence_parallel:      # every rank looks all ids up; each keeps its rows of the sum
            return reduce_scatter_rows(out, pm.PARALLEL_1D)
        return reduce_input(out, pm.PARALLEL_1D)


class Dropout1D(nn.Module):
    """Dropout that draws from the per-rank TENSOR stream when its input is sharded, and from the
    shared default stream when it is replicated (parallel_1d/module.py:458-472)."""

    def __init__(self, p: float = 0.5, inplace: bool = False, sequence_parallel=False):
        super().__init__()
        self.parallel_input = get_parallel_input() or sequence_parallel   # row shards differ per rank too
        self.p, self.inplace = p, inplace

    def forward(self, x):
        if self.p == 0.0 or not self.training:
            return x
        if self.parallel_input:
            with seed(pm.TENSOR):
                return F.dropout(x, self.p, self.training, self.inplace)
        return F.dropout(x, self.p, self.training, self.inplace)


class PatchEmbedding1D(nn.Module):
    """Replicated patch embedding (every rank computes the full embedding)."""

    def __init__(self, img_size, patch_size, in_chans, embed_size, flatten=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT,
                 position_embed_initializer: Callable = init.zeros_()):
        super().__init__()
        self.embed = PatchEmbeddingSTD(img_size, patch_size, in_chans, embed_size, flatten=flatten,
                                       weight_initializer=weight_initializer, bias_initializer=bias_initializer,
                                       position_embed_initializer=position_embed_initializer)

    def forward(self, *args, **kwargs):
        return self.embed(*args, **kwargs)

    weight = property(lambda self: self.embed.weight)
    bias = property(lambda self: self.embed.bias)
    cls_token = property(lambda self: self.embed.cls_token)
    pos_embed = property(lambda self: self.embed.pos_embed)
