"""User-facing layers that dispatch on the active tensor-parallel mode.

Parity: cubework/module/modules.py:19-296 — ``Linear``, ``LayerNorm``, ``Embedding``, ``Classifier``,
``PatchEmbedding``, ``Dropout``, ``DropPath``, ``partition_batch``.  ``Classifier`` builds the
vocab-parallel variant when the last embedding/classifier set ``env.vocab_parallel`` (:158-176);
``Dropout`` draws from the per-rank TENSOR stream in 2D/3D (:291-296).

Extension: ``Linear(..., activation="gelu"|"relu")`` fuses bias + activation into the GEMM epilogue
(1D column-parallel and unsharded linears); other modes apply the activation after the layer.

Extension: ``sequence_parallel=True`` on ``Linear`` / ``LayerNorm`` / ``Embedding`` / ``Classifier`` /
``Dropout`` selects, in 1D mode, the layout in which activations between column/row linear pairs are
sharded along their leading dimension (see :mod:`cubework_b200.parallel.layers_1d`).  The other modes
shard their activations already and ignore the flag.  :func:`sequence_parallel_size` tells a model by how
much the leading dimension shrinks.
"""
import math
from typing import Callable

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..global_vars import env
from ..utils.common import seed
from . import init
from .common import get_tensor_parallel_mode
from .functional import add_layer_norm, layer_norm, local_linear, masked_embedding
from .layers_1d import (Classifier1D, Dropout1D, Embedding1D, LayerNorm1D, Linear1D, PatchEmbedding1D,
                        VocabParallelClassifier1D, VocabParallelEmbedding1D)
from .layers_2d import (Classifier2D, Embedding2D, LayerNorm2D, Linear2D, PatchEmbedding2D,
                        VocabParallelClassifier2D, VocabParallelEmbedding2D)
from .layers_3d import (Classifier3D, Embedding3D, LayerNorm3D, Linear3D, PatchEmbedding3D,
                        VocabParallelClassifier3D, VocabParallelEmbedding3D)
from .mesh import pm
from .ops_2d import split_batch_2d
from .ops_3d import split_batch_3d
from .std import ClassifierSTD, DropPath, PatchEmbeddingSTD

_W_INIT = init.kaiming_uniform_(a=math.sqrt(5))
_B_INIT = init.xavier_uniform_(a=1, scale=1)

_parallel_layernorm = {"1d": LayerNorm1D, "2d": LayerNorm2D, "3d": LayerNorm3D}


def _linear_1d(*args, **kwargs):
    """Column or row layer directly (no ``Linear1D`` wrapper), so parameter names are the same in every mode."""
    return Linear1D(*args, **kwargs).linear


def _patch_embedding_1d(*args, **kwargs):
    return PatchEmbedding1D(*args, **kwargs).embed


_parallel_linear = {"1d": _linear_1d, "2d": Linear2D, "3d": Linear3D}
_parallel_classifier = {None: ClassifierSTD, "1d": Classifier1D, "2d": Classifier2D, "3d": Classifier3D}
_vocab_parallel_classifier = {"1d": VocabParallelClassifier1D, "2d": VocabParallelClassifier2D,
                              "3d": VocabParallelClassifier3D}
_parallel_embedding = {"1d": Embedding1D, "2d": Embedding2D, "3d": Embedding3D}
_vocab_parallel_embedding = {"1d": VocabParallelEmbedding1D, "2d": VocabParallelEmbedding2D,
                             "3d": VocabParallelEmbedding3D}
_parallel_patchembedding = {None: PatchEmbeddingSTD, "1d": _patch_embedding_1d, "2d": PatchEmbedding2D,
                            "3d": PatchEmbedding3D}
_parallel_split_batch = {"2d": split_batch_2d, "3d": split_batch_3d}

__all__ = ["Linear", "LayerNorm", "Embedding", "Classifier", "PatchEmbedding", "Dropout", "DropPath",
           "partition_batch", "sequence_parallel_size", "scatter_rows", "gather_rows", "mark_partial_grad",
           "sum_grad_over_rows"]


def sequence_parallel_size():
    """Number of row shards that ``sequence_parallel=True`` layers use: the 1D group size, else 1."""
    if get_tensor_parallel_mode() == "1d" and pm.PARALLEL_1D.is_initialized():
        return pm.PARALLEL_1D.world_size
    return 1


def scatter_rows(x):
    """This rank's block of the leading dimension of a replicated tensor (identity outside 1D mode)."""
    from .ops_1d import scatter_rows as _s
    return _s(x, pm.PARALLEL_1D) if sequence_parallel_size() > 1 else x


def gather_rows(x):
    """Inverse of :func:`scatter_rows`."""
    from .ops_1d import gather_rows as _g
    return _g(x, pm.PARALLEL_1D) if sequence_parallel_size() > 1 else x


def sum_grad_over_rows(x):
    """Identity; in backward the gradient is summed over the 1D group.  For a replicated tensor (a position
    table's rows, a broadcast bias) that is consumed by row-sharded computation and produced by sharded
    parameters, where completing the parameter gradient afterwards would mix different shards."""
    from .ops_1d import reduce_grad
    return reduce_grad(x, pm.PARALLEL_1D) if sequence_parallel_size() > 1 else x


def mark_partial_grad(param):
    """Declare that ``param`` is replicated but applied to row-sharded activations (1D ``sequence_parallel``), so
    its gradient must be summed over the group after the backward pass (the ``Trainer`` does it)."""
    from .ops_1d import mark_partial_grad as _m
    if sequence_parallel_size() > 1:
        _m(param)


def _sp_kwargs(mode, sequence_parallel):
    return dict(sequence_parallel=True) if (sequence_parallel and mode == "1d") else {}


def partition_batch(input_):
    """This rank's slice of a batch (tensor, tuple/list or dict of tensors); identity for 1D / none."""
    split = _parallel_split_batch.get(get_tensor_parallel_mode())
    if split is None:
        return input_
    if isinstance(input_, dict):
        return {k: split(v) for k, v in input_.items()}
    if isinstance(input_, (tuple, list)):
        return type(input_)(split(x) for x in input_)
    return split(input_)


class _PlainLinear(nn.Module):
    """Unsharded linear on this package's GEMM (used when no tensor parallelism is active)."""

    def __init__(self, in_features, out_features, bias, activation=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.empty(out_features)) if bias else None
        self.activation = activation

    def forward(self, x):
        return local_linear(x, self.weight, self.bias, True, self.activation)


class _PlainLayerNorm(nn.Module):

    def __init__(self, normalized_shape, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(normalized_shape))
        self.bias = nn.Parameter(torch.zeros(normalized_shape))
        self.eps = eps

    def forward(self, x, residual=None):
        if residual is not None:
            return add_layer_norm(x, residual, self.weight, self.bias, self.eps)
        return layer_norm(x, self.weight, self.bias, self.eps)


class _PlainEmbedding(nn.Module):

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim))
        self.padding_idx = padding_idx

    def forward(self, ids):
        return masked_embedding(ids, self.weight, 0)


def _to(module, dtype):
    return module.to(dtype) if dtype is not None else module


class LayerNorm(nn.Module):

    def __init__(self, normalized_shape: int, eps=1e-05, dtype=None, sequence_parallel=False):
        super().__init__()
        mode = get_tensor_parallel_mode()
        norm = _PlainLayerNorm(normalized_shape, eps) if mode is None else \
            _parallel_layernorm[mode](normalized_shape, eps=eps, **_sp_kwargs(mode, sequence_parallel))
        self._fused_residual = mode in (None, "1d")
        self.norm = _to(norm, dtype)

    def forward(self, x, residual=None):
        """``LN(x)``.  With ``residual`` the layer returns ``(x + residual, LN(x + residual))``: unsharded and 1D norms
        compute both in one kernel, the 2D / 3D norms add first."""
        if residual is None:
            return self.norm(x)
        if self._fused_residual:
            return self.norm(x, residual)
        total = x + residual
        return total, self.norm(total)

    weight = property(lambda self: self.norm.weight)
    bias = property(lambda self: self.norm.bias)


class Linear(nn.Module):

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=None,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT, activation=None,
                 sequence_parallel=False, **kwargs):
        super().__init__()
        mode = get_tensor_parallel_mode()
        kwargs.update(_sp_kwargs(mode, sequence_parallel))
        self._post_act = None
        if mode is None:
            lin = _PlainLinear(in_features, out_features, bias, activation)
            weight_initializer(lin.weight, fan_in=in_features, fan_out=out_features)
            if bias:
                bias_initializer(lin.bias, fan_in=in_features)
        else:
            if activation is not None:
                if mode == "1d" and not env.parallel_input_1d and not kwargs.get("gather_output", False) \
                        and not kwargs.get("skip_bias_add", False):
                    kwargs["activation"] = activation
                else:
                    self._post_act = activation
            lin = _parallel_linear[mode](in_features, out_features, bias=bias, weight_initializer=weight_initializer,
                                         bias_initializer=bias_initializer, **kwargs)
        self.linear = _to(lin, dtype)

    def forward(self, *args, **kwargs):
        y = self.linear(*args, **kwargs)
        if self._post_act is not None:
            fn = F.gelu if self._post_act == "gelu" else F.relu
            y = (fn(y[0]), y[1]) if isinstance(y, tuple) else fn(y)
        return y

    weight = property(lambda self: self.linear.weight)
    bias = property(lambda self: self.linear.bias)


class Classifier(nn.Module):

    def __init__(self, in_features: int, num_classes: int, weight: nn.Parameter = None, bias: bool = True,
                 dtype=None, weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT,
                 sequence_parallel=False):
        super().__init__()
        mode = get_tensor_parallel_mode()
        vocab_parallel = env.vocab_parallel and mode is not None
        table = _vocab_parallel_classifier if vocab_parallel else _parallel_classifier
        if sequence_parallel and mode == "1d" and not vocab_parallel:
            raise ValueError("sequence_parallel needs the vocab-parallel classifier in 1D mode")
        lin = table[mode](in_features, num_classes, weight=weight, bias=bias, weight_initializer=weight_initializer,
                          bias_initializer=bias_initializer, **_sp_kwargs(mode, sequence_parallel))
        self.linear = _to(lin, dtype)

    def forward(self, *args, **kwargs):
        return self.linear(*args, **kwargs)

    weight = property(lambda self: self.linear.weight)
    bias = property(lambda self: self.linear.bias)


class Embedding(nn.Module):

    def __init__(self, num_embeddings: int, embedding_dim: int, vocab_parallel: bool = False,
                 padding_idx: int = None, dtype=None, weight_initializer: Callable = init.normal_(),
                 sequence_parallel=False, *args, **kwargs):
        super().__init__()
        mode = get_tensor_parallel_mode()
        if vocab_parallel:
            kwargs.update(_sp_kwargs(mode, sequence_parallel))
        if mode is None:
            emb = _PlainEmbedding(num_embeddings, embedding_dim, padding_idx)
            weight_initializer(emb.weight, fan_in=num_embeddings, fan_out=embedding_dim)
            if padding_idx is not None:
                with torch.no_grad():
                    emb.weight[padding_idx].fill_(0)
        else:
            table = _vocab_parallel_embedding if vocab_parallel else _parallel_embedding
            emb = table[mode](num_embeddings, embedding_dim, padding_idx=padding_idx,
                              weight_initializer=weight_initializer, *args, **kwargs)
        self.embed = _to(emb, dtype)

    def forward(self, *args, **kwargs):
        return self.embed(*args, **kwargs)

    weight = property(lambda self: self.embed.weight)


class PatchEmbedding(nn.Module):

    def __init__(self, img_size: int, patch_size: int, in_chans: int, embed_size: int, flatten: bool = True,
                 dtype=None, weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT,
                 position_embed_initializer: Callable = init.zeros_()):
        super().__init__()
        emb = _parallel_patchembedding[get_tensor_parallel_mode()](
            img_size, patch_size, in_chans, embed_size, flatten=flatten, weight_initializer=weight_initializer,
            bias_initializer=bias_initializer, position_embed_initializer=position_embed_initializer)
        self.embed = _to(emb, dtype)

    def forward(self, *args, **kwargs):
        return self.embed(*args, **kwargs)

    weight = property(lambda self: self.embed.weight)
    bias = property(lambda self: self.embed.bias)
    cls_token = property(lambda self: self.embed.cls_token)
    pos_embed = property(lambda self: self.embed.pos_embed)


class Dropout(nn.Module):

    def __init__(self, p: float = 0.5, inplace: bool = False, sequence_parallel=False):
        super().__init__()
        self.tensor_parallel = get_tensor_parallel_mode()
        self.p = p
        self.drop = Dropout1D(p, inplace, **_sp_kwargs("1d", sequence_parallel)) if self.tensor_parallel == "1d" \
            else nn.Dropout(p, inplace)

    def forward(self, x):
        if self.p == 0.0 or not self.training:
            return x
        if self.tensor_parallel in (None, "1d"):
            return self.drop(x)
        with seed(pm.TENSOR):
            return self.drop(x)
