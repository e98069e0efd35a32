"""2D (SUMMA) tensor-parallel layers on a ``q x q`` grid.

Parity: cubework/module/parallel_2d/module.py:25-506 — ``Linear2D`` (W ``[in/q, out/q]``, b
``[out/q^2]``), ``LayerNorm2D`` (gamma, beta ``[H/q^2]``), ``PatchEmbedding2D`` (all parameters split
``q^2`` ways on the embedding dim), ``Embedding2D`` (W ``[V, H/q^2]``), ``VocabParallelEmbedding2D``
(W ``[V/q, H/q]``), ``Classifier2D`` (W ``[C, H/q^2]``, replicated bias), ``VocabParallelClassifier2D``
(W ``[C/q, H/q]``, b ``[C/q^2]``).  Activations are ``[B/q, S, H/q]``: batch split by grid row,
hidden by grid column.
"""
import math
from typing import Callable

import torch
import torch.nn as nn
from torch.nn import Parameter

from ..global_vars import env
from ..utils.common import seed
from . import init
from .collective import broadcast
from .common import set_tensor_parallel_attribute_by_partition as _stamp
from .common import to_2tuple
from .functional import masked_embedding
from .mesh import pm
from .ops_2d import (add_bias_2d, all_gather_tensor_2d, assert_summa_initialization, classifier_2d,
                     get_summa_dim_from_env, layer_norm_sharded, reduce_scatter_tensor_2d, split_batch_2d,
                     summa_AB, summa_ABT)
from .std import assemble_tokens, patchify_linear

_W_INIT = init.kaiming_uniform_(a=math.sqrt(5))
_B_INIT = init.xavier_uniform_(a=1, scale=1)
ROW, COL = "PARALLEL_2D_ROW", "PARALLEL_2D_COL"


class _Grid2D(nn.Module):

    def _grid(self):
        assert_summa_initialization()
        self.summa_dim = get_summa_dim_from_env()
        self.row_rank = pm.PARALLEL_2D_COL.local_rank
        self.col_rank = pm.PARALLEL_2D_ROW.local_rank
        return self.summa_dim

    @staticmethod
    def _div(a, n, what):
        if a % n != 0:
            raise ValueError(f"{what} ({a}) is not divisible by {n}")
        return a // n


class Linear2D(_Grid2D):

    def __init__(self, in_features, out_features, bias=True, skip_bias_add=False,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT):
        super().__init__()
        self.in_features, self.out_features, self.skip_bias_add = in_features, out_features, skip_bias_add
        q = self._grid()
        self.input_size_per_partition = self._div(in_features, q, "in_features")
        self.hidden_size_per_partition = self._div(out_features, q, "out_features")
        self.weight = Parameter(torch.empty(self.input_size_per_partition, self.hidden_size_per_partition))
        if bias:
            self.bias = Parameter(torch.empty(self._div(out_features, q * q, "out_features")))
        else:
            self.register_parameter("bias", None)
        with seed(pm.TENSOR):
            weight_initializer(self.weight, fan_in=in_features, fan_out=out_features)
            if bias:
                bias_initializer(self.bias, fan_in=in_features)
        _stamp(self.weight, q * q, [(0, COL), (-1, ROW)])
        self.weight.STORED_IN_OUT = True   # [in, out]; checkpoints canonicalise to [out, in]
        if bias:
            _stamp(self.bias, q * q, [(-1, ROW), (-1, COL)])

    def forward(self, x):
        out_shape = x.shape[:-1] + (self.hidden_size_per_partition, )
        y = summa_AB(x, self.weight, self.summa_dim, out_shape, pm.PARALLEL_2D_ROW, pm.PARALLEL_2D_COL)
        if self.bias is None:
            return y
        if self.skip_bias_add:
            return y, add_bias_2d(None, self.bias, pm.PARALLEL_2D_ROW, pm.PARALLEL_2D_COL, True)
        return add_bias_2d(y, self.bias, pm.PARALLEL_2D_ROW, pm.PARALLEL_2D_COL, False)


class LayerNorm2D(_Grid2D):

    def __init__(self, normalized_shape: int, eps: float = 1e-05):
        super().__init__()
        self.normalized_shape, self.variance_epsilon = normalized_shape, eps
        q = self._grid()
        self.partitioned_partition = self._div(normalized_shape, q * q, "normalized_shape")
        self.weight = Parameter(torch.ones(self.partitioned_partition))
        self.bias = Parameter(torch.zeros(self.partitioned_partition))
        _stamp(self.weight, q * q, [(-1, ROW), (-1, COL)])
        _stamp(self.bias, q * q, [(-1, ROW), (-1, COL)])

    def forward(self, x):
        gamma = all_gather_tensor_2d(self.weight, -1, pm.PARALLEL_2D_COL)
        beta = all_gather_tensor_2d(self.bias, -1, pm.PARALLEL_2D_COL)
        # gradients of the gathered gamma/beta are summed over the batch shards by the gather's
        # reduce-scatter, so no extra reduction group is needed here
        return layer_norm_sharded(x, gamma, beta, self.variance_epsilon, self.normalized_shape, pm.PARALLEL_2D_ROW)


class PatchEmbedding2D(_Grid2D):

    def __init__(self, img_size, patch_size, in_chans, embed_size, flatten=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT,
                 position_embed_initializer: Callable = init.zeros_()):
        super().__init__()
        self.img_size, self.patch_size = to_2tuple(img_size), to_2tuple(patch_size)
        q = self._grid()
        self.grid_size = (self.img_size[0] // self.patch_size[0], self.img_size[1] // self.patch_size[1])
        self.num_patches = self.grid_size[0] * self.grid_size[1]
        self.flatten, self.embed_size = flatten, embed_size
        e = self.embed_size_per_partition = self._div(embed_size, q * q, "embed_size")
        self.weight = Parameter(torch.empty(e, in_chans, *self.patch_size))
        self.bias = Parameter(torch.empty(e))
        self.cls_token = Parameter(torch.zeros(1, 1, e))
        self.pos_embed = Parameter(torch.zeros(1, self.num_patches + 1, e))
        with seed(pm.TENSOR):
            fan_in = in_chans * self.patch_size[0] * self.patch_size[1]
            weight_initializer(self.weight, fan_in=fan_in, fan_out=embed_size)
            bias_initializer(self.bias, fan_in=fan_in)
            position_embed_initializer(self.pos_embed)
        for p in (self.weight, self.bias):
            _stamp(p, q * q, [(0, ROW), (0, COL)])
        for p in (self.cls_token, self.pos_embed):
            _stamp(p, q * q, [(-1, ROW), (-1, COL)])

    def forward(self, images):
        images = split_batch_2d(images)
        _, _, H, W = images.shape
        assert (H, W) == tuple(self.img_size), \
            f"Input image size ({H}*{W}) doesn't match model ({self.img_size[0]}*{self.img_size[1]})."
        col = pm.PARALLEL_2D_COL
        weight = all_gather_tensor_2d(self.weight, 0, col)
        bias = all_gather_tensor_2d(self.bias, 0, col)
        cls_token = all_gather_tensor_2d(self.cls_token, -1, col)
        pos_embed = all_gather_tensor_2d(self.pos_embed, -1, col)
        return assemble_tokens(patchify_linear(images, weight, bias, self.patch_size), cls_token, pos_embed)


class Embedding2D(_Grid2D):

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None,
                 weight_initializer: Callable = init.normal_(), *args, **kwargs):
        super().__init__()
        q = self._grid()
        self.num_embeddings, self.embed_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.weight = Parameter(torch.empty(num_embeddings, self._div(embedding_dim, q * q, "embedding_dim")))
        with seed(pm.TENSOR):
            weight_initializer(self.weight, fan_in=num_embeddings, fan_out=embedding_dim)
            if padding_idx is not None:
                with torch.no_grad():
                    self.weight[padding_idx].fill_(0)
        _stamp(self.weight, q * q, [(-1, ROW), (-1, COL)])

    def forward(self, ids):
        ids = split_batch_2d(ids)
        weight = all_gather_tensor_2d(self.weight, -1, pm.PARALLEL_2D_COL)
        return masked_embedding(ids, weight, 0)


class VocabParallelEmbedding2D(_Grid2D):

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None,
                 weight_initializer: Callable = init.normal_(), *args, **kwargs):
        super().__init__()
        q = self._grid()
        self.num_embeddings, self.embed_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.num_embeddings_per_partition = self._div(num_embeddings, q, "num_embeddings")
        self.embed_dim_per_partition = self._div(embedding_dim, q, "embedding_dim")
        self.vocab_start_index = pm.PARALLEL_2D_COL.local_rank * self.num_embeddings_per_partition
        self.vocab_end_index = self.vocab_start_index + self.num_embeddings_per_partition
        self.weight = Parameter(torch.empty(self.num_embeddings_per_partition, self.embed_dim_per_partition))
        with seed(pm.TENSOR):
            weight_initializer(self.weight, fan_in=num_embeddings, fan_out=embedding_dim)
            if padding_idx is not None and self.vocab_start_index <= padding_idx < self.vocab_end_index:
                with torch.no_grad():
                    self.weight[padding_idx - self.vocab_start_index].fill_(0)
        _stamp(self.weight, q * q, [(-1, ROW), (0, COL)])
        env.vocab_parallel = True

    def forward(self, ids):
        partial = masked_embedding(ids, self.weight, self.vocab_start_index)
        return reduce_scatter_tensor_2d(partial, 0, pm.PARALLEL_2D_COL)


class Classifier2D(_Grid2D):

    def __init__(self, in_features, num_classes, weight: Parameter = None, bias=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT):
        super().__init__()
        self.in_features, self.num_classes = in_features, num_classes
        q = self._grid()
        self.input_size_per_partition = self._div(in_features, q * q, "in_features")
        self.has_weight = weight is None
        self.weight = weight if weight is not None else Parameter(
            torch.empty(num_classes, self.input_size_per_partition))
        self.bias = Parameter(torch.zeros(num_classes)) if bias else None
        with seed(pm.TENSOR):
            if self.has_weight:
                weight_initializer(self.weight, fan_in=in_features, fan_out=num_classes)
            if bias:
                bias_initializer(self.bias, fan_in=in_features)
        if bias:
            with torch.no_grad():
                broadcast(self.bias.data, pm.PARALLEL_2D_COL.rank_by_idx(0), pm.PARALLEL_2D_COL)
                broadcast(self.bias.data, pm.PARALLEL_2D_ROW.rank_by_idx(0), pm.PARALLEL_2D_ROW)
        if self.has_weight:
            _stamp(self.weight, q * q, [(-1, ROW), (-1, COL)])

    def forward(self, x):
        out_shape = x.shape[:-1] + (self.num_classes, )
        return classifier_2d(x, self.weight, self.bias, self.summa_dim, out_shape, pm.PARALLEL_2D_ROW,
                             pm.PARALLEL_2D_COL)


class VocabParallelClassifier2D(_Grid2D):

    def __init__(self, in_features, num_classes, weight: Parameter = None, bias=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT):
        super().__init__()
        self.in_features, self.num_classes = in_features, num_classes
        q = self._grid()
        self.input_size_per_partition = self._div(in_features, q, "in_features")
        self.output_size_per_partition = self._div(num_classes, q, "num_classes")
        self.has_weight = weight is None
        self.weight = weight if weight is not None else Parameter(
            torch.empty(self.output_size_per_partition, self.input_size_per_partition))
        self.bias = Parameter(torch.empty(self._div(num_classes, q * q, "num_classes"))) if bias else None
        with seed(pm.TENSOR):
            if self.has_weight:
                weight_initializer(self.weight, fan_in=in_features, fan_out=num_classes)
            if bias:
                bias_initializer(self.bias, fan_in=in_features)
        if self.has_weight:
            _stamp(self.weight, q * q, [(0, COL), (-1, ROW)])
        if bias:
            _stamp(self.bias, q * q, [(0, ROW), (0, COL)])
        env.vocab_parallel = True

    def forward(self, x):
        out_shape = x.shape[:-1] + (self.output_size_per_partition, )
        y = summa_ABT(x, self.weight, self.summa_dim, out_shape, pm.PARALLEL_2D_ROW, pm.PARALLEL_2D_COL)
        if self.bias is not None:
            y = add_bias_2d(y, self.bias, pm.PARALLEL_2D_ROW, pm.PARALLEL_2D_COL, False)
        return y
