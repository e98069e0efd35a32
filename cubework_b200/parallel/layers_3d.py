"""3D (cube) tensor-parallel layers on a ``d x d x d`` grid.

Parity: cubework/module/parallel_3d/module.py:22-462 — ``LayerNorm3D`` (gamma, beta ``[H/d]``, default
eps 1e-12), ``Linear3D`` (W ``[in/d, out/d^2]``, b ``[out/d]``; swaps the input/output group roles
after construction, :98), ``Classifier3D`` (W ``[C, in/d]``), ``VocabParallelClassifier3D`` (W
``[C/d^2, in/d]``, b ``[C/d]``; swaps), ``PatchEmbedding3D`` and ``Embedding3D`` (parameters ``[.., E/d]``
replicated over the input x weight plane, kept consistent by an init broadcast and a gradient
all-reduce hook), ``VocabParallelEmbedding3D`` (W ``[V/d^2, H/d]``).  Activations are
``[B/d^2, S, H/d]``.
"""
import math
from typing import Callable

import torch
import torch.nn as nn
from torch.nn import Parameter

from ..global_vars import env
from ..utils.common import seed
from . import init
from .collective import all_reduce, broadcast
from .common import set_tensor_parallel_attribute_by_partition as _stamp
from .common import split_tensor, to_2tuple
from .functional import masked_embedding
from .mesh import pm
from .ops_3d import (all_gather_weight_3d, classifier_3d, get_depth_from_env, get_input_parallel_mode,
                     get_input_x_weight_parallel_mode, get_output_parallel_mode,
                     get_output_x_weight_parallel_mode, get_weight_parallel_mode, layernorm_3d, linear_3d,
                     reduce_scatter_tensor_3d, split_batch_3d, swap_in_out_group, vocab_parallel_classifier_3d)
from .std import assemble_tokens, patchify_linear

_W_INIT = init.kaiming_uniform_(a=math.sqrt(5))
_B_INIT = init.xavier_uniform_(a=1, scale=1)


def _div(a, n, what):
    if a % n != 0:
        raise ValueError(f"{what} ({a}) is not divisible by {n}")
    return a // n


class _Cube(nn.Module):

    def _capture(self):
        """Freeze the group roles that are current while this layer is being built."""
        self.depth = get_depth_from_env()
        self.input_parallel_mode = get_input_parallel_mode()
        self.weight_parallel_mode = get_weight_parallel_mode()
        self.output_parallel_mode = get_output_parallel_mode()
        self.input_x_weight_parallel_mode = get_input_x_weight_parallel_mode()
        self.output_x_weight_parallel_mode = get_output_x_weight_parallel_mode()
        return self.depth

    def _replicate(self, params, mode):
        """Make ``params`` identical over ``mode`` now and keep their gradients summed over it."""
        for p in params:
            with torch.no_grad():
                broadcast(p.data, mode.rank_by_idx(0), mode)
            if mode.world_size > 1:
                p.register_hook(lambda g, m=mode: all_reduce(g.contiguous().clone(), m))


class LayerNorm3D(_Cube):

    def __init__(self, normalized_shape: int, eps: float = 1e-12):
        super().__init__()
        d = self._capture()
        self.normalized_shape, self.variance_epsilon = normalized_shape, eps
        self.normalized_shape_per_partition = _div(normalized_shape, d, "normalized_shape")
        self.weight = Parameter(torch.ones(self.normalized_shape_per_partition))
        self.bias = Parameter(torch.zeros(self.normalized_shape_per_partition))
        _stamp(self.weight, d, [(0, self.output_parallel_mode)])
        _stamp(self.bias, d, [(0, self.output_parallel_mode)])

    def forward(self, x):
        return layernorm_3d(x, self.weight, self.bias, self.normalized_shape, self.variance_epsilon,
                            self.input_parallel_mode, self.weight_parallel_mode, self.output_parallel_mode,
                            self.input_x_weight_parallel_mode)


class Linear3D(_Cube):

    def __init__(self, in_features, out_features, bias=True, weight_initializer: Callable = _W_INIT,
                 bias_initializer: Callable = _B_INIT):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        d = self._capture()
        self.in_features_per_partition = _div(in_features, d, "in_features")
        self.out_features_per_partition = _div(out_features, d * d, "out_features")
        self.bias_features_per_partition = _div(out_features, d, "out_features")
        self.weight = Parameter(torch.empty(self.in_features_per_partition, self.out_features_per_partition))
        self.bias = Parameter(torch.zeros(self.bias_features_per_partition)) if bias else None
        with seed(pm.TENSOR):
            weight_initializer(self.weight, fan_in=in_features, fan_out=out_features)
            if bias:
                bias_initializer(self.bias, fan_in=in_features)
        if bias:
            with torch.no_grad():
                m = self.output_x_weight_parallel_mode
                broadcast(self.bias.data, m.rank_by_idx(0), m)
        _stamp(self.weight, d**3, [(0, self.output_parallel_mode), (-1, self.input_parallel_mode),
                                   (-1, self.weight_parallel_mode)])
        self.weight.STORED_IN_OUT = True   # [in, out]; checkpoints canonicalise to [out, in]
        if bias:
            _stamp(self.bias, d, [(0, self.input_parallel_mode)])
        swap_in_out_group()

    def forward(self, x):
        return linear_3d(x, self.weight, self.bias, self.input_parallel_mode, self.weight_parallel_mode,
                         self.output_parallel_mode)


class Classifier3D(_Cube):

    def __init__(self, in_features, num_classes, weight: Parameter = None, bias=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT):
        super().__init__()
        self.in_features, self.num_classes = in_features, num_classes
        d = self._capture()
        self.in_features_per_partition = _div(in_features, d, "in_features")
        self.has_weight = weight is None
        self.weight = weight if weight is not None else Parameter(
            torch.empty(num_classes, self.in_features_per_partition))
        self.bias = Parameter(torch.zeros(num_classes)) if bias else None
        with seed(pm.TENSOR):
            if self.has_weight:
                weight_initializer(self.weight, fan_in=in_features, fan_out=num_classes)
            if bias:
                bias_initializer(self.bias, fan_in=in_features)
        with torch.no_grad():
            if self.has_weight:
                m = self.input_x_weight_parallel_mode
                broadcast(self.weight.data, m.rank_by_idx(0), m)
            if bias:
                broadcast(self.bias.data, pm.TENSOR.rank_by_idx(0), pm.TENSOR)
        if self.has_weight:
            _stamp(self.weight, d, [(-1, self.output_parallel_mode)])

    def forward(self, x):
        return classifier_3d(x, self.weight, self.bias, self.input_parallel_mode, self.weight_parallel_mode,
                             self.output_parallel_mode, self.input_x_weight_parallel_mode,
                             reduce_weight_grad=self.has_weight)


class VocabParallelClassifier3D(_Cube):

    def __init__(self, in_features, num_classes, weight: Parameter = None, bias=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT):
        super().__init__()
        self.in_features, self.num_classes = in_features, num_classes
        d = self._capture()
        self.in_features_per_partition = _div(in_features, d, "in_features")
        self.out_features_per_partition = _div(num_classes, d * d, "num_classes")
        self.bias_features_per_partition = _div(num_classes, d, "num_classes")
        self.has_weight = weight is None
        self.weight = weight if weight is not None else Parameter(
            torch.empty(self.out_features_per_partition, self.in_features_per_partition))
        self.bias = Parameter(torch.zeros(self.bias_features_per_partition)) if bias else None
        with seed(pm.TENSOR):
            if self.has_weight:
                weight_initializer(self.weight, fan_in=in_features, fan_out=num_classes)
            if bias:
                bias_initializer(self.bias, fan_in=in_features)
        if bias:
            with torch.no_grad():
                m = self.output_x_weight_parallel_mode
                broadcast(self.bias.data, m.rank_by_idx(0), m)
        if self.has_weight:
            _stamp(self.weight, d**3, [(0, self.input_parallel_mode), (0, self.weight_parallel_mode),
                                       (-1, self.output_parallel_mode)])
        if bias:
            _stamp(self.bias, d, [(0, self.input_parallel_mode)])
        swap_in_out_group()
        env.vocab_parallel = True

    def forward(self, x):
        return vocab_parallel_classifier_3d(x, self.weight, self.bias, self.input_parallel_mode,
                                            self.weight_parallel_mode, self.output_parallel_mode)


class PatchEmbedding3D(_Cube):

    def __init__(self, img_size, patch_size, in_chans, embed_size, flatten=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT,
                 position_embed_initializer: Callable = init.zeros_()):
        super().__init__()
        d = self._capture()
        self.img_size, self.patch_size = to_2tuple(img_size), to_2tuple(patch_size)
        self.grid_size = (self.img_size[0] // self.patch_size[0], self.img_size[1] // self.patch_size[1])
        self.num_patches = self.grid_size[0] * self.grid_size[1]
        self.embed_size, self.flatten = embed_size, flatten
        e = _div(embed_size, d, "embed_size")
        self.weight = Parameter(torch.empty(e, in_chans, *self.patch_size))
        self.bias = Parameter(torch.empty(e))
        self.cls_token = Parameter(torch.zeros(1, 1, e))
        self.pos_embed = Parameter(torch.zeros(1, self.num_patches + 1, e))
        with seed(pm.TENSOR):
            fan_in = in_chans * self.patch_size[0] * self.patch_size[1]
            weight_initializer(self.weight, fan_in=fan_in, fan_out=embed_size)
            bias_initializer(self.bias, fan_in=fan_in)
            position_embed_initializer(self.pos_embed)
        params = (self.weight, self.bias, self.cls_token, self.pos_embed)
        self._replicate(params, self.input_x_weight_parallel_mode)
        for p in (self.weight, self.bias):
            _stamp(p, d, [(0, self.output_parallel_mode)])
        for p in (self.cls_token, self.pos_embed):
            _stamp(p, d, [(-1, self.output_parallel_mode)])

    def forward(self, images):
        images = split_batch_3d(images, input_parallel_mode=self.input_parallel_mode,
                                weight_parallel_mode=self.weight_parallel_mode)
        return assemble_tokens(patchify_linear(images, self.weight, self.bias, self.patch_size), self.cls_token,
                               self.pos_embed)


class Embedding3D(_Cube):

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None,
                 weight_initializer: Callable = init.normal_(), *args, **kwargs):
        super().__init__()
        d = self._capture()
        self.num_embeddings, self.embed_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.weight = Parameter(torch.empty(num_embeddings, _div(embedding_dim, d, "embedding_dim")))
        with seed(pm.TENSOR):
            weight_initializer(self.weight, fan_in=num_embeddings, fan_out=embedding_dim)
            if padding_idx is not None:
                with torch.no_grad():
                    self.weight[padding_idx].fill_(0)
        self._replicate((self.weight, ), self.input_x_weight_parallel_mode)
        _stamp(self.weight, d, [(-1, self.output_parallel_mode)])

    def forward(self, ids):
        ids = split_batch_3d(ids, input_parallel_mode=self.input_parallel_mode,
                             weight_parallel_mode=self.weight_parallel_mode)
        return masked_embedding(ids, self.weight, 0)


class VocabParallelEmbedding3D(_Cube):

    def __init__(self, num_embeddings, embedding_dim, padding_idx=None,
                 weight_initializer: Callable = init.normal_(), *args, **kwargs):
        super().__init__()
        d = self._capture()
        self.num_embeddings, self.embed_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.num_embeddings_per_partition = _div(num_embeddings, d * d, "num_embeddings")
        self.embed_dim_per_partition = _div(embedding_dim, d, "embedding_dim")
        span = self.num_embeddings_per_partition * d
        self.vocab_start_index = self.input_parallel_mode.local_rank * span
        self.vocab_end_index = self.vocab_start_index + span
        self.weight = Parameter(torch.empty(self.num_embeddings_per_partition, self.embed_dim_per_partition))
        with seed(pm.TENSOR):
            weight_initializer(self.weight, fan_in=num_embeddings, fan_out=embedding_dim)
            own_start = self.vocab_start_index + self.weight_parallel_mode.local_rank * \
                self.num_embeddings_per_partition
            if padding_idx is not None and own_start <= padding_idx < own_start + self.num_embeddings_per_partition:
                with torch.no_grad():
                    self.weight[padding_idx - own_start].fill_(0)
        _stamp(self.weight, d**3, [(0, self.input_parallel_mode), (0, self.weight_parallel_mode),
                                   (-1, self.output_parallel_mode)])
        env.vocab_parallel = True

    def forward(self, ids):
        ids = split_tensor(ids, 0, self.weight_parallel_mode)
        weight = all_gather_weight_3d(self.weight, 0, self.weight_parallel_mode)
        partial = masked_embedding(ids, weight, self.vocab_start_index)
        return reduce_scatter_tensor_3d(partial, 0, self.input_parallel_mode)
