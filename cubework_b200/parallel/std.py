"""Unsharded layers used when no tensor parallelism is active (and by the 1D patch embedding).

Parity: cubework/module/module_std.py:17-133 — ``drop_path``/``DropPath`` (stochastic depth per
sample), ``PatchEmbeddingSTD`` (stride-``p`` conv patchify + class token + position embedding),
``ClassifierSTD`` (linear head with an optional tied weight).

The patchify convolution has stride == kernel, so it is an im2col reshape followed by one GEMM;
:func:`patchify_linear` does exactly that, which puts it on this package's tensor-core GEMM instead of
a cuDNN convolution.
"""
import math
from typing import Callable

import torch
import torch.nn as nn

from . import init
from .common import to_2tuple
from .functional import local_linear

_W_INIT = init.kaiming_uniform_(a=math.sqrt(5))
_B_INIT = init.xavier_uniform_(a=1, scale=1)


def drop_path(x, drop_prob: float = 0.0, training: bool = False):
    if not training or not drop_prob:
        return x
    keep = 1.0 - drop_prob
    mask = torch.empty((x.shape[0], ) + (1, ) * (x.dim() - 1), dtype=x.dtype, device=x.device).bernoulli_(keep)
    return x * (mask / keep)


class DropPath(nn.Module):

    def __init__(self, drop_prob=None):
        super().__init__()
        self.drop_prob = drop_prob

    def forward(self, x):
        return drop_path(x, self.drop_prob or 0.0, self.training)


def patchify_linear(images, weight, bias, patch_size):
    """``conv2d(images, weight, bias, stride=patch)`` -> ``[B, num_patches, E]`` via im2col + GEMM."""
    B, C, H, W = images.shape
    ph, pw = patch_size
    gh, gw = H // ph, W // pw
    cols = images.reshape(B, C, gh, ph, gw, pw).permute(0, 2, 4, 1, 3, 5).reshape(B, gh * gw, C * ph * pw)
    return local_linear(cols, weight.reshape(weight.shape[0], -1), bias, w_is_out_in=True)


def assemble_tokens(patches, cls_token, pos_embed):
    cls = cls_token.to(patches.dtype).expand(patches.shape[0], -1, -1)
    return torch.cat((cls, patches), dim=1) + pos_embed.to(patches.dtype)


class PatchEmbeddingSTD(nn.Module):

    def __init__(self, img_size, patch_size, in_chans, embed_size, flatten=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT,
                 position_embed_initializer: Callable = init.zeros_()):
        super().__init__()
        self.img_size, self.patch_size = to_2tuple(img_size), to_2tuple(patch_size)
        self.grid_size = (self.img_size[0] // self.patch_size[0], self.img_size[1] // self.patch_size[1])
        self.num_patches = self.grid_size[0] * self.grid_size[1]
        self.flatten = flatten
        self.weight = nn.Parameter(torch.empty(embed_size, in_chans, *self.patch_size))
        self.bias = nn.Parameter(torch.empty(embed_size))
        self.cls_token = nn.Parameter(torch.zeros(1, 1, embed_size))
        self.pos_embed = nn.Parameter(torch.zeros(1, self.num_patches + 1, embed_size))
        fan_in = in_chans * self.patch_size[0] * self.patch_size[1]
        fan_out = embed_size * self.patch_size[0] * self.patch_size[1]
        weight_initializer(self.weight, fan_in=fan_in, fan_out=fan_out)
        bias_initializer(self.bias, fan_in=fan_in)
        position_embed_initializer(self.pos_embed)

    def forward(self, images):
        _, _, H, W = images.shape
        assert (H, W) == tuple(self.img_size), \
            f"Input image size ({H}*{W}) doesn't match model ({self.img_size[0]}*{self.img_size[1]})."
        assert self.flatten, "only the flattened [B, N, C] token layout is supported"
        return assemble_tokens(patchify_linear(images, self.weight, self.bias, self.patch_size), self.cls_token,
                               self.pos_embed)


class ClassifierSTD(nn.Module):

    def __init__(self, in_features, num_classes, weight: nn.Parameter = None, bias=True,
                 weight_initializer: Callable = _W_INIT, bias_initializer: Callable = _B_INIT):
        super().__init__()
        self.in_features, self.num_classes = in_features, num_classes
        self.has_weight = weight is None
        self.weight = weight if weight is not None else nn.Parameter(torch.empty(num_classes, in_features))
        self.bias = nn.Parameter(torch.zeros(num_classes)) if bias else None
        if self.has_weight:
            weight_initializer(self.weight, fan_in=in_features, fan_out=num_classes)
        if bias:
            bias_initializer(self.bias, fan_in=in_features)

    def forward(self, x):
        return local_linear(x, self.weight, self.bias, w_is_out_in=True)
