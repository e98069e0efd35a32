"""Vision Transformer family on the parallel layers.

Parity: benchmark/vit/vit.py:18-356 — patch embedding (lecun-normal weight, zero bias, truncated-normal
position embedding) + dropout, pre-LN blocks with optional stochastic depth, GELU MLP, classification
head on the class token through ``Classifier`` (zero-initialised), optional representation layer,
presets ``vit_small ... vit_12b`` (``vit_base``: hidden 768, 16 heads, 12 layers); plus the mixup loss
and accuracy used by the CIFAR-10 recipe (:357-392).
"""
import torch
import torch.nn as nn

from .. import module as cube_nn
from .common import MLP, SelfAttention, mark_block_output, maybe_checkpoint


def _lin_kw():
    return dict(weight_initializer=cube_nn.init.xavier_uniform_(), bias_initializer=cube_nn.init.normal_(std=1e-6))


class ViTEmbedding(nn.Module):

    def __init__(self, img_size, patch_size, in_chans, embedding_size, dropout, flatten=True):
        super().__init__()
        self.patch_embed = cube_nn.PatchEmbedding(
            img_size, patch_size, in_chans, embedding_size, flatten=flatten,
            weight_initializer=cube_nn.init.lecun_normal_(), bias_initializer=cube_nn.init.zeros_(),
            position_embed_initializer=cube_nn.init.trunc_normal_(std=0.02))
        self.dropout = cube_nn.Dropout(dropout)

    def forward(self, x):
        return self.dropout(self.patch_embed(x))


class ViTHead(nn.Module):

    def __init__(self, hidden_size, num_classes, representation_size=None, bias=True):
        super().__init__()
        zeros = dict(weight_initializer=cube_nn.init.zeros_(), bias_initializer=cube_nn.init.zeros_())
        if representation_size:
            self.representation = cube_nn.Linear(hidden_size, representation_size, bias=bias, **zeros)
        else:
            self.representation, representation_size = None, hidden_size
        self.dense = cube_nn.Classifier(representation_size, num_classes, bias=bias, **zeros)

    def forward(self, x):
        x = x[:, 0]
        if self.representation is not None:
            x = self.representation(x)
        return self.dense(x)


class ViTBlock(nn.Module):

    def __init__(self, hidden_size, num_heads, intermediate_size, attention_dropout=0.0, dropout=0.0, drop_path=0.0,
                 layernorm_epsilon=1e-6, bias=True, checkpoint=False):
        super().__init__()
        self.checkpoint = checkpoint
        self.norm1 = cube_nn.LayerNorm(hidden_size, eps=layernorm_epsilon)
        self.attn = SelfAttention(hidden_size, num_heads, attention_dropout, dropout, bias=bias, causal=False,
                                  qkv_kw=_lin_kw(), out_kw=_lin_kw())
        self.drop_path = cube_nn.DropPath(drop_path) if drop_path > 0.0 else nn.Identity()
        self.norm2 = cube_nn.LayerNorm(hidden_size, eps=layernorm_epsilon)
        self.mlp = MLP(hidden_size, intermediate_size, "gelu", dropout, bias=bias, kw1=_lin_kw(), kw2=_lin_kw(),
                       inner_dropout=dropout)
        mark_block_output(self.mlp.dense_2)

    def _forward(self, x):
        x = x + self.drop_path(self.attn(self.norm1(x)))
        return x + self.drop_path(self.mlp(self.norm2(x)))

    def forward(self, x):
        return maybe_checkpoint(self._forward, self.checkpoint, x)


class VisionTransformer(nn.Module):

    def __init__(self, img_size=224, patch_size=16, in_chans=3, num_classes=1000, depth=12, hidden_size=768,
                 num_heads=12, intermediate_size=3072, representation_size=None, attention_dropout=0.0, dropout=0.1,
                 drop_path=0.0, layernorm_epsilon=1e-6, bias=True, checkpoint=False):
        super().__init__()
        self.img_size, self.patch_size = img_size, patch_size
        self.embed = ViTEmbedding(img_size, patch_size, in_chans, hidden_size, dropout)
        self.num_patches = self.embed.patch_embed.embed.num_patches
        self.flop_tokens_per_sample = self.num_patches + 1      # what the FLOP model counts per image (patches + class token)
        dpr = [x.item() for x in torch.linspace(0, drop_path, depth)]
        self.blocks = nn.ModuleList([
            ViTBlock(hidden_size, num_heads, intermediate_size, attention_dropout, dropout, dpr[i], layernorm_epsilon,
                     bias, checkpoint) for i in range(depth)
        ])
        self.norm = cube_nn.LayerNorm(hidden_size, eps=layernorm_epsilon)
        self.head = ViTHead(hidden_size, num_classes, representation_size, bias)

    def forward(self, pixel_values):
        x = self.embed(pixel_values)
        for block in self.blocks:
            x = block(x)
        return self.head(self.norm(x))


class MixupLoss(nn.Module):
    """``lam * CE(x, a) + (1 - lam) * CE(x, b)`` for mixup targets ``(a, b, lam)``; plain CE otherwise."""

    def __init__(self):
        super().__init__()
        self.loss = cube_nn.CrossEntropyLoss()

    def forward(self, logits, targets):
        if isinstance(targets, (tuple, list)):
            a, b, lam = targets
            return lam * self.loss(logits, a) + (1 - lam) * self.loss(logits, b)
        return self.loss(logits, targets)


class MixupAccuracy(nn.Module):

    def __init__(self):
        super().__init__()
        self.acc = cube_nn.Accuracy()
        self.name = self.acc.name

    def reset(self):
        self.acc.reset()

    def forward(self, logits, targets, loss=None):
        if isinstance(targets, (tuple, list)):
            a, b, lam = targets
            return lam * self.acc(logits, a, loss) + (1 - lam) * self.acc(logits, b, loss)
        return self.acc(logits, targets, loss)

    def value(self):
        return self.acc.value()

    def to_str(self):
        return self.acc.to_str()


def mixup_collate(images, labels, alpha=0.8, generator=None):
    """Mix a batch with a permutation of itself; returns ``images, (labels, permuted labels, lam)``."""
    lam = float(torch.distributions.Beta(alpha, alpha).sample()) if alpha > 0 else 1.0
    perm = torch.randperm(images.shape[0], generator=generator)
    return lam * images + (1 - lam) * images[perm], (labels, labels[perm], lam)


_PRESETS = {
    "vit_tiny": dict(img_size=32, patch_size=8, hidden_size=64, num_heads=4, intermediate_size=128, depth=2,
                     num_classes=16),
    "vit_small": dict(patch_size=16, hidden_size=384, num_heads=16, intermediate_size=1536, depth=12),
    "vit_base": dict(patch_size=16, hidden_size=768, num_heads=16, intermediate_size=3072, depth=12),
    "vit_large": dict(patch_size=16, hidden_size=1024, num_heads=16, intermediate_size=4096, depth=24),
    "vit_huge": dict(patch_size=14, hidden_size=1280, num_heads=16, intermediate_size=5120, depth=32),
    "vit_g": dict(patch_size=14, hidden_size=1664, num_heads=64, intermediate_size=8192, depth=48),
    "vit_3b": dict(patch_size=14, hidden_size=1920, num_heads=64, intermediate_size=7680, depth=64),
    "vit_6b": dict(patch_size=14, hidden_size=2560, num_heads=64, intermediate_size=10240, depth=72),
    "vit_12b": dict(patch_size=14, hidden_size=3200, num_heads=64, intermediate_size=12800, depth=96),
}


def build_model(name, checkpoint=False, **overrides):
    cfg = dict(img_size=224)
    cfg.update(_PRESETS[name])
    cfg.update(checkpoint=checkpoint)
    cfg.update(overrides)
    return VisionTransformer(**cfg)


def _preset(name):
    def f(checkpoint=False, **kw):
        return build_model(name, checkpoint, **kw)
    f.__name__ = name
    return f


for _n in _PRESETS:
    globals()[_n] = _preset(_n)
