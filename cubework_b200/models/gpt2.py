"""GPT-2 family on the parallel layers.

Parity: benchmark/gpt2/gpt2.py:16-373 — vocab-parallel word embedding + position embedding, pre-LN
blocks (optional post-LN), packed per-head QKV, GELU MLP, LM head tied to the word-embedding table,
shifted causal-LM loss, presets ``gpt2_small ... gpt2_40b`` (``gpt2_xl``: hidden 1600, 64 heads,
48 layers).  The attention is a fused causal kernel instead of materialised ``[b, heads, T, T]``
scores with a ``tril`` mask rebuilt every call (gpt2.py:75-91).
"""
import torch
import torch.nn as nn

from .. import module as cube_nn
from ..parallel.loss import IGNORE_INDEX
from .common import MLP, SelfAttention, key_bias_from_mask, mark_block_output, maybe_checkpoint, normal_init


class GPT2Embedding(nn.Module):

    def __init__(self, embedding_size, vocab_size, max_position_embeddings, padding_idx=None, dropout=0.0,
                 init_std=None, sequence_parallel=False):
        super().__init__()
        kw = {} if init_std is None else dict(weight_initializer=normal_init(init_std))
        self.word_embeddings = cube_nn.Embedding(vocab_size, embedding_size, vocab_parallel=True,
                                                 padding_idx=padding_idx, sequence_parallel=sequence_parallel, **kw)
        self.position_embeddings = cube_nn.Embedding(max_position_embeddings, embedding_size, **kw)
        self.sequence_parallel = sequence_parallel
        self.dropout = cube_nn.Dropout(dropout, sequence_parallel=sequence_parallel)

    def forward(self, input_ids):
        t = input_ids.size(1)
        pos = torch.arange(t, dtype=torch.long, device=input_ids.device).unsqueeze(0)
        pe = self.position_embeddings(pos)
        if self.sequence_parallel:    # the [1, T, H] position rows are added to this rank's sequences only
            pe = cube_nn.sum_grad_over_rows(pe)
        return self.dropout(self.word_embeddings(input_ids) + pe)


class GPT2Block(nn.Module):

    def __init__(self, hidden_size, num_heads, intermediate_size, attention_dropout=0.0, dropout=0.0,
                 layernorm_epsilon=1e-5, bias=True, apply_post_layernorm=False, checkpoint=False, init_std=None,
                 out_std=None, sequence_parallel=False):
        super().__init__()
        self.checkpoint, self.apply_post_layernorm = checkpoint, apply_post_layernorm
        wi = None if init_std is None else dict(weight_initializer=normal_init(init_std))
        wo = None if out_std is None else dict(weight_initializer=normal_init(out_std))
        sp = dict(sequence_parallel=sequence_parallel)
        self.norm1 = cube_nn.LayerNorm(hidden_size, eps=layernorm_epsilon, **sp)
        self.attn = SelfAttention(hidden_size, num_heads, attention_dropout, dropout, bias=bias, causal=True,
                                  qkv_kw=wi, out_kw=wo, **sp)
        self.norm2 = cube_nn.LayerNorm(hidden_size, eps=layernorm_epsilon, **sp)
        self.mlp = MLP(hidden_size, intermediate_size, "gelu", dropout, bias=bias, kw1=wi, kw2=wo, **sp)
        mark_block_output(self.mlp.dense_2)     # its output only feeds dropout and the residual add

    def _forward(self, x, pending, key_bias=None):
        """``x``: residual stream; ``pending``: the previous block's contribution that has not been added yet (or
        None).  Returns ``(stream, pending)`` again, so every residual add is done by the layer norm that follows it
        (one kernel computes the sum and its normalised value)."""
        if self.apply_post_layernorm:
            if pending is not None:
                x = x + pending
            h = self.norm1(x)
            x = h + self.attn(h, key_bias)
            h = self.norm2(x)
            return h, self.mlp(h)
        if pending is None:
            h = self.norm1(x)
        else:
            x, h = self.norm1(x, residual=pending)
        x, h = self.norm2(x, residual=self.attn(h, key_bias))
        return x, self.mlp(h)

    def forward(self, x, pending=None, key_bias=None):
        return maybe_checkpoint(self._forward, self.checkpoint and self.training, x, pending, key_bias)


class GPT2LMLoss(nn.Module):
    """Next-token loss: logits at position t against the label at t+1."""

    def __init__(self):
        super().__init__()
        self.loss = cube_nn.CrossEntropyLoss()

    def forward(self, logits, labels):
        # logits at position t are scored against the label at t+1; instead of copying the logits without their
        # last position, the labels are shifted and the last position of every sequence is marked as ignored
        pad = labels.new_full(labels.shape[:-1] + (1, ), IGNORE_INDEX)
        shift_labels = torch.cat([labels[..., 1:], pad], dim=-1)
        return self.loss(logits.reshape(-1, logits.size(-1)), shift_labels.reshape(-1))


class GPT2(nn.Module):

    def __init__(self, vocab_size=50304, max_position_embeddings=1024, hidden_size=768, num_heads=12,
                 intermediate_size=3072, depth=12, dropout=0.1, embedding_dropout=0.1, attention_dropout=0.0,
                 layernorm_epsilon=1e-5, padding_idx=None, bias=True, apply_post_layernorm=False, checkpoint=False,
                 init_std=None, sequence_parallel=False):
        """``sequence_parallel`` (1D tensor parallelism only; ignored elsewhere): hidden states between the
        attention / MLP pairs hold ``batch / tp`` sequences per rank instead of being replicated; the batch
        size must be a multiple of the 1D group size."""
        super().__init__()
        out_std = None if init_std is None else init_std
        sp = dict(sequence_parallel=sequence_parallel)
        self.sp_size = cube_nn.sequence_parallel_size() if sequence_parallel else 1
        self.embed = GPT2Embedding(hidden_size, vocab_size, max_position_embeddings, padding_idx, embedding_dropout,
                                   init_std, **sp)
        self.blocks = nn.ModuleList([
            GPT2Block(hidden_size, num_heads, intermediate_size, attention_dropout, dropout, layernorm_epsilon, bias,
                      apply_post_layernorm, checkpoint, init_std, out_std, **sp) for _ in range(depth)
        ])
        self.norm = cube_nn.LayerNorm(hidden_size, eps=layernorm_epsilon, **sp)
        self.head = cube_nn.Classifier(hidden_size, vocab_size, weight=self.embed.word_embeddings.weight, bias=False,
                                       **sp)

    def forward(self, input_ids, attention_mask=None):
        if self.sp_size > 1 and input_ids.size(0) % self.sp_size != 0:
            raise ValueError(f"sequence_parallel needs a batch ({input_ids.size(0)}) divisible by the tensor "
                             f"parallel size ({self.sp_size})")
        x = self.embed(input_ids)
        key_bias = key_bias_from_mask(attention_mask)
        pending = None
        for block in self.blocks:
            x, pending = block(x, pending, key_bias)
        h = self.norm(x) if pending is None else self.norm(x, residual=pending)[1]
        return self.head(h)


_PRESETS = {
    "gpt2_small": dict(hidden_size=768, intermediate_size=3072, depth=12, num_heads=16),
    "gpt2_medium": dict(hidden_size=1024, intermediate_size=4096, depth=24, num_heads=16),
    "gpt2_large": dict(hidden_size=1280, intermediate_size=5120, depth=36, num_heads=20),
    "gpt2_xl": dict(hidden_size=1600, intermediate_size=6400, depth=48, num_heads=64),
    "gpt2_5b": dict(hidden_size=2880, intermediate_size=11520, depth=50, num_heads=64),
    "gpt2_10b": dict(hidden_size=4096, intermediate_size=16384, depth=50, num_heads=64),
    "gpt2_20b": dict(hidden_size=5760, intermediate_size=23040, depth=50, num_heads=64),
    "gpt2_40b": dict(hidden_size=8192, intermediate_size=32768, depth=50, num_heads=64),
    "gpt2_tiny": dict(hidden_size=128, intermediate_size=512, depth=2, num_heads=4, vocab_size=1024),
}


def build_model(name, max_position_embeddings=1024, checkpoint=False, **overrides):
    cfg = dict(_PRESETS[name])
    cfg.update(max_position_embeddings=max_position_embeddings, checkpoint=checkpoint)
    cfg.update(overrides)
    return GPT2(**cfg)


def _preset(name):
    def f(max_position_embeddings=1024, checkpoint=False, **kw):
        return build_model(name, max_position_embeddings, checkpoint, **kw)
    f.__name__ = name
    return f


for _n in _PRESETS:
    globals()[_n] = _preset(_n)
