"""OPT decoder family on the parallel layers.

Parity: benchmark/opt/opt.py:20-653 — vocab-parallel token embedding, learned positions with the
offset-2 table indexed by the running count of non-pad tokens (:20-40), pre-LN (or post-LN for the
350m layout) decoder layers with packed per-head QKV, ReLU FFN, tied LM head, shifted LM loss, KV
cache for incremental decoding, presets ``opt_125m ... opt_175b`` (``opt_13b``: hidden 5120, ffn 20480,
40 layers, 64 heads).  Training attention is the fused causal kernel; the incremental-decoding path
(a few query rows against a cache) uses the plain formulation.
"""
import torch
import torch.nn as nn

from .. import module as cube_nn
from .. import ops
from ..parallel.loss import IGNORE_INDEX
from .common import MLP, SelfAttention, key_bias_from_mask, mark_block_output, maybe_checkpoint, normal_init


def _init_kw(init_std):
    return {} if init_std is None else dict(weight_initializer=normal_init(init_std))


class OPTLearnedPositionalEmbedding(nn.Module):
    """Positions = (cumulative count of real tokens) - 1, shifted by 2 into a ``[max_pos + 2, H]`` table."""

    def __init__(self, num_embeddings, embedding_dim, dtype=None, init_std=None):
        super().__init__()
        self.offset = 2
        self.embed = cube_nn.Embedding(num_embeddings + self.offset, embedding_dim, dtype=dtype, **_init_kw(init_std))

    def forward(self, attention_mask, past_key_values_length=0):
        m = attention_mask.long()
        positions = (torch.cumsum(m, dim=1) * m) - 1
        return self.embed(positions[:, past_key_values_length:] + self.offset)

    weight = property(lambda self: self.embed.weight)


class OPTAttention(SelfAttention):

    def __init__(self, embed_dim, num_heads, dropout=0.0, bias=True, dtype=None, init_std=None):
        kw = dict(dtype=dtype, **_init_kw(init_std))
        super().__init__(embed_dim, num_heads, attention_dropout=dropout, dropout=0.0, bias=bias, causal=True,
                         qkv_kw=kw, out_kw=kw, out_bias=bias)

    def forward_cached(self, x, past_key_value=None, key_bias=None):
        """Incremental decoding: returns (output, (k, v)) with ``k, v`` of shape ``[B, heads, T_total, dh]``."""
        qkv = self.query_key_value(x)
        b, t, w = qkv.shape
        heads = w // (3 * self.head_dim)
        q, k, v = qkv.view(b, t, heads, 3 * self.head_dim).permute(0, 2, 1, 3).chunk(3, dim=-1)
        if past_key_value is not None:
            k = torch.cat([past_key_value[0], k], dim=2)
            v = torch.cat([past_key_value[1], v], dim=2)
        o = ops.attention_reference(q, k, v, causal=True, key_bias=key_bias)
        o = o.transpose(1, 2).reshape(b, t, heads * self.head_dim)
        return self.dense(o), (k, v)


class OPTDecoderLayer(nn.Module):

    def __init__(self, hidden_size=768, ffn_dim=3072, num_attention_heads=12, attention_dropout=0.0, dropout=0.1,
                 do_layer_norm_before=True, activation_function="relu", gradient_checkpointing=False, dtype=None,
                 init_std=None):
        super().__init__()
        self.do_layer_norm_before = do_layer_norm_before
        self.gradient_checkpointing = gradient_checkpointing
        self.self_attn = OPTAttention(hidden_size, num_attention_heads, attention_dropout, dtype=dtype,
                                      init_std=init_std)
        self.dropout = cube_nn.Dropout(dropout)
        self.self_attn_layer_norm = cube_nn.LayerNorm(hidden_size, dtype=dtype)
        kw = dict(dtype=dtype, **_init_kw(init_std))
        self.ffn = MLP(hidden_size, ffn_dim, activation_function, dropout, kw1=kw, kw2=kw)
        if do_layer_norm_before:                # (the post-LN layout normalises the sum, which needs its value)
            mark_block_output(self.ffn.dense_2)
        self.final_layer_norm = cube_nn.LayerNorm(hidden_size, dtype=dtype)

    fc1 = property(lambda self: self.ffn.dense_1)
    fc2 = property(lambda self: self.ffn.dense_2)

    def _forward(self, h, key_bias=None, past_key_value=None, use_cache=False):
        residual = h
        if self.do_layer_norm_before:
            h = self.self_attn_layer_norm(h)
        present = None
        if use_cache or past_key_value is not None:
            h, present = self.self_attn.forward_cached(h, past_key_value, key_bias)
        else:
            h = self.self_attn(h, key_bias)
        h = residual + self.dropout(h)
        if not self.do_layer_norm_before:
            h = self.self_attn_layer_norm(h)
        residual = h
        if self.do_layer_norm_before:
            h = self.final_layer_norm(h)
        h = residual + self.ffn(h)
        if not self.do_layer_norm_before:
            h = self.final_layer_norm(h)
        return h, present

    def forward(self, h, key_bias=None, past_key_value=None, use_cache=False):
        if self.gradient_checkpointing and self.training and not use_cache:
            return maybe_checkpoint(lambda a, b: self._forward(a, b)[0], True, h, key_bias), None
        return self._forward(h, key_bias, past_key_value, use_cache)


class OPTLMLoss(nn.Module):

    def __init__(self):
        super().__init__()
        self.loss = cube_nn.CrossEntropyLoss()

    def forward(self, logits, labels):
        # logits at position t are scored against the label at t+1; instead of copying the logits without their
        # last position, the labels are shifted and the last position of every sequence is marked as ignored
        pad = labels.new_full(labels.shape[:-1] + (1, ), IGNORE_INDEX)
        shift_labels = torch.cat([labels[..., 1:], pad], dim=-1)
        return self.loss(logits.reshape(-1, logits.size(-1)), shift_labels.reshape(-1))


class OPT(nn.Module):

    def __init__(self, vocab_size=50304, hidden_size=768, num_hidden_layers=12, ffn_dim=3072, num_attention_heads=12,
                 max_position_embeddings=1024, do_layer_norm_before=True, dropout=0.1, attention_dropout=0.0,
                 layerdrop=0.0, padding_idx=1, activation_function="relu", gradient_checkpointing=False, dtype=None,
                 init_std=None):
        """``init_std``: every weight matrix and embedding table is drawn from N(0, init_std) (the HF OPT recipe uses
        0.02; ``None`` keeps the layers' own defaults).  ``dtype``: parameter dtype; a 16-bit dtype gives the pure
        16-bit-parameter mode of the reference's ``-O3`` (benchmark/opt/opt.py:541), without fp32 master copies."""
        super().__init__()
        self.layerdrop, self.padding_idx, self.vocab_size = layerdrop, padding_idx, vocab_size
        self.max_target_positions = max_position_embeddings
        self.embed_tokens = cube_nn.Embedding(vocab_size, hidden_size, vocab_parallel=True, padding_idx=padding_idx,
                                              dtype=dtype, **_init_kw(init_std))
        self.embed_positions = OPTLearnedPositionalEmbedding(max_position_embeddings, hidden_size, dtype=dtype,
                                                             init_std=init_std)
        self.layers = nn.ModuleList([
            OPTDecoderLayer(hidden_size, ffn_dim, num_attention_heads, attention_dropout, dropout,
                            do_layer_norm_before, activation_function, gradient_checkpointing, dtype, init_std)
            for _ in range(num_hidden_layers)
        ])
        self.final_layer_norm = cube_nn.LayerNorm(hidden_size, dtype=dtype) if do_layer_norm_before else None
        self.lm_head = cube_nn.Classifier(hidden_size, vocab_size, weight=self.embed_tokens.weight, bias=False,
                                          dtype=dtype)

    def forward(self, input_ids, attention_mask=None, past_key_values=None, use_cache=False):
        input_ids = input_ids.view(-1, input_ids.shape[-1])
        past_len = past_key_values[0][0].shape[2] if past_key_values is not None else 0
        h = self.embed_tokens(input_ids)
        if attention_mask is None:
            mask_full = torch.ones(input_ids.shape[0], input_ids.shape[1] + past_len, dtype=torch.bool,
                                   device=input_ids.device)
            key_bias = None
        else:
            mask_full = attention_mask
            key_bias = key_bias_from_mask(attention_mask)
        h = h + self.embed_positions(mask_full, past_len)
        cache = () if use_cache else None
        for idx, layer in enumerate(self.layers):
            if self.training and self.layerdrop > 0 and torch.rand(()).item() < self.layerdrop:
                continue
            past = past_key_values[idx] if past_key_values is not None else None
            h, present = layer(h, key_bias, past, use_cache)
            if use_cache:
                cache += (present, )
        if self.final_layer_norm is not None:
            h = self.final_layer_norm(h)
        logits = self.lm_head(h)
        return (logits, cache) if use_cache else (logits, )


_PRESETS = {
    "opt_125m": dict(hidden_size=768, ffn_dim=3072, num_hidden_layers=12, num_attention_heads=16),
    "opt_350m": dict(hidden_size=1024, ffn_dim=4096, num_hidden_layers=24, num_attention_heads=16),
    "opt_1b": dict(hidden_size=2048, ffn_dim=8192, num_hidden_layers=24, num_attention_heads=32),
    "opt_3b": dict(hidden_size=2560, ffn_dim=10240, num_hidden_layers=32, num_attention_heads=32),
    "opt_6b": dict(hidden_size=4096, ffn_dim=16384, num_hidden_layers=32, num_attention_heads=32),
    "opt_13b": dict(hidden_size=5120, ffn_dim=20480, num_hidden_layers=40, num_attention_heads=64),
    "opt_30b": dict(hidden_size=7168, ffn_dim=28672, num_hidden_layers=48, num_attention_heads=64),
    "opt_66b": dict(hidden_size=9216, ffn_dim=36864, num_hidden_layers=64, num_attention_heads=64),
    "opt_175b": dict(hidden_size=12288, ffn_dim=49152, num_hidden_layers=96, num_attention_heads=128),
    "opt_tiny": dict(hidden_size=64, ffn_dim=256, num_hidden_layers=2, num_attention_heads=4, vocab_size=512),
}


def build_model(name, max_position_embeddings=1024, checkpoint=False, dtype=None, **overrides):
    cfg = dict(_PRESETS[name])
    cfg.update(max_position_embeddings=max_position_embeddings, gradient_checkpointing=checkpoint, dtype=dtype)
    cfg.update(overrides)
    return OPT(**cfg)


def _preset(name):
    def f(max_position_embeddings=1024, checkpoint=False, dtype=None, **kw):
        return build_model(name, max_position_embeddings, checkpoint, dtype, **kw)
    f.__name__ = name
    return f


for _n in _PRESETS:
    globals()[_n] = _preset(_n)
