"""Cross-entropy losses for every tensor-parallel mode.

Parity: cubework/module/loss/losses.py:21-35 (façade ``CrossEntropyLoss(reduction: bool)``),
loss_1d.py:11-91, loss_2d.py:13-110, loss_3d.py:12-110 (``CrossEntropyLoss{2,3}D``,
``VocabParallelCrossEntropyLoss{1,2,3}D``).

The vocab-parallel loss exchanges ONE ``[rows, 3]`` fp32 block per rank — (row max, sum of
exponentials relative to that max, target logit if the target is local) — and merges the blocks
locally, where the reference runs three dependent all-reduces (MAX, SUM, SUM) and about six passes
over the fp32 logits (loss_1d.py:14-79).  Forward reads the logits once, backward reads them once and
writes the gradient once, both in a hand-written kernel on CUDA.
"""
import torch
import torch.nn as nn

from .. import ops
from ..global_vars import env
from .collective import all_gather
from .common import get_tensor_parallel_mode
from .mesh import pm
from .ops_2d import reduce_by_batch_2d, split_batch_2d
from .ops_3d import (get_input_parallel_mode, get_output_parallel_mode, get_weight_parallel_mode,
                     reduce_by_batch_3d, split_batch_3d)


def merge_ce_stats(blocks):
    """``blocks``: ``[n, rows, 3]`` per-shard (max, sumexp, target) -> (global max, global sumexp, target)."""
    mx, se, tl = blocks[..., 0], blocks[..., 1], blocks[..., 2]
    gmax = mx.max(dim=0).values
    gsum = (se * torch.exp(mx - gmax)).sum(dim=0)
    return gmax, gsum, tl.sum(dim=0)


IGNORE_INDEX = -100


class _ShardedCrossEntropy(torch.autograd.Function):
    """Per-row loss of logits whose class dimension is split over ``mode`` (or not split: ``None``).
    Rows whose target is ``IGNORE_INDEX`` get zero loss and zero gradient."""

    @staticmethod
    def forward(ctx, logits, targets, mode):
        n = mode.world_size if mode is not None else 1
        cd = logits.dtype
        l2 = logits.reshape(-1, logits.shape[-1]).contiguous()
        t1 = targets.reshape(-1).contiguous()
        vocab_start = (mode.local_rank if mode is not None else 0) * l2.shape[-1]
        stats = ops.ce_local_stats(l2, t1, vocab_start)
        if n > 1:
            blocks = all_gather(stats.unsqueeze(0), 0, mode)
        else:
            blocks = stats.unsqueeze(0)
        gmax, gsum, tl = merge_ce_stats(blocks)
        valid = t1 != IGNORE_INDEX
        loss = (torch.log(gsum) + gmax - tl) * valid
        ctx.save_for_backward(l2, t1, gmax, gsum)
        ctx.vocab_start, ctx.shape, ctx.dtype = vocab_start, logits.shape, cd
        return loss.view(targets.shape)

    @staticmethod
    def backward(ctx, g):
        l2, t1, gmax, gsum = ctx.saved_tensors
        scale = g.reshape(-1).float() * (t1 != IGNORE_INDEX)
        grad = ops.ce_grad(l2, t1, ctx.vocab_start, gmax, gsum, scale.contiguous())
        return grad.view(ctx.shape), None, None


def sharded_cross_entropy(logits, targets, mode=None):
    return _ShardedCrossEntropy.apply(logits, targets, mode)


def masked_mean(loss, targets):
    """Mean over the rows whose target is not ``IGNORE_INDEX``."""
    valid = (targets.reshape(-1) != IGNORE_INDEX).sum().clamp_min(1)
    return loss.sum() / valid


class _LossBase(nn.Module):

    def __init__(self, reduction=True):
        super().__init__()
        self.reduction_mean = reduction


class CrossEntropyLossSTD(_LossBase):
    """Unsharded classes, unsharded batch (no tensor parallelism, or 1D with a gathered classifier)."""

    def forward(self, logits, targets):
        loss = sharded_cross_entropy(logits, targets, None)
        return masked_mean(loss, targets) if self.reduction_mean else loss


class VocabParallelCrossEntropyLoss1D(_LossBase):

    def forward(self, logits, targets):
        loss = sharded_cross_entropy(logits, targets, pm.PARALLEL_1D)
        return masked_mean(loss, targets) if self.reduction_mean else loss


class CrossEntropyLoss2D(_LossBase):

    def forward(self, logits, targets):
        targets = split_batch_2d(targets)
        loss = sharded_cross_entropy(logits, targets, None)
        if self.reduction_mean:
            loss = reduce_by_batch_2d(masked_mean(loss, targets), True)
        return loss


class VocabParallelCrossEntropyLoss2D(_LossBase):

    def forward(self, logits, targets):
        targets = split_batch_2d(targets)
        loss = sharded_cross_entropy(logits, targets, pm.PARALLEL_2D_ROW)
        if self.reduction_mean:
            loss = reduce_by_batch_2d(masked_mean(loss, targets), True)
        return loss


class _Loss3D(_LossBase):

    def __init__(self, reduction=True):
        super().__init__(reduction)
        self.input_parallel_mode = get_input_parallel_mode()
        self.weight_parallel_mode = get_weight_parallel_mode()
        self.output_parallel_mode = get_output_parallel_mode()

    def _finish(self, loss, targets):
        if self.reduction_mean:
            loss = reduce_by_batch_3d(masked_mean(loss, targets), self.input_parallel_mode,
                                      self.weight_parallel_mode, True)
        return loss

    def _targets(self, targets):
        return split_batch_3d(targets, 0, self.input_parallel_mode, self.weight_parallel_mode)


class CrossEntropyLoss3D(_Loss3D):

    def forward(self, logits, targets):
        targets = self._targets(targets)
        return self._finish(sharded_cross_entropy(logits, targets, None), targets)


class VocabParallelCrossEntropyLoss3D(_Loss3D):

    def forward(self, logits, targets):
        targets = self._targets(targets)
        return self._finish(sharded_cross_entropy(logits, targets, self.output_parallel_mode), targets)


_parallel_cross_entropy = {None: CrossEntropyLossSTD, "1d": CrossEntropyLossSTD, "2d": CrossEntropyLoss2D,
                           "3d": CrossEntropyLoss3D}
_vocab_parallel_cross_entropy = {"1d": VocabParallelCrossEntropyLoss1D, "2d": VocabParallelCrossEntropyLoss2D,
                                 "3d": VocabParallelCrossEntropyLoss3D}


class CrossEntropyLoss(nn.Module):
    """Picks the loss that matches the logits produced by the most recently built classifier."""

    def __init__(self, reduction: bool = True):
        super().__init__()
        mode = get_tensor_parallel_mode()
        if mode is not None and env.vocab_parallel:
            self.loss = _vocab_parallel_cross_entropy[mode](reduction=reduction)
        else:
            self.loss = _parallel_cross_entropy[mode](reduction=reduction)

    def forward(self, *args, **kwargs):
        return self.loss(*args, **kwargs)
