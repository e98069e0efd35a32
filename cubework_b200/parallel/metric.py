"""Evaluation metrics.

Parity: cubework/module/metric/metrics.py:22-89 (``Metric``, ``Accuracy``, ``Perplexity`` with
``reset/forward/value/to_str``) and metric_{std,2d,3d}.py (``Accuracy{STD,2D,3D}``: argmax == target,
counted over the batch shards of the 2D / 3D grid).  Totals are combined over the DATA group.
"""
from abc import abstractmethod

import torch
import torch.nn as nn

from ..utils.common import get_current_device
from .collective import all_reduce
from .common import get_tensor_parallel_mode
from .mesh import pm
from .ops_2d import reduce_by_batch_2d, split_batch_2d
from .ops_3d import get_input_parallel_mode, get_weight_parallel_mode, reduce_by_batch_3d, split_batch_3d


class AccuracySTD(nn.Module):

    def forward(self, logits, targets):
        return (logits.argmax(dim=-1) == targets).sum()


class Accuracy2D(nn.Module):

    def forward(self, logits, targets):
        with torch.no_grad():
            targets = split_batch_2d(targets)
            return reduce_by_batch_2d((logits.argmax(dim=-1) == targets).sum())


class Accuracy3D(nn.Module):

    def __init__(self):
        super().__init__()
        self.input_parallel_mode = get_input_parallel_mode()
        self.weight_parallel_mode = get_weight_parallel_mode()

    def forward(self, logits, targets):
        with torch.no_grad():
            targets = split_batch_3d(targets, 0, self.input_parallel_mode, self.weight_parallel_mode)
            correct = (logits.argmax(dim=-1) == targets).sum()
            return reduce_by_batch_3d(correct, self.input_parallel_mode, self.weight_parallel_mode)


_parallel_accuracy = {None: AccuracySTD, "1d": AccuracySTD, "2d": Accuracy2D, "3d": Accuracy3D}


class Metric(nn.Module):

    def __init__(self, name):
        super().__init__()
        self.name = name

    @abstractmethod
    def reset(self):
        ...

    @abstractmethod
    def forward(self, logits, targets, loss):
        ...

    @abstractmethod
    def value(self):
        ...


class Accuracy(Metric):

    def __init__(self):
        super().__init__("Accuracy")
        self.acc = _parallel_accuracy[get_tensor_parallel_mode()]()
        self.reset()

    def reset(self):
        dev = get_current_device()
        self.total_correct = torch.zeros((), dtype=torch.float64 if dev.type == "cpu" else torch.float32, device=dev)
        self.total_samples = torch.zeros_like(self.total_correct)

    def forward(self, logits, targets, loss=None):
        with torch.no_grad():
            batch_size = targets.size(0)
            correct = self.acc(logits, targets).to(self.total_correct.dtype)
            self.total_samples += batch_size
            self.total_correct += correct
            return correct / batch_size

    def value(self):
        with torch.no_grad():
            both = torch.stack([self.total_correct, self.total_samples])
            if pm.DATA.is_initialized():
                both = all_reduce(both, pm.DATA)
            return both[0] / both[1]

    def to_str(self):
        return f"{self.value().item() * 100:.2f} %"


class Perplexity(Metric):

    def __init__(self):
        super().__init__("Perplexity")
        self.reset()

    def reset(self):
        self.cnt = 0
        self.total_loss = torch.zeros((), dtype=torch.float32, device=get_current_device())

    def forward(self, logits, targets, loss):
        with torch.no_grad():
            self.cnt += 1
            self.total_loss += loss.detach().float()
            return torch.exp(loss.detach().float())

    def value(self):
        with torch.no_grad():
            total = self.total_loss.clone()
            world = 1
            if pm.DATA.is_initialized():
                total = all_reduce(total, pm.DATA)
                world = pm.DATA.world_size
            return torch.exp(total / (max(self.cnt, 1) * world))

    def to_str(self):
        return f"{self.value().item():.5g}"
