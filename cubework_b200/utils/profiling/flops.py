"""Model size and model-FLOPs throughput.

Parity: cubework/utils/profiling/flops.py:9-37 — ``calc_model_size`` counts each sharded parameter
``NUM_PARTITIONS`` times and averages over the TENSOR group; ``calc_tflops = 2*numel*tokens*(1 + 2*bwd
+ 1*ckpt) / (1e12*world) / time``.
"""
import torch

from ...global_vars import NUM_PARTITIONS
from ...parallel.collective import all_reduce
from ...parallel.mesh import pm
from ..common import get_current_device


def calc_model_size(model: torch.nn.Module):
    tp = pm.TENSOR.world_size if pm.TENSOR.is_initialized() else 0
    numel = 0
    numel_per_device = 0
    for p in model.parameters():
        parts = getattr(p, NUM_PARTITIONS, 0)
        numel += p.numel() * parts if (tp > 1 and parts > 1) else p.numel()
        numel_per_device += p.numel()
    if tp > 1:
        t = torch.tensor([float(numel)], dtype=torch.float64, device=get_current_device())
        if t.device.type == "cuda":
            t = t.float()
        numel = int(round((all_reduce(t, pm.TENSOR) / tp).item()))
    return numel, numel_per_device


def calc_tflops(numel: int, num_tokens: int, iter_time: float, with_backward=True, use_checkpoint=False) -> float:
    multiple = 1 + (2 if with_backward else 0) + (1 if use_checkpoint else 0)
    world = pm.GLOBAL.world_size if pm.GLOBAL.is_initialized() else 1
    return (numel * num_tokens * 2 * multiple / (1e12 * world)) / (iter_time + 1e-12)
