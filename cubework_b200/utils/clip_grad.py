"""Global-norm gradient clipping that understands sharded parameters.

Parity: cubework/utils/clip_grad.py:16-70.  A parameter stamped with ``NUM_PARTITIONS = p`` is held in
``p`` distinct shards across the TENSOR group and replicated ``tp / p`` times, so each rank adds
``|g|^k * p`` and the group sum is divided by ``tp``; unstamped (fully replicated) parameters are
counted once, locally (clip_grad.py:36-55).  The infinity norm uses a MAX all-reduce
(clip_grad.py:28-34).  On CUDA the per-tensor norms and the scaling are one multi-tensor kernel each.
"""
import math

import torch
from torch.distributed import ReduceOp

from ..global_vars import NUM_PARTITIONS
from ..parallel.collective import all_reduce
from ..parallel.mesh import pm


def _grads(parameters):
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    return [p for p in parameters if p.grad is not None]


def clip_grad_norm(parameters, max_norm, norm_type=2):
    params = _grads(parameters)
    max_norm = float(max_norm)
    norm_type = float(norm_type)
    if len(params) == 0:
        return 0.0
    tp_on = pm.TENSOR.is_initialized() and pm.TENSOR.world_size > 1
    dp_on = pm.DATA.is_initialized() and pm.DATA.world_size > 1
    device = params[0].grad.device
    from .. import ops
    # shards of fully-sharded data parallelism hold 1/dp of a gradient: their sums also run over the DATA group
    sharded = [p for p in params if getattr(p, "fsdp_sharded", False)]
    whole = [p for p in params if not getattr(p, "fsdp_sharded", False)]
    if math.isinf(norm_type):
        total = torch.stack([p.grad.detach().abs().max().float() for p in params]).max().reshape(1)
        if tp_on:
            total = all_reduce(total, pm.TENSOR, op=ReduceOp.MAX)
        if sharded and dp_on:
            total = all_reduce(total, pm.DATA, op=ReduceOp.MAX)
        total_norm = total
    else:
        zero = torch.zeros(1, dtype=torch.float32, device=device)

        def acc(subset):
            """fp32 tensor [1] = sum_i w_i * |g_i|^k over the subset, tensor-parallel shards counted once"""
            if not subset:
                return zero
            tp_params = [p for p in subset if getattr(p, NUM_PARTITIONS, 0) > 0]
            std_params = [p for p in subset if getattr(p, NUM_PARTITIONS, 0) <= 0]
            std_acc = ops.grad_norm_pow(std_params, [1.0] * len(std_params), norm_type) if std_params else zero
            tp_acc = zero
            if tp_params:
                tp_acc = ops.grad_norm_pow(tp_params, [float(getattr(p, NUM_PARTITIONS)) for p in tp_params], norm_type)
                if tp_on:
                    tp_acc = all_reduce(tp_acc, pm.TENSOR) / pm.TENSOR.world_size
            return std_acc + tp_acc

        total = acc(whole)
        if sharded:
            part = acc(sharded)
            if dp_on:
                part = all_reduce(part.clone(), pm.DATA)
            total = total + part
        total_norm = total.pow(1.0 / norm_type)
    clip_coef = (max_norm / (total_norm + 1e-6)).clamp(max=1.0)
    ops.scale_grads(params, clip_coef)
    return total_norm.to(device)
