"""Fully sharded data parallelism (ZeRO stage 3) over the DATA group.

The reference offers it for OPT through ``torch.distributed.fsdp`` with ``FULL_SHARD``, one wrapped unit per
decoder layer, composed with 1D tensor parallelism (benchmark/opt/opt.py:544-562, flag ``--fsdp`` in
benchmark/opt/train.py:312).  This wrapper does the same job for the layers of this package:

* the parameters of every *unit* (a module of one of ``unit_classes``; everything else forms the root unit) are
  flattened into fp32 buffers, one per group of parameters with the same tensor-parallel partition count, and
  each rank of the DATA group keeps ``1 / dp`` of each buffer as the only persistent copy (an ``nn.Parameter``
  the optimizer updates);
* a unit's buffers are all-gathered right before its forward and again right before its backward, and dropped
  right after each (the root unit, whose parameters are used at both ends of the network, stays gathered from
  the start of forward to the end of backward);
* when every parameter of a buffer has its gradient, the flat gradient is reduce-scattered (averaged) into the
  shard's ``.grad`` and the full-size gradients are dropped.

Collectives go through the package's wrappers, so the communication profiler sees this traffic.  Gradient
clipping (:func:`cubework_b200.utils.clip_grad_norm`) recognises the shards by their ``fsdp_sharded`` stamp.
"""
from contextlib import contextmanager

import torch
import torch.nn as nn
from torch.autograd import Variable

from .. import ops
from ..global_vars import NUM_PARTITIONS
from .collective import all_gather, broadcast, reduce_scatter
from .mesh import pm

FSDP_SHARDED = "fsdp_sharded"


class _FlatGroup:
    """Parameters of one unit that share dtype and partition count, stored as one flat buffer."""

    def __init__(self, params, names, mode, root):
        self.params, self.names, self.mode, self.root = params, names, mode, root
        self.shapes = [p.shape for p in params]
        self.numels = [p.numel() for p in params]
        dp = mode.world_size
        total = sum(self.numels)
        self.padded = (total + dp - 1) // dp * dp
        flat = torch.zeros(self.padded, dtype=params[0].dtype, device=params[0].device)
        off = 0
        for p, n in zip(params, self.numels):
            flat[off:off + n] = p.data.reshape(-1)
            off += n
        if dp > 1:      # replicas start from identical values, like DistributedDataParallel's initial broadcast
            broadcast(flat, mode.rank_by_idx(0), mode)
        per = self.padded // dp
        self.shard = nn.Parameter(flat[mode.local_rank * per:(mode.local_rank + 1) * per].clone())
        setattr(self.shard, FSDP_SHARDED, True)
        parts = getattr(params[0], NUM_PARTITIONS, 0)
        if parts > 0:
            setattr(self.shard, NUM_PARTITIONS, parts)
        self.full = None
        self.ready = 0
        self.empty = torch.empty(0, dtype=flat.dtype, device=flat.device)
        for p in params:
            p.data = self.empty

    def gather(self):
        if self.full is not None:
            return
        self.full = all_gather(self.shard.data, 0, self.mode).contiguous() if self.mode.world_size > 1 \
            else self.shard.data.clone()
        off = 0
        for p, n, shape in zip(self.params, self.numels, self.shapes):
            p.data = self.full[off:off + n].view(shape)
            ops.drop_shadow(p)
            off += n

    def release(self):
        if self.full is None:
            return
        for p in self.params:
            p.data = self.empty
            ops.drop_shadow(p)
        self.full = None

    def reduce_grads(self):
        """Flat gradient -> reduce-scatter (mean over the DATA group) -> ``shard.grad``; full gradients dropped."""
        flat = torch.zeros(self.padded, dtype=self.shard.dtype, device=self.shard.device)
        off = 0
        for p, n in zip(self.params, self.numels):
            if p.grad is not None:
                flat[off:off + n] = p.grad.reshape(-1)
                p.grad = None
            off += n
        dp = self.mode.world_size
        if dp > 1:
            flat.div_(dp)
            g = reduce_scatter(flat, 0, self.mode).contiguous()
        else:
            g = flat
        if self.shard.grad is None:
            self.shard.grad = g
        else:
            self.shard.grad.add_(g)
        self.ready = 0


class FullyShardedDataParallel(nn.Module):

    def __init__(self, module, unit_classes=(), mode=None):
        super().__init__()
        self.module = module
        self.mode = mode or pm.DATA
        unit_classes = tuple(unit_classes)
        claimed = set()
        self._groups = []
        self._group_of = {}
        self._callback_queued = False
        self._in_backward = False
        units = [m for m in module.modules() if unit_classes and isinstance(m, unit_classes)]
        for unit in units + [module]:
            root = unit is module
            named = [(n, p) for n, p in unit.named_parameters() if id(p) not in claimed and p.requires_grad]
            if not named:
                continue
            claimed.update(id(p) for _, p in named)
            buckets = {}
            for n, p in named:
                buckets.setdefault((p.dtype, getattr(p, NUM_PARTITIONS, 0)), []).append((n, p))
            groups = []
            for items in buckets.values():
                g = _FlatGroup([p for _, p in items], [n for n, _ in items], self.mode, root)
                groups.append(g)
                self._groups.append(g)
                for p in g.params:
                    self._group_of[p] = g
                    p.register_post_accumulate_grad_hook(self._on_grad)
            if root:
                self._root_groups = groups
                module.register_forward_pre_hook(lambda m, a, gs=groups: self._gather(gs))
                # without a backward pass to end the step (evaluation) everything is dropped after the forward
                module.register_forward_hook(
                    lambda m, a, o: None if torch.is_grad_enabled() else self._release(self._groups))
            else:
                unit.register_forward_pre_hook(lambda m, a, gs=groups: self._gather(gs))
                unit.register_forward_hook(lambda m, a, o, gs=groups: self._release(gs))
                unit.register_full_backward_pre_hook(lambda m, go, gs=groups: self._gather(gs))
        if not hasattr(self, "_root_groups"):
            self._root_groups = []
        self._shards = nn.ParameterList([g.shard for g in self._groups])

    # ---- the optimizer, clipping and checkpoints see the shards, not the (mostly empty) original parameters
    def parameters(self, recurse=True):
        return iter(self._shards)

    def named_parameters(self, prefix="", recurse=True, remove_duplicate=True):
        for i, s in enumerate(self._shards):
            yield f"{prefix}{'.' if prefix else ''}_shards.{i}", s

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def _gather(self, groups):
        for g in groups:
            g.gather()

    def _release(self, groups):
        for g in groups:
            g.release()

    def _on_grad(self, p):
        g = self._group_of[p]
        g.ready += 1
        if not self._callback_queued:
            Variable._execution_engine.queue_callback(self._finish_backward)
            self._callback_queued = True
        if g.ready == len(g.params):
            g.reduce_grads()
            if not g.root:
                g.release()

    def _finish_backward(self):
        for g in self._groups:
            if g.ready > 0 or any(p.grad is not None for p in g.params):
                g.reduce_grads()
            g.release()
        self._callback_queued = False

    @contextmanager
    def summon_full_params(self):
        """All parameters gathered (read-only use: evaluation without hooks firing, checkpoints, tests)."""
        self._gather(self._groups)
        try:
            yield self.module
        finally:
            self._release(self._groups)

    def full_state_dict(self):
        """Unsharded (over the DATA group) copy of every parameter, by its name in the wrapped module."""
        out = {}
        with self.summon_full_params():
            for n, p in self.module.named_parameters():
                out[n] = p.detach().clone()
        return out

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)
