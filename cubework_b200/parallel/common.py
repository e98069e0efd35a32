"""Small helpers shared by the parallel layers.

Parity: cubework/module/utils.py:10-92 — ``set_tensor_parallel_attribute_by_partition``,
``get_tensor_parallel_mode``, ``to_2tuple``, ``split_tensor`` and the asynchronous gradient bucket
(``push_async_grad`` / ``register_async_grad_hook`` / ``synchronize``).

The bucket differs from the reference's: the reference returns a *zero* gradient to autograd and adds
the real one from a tensor hook (module/utils.py:47-49,79-81).  Here the in-flight reduction is
attached to the gradient tensor that autograd delivers, and the hook only waits for it, so there is no
zero-fill and no extra add; ``synchronize`` drains whatever no hook consumed.
"""
import collections.abc
from itertools import repeat

import torch

from ..global_vars import NUM_PARTITIONS, env


SHARD_SPEC = "SHARD_SPEC"


def set_tensor_parallel_attribute_by_partition(param, num_partitions, spec=None):
    """Stamp the number of distinct shards and, optionally, how the shard was cut.

    ``spec`` is a list of ``(dim, group name)`` in nesting order: the logical tensor is chunked along
    ``dim`` over the named group, then the result along the next entry, and so on.  Parameters without
    a spec are replicated.  The checkpoint code gathers / reshards from this record alone.
    """
    setattr(param, NUM_PARTITIONS, num_partitions)
    if spec is not None:
        setattr(param, SHARD_SPEC, [(int(d), m if isinstance(m, str) else m.name) for d, m in spec])


def get_shard_spec(param):
    return list(getattr(param, SHARD_SPEC, []))


def get_tensor_parallel_mode():
    return env.mode


def to_2tuple(x):
    if isinstance(x, collections.abc.Iterable):
        return tuple(x)
    return tuple(repeat(x, 2))


def split_tensor(tensor, dim, parallel_mode):
    """This rank's chunk of ``tensor`` along ``dim`` for the given group."""
    if tensor.size(dim) <= 1 or parallel_mode.world_size == 1:
        return tensor
    return torch.chunk(tensor, parallel_mode.world_size, dim=dim)[parallel_mode.local_rank].contiguous()


class AsyncGradientBucket(object):
    """In-flight parameter-gradient reductions keyed by ``id(param)``."""

    def __init__(self):
        self.pending = {}

    def __len__(self):
        return len(self.pending)

    def push(self, work, grad, param_id):
        """Remember ``work`` (may be None) that is still writing ``grad``; returns ``grad``."""
        self.pending.setdefault(param_id, []).append(work)
        return grad

    def wait(self, param_id):
        for w in self.pending.pop(param_id, []):
            if w is not None:
                w.wait()

    def synchronize(self, params=()):
        for p in params:
            self.wait(id(p))
        for pid in list(self.pending):
            self.wait(pid)


_bucket = AsyncGradientBucket()


def push_async_grad(work, grad, param_id):
    return _bucket.push(work, grad, param_id)


def register_async_grad_hook(param):
    pid = id(param)

    def _hook(grad):
        _bucket.wait(pid)
        return grad

    param.register_hook(_hook)


def synchronize(params=(), host_sync=True):
    """Wait for every outstanding asynchronous parameter-gradient reduction.

    The reductions are awaited on the current stream (``work.wait()`` orders the stream behind the collective, it does
    not block the host).  ``host_sync`` additionally blocks the host until the stream has drained, which is what a
    caller that is about to read gradients on the host wants (the reference's ``synchronize``, module/utils.py:88-92);
    the training engine passes ``False`` so that the host keeps running ahead of the device."""
    _bucket.synchronize(params)
    if host_sync and torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()
    if len(_bucket) > 0:
        raise RuntimeError(f"{len(_bucket)} asynchronous gradient(s) not collected.")
