"""Data loading helpers.

Parity: cubework/utils/data.py:9-26 (``get_dataloader`` = ``DataLoader`` + ``DistributedSampler``).
The sampler here shards over the DATA group (replica index / replica count), so tensor-parallel peers
read identical samples; the reference shards over the global world instead.  ``SyntheticLoader``
produces fixed-shape random batches in pinned host memory for the benchmark entry points.
"""
import torch
from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler

from ..parallel.mesh import pm


def get_dataloader(dataset, shuffle=False, seed=1024, add_sampler=True, drop_last=False, pin_memory=False,
                   num_workers=0, **kwargs):
    _kwargs = dict(kwargs)
    if add_sampler and pm.DATA.is_initialized() and pm.DATA.world_size > 1:
        sampler = DistributedSampler(dataset, num_replicas=pm.DATA.world_size, rank=pm.DATA.local_rank,
                                     shuffle=shuffle, seed=seed, drop_last=drop_last)
        return DataLoader(dataset, sampler=sampler, drop_last=drop_last, pin_memory=pin_memory,
                          num_workers=num_workers, **_kwargs)
    return DataLoader(dataset, shuffle=shuffle, drop_last=drop_last, pin_memory=pin_memory,
                      num_workers=num_workers, **_kwargs)


class SyntheticLoader:
    """Endless iterator over ``n_distinct`` pre-generated batches held in pinned host memory.

    ``make_batch(generator) -> dict[str, Tensor]`` builds one CPU batch.  Batches are identical on
    every rank of a DATA replica because the generator is seeded from the replica index only.
    """

    def __init__(self, make_batch, n_distinct=4, seed=1234, length=None):
        replica = pm.DATA.local_rank if pm.DATA.is_initialized() else 0
        g = torch.Generator().manual_seed(seed + 7919 * replica)
        pin = torch.cuda.is_available()
        self.batches = []
        for _ in range(n_distinct):
            b = make_batch(g)
            self.batches.append({k: (v.pin_memory() if pin else v) for k, v in b.items()})
        self.length = length
        self._i = 0

    def __len__(self):
        return self.length if self.length is not None else 1 << 30

    def __iter__(self):
        return self

    def __next__(self):
        b = self.batches[self._i % len(self.batches)]
        self._i += 1
        return b

    def bytes_per_batch(self):
        return sum(v.numel() * v.element_size() for v in self.batches[0].values())
