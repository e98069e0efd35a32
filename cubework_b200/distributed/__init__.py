"""``cubework.distributed`` API surface (reference: cubework/distributed/__init__.py:1-11)."""
from ..parallel.collective import all_gather, all_reduce, barrier, broadcast, reduce, reduce_scatter
from ..parallel.mesh import (ParallelManager, ParallelMode, build_rank_table, destroy_distributed,
                             init_1d_parallel, init_2d_parallel, init_3d_parallel, init_data_parallel,
                             init_global, init_tensor_parallel)

__all__ = [
    "all_gather", "all_reduce", "barrier", "broadcast", "reduce", "reduce_scatter", "ParallelManager",
    "ParallelMode", "build_rank_table", "destroy_distributed", "init_1d_parallel", "init_2d_parallel",
    "init_3d_parallel", "init_data_parallel", "init_global", "init_tensor_parallel"
]
