from . import init
from .collective import all_gather, all_reduce, barrier, broadcast, reduce, reduce_scatter
from .common import (AsyncGradientBucket, get_tensor_parallel_mode, push_async_grad, register_async_grad_hook,
                     set_tensor_parallel_attribute_by_partition, split_tensor, synchronize, to_2tuple)
from .facade import (Classifier, DropPath, Dropout, Embedding, LayerNorm, Linear, PatchEmbedding,
                     partition_batch)
from .loss import CrossEntropyLoss
from .mesh import (ParallelManager, ParallelMode, build_rank_table, destroy_distributed, grid_coords,
                   init_1d_parallel, init_2d_parallel, init_3d_parallel, init_data_parallel, init_global,
                   init_tensor_parallel, pm)
from .metric import Accuracy, Perplexity
