"""``cubework.module`` API surface (reference: cubework/module/__init__.py:1-6): the mode-dispatching
layers, loss, metrics, initializers, plus the per-mode classes under their reference names."""
from ..parallel import init
from ..parallel.common import synchronize
from ..parallel.facade import (Classifier, DropPath, Dropout, Embedding, LayerNorm, Linear, PatchEmbedding,
                               gather_rows, mark_partial_grad, partition_batch, scatter_rows,
                               sequence_parallel_size, sum_grad_over_rows)
from ..parallel.init import *  # noqa: F401,F403
from ..parallel.layers_1d import (Classifier1D, Dropout1D, Embedding1D, LayerNorm1D, Linear1D, Linear1D_Col,
                                  Linear1D_Row, PatchEmbedding1D, VocabParallelClassifier1D,
                                  VocabParallelEmbedding1D)
from ..parallel.layers_2d import (Classifier2D, Embedding2D, LayerNorm2D, Linear2D, PatchEmbedding2D,
                                  VocabParallelClassifier2D, VocabParallelEmbedding2D)
from ..parallel.layers_3d import (Classifier3D, Embedding3D, LayerNorm3D, Linear3D, PatchEmbedding3D,
                                  VocabParallelClassifier3D, VocabParallelEmbedding3D)
from ..parallel.loss import (CrossEntropyLoss, CrossEntropyLoss2D, CrossEntropyLoss3D,
                             VocabParallelCrossEntropyLoss1D, VocabParallelCrossEntropyLoss2D,
                             VocabParallelCrossEntropyLoss3D)
from ..parallel.metric import Accuracy, Perplexity
from ..parallel.std import ClassifierSTD, PatchEmbeddingSTD
