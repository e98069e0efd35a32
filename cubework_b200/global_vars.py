"""Process-group kind names and the construction-time environment singleton.

Parity: cubework/global_vars.py:1-80 (constants, ``TensorParallelEnv`` with ``load``/``save``).
The environment holds the *mutable* state that user model code relies on while it builds
layers one after another (1D column/row alternation, 3D input/output group swapping, the
vocab-parallel flag).  Everything that is fixed once the process groups exist lives in
:mod:`cubework_b200.parallel.mesh` instead.
"""
from typing import Optional

ALLOWED_MODES = [None, "1d", "2d", "3d"]

GLOBAL = "GLOBAL"
DATA = "DATA"
TENSOR = "TENSOR"
NUM_PARTITIONS = "NUM_PARTITIONS"
VOCAB_PARALLEL = "VOCAB_PARALLEL"
PARALLEL_1D = "PARALLEL_1D"
PARALLEL_2D_ROW = "PARALLEL_2D_ROW"
PARALLEL_2D_COL = "PARALLEL_2D_COL"
PARALLEL_3D_INPUT = "PARALLEL_3D_INPUT"
PARALLEL_3D_WEIGHT = "PARALLEL_3D_WEIGHT"
PARALLEL_3D_OUTPUT = "PARALLEL_3D_OUTPUT"
PARALLEL_3D_INPUT_X_WEIGHT = "PARALLEL_3D_INPUT_X_WEIGHT"
PARALLEL_3D_OUTPUT_X_WEIGHT = "PARALLEL_3D_OUTPUT_X_WEIGHT"

ALL_MODE_NAMES = [
    DATA, GLOBAL, TENSOR, PARALLEL_1D, PARALLEL_2D_COL, PARALLEL_2D_ROW, PARALLEL_3D_INPUT,
    PARALLEL_3D_WEIGHT, PARALLEL_3D_OUTPUT, PARALLEL_3D_INPUT_X_WEIGHT, PARALLEL_3D_OUTPUT_X_WEIGHT
]

_FIELDS = dict(
    mode=None,
    vocab_parallel=False,
    parallel_input_1d=False,
    summa_dim=None,
    depth_3d=None,
    input_group_3d=None,
    weight_group_3d=None,
    output_group_3d=None,
    input_x_weight_group_3d=None,
    output_x_weight_group_3d=None,
)


class TensorParallelEnv(object):
    """Singleton; ``env.load(**state)`` / ``env.save()`` round-trip a plain dict."""
    _instance = None

    def __new__(cls, *args, **kwargs):
        if cls._instance is None:
            cls._instance = object.__new__(cls)
        return cls._instance

    def __init__(self, *args, **kwargs):
        self.load(*args, **kwargs)

    def load(self, mode: Optional[str] = None, **kwargs):
        state = dict(_FIELDS)
        state["mode"] = mode
        unknown = set(kwargs) - set(_FIELDS)
        if unknown:
            raise TypeError(f"unknown env fields: {sorted(unknown)}")
        state.update(kwargs)
        for k, v in state.items():
            setattr(self, k, v)

    def save(self):
        return {k: getattr(self, k) for k in _FIELDS}

    def swap_in_out_3d(self):
        """Exchange the roles of the 3D input and output groups (and the two x-weight groups)."""
        self.input_group_3d, self.output_group_3d = self.output_group_3d, self.input_group_3d
        self.input_x_weight_group_3d, self.output_x_weight_group_3d = (self.output_x_weight_group_3d,
                                                                       self.input_x_weight_group_3d)


env = TensorParallelEnv()
