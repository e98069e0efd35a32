"""Process-group topology: a declarative rank table + the ``ParallelMode`` registry built from it.

Parity: cubework/distributed/utils.py:21-452 (``ParallelMode``, ``ParallelManager``, ``init_global``,
``init_data_parallel``, ``init_{1d,2d,3d}_parallel``, ``init_tensor_parallel``,
``destroy_distributed``).  The rank formulas are the reference's:

* DATA group ``i``     = ``[i + j*tp for j < dp]``                       (utils.py:129-152)
* TENSOR group ``i``   = ``[i*tp + j for j < tp]``; seed ``seed+1024+tp_rank``   (utils.py:410-443)
* 2D, in-TP rank ``r = row*q + col``: COL group varies ``row``, ROW group varies ``col`` (utils.py:189-248)
* 3D, in-TP rank ``r = i + d*(j + d*k)``: INPUT varies ``j``, WEIGHT varies ``i``, OUTPUT varies ``k``,
  INPUT_X_WEIGHT varies ``(j, i)`` at fixed ``k``, OUTPUT_X_WEIGHT varies ``(k, i)`` at fixed ``j``
  (utils.py:251-400)

Design difference: the table of groups is computed by a pure function (:func:`build_rank_table`) that
needs no process group, so layouts are unit-testable on one CPU process and are what the checkpoint
metadata records.  Group creation is then one loop over that table.  RNG capture works without CUDA.
"""
import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import global_vars as gv
from ..global_vars import env


def build_rank_table(world_size: int, tp_size: Optional[int], mode: Optional[str]) -> Dict[str, List[List[int]]]:
    """Every process group of every kind, as lists of global ranks, for the whole job."""
    table: Dict[str, List[List[int]]] = {gv.GLOBAL: [list(range(world_size))]}
    tp = tp_size if (mode is not None and tp_size) else 1
    if world_size % tp != 0:
        raise ValueError(f"world size {world_size} is not a multiple of tensor parallel size {tp}")
    dp = world_size // tp
    table[gv.DATA] = [[i + j * tp for j in range(dp)] for i in range(tp)]
    if mode is None:
        return table
    n_rep = world_size // tp
    table[gv.TENSOR] = [[h * tp + j for j in range(tp)] for h in range(n_rep)]
    if mode == "1d":
        table[gv.PARALLEL_1D] = [list(g) for g in table[gv.TENSOR]]
    elif mode == "2d":
        q = int(math.isqrt(tp))
        if q * q != tp:
            raise ValueError(f"2D tensor parallelism needs a square size, got {tp}")
        table[gv.PARALLEL_2D_COL] = [[h * tp + row * q + col for row in range(q)] for h in range(n_rep)
                                     for col in range(q)]
        table[gv.PARALLEL_2D_ROW] = [[h * tp + row * q + col for col in range(q)] for h in range(n_rep)
                                     for row in range(q)]
    elif mode == "3d":
        d = round(tp**(1 / 3))
        if d**3 != tp:
            raise ValueError(f"3D tensor parallelism needs a cubic size, got {tp}")

        def r(h, i, j, k):
            return h * tp + i + d * (j + d * k)

        R = range(d)
        table[gv.PARALLEL_3D_INPUT] = [[r(h, i, j, k) for j in R] for h in range(n_rep) for i in R for k in R]
        table[gv.PARALLEL_3D_WEIGHT] = [[r(h, i, j, k) for i in R] for h in range(n_rep) for k in R for j in R]
        table[gv.PARALLEL_3D_OUTPUT] = [[r(h, i, j, k) for k in R] for h in range(n_rep) for i in R for j in R]
        table[gv.PARALLEL_3D_INPUT_X_WEIGHT] = [[r(h, i, j, k) for j in R for i in R] for h in range(n_rep)
                                                for k in R]
        table[gv.PARALLEL_3D_OUTPUT_X_WEIGHT] = [[r(h, i, j, k) for k in R for i in R] for h in range(n_rep)
                                                 for j in R]
    else:
        raise ValueError(f"unknown tensor parallel mode {mode!r}")
    return table


def grid_coords(mode: Optional[str], tp_size: int, tp_rank: int) -> Dict[str, int]:
    """Grid coordinates of an in-TP rank: 1D ``{r}``, 2D ``{row, col}``, 3D ``{i, j, k}``."""
    if mode == "1d":
        return {"r": tp_rank}
    if mode == "2d":
        q = int(math.isqrt(tp_size))
        return {"row": tp_rank // q, "col": tp_rank % q}
    if mode == "3d":
        d = round(tp_size**(1 / 3))
        return {"i": tp_rank % d, "j": (tp_rank // d) % d, "k": tp_rank // (d * d)}
    return {}


class ParallelMode(object):
    """One process-group kind as seen from this rank (name, ranks, NCCL/gloo handles, RNG stream)."""

    def __init__(self, name):
        self._name = name
        self._reset()

    def _reset(self):
        self._initialized = False
        self._rank = None
        self._local_rank = None
        self._world_size = None
        self._group = None
        self._cpu_group = None
        self._ranks_in_group = None
        self._rng_state = None
        self._cuda_rng_state = None
        self._owns_group = False

    name = property(lambda self: self._name)
    rank = property(lambda self: self._rank)
    local_rank = property(lambda self: self._local_rank)
    world_size = property(lambda self: self._world_size)
    group = property(lambda self: self._group)
    cpu_group = property(lambda self: self._cpu_group)
    ranks_in_group = property(lambda self: self._ranks_in_group)
    rng_state = property(lambda self: self._rng_state)
    cuda_rng_state = property(lambda self: self._cuda_rng_state)

    def rank_by_idx(self, idx):
        return self._ranks_in_group[idx]

    def is_initialized(self):
        return self._initialized

    def group_for(self, tensor):
        """gloo twin for host tensors, the device group otherwise (collective.py:19 in the reference)."""
        return self._cpu_group if tensor.device.type == "cpu" else self._group

    def init(self, rank, local_rank, world_size, process_group, cpu_group, ranks_in_group, seed=None,
             owns_group=True):
        self._initialized = True
        self._rank = rank
        self._local_rank = local_rank
        self._world_size = world_size
        self._group = process_group
        self._cpu_group = cpu_group
        self._ranks_in_group = list(ranks_in_group)
        self._owns_group = owns_group and process_group is not None
        use_cuda = torch.cuda.is_available()
        if seed is not None:
            cur = torch.get_rng_state()
            cur_cuda = torch.cuda.get_rng_state() if use_cuda else None
            torch.manual_seed(seed)
            self._rng_state = torch.get_rng_state()
            self._cuda_rng_state = torch.cuda.get_rng_state() if use_cuda else None
            torch.set_rng_state(cur)
            if use_cuda:
                torch.cuda.set_rng_state(cur_cuda)
        else:
            self._rng_state = torch.get_rng_state()
            self._cuda_rng_state = torch.cuda.get_rng_state() if use_cuda else None

    def set_rng_states(self, cpu_state, cuda_state=None):
        self._rng_state = cpu_state
        if cuda_state is not None:
            self._cuda_rng_state = cuda_state

    def destroy(self):
        if self._owns_group and self._group is not None:
            try:
                dist.destroy_process_group(self._group)
            except Exception:
                pass
        if self._cpu_group is not None and self._cpu_group is not self._group:
            try:
                dist.destroy_process_group(self._cpu_group)
            except Exception:
                pass
        self._reset()

    def __repr__(self):
        return f"ParallelMode({self._name}, local_rank={self._local_rank}, ranks={self._ranks_in_group})"


class ParallelManager(object):
    """Registry of the 11 group kinds (reference: distributed/utils.py:104-115); aliased ``pm``."""
    DATA = ParallelMode(gv.DATA)
    GLOBAL = ParallelMode(gv.GLOBAL)
    TENSOR = ParallelMode(gv.TENSOR)
    PARALLEL_1D = ParallelMode(gv.PARALLEL_1D)
    PARALLEL_2D_COL = ParallelMode(gv.PARALLEL_2D_COL)
    PARALLEL_2D_ROW = ParallelMode(gv.PARALLEL_2D_ROW)
    PARALLEL_3D_INPUT = ParallelMode(gv.PARALLEL_3D_INPUT)
    PARALLEL_3D_WEIGHT = ParallelMode(gv.PARALLEL_3D_WEIGHT)
    PARALLEL_3D_OUTPUT = ParallelMode(gv.PARALLEL_3D_OUTPUT)
    PARALLEL_3D_INPUT_X_WEIGHT = ParallelMode(gv.PARALLEL_3D_INPUT_X_WEIGHT)
    PARALLEL_3D_OUTPUT_X_WEIGHT = ParallelMode(gv.PARALLEL_3D_OUTPUT_X_WEIGHT)

    # filled by init_*: the rank table and this rank's grid position (recorded in checkpoints)
    table: Dict[str, List[List[int]]] = {}
    tp_size: int = 1
    dp_size: int = 1

    @classmethod
    def get(cls, name: str) -> ParallelMode:
        return getattr(cls, name)

    @classmethod
    def modes(cls):
        return [m for m in vars(cls).values() if isinstance(m, ParallelMode)]

    @classmethod
    def coords(cls) -> Dict[str, int]:
        if env.mode is None or not cls.TENSOR.is_initialized():
            return {}
        return grid_coords(env.mode, cls.TENSOR.world_size, cls.TENSOR.local_rank)


pm = ParallelManager


def _make_groups(kind: str, groups: List[List[int]], seed=None, reuse_default=False):
    """Create every group of one kind on every rank (``new_group`` is collective) and register ours."""
    rank = dist.get_rank()
    backend = dist.get_backend()
    mine = None
    for ranks in groups:
        if reuse_default and len(ranks) == dist.get_world_size():
            group = None
            owns = False
        else:
            group = dist.new_group(ranks)
            owns = True
        cpu_group = dist.new_group(ranks, backend="gloo") if backend != "gloo" else group
        if rank in ranks:
            mine = (ranks, group, cpu_group, owns)
    assert mine is not None, f"rank {rank} is in no {kind} group"
    ranks, group, cpu_group, owns = mine
    if group is None:
        group = dist.group.WORLD
    if cpu_group is None:
        cpu_group = dist.group.WORLD
    pm.get(kind).init(rank, ranks.index(rank), len(ranks), group, cpu_group, ranks, seed=seed, owns_group=owns)


def init_global():
    assert dist.is_initialized()
    world = dist.get_world_size()
    pm.table = {gv.GLOBAL: [list(range(world))]}
    _make_groups(gv.GLOBAL, pm.table[gv.GLOBAL], reuse_default=True)


def init_data_parallel(data_parallel_size):
    assert dist.is_initialized()
    world = dist.get_world_size()
    tp = world // data_parallel_size
    groups = [[i + j * tp for j in range(data_parallel_size)] for i in range(tp)]
    pm.table[gv.DATA] = groups
    pm.dp_size = data_parallel_size
    _make_groups(gv.DATA, groups)


def init_1d_parallel(tensor_parallel_size, seed):
    table = build_rank_table(dist.get_world_size(), tensor_parallel_size, "1d")
    pm.table[gv.PARALLEL_1D] = table[gv.PARALLEL_1D]
    # the 1D group is the TENSOR group: share its handles instead of creating a second communicator
    t = pm.TENSOR
    pm.PARALLEL_1D.init(t.rank, t.local_rank, t.world_size, t.group, t.cpu_group, t.ranks_in_group, seed=seed,
                        owns_group=False)
    env.parallel_input_1d = False


def init_2d_parallel(tensor_parallel_size, seed):
    table = build_rank_table(dist.get_world_size(), tensor_parallel_size, "2d")
    env.summa_dim = int(math.isqrt(tensor_parallel_size))
    for kind in (gv.PARALLEL_2D_COL, gv.PARALLEL_2D_ROW):
        pm.table[kind] = table[kind]
        _make_groups(kind, table[kind], seed=seed)


def init_3d_parallel(tensor_parallel_size, seed):
    table = build_rank_table(dist.get_world_size(), tensor_parallel_size, "3d")
    env.depth_3d = round(tensor_parallel_size**(1 / 3))
    for kind in (gv.PARALLEL_3D_INPUT, gv.PARALLEL_3D_WEIGHT, gv.PARALLEL_3D_OUTPUT,
                 gv.PARALLEL_3D_INPUT_X_WEIGHT, gv.PARALLEL_3D_OUTPUT_X_WEIGHT):
        pm.table[kind] = table[kind]
        _make_groups(kind, table[kind], seed=seed)
    env.input_group_3d = gv.PARALLEL_3D_INPUT
    env.weight_group_3d = gv.PARALLEL_3D_WEIGHT
    env.output_group_3d = gv.PARALLEL_3D_OUTPUT
    env.input_x_weight_group_3d = gv.PARALLEL_3D_INPUT_X_WEIGHT
    env.output_x_weight_group_3d = gv.PARALLEL_3D_OUTPUT_X_WEIGHT


_TENSOR_PARALLEL_INIT_FUNCS = {"1d": init_1d_parallel, "2d": init_2d_parallel, "3d": init_3d_parallel}


def init_tensor_parallel(tensor_parallel_size, seed):
    assert dist.is_initialized()
    world = dist.get_world_size()
    table = build_rank_table(world, tensor_parallel_size, env.mode)
    pm.table[gv.TENSOR] = table[gv.TENSOR]
    pm.tp_size = tensor_parallel_size
    _make_groups(gv.TENSOR, table[gv.TENSOR], reuse_default=True)
    tp_seed = seed + 1024 + pm.TENSOR.local_rank
    t = pm.TENSOR
    t.init(t.rank, t.local_rank, t.world_size, t.group, t.cpu_group, t.ranks_in_group, seed=tp_seed,
           owns_group=t._owns_group)
    _TENSOR_PARALLEL_INIT_FUNCS[env.mode](tensor_parallel_size, tp_seed)


def destroy_distributed():
    from . import symm
    symm.release_all()
    for mode in pm.modes():
        if mode.name != gv.GLOBAL and mode.is_initialized():
            mode.destroy()
    pm.GLOBAL._reset()
    pm.table = {}
    pm.tp_size = 1
    pm.dp_size = 1
    env.load()
    if dist.is_initialized():
        dist.destroy_process_group()
