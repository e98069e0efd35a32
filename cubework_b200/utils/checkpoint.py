"""Sharded checkpoints with an explicit layout record.

The reference has no save/load code; its layout is implicit in each rank's ``state_dict()``
(see the slicing recipes in tests/test_{1,2,3}d/check_*_modules.py).  Here the layout is written down:

    <dir>/step_<N>/meta.json          mode, tp/dp sizes, rank table, and per parameter: global shape,
                                      shard spec [(dim, group name), ...] in nesting order, orientation
    <dir>/step_<N>/tp<r>_dp<d>.pt     that rank's model shards, optimizer state shards, per-group RNG
                                      streams, step / scheduler / scaler state

Data-parallel replicas hold identical shards, so only replica 0 (``dp0``) writes them - unless the model is
wrapped in :class:`~cubework_b200.parallel.fsdp.FullyShardedDataParallel`, whose flat shards and optimizer moments
differ on every DATA rank: then every rank writes its own ``tp<r>_dp<d>.pt``, ``meta.json`` records ``fsdp`` and the
data-parallel size, and a resume refuses a different one.  Consolidating such a checkpoint goes through the wrapper
(``FullyShardedDataParallel.full_state_dict``), which knows the original parameter names.

``gather_tensor`` / ``shard_tensor`` invert each other from the spec alone, so a checkpoint can be
consolidated (``full_state_dict``) and loaded into a different mode or tensor-parallel size
(``load_full_state_dict``): 1D <-> 2D <-> 3D.  Linear weights stored ``[in, out]`` (2D/3D) are
canonicalised to ``[out, in]`` in the consolidated form.
"""
import json
import os

import torch

from ..global_vars import env
from ..parallel.collective import all_gather
from ..parallel.common import get_shard_spec
from ..parallel.mesh import pm


def _norm_dim(d, ndim):
    return d % ndim


def shard_tensor(full, spec):
    """Local shard of ``full`` for this rank: chunk along each (dim, group) in nesting order."""
    out = full
    for dim, name in spec:
        m = pm.get(name)
        out = torch.chunk(out, m.world_size, dim=_norm_dim(dim, out.dim()))[m.local_rank]
    return out.contiguous()


def gather_tensor(local, spec):
    """Inverse of :func:`shard_tensor`: all-gather along each (dim, group) in reverse nesting order."""
    out = local
    for dim, name in reversed(spec):
        out = all_gather(out.contiguous(), _norm_dim(dim, out.dim()), pm.get(name)).contiguous()
    return out


def global_shape(local_shape, spec):
    shape = list(local_shape)
    for dim, name in spec:
        shape[_norm_dim(dim, len(shape))] *= pm.get(name).world_size
    return shape


def _named_unique_params(model):
    seen = {}
    for name, p in model.named_parameters(remove_duplicate=False):
        if id(p) in seen:
            continue
        seen[id(p)] = name
        yield name, p


def _strip(name):
    return name[len("module."):] if name.startswith("module.") else name


def _is_fsdp(model):
    return any(getattr(p, "fsdp_sharded", False) for p in model.parameters())


def _unwrap_fsdp(model):
    """The wrapper whose ``summon_full_params`` restores the original parameters, or None."""
    m = model
    while m is not None:
        if hasattr(m, "summon_full_params") and hasattr(m, "_shards"):
            return m
        m = getattr(m, "module", None)
    return None


def full_state_dict(model):
    """Every parameter gathered to its logical (unsharded, ``[out, in]``) form, on every rank.  A fully sharded
    data-parallel wrapper is gathered over the DATA group first, then each parameter over its tensor-parallel
    groups."""
    if _is_fsdp(model):
        w = _unwrap_fsdp(model)
        if w is None:
            raise ValueError("the model holds fully-sharded (DATA group) parameters but no wrapper that can gather them")
        with w.summon_full_params() as inner:
            # the gathered parameters are views of transient buffers: full_state_dict copies (all_gather / clone)
            return {k: v.clone() for k, v in full_state_dict(inner).items()}
    out, done = {}, {}
    with torch.no_grad():
        for name, p in model.named_parameters(remove_duplicate=False):
            if id(p) not in done:   # tied parameters appear under every name they have
                t = gather_tensor(p.detach(), get_shard_spec(p))
                if getattr(p, "STORED_IN_OUT", False):
                    t = t.t().contiguous()
                done[id(p)] = t
            out[_strip(name)] = done[id(p)]
    return out


def load_full_state_dict(model, full):
    """Slice logical tensors into this rank's shards (any mode / tensor-parallel size)."""
    if _is_fsdp(model):
        raise ValueError("load the logical tensors into the plain model first, then wrap it in FullyShardedDataParallel")
    with torch.no_grad():
        for name, p in _named_unique_params(model):
            t = full[_strip(name)]
            if getattr(p, "STORED_IN_OUT", False):
                t = t.t()
            p.copy_(shard_tensor(t.to(p.device), get_shard_spec(p)).to(p.dtype))


def layout_meta(model):
    params = {}
    for name, p in _named_unique_params(model):
        spec = get_shard_spec(p)
        params[_strip(name)] = dict(local_shape=list(p.shape), global_shape=global_shape(p.shape, spec), spec=spec,
                                    stored_in_out=bool(getattr(p, "STORED_IN_OUT", False)), dtype=str(p.dtype))
    # tied parameters are stored once, under the first of their names; the others are recorded as aliases
    first, aliases = {}, {}
    for name, p in model.named_parameters(remove_duplicate=False):
        if id(p) in first:
            aliases[_strip(name)] = first[id(p)]
        else:
            first[id(p)] = _strip(name)
    return dict(mode=env.mode, tp_size=pm.tp_size, dp_size=pm.dp_size, summa_dim=env.summa_dim,
                depth_3d=env.depth_3d, rank_table=pm.table, params=params, aliases=aliases, fsdp=_is_fsdp(model))


def _rng_states():
    out = {"cpu": torch.get_rng_state()}
    if torch.cuda.is_available():
        out["cuda"] = torch.cuda.get_rng_state()
    for m in pm.modes():
        if m.is_initialized():
            out[m.name] = (m.rng_state, m.cuda_rng_state)
    return out


def _set_rng_states(st):
    torch.set_rng_state(st["cpu"])
    if "cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["cuda"])
    for m in pm.modes():
        if m.is_initialized() and m.name in st:
            m.set_rng_states(*st[m.name])


def _ranks():
    tp_rank = pm.TENSOR.local_rank if pm.TENSOR.is_initialized() else 0
    dp_rank = pm.DATA.local_rank if pm.DATA.is_initialized() else 0
    return tp_rank, dp_rank


def step_dir(root, step):
    return os.path.join(root, f"step_{step}")


def save_checkpoint(root, step, model, optimizer=None, lr_scheduler=None, scaler=None, extra=None):
    """Every rank that holds distinct state writes its own shard file; global rank 0 also writes ``meta.json``.

    Data-parallel replicas hold identical model shards and optimizer state, so only replica 0 writes them; under
    fully sharded data parallelism every DATA rank holds a different slice and writes ``tp<r>_dp<d>.pt``."""
    d = step_dir(root, step)
    os.makedirs(d, exist_ok=True)
    tp_rank, dp_rank = _ranks()
    meta = layout_meta(model)
    meta["step"] = step
    if pm.GLOBAL.rank in (0, None):
        with open(os.path.join(d, "meta.json"), "w") as f:
            json.dump(meta, f, indent=1)
    fsdp = meta["fsdp"]
    if dp_rank == 0 or fsdp:
        payload = dict(step=step, model={_strip(k): v.detach().cpu() for k, v in _named_unique_params(model)},
                       rng=_rng_states(), extra=extra)
        if optimizer is not None:
            payload["optimizer"] = optimizer.state_dict()
        if lr_scheduler is not None:
            payload["lr_scheduler"] = lr_scheduler.state_dict()
        if scaler is not None:
            payload["scaler"] = scaler.state_dict()
        torch.save(payload, os.path.join(d, f"tp{tp_rank}_dp{dp_rank if fsdp else 0}.pt"))
    if torch.distributed.is_initialized():
        torch.distributed.barrier(group=pm.GLOBAL.cpu_group if pm.GLOBAL.is_initialized() else None)
    return d


def load_checkpoint(root, step, model, optimizer=None, lr_scheduler=None, scaler=None, restore_rng=True):
    """Resume into the *same* layout the checkpoint was written with (checked against ``meta.json``)."""
    d = step_dir(root, step)
    with open(os.path.join(d, "meta.json")) as f:
        meta = json.load(f)
    if meta["mode"] != env.mode or meta["tp_size"] != pm.tp_size:
        raise ValueError(f"checkpoint layout (mode={meta['mode']}, tp={meta['tp_size']}) differs from the running "
                         f"one (mode={env.mode}, tp={pm.tp_size}); consolidate it and use load_full_state_dict")
    fsdp = bool(meta.get("fsdp", False))
    if fsdp != _is_fsdp(model):
        raise ValueError(f"checkpoint was written {'with' if fsdp else 'without'} fully sharded data parallelism, the "
                         f"running model is {'' if _is_fsdp(model) else 'not '}wrapped in it")
    if fsdp and meta["dp_size"] != pm.dp_size:
        raise ValueError(f"fully sharded checkpoint of {meta['dp_size']} data-parallel ranks cannot be resumed on "
                         f"{pm.dp_size}; consolidate it through the wrapper's full_state_dict instead")
    tp_rank, dp_rank = _ranks()
    payload = torch.load(os.path.join(d, f"tp{tp_rank}_dp{dp_rank if fsdp else 0}.pt"), map_location="cpu",
                         weights_only=False)
    with torch.no_grad():
        for name, p in _named_unique_params(model):
            p.copy_(payload["model"][_strip(name)].to(p.device))
    if optimizer is not None and "optimizer" in payload:
        optimizer.load_state_dict(payload["optimizer"])
    if lr_scheduler is not None and "lr_scheduler" in payload:
        lr_scheduler.load_state_dict(payload["lr_scheduler"])
    if scaler is not None and "scaler" in payload:
        scaler.load_state_dict(payload["scaler"])
    if restore_rng:
        _set_rng_states(payload["rng"])
    return payload["step"], payload.get("extra")


def consolidate(root, step):
    """Offline (single process, no process group): rebuild every logical tensor from the shard files."""
    d = step_dir(root, step)
    with open(os.path.join(d, "meta.json")) as f:
        meta = json.load(f)
    if meta.get("fsdp", False):
        raise ValueError("a fully sharded (DATA group) checkpoint stores flat buffers without parameter names; "
                         "consolidate it online with FullyShardedDataParallel.full_state_dict / full_state_dict(model)")
    tp = meta["tp_size"] if meta["mode"] is not None else 1
    shards = [torch.load(os.path.join(d, f"tp{r}_dp0.pt"), map_location="cpu", weights_only=False)["model"]
              for r in range(tp)]
    table = meta["rank_table"]
    full = {}
    for name, info in meta["params"].items():

        def build(level, members):
            """``members``: tp ranks that agree on the chunk indices of spec[:level]."""
            if level == len(info["spec"]):
                return shards[members[0]][name]
            dim, group = info["spec"][level]
            groups = [g for g in table[group] if g[0] < tp]   # replica 0's groups (global rank == tp rank)
            n = len(groups[0])
            pieces = []
            for idx in range(n):
                sub = [r for r in members if any(r in g and g.index(r) == idx for g in groups)]
                pieces.append(build(level + 1, sub))
            return torch.cat(pieces, dim=dim % pieces[0].dim())

        t = build(0, list(range(tp)))
        if info["stored_in_out"]:
            t = t.t().contiguous()
        full[name] = t
    for alias, name in meta.get("aliases", {}).items():
        full[alias] = full[name]
    return full, meta
