"""Process start-up.

Parity: cubework/initialize.py:24-59 — reads ``RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR /
MASTER_PORT``, creates the default process group, the logger, binds the device, then the GLOBAL and
DATA groups (``dp = world // tp_size``), seeds the RNGs (default 1024), records the mode in ``env`` and
builds the tensor-parallel groups.  The backend defaults to NCCL on a GPU host and gloo otherwise, so
the same entry point runs the CPU oracle.
"""
import datetime
import os

import torch
import torch.distributed as dist

from .arguments import parse_args
from .global_vars import ALLOWED_MODES, env
from .parallel import mesh
from .utils.common import set_device, set_seed
from .utils.logging import get_logger, init_logger

_DEFAULT_SEED = 1024


def _get_version():
    """``version.txt`` of a checkout, the installed distribution's version otherwise (reference: initialize.py:13-21
    reads ``version.txt`` and falls back to 0.0.0)."""
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "version.txt")
    try:
        with open(path) as f:
            return f.read().strip() or "0.0.0"
    except OSError:
        pass
    try:
        from importlib.metadata import version
        return version("cubework_b200")
    except Exception:  # noqa: BLE001
        return "0.0.0"


__version__ = _get_version()


def initialize_distributed(parser=None, argv=None, timeout_s: float = 1800.0):
    args = parse_args(parser, argv)
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    world_size = int(os.environ["WORLD_SIZE"])
    addr = os.environ["MASTER_ADDR"]
    port = int(os.environ["MASTER_PORT"])

    backend = args.backend or ("nccl" if torch.cuda.is_available() else "gloo")
    set_device(local_rank)
    kwargs = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(rank=rank, world_size=world_size, backend=backend, init_method=f"tcp://{addr}:{port}",
                            timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    init_logger()
    logger = get_logger()
    logger.info(f"cubework_b200 v{__version__}")

    mesh.init_global()
    tp = args.tensor_parallel_size if (args.tensor_parallel is not None and args.tensor_parallel_size) else None
    if args.tensor_parallel is not None and tp is None:
        tp = world_size
        args.tensor_parallel_size = tp
    dp = world_size if tp is None else world_size // tp
    mesh.init_data_parallel(dp)

    seed = args.seed if args.seed is not None else _DEFAULT_SEED
    set_seed(seed)

    env.load(mode=args.tensor_parallel)
    assert env.mode in ALLOWED_MODES
    if env.mode is not None:
        mesh.init_tensor_parallel(tp, seed)
        logger.info(f"Using {env.mode.upper()} tensor parallelism (tp={tp}, dp={dp})")
    else:
        logger.info(f"Using data parallelism (dp={dp})")
    return args
