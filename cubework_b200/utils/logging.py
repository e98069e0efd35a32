"""Rank-aware logger.

Parity: cubework/utils/logging.py:8-61 — logger ``"cubework"``, INFO on global rank 0 and ERROR on the
other ranks, third-party loggers quietened, optional per-rank log file ``name_rank_N.ext``.
``rich`` formatting is used when the package is importable and plain ``logging`` otherwise.
"""
import logging
import os

import torch.distributed as dist

_NAME = "cubework"
_FORMAT = "%(asctime)s %(levelname)s %(message)s"


def get_logger():
    return logging.getLogger(_NAME)


def _rank():
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else int(os.environ.get("RANK", 0))


def init_logger(quiet_others: bool = True):
    logger = get_logger()
    for h in list(logger.handlers):
        logger.removeHandler(h)
    try:
        from rich.logging import RichHandler
        handler = RichHandler(show_path=False, markup=False)
        handler.setFormatter(logging.Formatter("%(message)s"))
    except Exception:
        handler = logging.StreamHandler()
        handler.setFormatter(logging.Formatter(_FORMAT))
    logger.addHandler(handler)
    logger.propagate = False
    logger.setLevel(logging.INFO if _rank() == 0 else logging.ERROR)
    if quiet_others:
        for name in list(logging.root.manager.loggerDict):
            if not name.startswith(_NAME):
                logging.getLogger(name).setLevel(logging.ERROR)
    return logger


def write_logger_to_file(path, mode="a", level=logging.INFO):
    """Add a file handler writing to ``<stem>_rank_<N><ext>``; every rank logs at ``level`` there."""
    stem, ext = os.path.splitext(path)
    fname = f"{stem}_rank_{_rank()}{ext}"
    os.makedirs(os.path.dirname(os.path.abspath(fname)), exist_ok=True)
    handler = logging.FileHandler(fname, mode=mode)
    handler.setLevel(level)
    handler.setFormatter(logging.Formatter(_FORMAT))
    logger = get_logger()
    logger.addHandler(handler)
    if logger.level > level:
        logger.setLevel(level)
        for h in logger.handlers:
            if not isinstance(h, logging.FileHandler) and _rank() != 0:
                h.setLevel(logging.ERROR)
    return fname
